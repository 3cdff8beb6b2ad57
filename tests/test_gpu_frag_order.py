"""Fragment-order HUFPAIR tensors (16-row bands in mma A-fragment order, the layout the reference's vLLM policy picks for
experts, linear layers and lm_head): bit-exact device reconstruction and verify, row gather, and the decode GEMV against
FP64 over the exact weights for 1..8 dense tokens and for routed (token, slot) columns. Shapes and seeds follow the
fragment-order cases of the reference's tests/core/test_roundtrip.py and test_kernels.py."""
import numpy as np
import pytest
import torch

from conftest import GEMV_REL, bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
HP = 3


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


def fo(ops, bits):
    plane, aux, meta = ops.encode(to_bf16_tensor(bits), HP, 16, False, True)
    assert meta.frag_order and meta.R == 16
    return ops.upload(plane, aux, meta, "cuda")


def act(shape, seed):
    xb = o.f32_to_bf16_bits(np.random.default_rng(500 + seed).standard_normal(shape).astype(np.float32))
    return to_bf16_tensor(xb).cuda(), o.bf16_bits_to_f32(xb).astype(np.float64)


@pytest.mark.parametrize("rows,K", [(16, 512), (64, 512), (2048, 512), (512, 2048), (48, 1024), (32, 4096)])
def test_roundtrip_and_verify(ops, rows, K):
    bits = o.with_specials(o.weights_like(rows, K, rows + K), rows + K).reshape(rows, K)  # NaN, infinities, denormals, zeros too
    w = fo(ops, bits)
    src = to_bf16_tensor(bits).cuda()
    assert torch.equal(ops.dequant(w).view(torch.int16), src.view(torch.int16))
    assert ops.mismatches(w, src) == 0
    if rows >= 48:  # a band range in the middle
        assert torch.equal(ops.dequant(w, 16, 32).view(torch.int16), src[16:48].view(torch.int16))
    bad = src.clone()
    bad.view(torch.int16)[rows - 1, K - 3] ^= 0x0100
    bad.view(torch.int16)[0, 17] ^= 0x0001
    assert ops.mismatches(w, bad) == 2


def test_matches_the_oracle_decoder_bytes(ops):
    bits = o.weights_like(64, 1024, 9)
    plane, aux, meta = ops.encode(to_bf16_tensor(bits), HP, 16, False, True)
    op, oa, _ = o.encode(bits, HP, 16, False, True)
    assert np.array_equal(plane.numpy().ravel(), op.ravel()) and np.array_equal(aux.numpy(), oa)
    assert np.array_equal(o.decode(op, oa), bits)


@pytest.mark.parametrize("T", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("rows,K", [(2048, 512), (512, 2048), (160, 1024)])
def test_dense_gemv_against_fp64(ops, rows, K, T):
    bits = o.weights_like(rows, K, 3 * rows + K)
    w = fo(ops, bits)
    x, x64 = act((T, K), T)
    w64 = o.bf16_bits_to_f32(bits).astype(np.float64)
    ref, s = x64 @ w64.T, np.abs(x64) @ np.abs(w64).T
    y = ops.mmv(x, w)
    assert y.shape == (T, rows) and y.dtype == torch.float32
    assert (np.abs(y.cpu().numpy() - ref) <= GEMV_REL * s).all()
    # several BF16 tokens run on the tensor cores, one token and FP32 activations on FMAs: all within the bound, and a
    # column's result does not depend on what it is batched with (first column of a 2-token batch vs of the full batch)
    yf = ops.mmv(x.float(), w)
    assert (np.abs(yf.cpu().numpy() - ref) <= GEMV_REL * s).all()
    if T >= 2:
        assert torch.equal(ops.mmv(x[:2].contiguous(), w)[0], y[0])
    yb = ops.mmv(x, w, out_dtype=torch.bfloat16)
    assert torch.equal(yb.view(torch.int16), y.to(torch.bfloat16).view(torch.int16))


@pytest.mark.parametrize("K,T", [(512, 1), (512, 8), (2048, 1), (2048, 5)])
def test_large_matrix_kernel(ops, K, T):
    """At least 16 bands per SM: the persistent kernel with bulk-copy staged streams (also for one token)."""
    rows = 16 * 16 * 160
    bits = o.weights_like(rows, K, K + T)
    w = fo(ops, bits)
    x, x64 = act((T, K), 30 + T)
    w64 = o.bf16_bits_to_f32(bits).astype(np.float64)
    ref, s = x64 @ w64.T, np.abs(x64) @ np.abs(w64).T
    y = ops.mmv(x, w)
    assert (np.abs(y.cpu().numpy() - ref) <= GEMV_REL * s).all()
    assert torch.equal(ops.mmv(x[:1].contiguous(), w)[0], y[0])  # a column does not depend on its batch


@pytest.mark.parametrize("K,rows_e", [(512, 512), (2048, 80), (1024, 48)])
@pytest.mark.parametrize("fp32_x", [False, True])
def test_routed_columns(ops, K, rows_e, fp32_x):
    """Routed columns (expert ids): the kernel that puts a band's slabs on separate warps, 1, 4 and 2 slabs per band,
    bands that do not fill the last block, BF16 and FP32 activations."""
    E, T, k = 4, 3, 2
    bits = o.weights_like(E * rows_e, K, 77 + K)
    w = fo(ops, bits)
    ids = torch.tensor([[0, 3], [2, 2], [1, 0]], dtype=torch.int32, device="cuda")
    x, x64 = act((T, k, K), 4)
    y = ops.mmv(x.float() if fp32_x else x, w, ids, rows_e)
    assert y.shape == (T, k, rows_e)
    w64 = o.bf16_bits_to_f32(bits).astype(np.float64).reshape(E, rows_e, K)
    for t in range(T):
        for s_ in range(k):
            e = int(ids[t, s_])
            ref, s = w64[e] @ x64[t, s_], np.abs(w64[e]) @ np.abs(x64[t, s_])
            assert (np.abs(y[t, s_].cpu().numpy() - ref) <= GEMV_REL * s).all()


@pytest.mark.parametrize("K,rows_e,per_slot", [(2048, 64, False), (512, 96, True)])
@pytest.mark.parametrize("fp32_x", [False, True])
def test_columns_of_one_expert_share_a_decode_with_the_same_bits(ops, K, rows_e, per_slot, fp32_x):
    """Routed columns of 4..8 tokens are grouped by expert inside the kernel (two columns per decode; a third starts a
    new group): every (token, slot) pair gets the bits it gets when its token is multiplied alone, whatever
    else is in the batch. Routings: every token picks the same experts, one expert in every slot of every token, and a
    mix with unshared experts."""
    E, k = 6, 4
    bits = o.weights_like(E * rows_e, K, 91 + K)
    w = fo(ops, bits)
    for T, routing in [(8, "same"), (7, "one_expert"), (5, "mixed"), (4, "same"), (2, "same")]:
        g = np.random.default_rng(T)
        if routing == "same":
            ids_np = np.tile(g.permutation(E)[:k], (T, 1))
        elif routing == "one_expert":
            ids_np = np.full((T, k), 3)
        else:
            ids_np = np.stack([g.permutation(E)[:k] for _ in range(T)])
        ids = torch.from_numpy(ids_np.astype(np.int32)).cuda()
        x, _ = act((T, k, K) if per_slot else (T, K), 11 + T)
        x = x.float() if fp32_x else x
        y = ops.mmv(x, w, ids, rows_e)
        for t in range(T):
            alone = ops.mmv(x[t:t + 1], w, ids[t:t + 1], rows_e)
            assert torch.equal(y[t:t + 1], alone), (routing, T, t)
    assert ops.fault_status() == 0


def test_get_rows_and_linear(ops):
    rows, K = 256, 2048
    bits = o.weights_like(rows, K, 5)
    w = fo(ops, bits)
    src = to_bf16_tensor(bits).cuda()
    ids = torch.tensor([0, 255, 17, 8, 129, 17], dtype=torch.int64, device="cuda")
    assert torch.equal(ops.get_rows(ids, w).view(torch.int16), src[ids].view(torch.int16))
    assert torch.equal(ops.get_rows(ids.int(), w, torch.float32), src[ids].float())
    x, _ = act((12, K), 6)  # more than 8 tokens: exact dequantisation + GEMM
    assert torch.equal(ops.linear(x, w).view(torch.int16), (x @ src.t()).view(torch.int16))


def test_batched_kernel_is_offered(ops):
    bits = o.weights_like(4 * 512, 2048, 6)
    w = fo(ops, bits)
    assert ops.mm_ids_supported(w) and ops.mm_ids_supported(w, w)  # the batched cases themselves: test_gpu_prefill.py
