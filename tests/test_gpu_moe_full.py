"""The MoE layer at the baseline's full size (hidden 2048, 256 routed experts of 512 x 2048 gate / up and 2048 x 512 down,
top-8) against the FP64 oracle layer over the exact weights: the fused decode step at 1, 2 and 4 tokens with the router
on the device, and the batched (prefill) layer at 2048 and 8192 tokens on a sample of tokens. Needs nothing but this
repository: every expert has its own seed, so the oracle regenerates only the experts the checked tokens use."""
import numpy as np
import pytest
import torch

from conftest import BF16_REL, HARD_REL, bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
E, TOPK, H, N = 256, 8, 2048, 512


def expert_bits(e: int):
    return o.weights_like(N, H, 7000 + 3 * e), o.weights_like(N, H, 7001 + 3 * e), o.weights_like(H, N, 7002 + 3 * e)


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


@pytest.fixture(scope="module")
def experts(ops):
    """All 256 experts encoded in the llama.cpp layout (chunk-major R = 8 gate / up, row-major R = 16 down)."""
    parts = [expert_bits(e) for e in range(E)]
    out = []
    for i, (R, cm) in enumerate(((8, True), (8, True), (16, False))):
        w = np.concatenate([p[i] for p in parts], axis=0)
        plane, aux, meta = ops.encode(to_bf16_tensor(w), 3, R, cm)
        assert meta.format == 3
        out.append(ops.upload(plane, aux, meta, "cuda"))
    return out


def oracle_layer(x_bits, wts, ids, bf16_act):
    """FP64 layer output for the given tokens, generating only the experts they use."""
    used = sorted({int(e) for e in ids.reshape(-1)})
    pos = {e: i for i, e in enumerate(used)}
    ws = [expert_bits(e) for e in used]
    gb, ub, db = (np.concatenate([w[i] for w in ws], axis=0) for i in range(3))
    ids_c = np.vectorize(lambda e: pos[int(e)])(ids).astype(np.int32)
    return o.moe_layer_f64(o.bf16_bits_to_f32(x_bits), gb, ub, db, wts, ids_c, len(used), bf16_act=bf16_act)


@pytest.mark.parametrize("T", [1, 2, 4])
def test_decode_step_full_size(ops, experts, T):
    gate, up, down = experts
    g = np.random.default_rng(100 + T)
    xb = o.f32_to_bf16_bits(g.standard_normal((T, H)).astype(np.float32))
    logits = g.standard_normal((T, E)).astype(np.float32)
    y, wts, ids = ops.moe_decode(to_bf16_tensor(xb).cuda(), gate, up, down, E, TOPK, router_logits=torch.from_numpy(logits).cuda())
    ids_ref, w_ref = o.softmax_topk(logits, TOPK)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert np.allclose(wts.cpu().numpy(), w_ref, rtol=1e-5)
    ref = oracle_layer(xb, wts.cpu().numpy(), ids.cpu().numpy(), False)
    assert np.abs(y.cpu().numpy() - ref).max() <= HARD_REL * np.abs(ref).max()
    assert ops.fault_status() == 0


@pytest.mark.parametrize("T", [2048, 8192])
def test_prefill_layer_full_size(ops, experts, T):
    gate, up, down = experts
    g = torch.Generator(device="cuda").manual_seed(200 + T)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    wts, ids = ops.moe_topk(torch.randn(T, E, device="cuda", generator=g), TOPK)
    y = ops.moe_experts(x, gate, up, down, wts, ids, E)          # BF16 [T, H]
    sample = [0, 1, T // 2, T - 1]
    ref = oracle_layer(bits_of(x[sample]), wts[sample].cpu().numpy(), ids[sample].cpu().numpy(), True)
    got = y[sample].float().cpu().numpy()
    assert np.abs(got - ref).max() <= BF16_REL * np.abs(ref).max()
    assert ops.fault_status() == 0
