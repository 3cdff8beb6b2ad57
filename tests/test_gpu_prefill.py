"""Batched (prefill) routed products on the tensor cores against FP64 references over the exact weights: gate only,
fused gate/up + SwiGLU, down with per-slot activations, and the whole > 8 token MoE layer; token counts around the tile
sizes, skewed routing (one expert takes every token, half of the experts empty), int32 / int64 ids. Mirrors the
reference's tests/core/test_kernels.py MoE cases (T in {9, 48, 97, 128, 129, ...} x routing kinds)."""
import numpy as np
import pytest
import torch

from conftest import BF16_REL, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
E, TOPK, H, N = 8, 4, 2048, 512
MMA_REL = 2e-6  # FP32 tensor-core accumulation, relative to sum |w x| (the reference measures <= 7e-7 for its batched path)


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


@pytest.fixture(scope="module", params=["lane_major", "lane_major_two_pass", "fragment_order"])
def layer(ops, request):
    """The expert weights in the llama.cpp layout (chunk-major R = 8 gate / up, row-major R = 16 down: tcgen05 kernels;
    once with the fused decode-and-multiply kernel, once with a workspace registered, i.e. the decode pass into operand
    tiles followed by the tensor-core pass) and in the vLLM layout (16-row fragment-order bands everywhere: the
    mma.m16n8k16 batched kernel)."""
    bits = {"gate": o.weights_like(E * N, H, 21), "up": o.weights_like(E * N, H, 22), "down": o.weights_like(E * H, N, 23)}
    fo = request.param == "fragment_order"

    def enc(w, R, cm):
        plane, aux, meta = ops.encode(to_bf16_tensor(w), 3, 16 if fo else R, False if fo else cm, fo)
        return ops.upload(plane, aux, meta, "cuda")

    enc_w = {"gate": enc(bits["gate"], 8, True), "up": enc(bits["up"], 8, True), "down": enc(bits["down"], 16, False)}
    f64 = {k: o.bf16_bits_to_f32(v).astype(np.float64) for k, v in bits.items()}
    if request.param == "lane_major_two_pass":
        assert ops.mm_ids_workspace_bytes(enc_w["gate"], enc_w["up"]) == 2 * E * N * H * 2
        assert ops.mm_ids_workspace_bytes(enc_w["down"]) == E * H * N * 2
        assert ops.ensure_workspace((enc_w["gate"], enc_w["up"]), (enc_w["down"], None)) >= 2 * E * N * H * 2
    elif fo:
        assert ops.mm_ids_workspace_bytes(enc_w["gate"], enc_w["up"]) == 0
    yield bits, enc_w, f64
    torch.cuda.synchronize()
    ops.set_workspace(None)
    assert ops.fault_status() == 0


def routing(T, kind, seed):
    g = np.random.default_rng(seed)
    if kind == "uniform":
        return np.stack([g.permutation(E)[:TOPK] for _ in range(T)]).astype(np.int64)
    if kind == "one_expert_all":  # expert 5 is in every token's list
        ids = np.stack([g.permutation(E - 1)[:TOPK - 1] for _ in range(T)]).astype(np.int64)
        ids = np.where(ids >= 5, ids + 1, ids)
        return np.concatenate([np.full((T, 1), 5), ids], axis=1)
    ids = np.stack([g.permutation(E // 2)[:TOPK] for _ in range(T)]).astype(np.int64)  # half_empty: experts 4..7 unused
    return ids


def act(shape, seed):
    xb = o.f32_to_bf16_bits(np.random.default_rng(seed).standard_normal(shape).astype(np.float32))
    return to_bf16_tensor(xb).cuda(), o.bf16_bits_to_f32(xb).astype(np.float64)


def expert_products(w64, rows, ids, x64, per_slot):
    """y[t, s, :] = W_e x and S = |W_e| |x| in FP64."""
    T, k = ids.shape
    y = np.zeros((T, k, rows))
    S = np.zeros((T, k, rows))
    for e in np.unique(ids):
        tt, ss = np.nonzero(ids == e)
        We = w64[e * rows:(e + 1) * rows]
        xe = x64[tt, ss] if per_slot else x64[tt]
        y[tt, ss] = xe @ We.T
        S[tt, ss] = np.abs(xe) @ np.abs(We).T
    return y, S


@pytest.mark.parametrize("T", [9, 48, 97, 128, 129, 300])
@pytest.mark.parametrize("kind", ["uniform", "one_expert_all", "half_empty"])
def test_gate_only_and_fused_glu(ops, layer, T, kind):
    bits, w, f64 = layer
    ids_np = routing(T, kind, T)
    ids = torch.from_numpy(ids_np).to(torch.int32 if T % 2 else torch.int64).cuda()
    x, x64 = act((T, H), T + 1)
    g_ref, Sg = expert_products(f64["gate"], N, ids_np, x64, False)
    u_ref, Su = expert_products(f64["up"], N, ids_np, x64, False)
    g = ops.moe_mm_ids(x, ids, w["gate"], E)
    assert g.shape == (T, TOPK, N) and g.dtype == torch.float32
    assert (np.abs(g.cpu().numpy() - g_ref) <= MMA_REL * Sg + 1e-30).all()
    a = ops.moe_mm_ids(x, ids, w["gate"], E, up=w["up"], out_dtype=torch.bfloat16)
    a_ref = o.silu(g_ref) * u_ref
    # error of the product of two sums + the BF16 rounding of the output
    bound = BF16_REL * np.abs(a_ref) + 4 * MMA_REL * (Sg * np.abs(u_ref) + np.abs(o.silu(g_ref)) * Su + Sg * Su) + 1e-30
    assert a.dtype == torch.bfloat16 and (np.abs(a.float().cpu().numpy() - a_ref) <= bound).all()
    a32 = ops.moe_mm_ids(x, ids, w["gate"], E, up=w["up"], out_dtype=torch.float32)
    assert torch.equal(a32.to(torch.bfloat16).view(torch.int16), a.view(torch.int16))


@pytest.mark.parametrize("T", [9, 64, 257, 700])
def test_down_with_per_slot_activations(ops, layer, T):
    bits, w, f64 = layer
    ids_np = routing(T, "uniform" if T != 257 else "one_expert_all", 3 * T)
    ids = torch.from_numpy(ids_np).to(torch.int32).cuda()
    a, a64 = act((T, TOPK, N), T + 7)
    y_ref, S = expert_products(f64["down"], H, ids_np, a64, True)
    y = ops.moe_mm_ids(a, ids, w["down"], E)
    assert y.shape == (T, TOPK, H)
    assert (np.abs(y.cpu().numpy() - y_ref) <= MMA_REL * S + 1e-30).all()
    yb = ops.moe_mm_ids(a, ids, w["down"], E, out_dtype=torch.bfloat16)
    assert torch.equal(yb.view(torch.int16), y.to(torch.bfloat16).view(torch.int16))


@pytest.mark.parametrize("T", [9, 127, 2048])
def test_moe_layer_batched_path(ops, layer, T):
    bits, w, f64 = layer
    x, x64 = act((T, H), T + 3)
    logits = np.random.default_rng(T).standard_normal((T, E)).astype(np.float32)
    wts, ids = ops.moe_topk(torch.from_numpy(logits).cuda(), TOPK)
    y = ops.moe_experts(x, w["gate"], w["up"], w["down"], wts, ids, E)
    assert y.shape == (T, H) and y.dtype == torch.bfloat16
    n = min(T, 64)  # the FP64 layer is slow: check a sample of tokens
    ref = o.moe_layer_f64(x64[:n].astype(np.float32), bits["gate"], bits["up"], bits["down"], wts.cpu().numpy()[:n],
                          ids.cpu().numpy()[:n], E, bf16_act=True)
    err = np.abs(y.float().cpu().numpy()[:n] - ref)
    assert err.max() <= 2.0 ** -6 * np.abs(ref).max()


def test_workspace_on_demand(ops, layer):
    """set_auto_workspace: the batched operator registers a workspace of the needed size itself (two-pass form from then
    on); results agree with the fused kernel to accumulation order."""
    bits, w, f64 = layer
    if w["gate"].meta.frag_order or ops.mm_ids_workspace_bytes(w["down"]) == 0:
        pytest.skip("lane-major experts only")
    x, _ = act((40, H), 5)
    ids = torch.from_numpy(routing(40, "uniform", 40).astype(np.int32)).cuda()
    had_workspace = ops._workspace is not None
    ops.set_workspace(None)
    fused = ops.moe_mm_ids(x, ids, w["gate"], E)
    ops.set_auto_workspace(True)
    try:
        two = ops.moe_mm_ids(x, ids, w["gate"], E)
        assert ops.ensure_workspace((w["gate"], None)) >= E * N * H * 2
    finally:
        ops.set_auto_workspace(False)
    assert torch.allclose(two, fused, rtol=0, atol=1e-5 * float(fused.abs().max()))
    torch.cuda.synchronize()
    ops.set_workspace(None)   # back to what the fixture set up for the other tests
    if had_workspace:
        ops.ensure_workspace((w["gate"], w["up"]), (w["down"], None))


def test_unsupported_shapes_are_rejected(ops, layer):
    bits, w, f64 = layer
    x, _ = act((9, H), 1)
    ids = torch.zeros((9, TOPK), dtype=torch.int32, device="cuda")
    plane, aux, meta = ops.encode(to_bf16_tensor(bits["gate"]), 3, 8, False)  # row-major K = 2048: no batched kernel
    rm = ops.upload(plane, aux, meta, "cuda")
    assert not ops.mm_ids_supported(rm) and ops.mm_ids_supported(w["gate"], w["up"]) and ops.mm_ids_supported(w["down"])
    with pytest.raises(ValueError, match="no batched kernel"):
        ops.moe_mm_ids(x, ids, rm, E)


def test_device_side_dispatch_on_one_rank(ops, layer):
    """The expert-parallel layer with its device-side exchange, degenerate on one rank (every row is sent to this rank's
    own inbox): bit-equal to the single-GPU layer, which pins the plan, inbox, routing-over-inbox and give-back kernels."""
    from orin_qwen_lossless_b200 import sharded
    bits, enc_w, _ = layer
    if enc_w["gate"].meta.frag_order:
        pytest.skip("lane-major experts only")
    fmp = sharded.FusedMoePrefill(enc_w["gate"], enc_w["up"], enc_w["down"], E, TOPK, 300)
    for T in (9, 130, 300):
        x, _ = act((T, H), 70 + T)
        ids = torch.from_numpy(routing(T, "uniform", T).astype(np.int32)).cuda()
        wts = torch.rand(T, TOPK, device="cuda")
        assert torch.equal(fmp(x, wts, ids), ops.moe_experts(x, enc_w["gate"], enc_w["up"], enc_w["down"], wts, ids, E))
    fmp.close()
