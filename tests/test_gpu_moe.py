"""The fused MoE decode step (router on the device, gate+up in one launch, SwiGLU folded into the down product,
combine) against the unfused operator chain (bitwise), the FP64 oracle layer, and under expert parallelism."""
import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
E, K_TOP, H, N = 16, 8, 2048, 512


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


@pytest.fixture(scope="module")
def layer(ops):
    bits = {"gate": o.weights_like(E * N, H, 11), "up": o.weights_like(E * N, H, 12), "down": o.weights_like(E * H, N, 13)}

    def enc(w, R, cm, lo=0, n=E):
        rows = w.shape[0] // E
        plane, aux, meta = ops.encode(to_bf16_tensor(w[lo * rows:(lo + n) * rows]), 3, R, cm)
        return ops.upload(plane, aux, meta, "cuda")

    return bits, enc


def inputs(T, seed, dtype=torch.bfloat16):
    g = np.random.default_rng(seed)
    xb = o.f32_to_bf16_bits(g.standard_normal((T, H)).astype(np.float32))
    logits = g.standard_normal((T, E)).astype(np.float32)
    return to_bf16_tensor(xb).cuda().to(dtype), o.bf16_bits_to_f32(xb), torch.from_numpy(logits).cuda(), logits


@pytest.mark.parametrize("T", [1, 2, 4, 8])
@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float32])
def test_fused_step_equals_operator_chain(ops, layer, T, xdt):
    bits, enc = layer
    g, u, d = enc(bits["gate"], 8, True), enc(bits["up"], 8, True), enc(bits["down"], 16, False)
    x, xf, logits, logits_np = inputs(T, T, xdt)
    y, wts, ids = ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits)
    ids_ref, w_ref = o.softmax_topk(logits_np, K_TOP)
    assert np.array_equal(ids.cpu().numpy(), ids_ref) and np.allclose(wts.cpu().numpy(), w_ref, rtol=1e-5)
    # the reference's five-launch chain with the same routing
    gg, uu = ops.mmv(x, g, ids, N), ops.mmv(x, u, ids, N)
    ys = ops.mmv(ops.swiglu(gg, uu), d, ids, H)
    chain = ops.moe_combine(ys, wts, torch.float32)
    assert torch.equal(y, chain)
    # routing given instead of logits, BF16 output = rounding of the FP32 output
    y2, _, _ = ops.moe_decode(x, g, u, d, E, K_TOP, topk_weights=wts, topk_ids=ids, out_dtype=torch.bfloat16)
    assert torch.equal(y2.view(torch.int16), y.to(torch.bfloat16).view(torch.int16))
    ref = o.moe_layer_f64(xf, bits["gate"], bits["up"], bits["down"], wts.cpu().numpy(), ids.cpu().numpy(), E)
    assert np.abs(y.cpu().numpy() - ref).max() <= 2.0 ** -10 * np.abs(ref).max()


@pytest.mark.parametrize("ranks", [2, 4])
def test_expert_parallel_partials_add_up(ops, layer, ranks):
    """Each rank holds a slice of the experts and adds zeros for the slots routed elsewhere: the partial outputs sum to
    the single-GPU result (up to the FP32 reassociation of the final sum)."""
    bits, enc = layer
    g, u, d = enc(bits["gate"], 8, True), enc(bits["up"], 8, True), enc(bits["down"], 16, False)
    x, _, logits, _ = inputs(4, 99)
    full, wts, ids = ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits)
    n = E // ranks
    total = torch.zeros_like(full, dtype=torch.float64)
    for r in range(ranks):
        gr, ur, dr = enc(bits["gate"], 8, True, r * n, n), enc(bits["up"], 8, True, r * n, n), enc(bits["down"], 16, False, r * n, n)
        part, w2, i2 = ops.moe_decode(x, gr, ur, dr, E, K_TOP, router_logits=logits, expert_lo=r * n, n_experts_local=n)
        assert torch.equal(i2, ids) and torch.equal(w2, wts)
        total += part.double()
    assert torch.allclose(total, full.double(), rtol=0, atol=2.0 ** -18 * float(full.abs().max()) * K_TOP)


@pytest.mark.parametrize("T", [1, 2, 4])
def test_step_over_fragment_order_experts(ops, layer, T):
    """The vLLM layout (16-row fragment-order bands for gate, up and down) through the same entry point: equal to the
    operator chain over the same weights (bitwise) and within the bound of the FP64 layer; an expert slice is refused."""
    bits, _ = layer

    def enc_fo(w):
        plane, aux, meta = ops.encode(to_bf16_tensor(w), 3, 16, False, True)
        return ops.upload(plane, aux, meta, "cuda")

    g, u, d = enc_fo(bits["gate"]), enc_fo(bits["up"]), enc_fo(bits["down"])
    x, xf, logits, _ = inputs(T, 40 + T)
    y, wts, ids = ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits)
    gg, uu = ops.mmv(x, g, ids, N), ops.mmv(x, u, ids, N)
    chain = ops.moe_combine(ops.mmv(ops.swiglu(gg, uu), d, ids, H), wts, torch.float32)
    assert torch.equal(y, chain)
    ref = o.moe_layer_f64(xf, bits["gate"], bits["up"], bits["down"], wts.cpu().numpy(), ids.cpu().numpy(), E)
    assert np.abs(y.cpu().numpy() - ref).max() <= 2.0 ** -10 * np.abs(ref).max()
    with pytest.raises(ValueError, match="no expert slice"):
        ops.moe_decode(x, g, u, d, 2 * E, K_TOP, topk_weights=wts, topk_ids=ids, expert_lo=0, n_experts_local=E)


def test_fused_step_in_a_cuda_graph(ops, layer):
    bits, enc = layer
    g, u, d = enc(bits["gate"], 8, True), enc(bits["up"], 8, True), enc(bits["down"], 16, False)
    x, _, logits, _ = inputs(2, 5)
    scratch = ops.moe_decode_scratch(2, K_TOP, g, d, E, x.device)
    out = torch.empty(2, H, device="cuda")
    wts = torch.empty(2, K_TOP, device="cuda")
    ids = torch.empty(2, K_TOP, dtype=torch.int32, device="cuda")
    ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits, topk_weights=wts, topk_ids=ids, scratch=scratch, out=out)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits, topk_weights=wts, topk_ids=ids, scratch=scratch, out=out)
    x2, _, logits2, _ = inputs(2, 6)
    x.copy_(x2), logits.copy_(logits2)
    gr.replay()
    torch.cuda.synchronize()
    want, _, _ = ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits)
    assert torch.equal(out, want)


def test_argument_errors(ops, layer):
    bits, enc = layer
    g, u, d = enc(bits["gate"], 8, True), enc(bits["up"], 8, True), enc(bits["down"], 16, False)
    x, _, logits, _ = inputs(1, 1)
    with pytest.raises(ValueError, match="chunk-major"):
        ops.moe_decode(x, enc(bits["gate"], 8, False), u, d, E, K_TOP, router_logits=logits)
    with pytest.raises(ValueError, match="scratch too small"):
        ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits, scratch=torch.empty(16, device="cuda"))
    with pytest.raises(ValueError, match="expert slice"):
        ops.moe_decode(x, g, u, d, E, K_TOP, router_logits=logits, expert_lo=8, n_experts_local=16)
