"""`torch.ops.bf16n` on the GPU: torch.library.opcheck on every op (schema, fake kernels against the real ones,
AOT dispatch with dynamic shapes), equality with the `ops` functions underneath, and CUDA-graph capture of a
decode-like step replaying bitwise what eager execution computes after the inputs change in place. Mirrors the
reference's tests/core/test_opcheck.py and tests/core/test_graphs.py (without the fragment-order cases)."""
import pytest
import torch

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
NIB, HP = 1, 3
E, N, H, TOPK = 8, 512, 2048, 4


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    from orin_qwen_lossless_b200 import torch_ops  # noqa: F401
    assert torch.cuda.is_available()
    torch.ops.bf16n.init()
    return m


@pytest.fixture(scope="module")
def m(ops):
    def enc(rows, K, seed, fmt, R=0, cm=False):
        plane, aux, meta = ops.encode(to_bf16_tensor(o.weights_like(rows, K, seed)), fmt, R, cm)
        return ops.upload(plane, aux, meta, "cuda")
    return {"hp": enc(512, 2048, 1, HP, 16), "nib": enc(1024, 2048, 2, NIB), "gate": enc(E * N, H, 3, HP, 8, True),
            "up": enc(E * N, H, 4, HP, 8, True), "down": enc(E * H, N, 5, HP, 16)}


def cases(m):
    b = torch.ops.bf16n
    g = torch.Generator().manual_seed(3)
    x4 = torch.randn(4, 2048, generator=g).to(torch.bfloat16).cuda()
    x12 = torch.randn(12, 2048, generator=g).to(torch.bfloat16).cuda()
    a12 = torch.randn(12, TOPK, 512, generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:TOPK] for _ in range(12)]).to(torch.int32).cuda()
    hp, nib, gate, up, down = m["hp"], m["nib"], m["gate"], m["up"], m["down"]
    w2 = to_bf16_tensor(o.weights_like(64, 2048, 9)).cuda()
    return {
        "dequant": (b.dequant, (hp.plane, hp.aux, hp.m, 16, 32)),
        "mmv_dense": (b.mmv, (x4, hp.plane, hp.aux, hp.m, None, 0, True)),
        "mmv_ids": (b.mmv, (x4, gate.plane, gate.aux, gate.m, ids[:4], 512, False)),
        "mmv_glu": (b.mmv_glu, (x4, nib.plane, nib.aux, nib.m, None, 0, True)),
        "linear_gemv": (b.linear, (x4, hp.plane, hp.aux, hp.m, None)),
        "linear_gemm": (b.linear, (x12.view(3, 4, 2048), hp.plane, hp.aux, hp.m, None)),
        "get_rows": (b.get_rows, (ids[:, 0].long(), hp.plane, hp.aux, hp.m, True)),
        "moe_mm_ids_glu": (b.moe_mm_ids, (x12, ids, gate.plane, gate.aux, gate.m, up.plane, up.aux, up.m, E, True)),
        "moe_mm_ids_down": (b.moe_mm_ids, (a12, ids, down.plane, down.aux, down.m, None, None, [], E, False)),
        "moe_combine": (b.moe_combine, (torch.randn(12, TOPK, 2048, device="cuda"), torch.rand(12, TOPK, device="cuda"), True)),
        "swiglu": (b.swiglu, (torch.randn(12, TOPK, 512, device="cuda"), torch.randn(12, TOPK, 512, device="cuda"))),
        "int2_quantize": (b.int2_quantize, (w2,)),
        "int2_gemv": (b.int2_gemv, (x4[:1], *b.int2_quantize(w2))),
        "int4_quantize": (b.int4_quantize, (w2,)),
        "int4_gemv": (b.int4_gemv, (x4[:1], *b.int4_quantize(w2))),
    }


NAMES = ["dequant", "mmv_dense", "mmv_ids", "mmv_glu", "linear_gemv", "linear_gemm", "get_rows", "moe_mm_ids_glu",
         "moe_mm_ids_down", "moe_combine", "swiglu", "int2_quantize", "int2_gemv", "int4_quantize", "int4_gemv"]


@pytest.mark.parametrize("name", NAMES)
def test_opcheck(ops, m, name):
    op, args = cases(m)[name]
    torch.library.opcheck(op, args, test_utils=("test_schema", "test_autograd_registration", "test_faketensor",
                                                "test_aot_dispatch_dynamic"))


def test_ops_equal_the_functions_underneath(ops, m):
    c = cases(m)
    hp, nib, gate, up = m["hp"], m["nib"], m["gate"], m["up"]
    x4, ids = c["mmv_dense"][1][0], c["moe_mm_ids_glu"][1][1]
    x12 = c["moe_mm_ids_glu"][1][0]

    def same(a, b):
        return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))

    b = torch.ops.bf16n
    assert same(b.dequant(hp.plane, hp.aux, hp.m, 16, 32), ops.dequant(hp, 16, 32))
    assert same(b.mmv(x4, hp.plane, hp.aux, hp.m, None, 0, True), ops.mmv(x4, hp, out_dtype=torch.bfloat16))
    assert same(b.mmv_glu(x4, nib.plane, nib.aux, nib.m, None, 0, False), ops.mmv_glu(x4, nib))
    assert same(b.linear(x4, hp.plane, hp.aux, hp.m, None), ops.linear(x4, hp))
    assert same(b.moe_mm_ids(x12, ids, gate.plane, gate.aux, gate.m, up.plane, up.aux, up.m, E, True),
                ops.moe_mm_ids(x12, ids, gate, E, up=up, out_dtype=torch.bfloat16))


def test_invalid_arguments_raise_value_error(ops, m):
    hp = m["hp"]
    x = torch.randn(4, 2048, device="cuda").to(torch.bfloat16)
    with pytest.raises(ValueError, match="whole units"):
        torch.ops.bf16n.dequant(hp.plane, hp.aux, hp.m, 8, 16)
    with pytest.raises(ValueError, match="meta must be"):
        torch.ops.bf16n.mmv(x, hp.plane, hp.aux, hp.m[:5], None, 0, True)


def step(ops, w, x, ids, wts):
    """One decode-like step through the ops a serving engine captures into its graphs."""
    b = torch.ops.bf16n
    hp, nib = w["hp"], w["nib"]
    return [b.linear(x, hp.plane, hp.aux, hp.m, None), b.mmv_glu(x, nib.plane, nib.aux, nib.m, None, 0, True),
            ops.moe_experts(x, w["gate"], w["up"], w["down"], wts, ids, E),
            b.get_rows(ids[:, 0].long(), hp.plane, hp.aux, hp.m, True)]


def inputs(T, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, 2048, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:TOPK] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, TOPK, generator=g)
    return x.cuda(), ids.cuda(), (w / w.sum(1, keepdim=True)).cuda()


@pytest.mark.parametrize("T", [1, 2, 4, 12])
def test_capture_replay_bitwise(ops, m, T):
    x, ids, wts = inputs(T, seed=T)
    step(ops, m, x, ids, wts)  # warm-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        outs = step(ops, m, x, ids, wts)
    for seed in (100 + T, 200 + T):  # new inputs written in place before each replay
        nx, nids, nw = inputs(T, seed)
        x.copy_(nx); ids.copy_(nids); wts.copy_(nw)
        g.replay()
        torch.cuda.synchronize()
        eager = step(ops, m, x, ids, wts)
        for a, e in zip(outs, eager):
            assert torch.equal(a.view(torch.int16), e.view(torch.int16))
