"""GEMV-family kernels against the CPU oracle: FP64 dot products over the exact weights with the reference's bound
|err| <= 1e-5 * sum|w x| (hard gate 2^-10), bitwise against the FP32 emulation of the reference summation order, and the
bitwise invariants of the reference's tests/core/test_kernels.py (BF16 vs FP32 staging, BF16 output = RNE of FP32,
multi-column = single column, fused GLU = unfused)."""
import numpy as np
import pytest
import torch

from conftest import BF16_REL, GEMV_REL, HARD_REL, bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
NIB, HUF, HP = 1, 2, 3
DENSE = {"nibble": (NIB, 0, 256), "huffman": (HUF, 8, 256), "hufpair": (HP, 16, 512)}
TOKENS = [1, 2, 4, 7, 8]


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


def up(ops, w_bits, fmt, R=0, cm=False):
    plane, aux, meta = ops.encode(to_bf16_tensor(w_bits), fmt, R, cm)
    return ops.upload(plane, aux, meta, "cuda")


def act(T, K, seed=0, dtype=torch.bfloat16):
    g = np.random.default_rng(1000 + seed)
    xb = o.f32_to_bf16_bits(g.standard_normal((T, K)).astype(np.float32))
    return to_bf16_tensor(xb).cuda().to(dtype), o.bf16_bits_to_f32(xb)


def ref64(w_bits, xf):
    ys, ss = zip(*(o.gemv_f64(w_bits, xf[t]) for t in range(xf.shape[0])))
    return np.stack(ys), np.stack(ss)


def assert_within(y, ref, S, rel=GEMV_REL, out_rel=0.0):
    err = np.abs(y.double().cpu().numpy().reshape(ref.shape) - ref)
    bound = rel * S + out_rel * np.abs(ref) + 1e-30
    worst = float((err / bound).max())
    assert worst <= 1.0, f"error {worst:.3g} x the bound"
    assert float((err / (HARD_REL * S + out_rel * np.abs(ref) + 1e-30)).max()) <= 1.0


@pytest.fixture(scope="module")
def dense(ops):
    out = {}
    for name, (fmt, R, rows) in DENSE.items():
        for K in (512, 2048, 4096):
            w = o.weights_like(rows, K, K + fmt, outliers=True)
            out[name, K] = (w, up(ops, w, fmt, R))
    return out


@pytest.mark.parametrize("name", list(DENSE))
@pytest.mark.parametrize("K", [512, 2048, 4096])
@pytest.mark.parametrize("T", TOKENS)
def test_mmv_dense(ops, dense, name, K, T):
    w, enc = dense[name, K]
    x, xf = act(T, K, seed=T)
    ref, S = ref64(w, xf)
    y32 = ops.mmv(x, enc)
    assert_within(y32, ref, S)
    assert torch.equal(ops.mmv(x.float(), enc), y32)                       # BF16 staging is exact
    assert torch.equal(ops.mmv(x, enc, out_dtype=torch.bfloat16).view(torch.int16), y32.to(torch.bfloat16).view(torch.int16))
    if T > 1:
        single = torch.cat([ops.mmv(x[t:t + 1], enc) for t in range(T)])
        assert torch.equal(y32, single)                                    # batch invariance, bitwise
        assert torch.equal(ops.mmv(x, enc, multi_col=False), y32)


@pytest.mark.parametrize("K", [512, 2048, 4096])
def test_mmv_summation_order_is_the_reference_order(ops, K):
    """Bitwise equal to the FP32 emulation of the reference kernels' order (row-major, chunk-major, NIBBLE + escapes)."""
    rows = 32
    w = o.weights_like(rows, K, 40 + K, outliers=True)
    x, xf = act(1, K, seed=K)
    for fmt, R, cm in [(HP, 8, False), (HP, 16, False), (HUF, 8, False)] + ([(HP, 8, True), (HP, 4, True)] if K > 512 else []):
        y = ops.mmv(x, up(ops, w, fmt, R, cm)).cpu().numpy()[0]
        assert np.array_equal(y.view(np.uint32), o.gemv_f32_order(w, xf[0], cm).view(np.uint32)), (fmt, R, cm)
    enc = up(ops, w, NIB)
    h = o.parse_header(enc.aux.cpu().numpy())
    aux = enc.aux.cpu().numpy()
    off = aux[h.off_c:h.off_c + 4 * (rows + 1)].view(np.uint32)
    rec = aux[h.off_d:h.off_d + 4 * max(h.n_a, 1)].view(np.uint32)
    esc = [list((rec[off[r]:off[r + 1]] & 0xFFF).astype(np.int32)) for r in range(rows)]
    y = ops.mmv(x, enc).cpu().numpy()[0]
    assert np.array_equal(y.view(np.uint32), o.gemv_f32_order(w, xf[0], False, esc).view(np.uint32))


@pytest.mark.parametrize("K", [512, 2048, 4096])
def test_mmv_full_machine(ops, K):
    """>= 512 units: the launch fills every SM with full blocks."""
    w = o.weights_like(8192, K, K)
    enc = up(ops, w, HP, 16)
    x, xf = act(1, K)
    ref, S = ref64(w, xf)
    y = ops.mmv(x, enc)
    assert_within(y, ref, S)
    assert torch.equal(ops.mmv(x.float(), enc), y)


def test_mmv_nibble_escapes(ops):
    w = o.weights_like(64, 2048, 5, outliers=True).copy()
    w[:, ::5] = 0x4000 | (np.arange(w[:, ::5].size).reshape(64, -1) % 128).astype(np.uint16)
    w[:, 1::97] = (((np.arange(w[:, 1::97].size).reshape(64, -1) % 40) + 70) << 7).astype(np.uint16)
    enc = up(ops, w, NIB)
    x, xf = act(3, 2048)
    ref, S = ref64(w, xf)
    assert_within(ops.mmv(x, enc), ref, S)


def test_one_hot_products_are_exact(ops):
    """x = e_k picks column k: the product is the weight itself, for every format (known-answer weights as in the
    reference's backend-op tests: (118 + ((i*7 + i/K) % 19)) << 7 | ((i*13 + i/K) & 127))."""
    rows, K = 32, 1024
    i = np.arange(rows * K)
    w = (((118 + ((i * 7 + i // K) % 19)) << 7) | ((i * 13 + i // K) & 127)).astype(np.uint16).reshape(rows, K)
    for fmt, R, cm in [(NIB, 0, False), (HUF, 8, False), (HP, 8, False), (HP, 8, True)]:
        enc = up(ops, w, fmt, R, cm)
        for k in (0, 1, 130, 511, 512, 1023):
            x = torch.zeros(1, K, dtype=torch.bfloat16, device="cuda")
            x[0, k] = 1.0
            y = ops.mmv(x, enc).cpu().numpy()[0]
            assert np.array_equal(y, o.bf16_bits_to_f32(w[:, k])), (fmt, cm, k)


@pytest.mark.parametrize("T", [1, 2, 8])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_merged_glu_equals_unfused(ops, T, xdt, ydt):
    N, K = 512, 2048
    enc = up(ops, o.weights_like(2 * N, K, 21, outliers=True), NIB)
    x, _ = act(T, K, seed=T, dtype=xdt)
    gu = ops.mmv(x, enc)
    unfused = ops.swiglu(gu[:, :N].contiguous(), gu[:, N:].contiguous())
    got = ops.mmv_glu(x, enc, out_dtype=ydt)
    assert got.dtype == ydt and torch.equal(got.view(torch.int16 if ydt == torch.bfloat16 else torch.int32),
                                             unfused.to(ydt).view(torch.int16 if ydt == torch.bfloat16 else torch.int32))


@pytest.mark.parametrize("fmt,R", [(NIB, 0), (HP, 1), (HP, 8), (HP, 16), (HUF, 8), (HUF, 16)])
@pytest.mark.parametrize("K", [512, 2048])
def test_separate_glu_equals_unfused(ops, fmt, R, K):
    N = 64
    g, u = up(ops, o.weights_like(N, K, 31), fmt, R), up(ops, o.weights_like(N, K, 32), fmt, R)
    x, _ = act(2, K, seed=3)
    want = ops.swiglu(ops.mmv(x, g), ops.mmv(x, u))
    assert torch.equal(ops.mmv_glu2(x, g, u), want)
    assert torch.equal(ops.mmv_glu2(x, g, u, out_dtype=torch.bfloat16).view(torch.int16), want.to(torch.bfloat16).view(torch.int16))


def test_glu_argument_errors(ops):
    K = 1024
    g = up(ops, o.weights_like(32, K, 1), HP, 8, True)
    u = up(ops, o.weights_like(32, K, 2), HP, 8, True)
    x, _ = act(1, K)
    with pytest.raises(ValueError, match="chunk-major"):
        ops.mmv_glu2(x, g, u)
    with pytest.raises(ValueError, match="NIBBLE"):
        ops.mmv_glu(x, up(ops, o.weights_like(32, K, 1), HP, 8))


def routed_case(ops, fmt, R, cm, K, rpm, n_exp, T, n_used, per_slot, ids_dtype, seed):
    w = o.weights_like(rpm * n_exp, K, seed)
    enc = up(ops, w, fmt, R, cm)
    g = np.random.default_rng(seed)
    ids = np.stack([g.permutation(n_exp)[:n_used] for _ in range(T)]).astype(np.int64)
    ids[0, -1] = ids[0, 0]  # a repeated expert inside one token is legal for the GEMV path
    shape = (T, n_used, K) if per_slot else (T, K)
    xb = o.f32_to_bf16_bits(g.standard_normal(shape).astype(np.float32))
    x = to_bf16_tensor(xb).cuda()
    xf = o.bf16_bits_to_f32(xb)
    y = ops.mmv(x, enc, torch.from_numpy(ids).to(ids_dtype).cuda(), rpm)
    assert y.shape == (T, n_used, rpm)
    for t in range(T):
        for s in range(n_used):
            e = ids[t, s]
            ref, S = o.gemv_f64(w[e * rpm:(e + 1) * rpm], xf[t, s] if per_slot else xf[t])
            assert_within(y[t, s], ref, S)
    return enc, x, ids, y


@pytest.mark.parametrize("ids_dtype", [torch.int32, torch.int64])
def test_mmv_routed(ops, ids_dtype):
    routed_case(ops, HP, 8, True, 2048, 64, 6, 3, 4, False, ids_dtype, 1)    # expert gate / up: chunk-major, x per token
    routed_case(ops, HP, 16, False, 512, 128, 5, 2, 4, True, ids_dtype, 2)   # expert down: x per slot
    routed_case(ops, NIB, 0, False, 1024, 32, 4, 2, 3, False, ids_dtype, 3)
    routed_case(ops, HUF, 8, False, 512, 32, 4, 1, 2, True, ids_dtype, 4)


def test_mmv_routed_padded_strides(ops):
    """ids and x rows taken from wider buffers (row strides larger than the rows)."""
    rpm, n_exp, K, T, n_used = 32, 8, 1024, 3, 2
    w = o.weights_like(rpm * n_exp, K, 9)
    enc = up(ops, w, HP, 8, True)
    ids_full = torch.randint(0, n_exp, (T, 8), dtype=torch.int32, device="cuda")
    ids = ids_full[:, :n_used]
    x_full, _ = act(T, 2 * K, seed=7)
    x = x_full[:, :K]
    y = ops.mmv(x, enc, ids, rpm)
    y2 = ops.mmv(x.contiguous(), enc, ids.contiguous(), rpm)
    assert torch.equal(y, y2)


def test_alignment_and_shape_rejection(ops):
    K = 1024
    enc = up(ops, o.weights_like(32, K, 1), HP, 8)
    buf = torch.zeros(2 * K + 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        ops.mmv(buf[1:K + 1].view(1, K), enc)
    with pytest.raises(RuntimeError, match="row strides must be multiples of 16 bytes"):
        ops.mmv(torch.as_strided(buf, (2, K), (K + 1, 1)), enc)
    with pytest.raises(RuntimeError, match="last dim must be K"):
        ops.mmv(buf[:512].view(1, 512), enc)
    ids = torch.zeros(1, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="whole units"):
        ops.mmv(buf[:K].view(1, K), enc, ids, 4)


@pytest.mark.parametrize("fmt,R", [(NIB, 0), (HP, 16), (HP, 1)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
def test_get_rows(ops, fmt, R, odt):
    w = o.weights_like(96, 1024, 17, outliers=True)
    w[5, 3] = 0x4123  # an escape for NIBBLE
    enc = up(ops, w, fmt, R)
    for idt in (torch.int32, torch.int64):
        ids = torch.tensor([0, 95, 5, 5, 17, 31, 32], dtype=idt, device="cuda")
        got = ops.get_rows(ids, enc, odt)
        want = to_bf16_tensor(w[ids.cpu().numpy()]).cuda().to(odt)
        assert torch.equal(got, want)
    assert ops.embedding(torch.tensor([[1, 2], [3, 4]], device="cuda"), enc).shape == (2, 2, 1024)
    assert ops.get_rows(torch.zeros(0, dtype=torch.int32, device="cuda"), enc).shape == (0, 1024)


def test_get_rows_rejections(ops):
    w = o.weights_like(32, 1024, 1)
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="chunk-major"):
        ops.get_rows(ids, up(ops, w, HP, 8, True))
    with pytest.raises(ValueError, match="single-symbol"):
        ops.get_rows(ids, up(ops, w, HUF, 8))


@pytest.mark.parametrize("name", ["nibble", "hufpair"])
@pytest.mark.parametrize("T", [1, 8, 9])
def test_linear_dispatch(ops, dense, name, T):
    w, enc = dense[name, 2048]
    x, xf = act(T, 2048, seed=T)
    bias = torch.randn(w.shape[0]).to(torch.bfloat16).cuda()
    y = ops.linear(x, enc)
    yb = ops.linear(x.view(1, T, 2048), enc, bias)
    assert y.dtype == torch.bfloat16 and y.shape == (T, w.shape[0]) and yb.shape == (1, T, w.shape[0])
    ref, S = ref64(w, xf)
    if T > ops.GEMV_MAX_TOKENS:
        wc = to_bf16_tensor(w).cuda()
        assert torch.equal(y.view(torch.int16), torch.nn.functional.linear(x, wc).view(torch.int16))
    else:
        assert_within(y, ref, S, out_rel=BF16_REL)
        b = bias.double().cpu().numpy()
        assert_within(yb[0], ref + b, S + np.abs(b), out_rel=BF16_REL)


def test_linear_host_round_trip(ops):
    w = o.weights_like(1024, 2048, 8)
    enc = up(ops, w, HP, 16)
    xh = torch.randn(1, 2048).to(torch.bfloat16).pin_memory()
    yh = torch.empty(1, 1024, dtype=torch.float32).pin_memory()
    xd, yd = torch.empty_like(xh, device="cuda"), torch.empty(1, 1024, dtype=torch.float32, device="cuda")
    ops.linear_host(xh, enc, yh, xd, yd)
    torch.cuda.synchronize()
    want = ops.mmv(xh.cuda(), enc).cpu()
    assert torch.equal(yh, want)
    yh.zero_()
    ops.linear_host(xh, enc, yh, xd)  # no device buffer: the kernel stores into the pinned host buffer itself
    torch.cuda.synchronize()
    assert torch.equal(yh, want)
    with pytest.raises(RuntimeError, match="pinned"):
        ops.mmv(xh.cuda(), enc, out=torch.empty(1, 1024))


# ---------------------------------------------------------------- MoE pieces


def test_topk_matches_oracle(ops):
    g = np.random.default_rng(0)
    for T, E, k in [(1, 256, 8), (4, 256, 8), (7, 64, 6), (3, 1000, 32), (2, 8, 8)]:
        logits = g.standard_normal((T, E)).astype(np.float32)
        wts, ids = ops.moe_topk(torch.from_numpy(logits).cuda(), k)
        ids_ref, w_ref = o.softmax_topk(logits, k)
        assert np.array_equal(ids.cpu().numpy(), ids_ref)
        assert np.allclose(wts.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-7)
        assert np.allclose(wts.sum(-1).cpu().numpy(), 1.0, atol=1e-5)
    logits = np.zeros((1, 256), np.float32)  # all tied: lowest indices win
    wts, ids = ops.moe_topk(torch.from_numpy(logits).cuda(), 8)
    assert ids.cpu().tolist() == [list(range(8))]


def test_swiglu_and_combine(ops):
    g = torch.randn(3, 8, 512, device="cuda")
    u = torch.randn(3, 8, 512, device="cuda")
    y = ops.swiglu(g, u)
    ref = (g.double() / (1 + torch.exp(-g.double()))) * u.double()
    assert torch.allclose(y.double(), ref, rtol=1e-5, atol=1e-6)
    wts = torch.rand(3, 8, device="cuda")
    c32 = ops.moe_combine(y, wts, torch.float32)
    acc = torch.zeros(3, 512, device="cuda")
    for k in range(8):  # slot order, fused multiply-add
        acc = torch.addcmul(acc, wts[:, k:k + 1], y[:, k])
    assert torch.allclose(c32, acc, rtol=1e-6, atol=1e-6)
    assert torch.equal(ops.moe_combine(y, wts).view(torch.int16), c32.to(torch.bfloat16).view(torch.int16))
    assert torch.equal(ops.moe_combine(y, wts.to(torch.bfloat16), torch.float32),
                       ops.moe_combine(y, wts.to(torch.bfloat16).float(), torch.float32))


@pytest.mark.parametrize("T", [1, 9, 127, 300])
@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_route_matches_oracle(ops, T, idt):
    E, k = 16, 4
    g = np.random.default_rng(T)
    ids = np.stack([g.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    ids[:, 0] = np.where(g.random(T) < 0.5, 3, ids[:, 0])  # skew: expert 3 is popular; fix duplicates below
    for t in range(T):
        if len(set(ids[t])) < k:
            ids[t] = g.permutation(E)[:k]
    ids[:, :] = np.where(ids == 7, 8, ids)  # expert 7 stays empty; may create duplicates
    for t in range(T):
        if len(set(ids[t])) < k:
            ids[t] = np.array([8, 9, 10, 11])
    for per_slot in (False, True):
        s1, d, b = ops.moe_route(torch.from_numpy(ids).to(idt).cuda(), E, per_slot)
        ny = k if per_slot else 1
        rs, rd, rb = o.route(ids, E, ny, ny)
        assert np.array_equal(b.cpu().numpy(), rb)
        assert np.array_equal(d.cpu().numpy(), rd) and np.array_equal(s1.cpu().numpy(), rs)


@pytest.mark.parametrize("T", [1, 2, 4, 8])
def test_moe_experts_decode(ops, T):
    """The <= 8 token MoE layer (routed GEMVs, SwiGLU, combine) against the FP64 layer over exact weights."""
    E, k, H, N = 8, 4, 1024, 512  # gate / up: [E*N, H]; down: [E*H, N]
    gate, upw, down = o.weights_like(E * N, H, 1), o.weights_like(E * N, H, 2), o.weights_like(E * H, N, 3)
    eg, eu, ed = up(ops, gate, HP, 8, True), up(ops, upw, HP, 8, True), up(ops, down, HP, 16)
    x, xf = act(T, H, seed=T)
    logits = np.random.default_rng(T).standard_normal((T, E)).astype(np.float32)
    wts, ids = ops.moe_topk(torch.from_numpy(logits).cuda(), k)
    y = ops.moe_experts(x, eg, eu, ed, wts, ids, E)
    assert y.dtype == torch.bfloat16 and y.shape == (T, H)
    ref = o.moe_layer_f64(xf, gate, upw, down, wts.cpu().numpy(), ids.cpu().numpy(), E)
    scale = np.abs(ref).max()
    assert np.abs(y.float().cpu().numpy() - ref).max() <= 2.0 ** -7 * scale


def test_cuda_graph_replay_equals_eager(ops, dense):
    """Every launcher only enqueues work: a captured decode-like step replays bitwise after its inputs change in place."""
    w, enc = dense["hufpair", 2048]
    wn, encn = dense["nibble", 2048]
    x, _ = act(2, 2048, seed=1)
    ys = [None, None]

    def step():
        ys[0] = ops.mmv(x, enc)
        ys[1] = ops.mmv_glu(x, encn)

    step()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            step()
    x2, _ = act(2, 2048, seed=2)
    x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in ys]
    assert torch.equal(got[0], ops.mmv(x, enc)) and torch.equal(got[1], ops.mmv_glu(x, encn))


@pytest.mark.parametrize("K,R,rows", [(2048, 16, 20480), (1024, 8, 12288), (512, 16, 24576), (2048, 4, 6144),
                                      (2048, 16, 40976), (1024, 8, 20480), (512, 16, 40960), (2048, 2, 5120),
                                      (2048, 16, 8192), (2048, 8, 4096), (1024, 16, 4112), (512, 16, 16384)])
def test_mmv_large_matrix_path(ops, K, R, rows):
    """Matrices from 256 units on take the persistent kernels that stage lane streams in shared memory (whole units
    by bulk copy: one unit per warp over all SMs below 8 units per SM, several above; per-lane rings with two units per
    warp from 16 units per SM and BF16 activations; 40976 rows = an odd number of units, 4112 rows = 257 units): same
    bits as the reference summation order, BF16 and FP32
    activations, BF16 output = rounding of the FP32 output."""
    w = o.weights_like(rows, K, rows + K, outliers=True)
    enc = up(ops, w, HP, R)
    x, xf = act(1, K, seed=R)
    y = ops.mmv(x, enc)
    ref, S = ref64(w, xf)
    assert_within(y, ref, S)
    want = o.gemv_f32_order(w, xf[0])
    assert np.array_equal(y.cpu().numpy()[0].view(np.uint32), want.view(np.uint32))
    assert torch.equal(ops.mmv(x.float(), enc), y)
    assert torch.equal(ops.mmv(x, enc, out_dtype=torch.bfloat16).view(torch.int16), y.to(torch.bfloat16).view(torch.int16))
    x2, _ = act(2, K, seed=R + 1)
    y2 = ops.mmv(x2, enc, multi_col=False)
    assert torch.equal(y2[0:1], ops.mmv(x2[0:1], enc)) and torch.equal(y2[1:2], ops.mmv(x2[1:2], enc))
    # 2..7 dense columns: groups of four and two share one decode (the ring kernel on the large shapes), same bits as
    # one column at a time
    x7, _ = act(7, K, seed=R + 2)
    singles = torch.cat([ops.mmv(x7[i:i + 1], enc) for i in range(7)])
    for T in (2, 3, 4, 7):
        assert torch.equal(ops.mmv(x7[:T], enc), singles[:T])
    assert ops.fault_status() == 0


@pytest.mark.parametrize("rows", [20480, 40960])
def test_mmv_large_matrix_long_codes(ops, rows):
    """Near-uniform exponents give ~12-bit codes, the most a row can consume: units then exceed the bulk-copy buffer
    (that kernel reads their streams from global memory instead) and drain the per-lane rings at the maximum rate."""
    K = 2048
    g = np.random.default_rng(3)
    ex = g.integers(64, 127, size=(rows, K)).astype(np.uint16)   # 63 x 63 = 3969 distinct pairs, all equally likely
    w = (ex << 7 | g.integers(0, 128, size=(rows, K)).astype(np.uint16)).astype(np.uint16)
    w[:256] = o.weights_like(256, K, 5)                          # the first units are short again
    enc = up(ops, w, HP, 16)
    assert enc.meta.format == HP
    x, xf = act(1, K, seed=9)
    y = ops.mmv(x, enc)
    idx = np.r_[0:512, rows - 512:rows]
    assert np.array_equal(y.cpu().numpy()[0, idx].view(np.uint32), o.gemv_f32_order(w[idx], xf[0]).view(np.uint32))
    assert np.array_equal(bits_of(ops.dequant(enc, 0, 512)), w[:512])


def test_mmv_group_equals_single_launches(ops):
    """Independent products in one call: the small NIBBLE matrices share a grid, a pair-Huffman matrix in the middle of
    the list is launched on its own; every result is bitwise what mmv gives, eagerly and replayed from a CUDA graph."""
    shapes = [(2048, 512, NIB, 0), (512, 2048, NIB, 0), (256, 2048, NIB, 0), (1024, 2048, HP, 16), (96, 4096, NIB, 0),
              (40, 1024, NIB, 0)] + [(64, 512, NIB, 0)] * 8          # more than eight groupable items: two grids
    ws = [up(ops, o.weights_like(r, K, 300 + i, outliers=True), fmt, R) for i, (r, K, fmt, R) in enumerate(shapes)]
    for T, xdt in ((1, torch.bfloat16), (3, torch.float32), (8, torch.bfloat16)):
        xs = [act(T, K, seed=50 + i)[0].to(xdt) for i, (r, K, fmt, R) in enumerate(shapes)]
        want = [ops.mmv(x, w) for x, w in zip(xs, ws)]
        got = ops.mmv_group(xs, ws)
        assert all(torch.equal(a, b) for a, b in zip(got, want))
    xs = [act(1, K, seed=70 + i)[0] for i, (r, K, fmt, R) in enumerate(shapes)]
    outs = [torch.empty(1, r, device="cuda") for (r, K, fmt, R) in shapes]
    ops.mmv_group(xs, ws, outs)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            ops.mmv_group(xs, ws, outs)
    for x in xs:
        x.copy_(act(1, x.shape[1], seed=int(x.shape[1]) + 5)[0])
    g.replay()
    torch.cuda.synchronize()
    assert all(torch.equal(y, ops.mmv(x, w)) for x, w, y in zip(xs, ws, outs))
    assert ops.mmv_group([], []) == []


def test_host_gathered_projection_on_one_gpu(ops):
    """The end-to-end projection (activation from pinned host memory, logits stored into host memory by the kernel, which
    then writes the step number the host waits for): eager, captured and replayed steps equal ops.mmv bitwise."""
    from orin_qwen_lossless_b200 import sharded
    rows, K, R = 16 * 148 * 16, 2048, 16
    w = up(ops, o.weights_like(rows, K, 21), HP, R, False)
    hg = sharded.HostGatheredLinear(w, rows, R, 2)
    try:
        for T in (1, 2):
            xh = torch.empty((T, K), dtype=torch.bfloat16).pin_memory()
            for i in range(5):
                xi = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(90 + i).standard_normal((T, K)).astype(np.float32)))
                xh.copy_(xi)
                got = hg.step(xh).clone()
                assert torch.equal(got, ops.mmv(xi.cuda(), w).cpu())
        assert ops.fault_status() == 0
        with pytest.raises(ValueError):
            hg.step(torch.empty((1, K), dtype=torch.bfloat16))   # not pinned
    finally:
        hg.close()
