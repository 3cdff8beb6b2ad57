"""Draft-only k-bit copies of an output head (csrc/draft.cu) under the contract of the reference's
tests/core/test_draft_head.py: every weight reads back as the documented level of its group, the GEMV is the product
with the stored matrix up to its FP16 partial sums, a column's scores do not depend on the batch, and draft_logits
gives every candidate its exact FP32 logit and everything else -inf. The stored formats are checked against a NumPy
restatement of the reference's quantisers (core/include/bf16n/draft_head.cuh:22-45, 117-145)."""
import numpy as np
import pytest
import torch

from conftest import bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
HP = 3


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


def model_like(rows, K, seed):
    return to_bf16_tensor(o.weights_like(rows, K, seed, outliers=True))


def readout(ops, bits, q, s, K):
    """The stored matrix [rows, K] as the GEMV sees it: one-hot inputs, four columns per call (exact in FP16)."""
    gemv = ops.int2_gemv if bits == 2 else ops.int4_gemv
    cols = []
    for c0 in range(0, K, 4):
        x = torch.zeros(4, K, dtype=torch.bfloat16, device="cuda")
        x[torch.arange(4), torch.arange(c0, c0 + 4)] = 1.0
        cols.append(gemv(x, q, s))
    return torch.cat(cols).t()


def int2_case(K, seed=0):
    w = model_like(8, K, seed).float()
    w[0, :128] = 0.0
    w[1, :8] = torch.tensor([-1.5, -1.0, -0.75, -0.5, 0.0, 0.5, 1.0, 1.5])
    w[1, 8:128] = torch.linspace(-1.4, 1.4, 120)
    return w.to(torch.bfloat16)


def np_int2(w):
    """Words and scales as the reference's 2-bit quantiser defines them."""
    wf = w.float().numpy().astype(np.float32)
    g = wf.reshape(wf.shape[0], -1, 128)
    s = (np.abs(g).max(-1) / np.float32(1.5)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        n = np.where(s[:, :, None] > 0, np.clip(np.floor(g / s[:, :, None]), -2, 1) + 2, 2).astype(np.uint32)
    n = n.reshape(wf.shape[0], -1, 16)
    words = (n << (2 * np.arange(16, dtype=np.uint32))).sum(-1).astype(np.uint32)
    return words.view(np.uint8).reshape(wf.shape[0], -1), s


def np_int4(w):
    wf = w.float().numpy().astype(np.float32)
    g = wf.reshape(wf.shape[0], -1, 128)
    amax = np.abs(g).max(-1)
    s = np.where(amax > 0, amax / np.float32(7.0), np.float32(1.0)).astype(np.float32)
    a = (np.clip(np.rint(g / s[:, :, None]), -8, 7) + 8).astype(np.uint8).reshape(wf.shape[0], -1)
    return (a[:, 0::2] | (a[:, 1::2] << 4)).astype(np.uint8), s


@pytest.mark.parametrize("K", [2048, 1024])
def test_stored_formats_are_the_reference_formats(ops, K):
    w = int2_case(K) if K == 2048 else model_like(24, K, 3)
    q2, s2 = ops.int2_quantize(w.cuda())
    wq, ws = np_int2(w)
    assert np.array_equal(s2.cpu().numpy(), ws) and np.array_equal(q2.cpu().numpy(), wq)
    q4, s4 = ops.int4_quantize(w.cuda())
    wq, ws = np_int4(w)
    assert np.array_equal(s4.cpu().numpy(), ws) and np.array_equal(q4.cpu().numpy(), wq)


def test_int2_weights_read_back_as_nearest_level(ops):
    K = 2048
    w = int2_case(K)
    q, s = ops.int2_quantize(w.cuda())
    d = readout(ops, 2, q, s, K).double().cpu()
    g = w.float().view(w.shape[0], -1, 128)
    assert torch.equal(s.cpu(), g.abs().amax(-1) / 1.5)
    step = s.cpu().double()[:, :, None].expand_as(g).reshape(w.shape)
    wd = w.double()
    nz = step > 0
    assert torch.equal(d[~nz], torch.zeros_like(d[~nz]))
    r2 = d[nz] / step[nz] * 2
    assert torch.isin(r2.round(), torch.tensor([-3.0, -1.0, 1.0, 3.0], dtype=torch.float64)).all()
    assert (r2 - r2.round()).abs().max() < 1e-6
    assert ((wd - d).abs() <= step / 2 * (1 + 1e-6))[nz].all()
    wf, sf = w.float(), step.float()
    ties = nz & ((wf == 0) | (wf == sf) | (wf == -sf))
    assert ties[1, :8].sum() == 3
    assert torch.allclose(d[ties], wd[ties] + step[ties] / 2, rtol=1e-6, atol=0)


@pytest.mark.parametrize("bits, K", [(2, 2048), (4, 1024), (4, 2048), (4, 4096)])
@pytest.mark.parametrize("T", [1, 2, 3, 4])
def test_kbit_gemv_is_the_product_with_the_stored_matrix(ops, bits, K, T):
    w = model_like(61, K, K + T)   # 61 rows: not a multiple of the 8 rows per block
    q, s = (ops.int2_quantize if bits == 2 else ops.int4_quantize)(w.cuda())
    d = readout(ops, bits, q, s, K).double()
    x = (torch.randn(T, K, generator=torch.Generator().manual_seed(T)) * 2).to(torch.bfloat16).cuda()
    y = (ops.int2_gemv if bits == 2 else ops.int4_gemv)(x, q, s).double()
    ref = x.double() @ d.t()
    bound = x.double().abs() @ d.abs().t()
    assert ((y - ref).abs() <= 2e-2 * bound + 1e-6).all()


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("T", [2, 3, 4])
def test_kbit_gemv_scores_each_column_as_alone(ops, bits, T):
    K = 2048
    q, s = (ops.int2_quantize if bits == 2 else ops.int4_quantize)(model_like(61, K, T).cuda())
    gemv = ops.int2_gemv if bits == 2 else ops.int4_gemv
    x = (torch.randn(T, K, generator=torch.Generator().manual_seed(10 + T)) * 2).to(torch.bfloat16).cuda()
    y = gemv(x, q, s)
    for t in range(T):
        assert torch.equal(y[t].view(torch.int32), gemv(x[t:t + 1].contiguous(), q, s)[0].view(torch.int32))


@pytest.mark.parametrize("fo", [False, True])
def test_draft_logits_rescore_every_candidate_exactly(ops, fo):
    V, K = 4096, 2048
    w = model_like(V, K, 7)
    h = (torch.randn(3, K, generator=torch.Generator().manual_seed(3)) * 3).to(torch.bfloat16)
    w[777] = (h[2].float() / h[2].float().norm() * 0.5).to(torch.bfloat16)   # row 2: a clear exact winner

    def enc(R, fo_):
        plane, aux, meta = ops.encode(w, HP, R, False, fo_)
        return ops.upload(plane, aux, meta, "cuda")

    e = enc(16, True) if fo else enc(4, False)
    q, s = ops.int2_quantize(w.cuda())
    head = ops.DraftHead(2, q, s, 128)
    h = h.cuda()
    out = ops.draft_logits(h, e, head, V)
    if fo:
        assert torch.equal(out, ops.draft_logits(h, enc(4, False), head, V))
    cand = head.scores(h).topk(128, dim=-1).indices
    finite = torch.isfinite(out)
    assert torch.equal(finite.sum(1), torch.full((3,), 128, device="cuda"))
    assert finite.gather(1, cand).all()
    exact = h.double() @ w.cuda().double().t()
    S = h.double().abs() @ w.cuda().double().abs().t()
    got = out.gather(1, cand).double()
    assert ((got - exact.gather(1, cand)).abs() <= 1e-5 * S.gather(1, cand)).all()
    best_cand = cand.gather(1, exact.gather(1, cand).argmax(1, keepdim=True)).squeeze(1)
    assert torch.equal(out.argmax(1), best_cand)
    assert out.argmax(1)[2].item() == 777 == exact.argmax(1)[2].item()


@pytest.mark.parametrize("bits, qcols, scols, cand, ok", [
    (2, 512, 16, 1, True), (2, 512, 16, 64, True), (2, 512, 16, 65, False), (2, 512, 16, 0, False),
    (4, 1024, 16, 32, True), (4, 512, 16, 32, False), (3, 768, 16, 32, False),
])
def test_draft_head_rejects_inconsistent_shapes(ops, bits, qcols, scols, cand, ok):
    q = torch.zeros(64, qcols, dtype=torch.uint8)
    s = torch.zeros(64, scols)
    if ok:
        assert ops.DraftHead(bits, q, s, cand).candidates == cand
    else:
        with pytest.raises(ValueError):
            ops.DraftHead(bits, q, s, cand)


@pytest.mark.parametrize("env, bits", [(None, 2), ("int2", 2), ("int4", 4), ("full", None)])
def test_draft_head_choice(ops, monkeypatch, env, bits):
    if env is None:
        monkeypatch.delenv("BF16N_DRAFT_HEAD", raising=False)
    else:
        monkeypatch.setenv("BF16N_DRAFT_HEAD", env)
    assert ops.draft_head_bits() == bits
    if env not in (None, "full"):
        monkeypatch.delenv("BF16N_DRAFT_CANDIDATES", raising=False)
        head = ops.make_draft_head(model_like(256, 2048, 1).cuda(), bits)
        assert (head.bits, head.candidates) == (bits, {2: 128, 4: 32}[bits])


@pytest.mark.parametrize("env", ["int8", "INT2", ""])
def test_draft_head_choice_rejects_unknown_values(ops, monkeypatch, env):
    monkeypatch.setenv("BF16N_DRAFT_HEAD", env)
    with pytest.raises(ValueError):
        ops.draft_head_bits()


@pytest.mark.parametrize("K", [1024, 4096])
def test_int2_gemv_rejects_other_widths(ops, K):
    q, s = ops.int2_quantize(model_like(16, K, 2).cuda())
    with pytest.raises(ValueError, match="K must be 2048"):
        ops.int2_gemv(torch.zeros(1, K, dtype=torch.bfloat16, device="cuda"), q, s)
