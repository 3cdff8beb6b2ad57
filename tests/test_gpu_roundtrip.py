"""GPU decode is bit-exact: host encode -> device dequant / verify equals the source for every format and layout, for
special values, escapes, the pair-alphabet boundary and unit-aligned row ranges; a flipped bit is detected. Mirrors the
reference's tests/core/test_roundtrip.py, with the CPU oracle as the second opinion."""
import numpy as np
import pytest
import torch

from conftest import bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    m.init()
    return m


def up(ops, w_bits, fmt, R=0, cm=False):
    plane, aux, meta = ops.encode(to_bf16_tensor(w_bits), fmt, R, cm)
    return ops.upload(plane, aux, meta, "cuda")


LAYOUTS = [(1, 0, False)] + [(f, R, False) for f in (2, 3) for R in (1, 2, 4, 8, 16)] + [(3, R, True) for R in (4, 8, 16)]


@pytest.mark.parametrize("K", [512, 2048, 4096])
def test_round_trip_all_layouts(ops, K):
    rows = 64
    w = o.with_specials(o.weights_like(rows, K, K, outliers=True), K).reshape(rows, K)
    src = to_bf16_tensor(w).cuda()
    for fmt, R, cm in LAYOUTS:
        if cm and K == 512:
            continue
        e = up(ops, w, fmt, R, cm)
        assert np.array_equal(bits_of(ops.dequant(e)), w), (fmt, R, cm)
        assert ops.mismatches(e, src) == 0, (fmt, R, cm)
        assert ops.roundtrip_equal(e, src, chunk_bytes=16 * K * 2)
        assert np.array_equal(o.decode(e.plane.cpu().numpy(), e.aux.cpu().numpy()), w)


def test_decodes_reference_encoded_tensors(ops, golden_vectors):
    """Tensors encoded by the reference encoder (the committed vectors carry its bytes) decode exactly on the GPU."""
    meta, blobs = golden_vectors
    n = 0
    for rec in meta:
        if rec["fo"] or rec["name"] + "__aux" not in blobs:
            continue
        aux = torch.from_numpy(blobs[rec["name"] + "__aux"].copy())
        plane = torch.from_numpy(blobs[rec["name"] + "__plane"].copy())
        e = ops.upload(plane, aux, ops.parse_header(aux), "cuda")
        assert np.array_equal(bits_of(ops.dequant(e)), blobs[rec["name"] + "__w"]), rec["name"]
        n += 1
    assert n >= 8


def test_special_values_every_format(ops):
    K = 1024
    w = np.tile(o.SPECIALS, 16 * K // o.SPECIALS.size + 1)[: 16 * K].reshape(16, K).copy()
    for fmt, R, cm in [(1, 0, False), (2, 8, False), (3, 8, False), (3, 8, True)]:
        e = up(ops, w, fmt, R, cm)
        assert np.array_equal(bits_of(ops.dequant(e)), w)


@pytest.mark.parametrize("n_exp", [14, 15, 16, 17])
def test_nibble_escape_counts(ops, n_exp):
    K = 2048
    ex = 90 + (np.arange(4 * K) % n_exp)
    w = (ex << 7 | (np.arange(4 * K) % 128)).astype(np.uint16).reshape(4, K)
    e = up(ops, w, 1)
    h = o.parse_header(e.aux.cpu().numpy())
    assert (h.n_a > 0) == (n_exp > 15)
    assert np.array_equal(bits_of(ops.dequant(e)), w)
    assert ops.mismatches(e, to_bf16_tensor(w).cuda()) == 0


def test_nibble_msb_exponents_escape(ops):
    w = o.weights_like(8, 512, 3).copy()
    w[:, ::9] = 0x4000 | (np.arange(w[:, ::9].size).reshape(8, -1) % 128).astype(np.uint16)
    e = up(ops, w, 1)
    assert o.parse_header(e.aux.cpu().numpy()).n_a == w[:, ::9].size
    assert np.array_equal(bits_of(ops.dequant(e)), w)


@pytest.mark.parametrize("n", [4095, 4096, 4097])
def test_pair_alphabet_boundary(ops, n):
    w = o.with_pairs(16, 1024, n)
    e = up(ops, w, 3, 4)
    assert e.meta.format == (3 if n <= 4096 else 2)
    assert np.array_equal(bits_of(ops.dequant(e)), w)


def test_unit_aligned_row_ranges(ops):
    w = o.weights_like(64, 2048, 9)
    for fmt, R, cm in [(1, 0, False), (2, 8, False), (3, 16, False), (3, 8, True)]:
        e = up(ops, w, fmt, R, cm)
        unit = max(R, 1)
        for r0, nr in [(0, unit), (unit, 2 * unit), (64 - unit, unit), (16, 32)]:
            assert np.array_equal(bits_of(ops.dequant(e, r0, nr)), w[r0:r0 + nr])
            assert ops.mismatches(e, to_bf16_tensor(w[r0:r0 + nr]).cuda(), r0, nr) == 0
        assert ops.dequant(e, 0, 0).shape == (0, 2048)
        if R > 1:
            with pytest.raises(ValueError, match="whole units"):
                ops.dequant(e, 1, R)


def test_flipped_bits_are_detected(ops):
    w = o.weights_like(32, 2048, 4)
    src = to_bf16_tensor(w).cuda()
    for fmt, R, cm in [(1, 0, False), (3, 16, False), (3, 8, True)]:
        e = up(ops, w, fmt, R, cm)
        e.plane[5, 77] ^= 0x10   # a mantissa bit
        assert ops.mismatches(e, src) == 1
        assert not ops.roundtrip_equal(e, src)
        e.plane[5, 77] ^= 0x10
        bad = src.clone()
        bad.view(torch.int16)[3, 100] ^= 0x0080  # an exponent bit of the source
        bad.view(torch.int16)[9, 0] ^= 0x0001
        assert ops.mismatches(e, bad) == 2


def test_large_tensor_verify_property(ops):
    """Encode -> verify at a size the CPU oracle would take long for: the mismatch count of the real source is 0 and of
    a source with k flipped words is exactly k."""
    rows, K = 16384, 2048
    w = o.weights_like(rows, K, 123)
    e = up(ops, w, 3, 16)
    src = to_bf16_tensor(w).cuda()
    assert ops.mismatches(e, src) == 0
    idx = torch.randperm(rows * K, device="cuda")[:1000]
    src.view(torch.int16).view(-1)[idx] ^= 0x0040
    assert ops.mismatches(e, src) == 1000
