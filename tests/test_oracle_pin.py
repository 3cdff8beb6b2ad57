"""Pins the CPU oracle (oracle/bf16n_oracle.cpp) to the reference: against the committed golden vectors made by the
reference encoder, against the reference encoder itself where oracle/_ref is built, and through the round-trip cases of
the reference's own host test (core/tests/test_encode.cpp:233-306)."""
import hashlib

import numpy as np
import pytest

from oracle import cpu_oracle as o


def test_oracle_matches_golden_vectors(golden_vectors):
    meta, blobs = golden_vectors
    for rec in meta:
        w = blobs[rec["name"] + "__w"]
        plane, aux, fmt = o.encode(w, rec["format"], rec["R"], rec["cm"], rec["fo"])
        assert fmt == rec["format_out"], rec["name"]
        assert aux.size == rec["aux_len"], rec["name"]
        assert hashlib.sha256(plane.tobytes()).hexdigest() == rec["plane_sha256"], rec["name"]
        assert hashlib.sha256(aux.tobytes()).hexdigest() == rec["aux_sha256"], rec["name"]
        if rec["name"] + "__aux" in blobs:
            assert np.array_equal(aux, blobs[rec["name"] + "__aux"])
            assert np.array_equal(plane, blobs[rec["name"] + "__plane"])
            assert np.array_equal(o.decode(blobs[rec["name"] + "__plane"], blobs[rec["name"] + "__aux"]), w)
        assert list(o.parse_header(aux).__dict__.values()) == rec["header"]


@pytest.mark.skipif(not o.have_ref(), reason="oracle/_ref (the reference's own encoder) not built here")
@pytest.mark.parametrize("K", [512, 2048, 4096])
def test_oracle_equals_reference_encoder(K):
    rows = 32
    w = o.with_specials(o.weights_like(rows, K, K, outliers=True), K).reshape(rows, K)
    cases = [(1, 0, 0)] + [(f, R, 0) for f in (2, 3) for R in (1, 2, 4, 8, 16)] + [(3, R, 1) for R in (4, 8, 16) if K > 512]
    for fmt, R, cm in cases:
        a = o.encode(w, fmt, R, cm)
        b = o.ref_encode(w, fmt, R, cm)
        assert a[2] == b[2] and np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]), (fmt, R, cm)
    a, b = o.encode(w, 3, 16, False, True), o.ref_encode(w, 3, 16, False, True)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("K", [512, 2048, 4096])
def test_round_trip_every_format_and_layout(K):  # test_encode.cpp:235-248
    rows = 32
    w = o.with_specials(o.weights_like(rows, K, K + 1, outliers=True), K).reshape(rows, K)
    plane, aux, fmt = o.encode(w, 1, 0)
    assert fmt == 1 and np.array_equal(o.decode(plane, aux), w)
    for R in (1, 2, 4, 8, 16):
        for f in (2, 3):
            plane, aux, fmt = o.encode(w, f, R)
            h = o.parse_header(aux)
            assert fmt == f and h.K == K and h.rows == rows and h.flags == 0
            assert np.array_equal(o.decode(plane, aux), w), (f, R)
        if K > 512 and R >= 4:
            plane, aux, fmt = o.encode(w, 3, R, True)
            assert o.parse_header(aux).flags == 1 and np.array_equal(o.decode(plane, aux), w)


@pytest.mark.parametrize("K,rows", [(512, 16), (512, 48), (2048, 16), (4096, 48)])
def test_round_trip_fragment_order(K, rows):  # test_encode.cpp:251-259
    w = o.with_specials(o.weights_like(rows, K, rows + K, outliers=True), K).reshape(rows, K)
    plane, aux, _ = o.encode(w, 3, 16, False, True)
    h = o.parse_header(aux)
    assert h.n_a == rows // 16 * (K // 512) and h.flags == 2
    assert np.array_equal(o.decode(plane, aux), w)


@pytest.mark.parametrize("n", [4095, 4096, 4097])
def test_pair_alphabet_boundary(n):  # test_encode.cpp:262-269
    want = 3 if n <= 4096 else 2
    w = o.with_pairs(16, 1024, n)
    for cm in (False, True):
        plane, aux, fmt = o.encode(w, 3, 4, cm)
        assert fmt == want
        assert o.parse_header(aux).flags == (1 if cm and want == 3 else 0)
        assert np.array_equal(o.decode(plane, aux), w)


def test_argument_boundaries():  # test_encode.cpp:272-306
    z = np.zeros((64, 4096 + 512), dtype=np.uint16)

    def bad(rows, K, fmt, R, cm=False, fo=False):
        with pytest.raises(ValueError):
            o.encode(z.reshape(-1)[: max(rows * K, 0)].reshape(max(rows, 0), K) if K else z[:0], fmt, R, cm, fo)

    def good(rows, K, fmt, R, cm=False, fo=False):
        o.encode(z.reshape(-1)[: rows * K].reshape(rows, K), fmt, R, cm, fo)

    for K in (511, 513, 4095, 4097, 4608):
        bad(16, K, 3, 4)
    for K in (512, 4096):
        good(16, K, 3, 4)
    good(1, 512, 1, 0)
    bad(16, 512, 1, 4)
    bad(16, 1024, 1, 0, True)
    for R in (0, 3, 32):
        bad(96, 512, 2, R)
    bad(15, 512, 3, 4), good(16, 512, 3, 4), bad(17, 512, 3, 4)
    bad(16, 1024, 2, 4, True)
    bad(16, 512, 3, 4, True), good(16, 1024, 3, 4, True), bad(16, 1024, 3, 2, True)
    bad(16, 512, 0, 4), bad(16, 512, 4, 4)
    good(16, 512, 3, 16, False, True), good(16, 1024, 3, 16, False, True)
    bad(16, 512, 3, 8, False, True), bad(32, 1024, 3, 16, True, True), bad(16, 512, 2, 16, False, True)
    bad(16, 512, 1, 0, False, True)


def test_nibble_escape_counts():
    """14/15/16/17 distinct exponents per row: 15 fit the table (exponent 0 holds entry 0), the rest escape; exponents
    >= 128 always escape (tests/core/test_roundtrip.py:120-130 in the reference)."""
    K = 512
    for n_exp in (14, 15, 16, 17):
        ex = 100 + (np.arange(K) % n_exp)
        w = (ex << 7 | 5).astype(np.uint16).reshape(1, K)
        plane, aux, _ = o.encode(w, 1, 0)
        h = o.parse_header(aux)
        counts = np.bincount(ex, minlength=256)
        kept = sorted(range(256), key=lambda e: (-counts[e], e))[:15]
        assert h.n_a == sum(counts[e] for e in range(256) if counts[e] and e not in kept)
        assert np.array_equal(o.decode(plane, aux), w)
    w = np.full((1, K), 0x3F80, dtype=np.uint16)
    w[0, 7] = 0x4120  # exponent 130
    plane, aux, _ = o.encode(w, 1, 0)
    assert o.parse_header(aux).n_a == 1 and np.array_equal(o.decode(plane, aux), w)


def test_policy_port_matches_reference_table(policy_table):
    for rows, K, n, engine, mode, expert, dfo, want in policy_table:
        got = o.choose(rows, K, n, engine=engine, mode=mode, expert=bool(expert), dense_frag_order=bool(dfo))
        assert (list(map(int, got)) if got else None) == want, (rows, K, n, engine, mode, expert, dfo)


def test_gemv_order_emulation_close_to_fp64():
    w = o.weights_like(64, 2048, 3)
    x = o.bf16_bits_to_f32(o.f32_to_bf16_bits(np.random.default_rng(5).standard_normal(2048).astype(np.float32)))
    y64, s = o.gemv_f64(w, x)
    for cm in (False, True):
        y = o.gemv_f32_order(w, x, cm)
        assert np.all(np.abs(y - y64) <= 1e-6 * s)
    plane, aux, _ = o.encode(w, 3, 8)
    y = o.decode_gemv_mt(plane, aux, x, 0, 8, 4)
    assert np.all(np.abs(y - y64) <= 1e-5 * s)
