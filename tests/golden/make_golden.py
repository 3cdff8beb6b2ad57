"""Generates tests/golden/*.npz from the REFERENCE encoder and policy (oracle/_ref, built from the reference's own
sources by oracle/Makefile). Run where the reference checkout exists:

    make -C oracle && python tests/golden/make_golden.py

Each encoder vector stores the seeded input (BF16 bits) with the SHA-256 of the plane and aux bytes the reference
produced, the aux header fields, and for the smallest cases the full bytes. The policy table stores the reference's
choice for the shape groups its own test lists (core/tests/test_policy.cpp:40-160) and a sweep around the thresholds.
"""
import hashlib
import itertools
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import cpu_oracle as o  # noqa: E402

CASES = [  # (name, rows, K, format, R, chunk_major, frag_order, data)
    ("nib_k512", 24, 512, 1, 0, 0, 0, "model"),
    ("nib_k2048", 9, 2048, 1, 0, 0, 0, "model"),
    ("nib_17exp", 4, 512, 1, 0, 0, 0, "exp17"),
    ("huf_k512_r1", 8, 512, 2, 1, 0, 0, "model"),
    ("huf_k1024_r8", 16, 1024, 2, 8, 0, 0, "model"),
    ("hp_k512_r1", 8, 512, 3, 1, 0, 0, "model"),
    ("hp_k512_r16", 32, 512, 3, 16, 0, 0, "model"),
    ("hp_k2048_r8", 16, 2048, 3, 8, 0, 0, "model"),
    ("hp_k2048_r8_cm", 16, 2048, 3, 8, 1, 0, "model"),
    ("hp_k1024_r4_cm", 8, 1024, 3, 4, 1, 0, "model"),
    ("hp_k4096_r2", 4, 4096, 3, 2, 0, 0, "model"),
    ("hp_k512_fo", 16, 512, 3, 16, 0, 1, "model"),
    ("hp_k1024_fo", 16, 1024, 3, 16, 0, 1, "model"),
    ("hp_pairs4096", 16, 1024, 3, 4, 0, 0, "pairs4096"),
    ("hp_pairs4097", 16, 1024, 3, 4, 0, 0, "pairs4097"),
    ("hp_ties", 16, 512, 3, 4, 0, 0, "ties"),
]


def data(kind, rows, K, seed):
    if kind == "model":
        return o.with_specials(o.weights_like(rows, K, seed, outliers=True), seed).reshape(rows, K)
    if kind == "exp17":  # 17 distinct exponents in one row: two escapes classes
        w = np.zeros((rows, K), dtype=np.uint16)
        ex = 100 + (np.arange(K) % 17)
        w[:] = (ex << 7 | (np.arange(K) % 128)).astype(np.uint16)
        w[1, ::7] |= 0x8000
        w[2, 5] = 0x4120  # exponent 130 >= 128: always an escape
        return w
    if kind.startswith("pairs"):
        return o.with_pairs(rows, K, int(kind[5:]))
    if kind == "ties":  # many equally frequent pairs: exercises the tie order of the length assignment
        g = np.random.default_rng(seed)
        ex = g.integers(110, 126, size=(rows, K)).astype(np.uint16)
        return (ex << 7 | g.integers(0, 128, size=(rows, K)).astype(np.uint16)).astype(np.uint16)
    raise ValueError(kind)


def main():
    assert o.have_ref(), "build oracle/_ref first (make -C oracle)"
    out, meta = {}, []
    for i, (name, rows, K, fmt, R, cm, fo, kind) in enumerate(CASES):
        w = data(kind, rows, K, 1000 + i)
        plane, aux, fmt_out = o.ref_encode(w, fmt, R, cm, fo)
        assert np.array_equal(o.decode(plane, aux), w), name
        h = o.parse_header(aux)
        rec = dict(name=name, rows=rows, K=K, format=fmt, R=R, cm=cm, fo=fo, format_out=fmt_out, aux_len=int(aux.size),
                   plane_sha256=hashlib.sha256(plane.tobytes()).hexdigest(),
                   aux_sha256=hashlib.sha256(aux.tobytes()).hexdigest(), header=list(h.__dict__.values()))
        out[name + "__w"] = w
        if rows * K <= 16 * 1024:
            out[name + "__plane"] = plane
            out[name + "__aux"] = aux
        meta.append(rec)
    np.savez_compressed(os.path.join(HERE, "encoder_vectors.npz"), **out)
    with open(os.path.join(HERE, "encoder_vectors.json"), "w") as f:
        json.dump(meta, f, indent=1)

    pol = []
    shapes = [(248320, 2048, 1), (8192, 2048, 1), (4096, 2048, 1), (2048, 4096, 1), (512, 2048, 256), (2048, 512, 256),
              (12288, 2048, 1), (9216, 2048, 1), (2048, 512, 1), (512, 2048, 1), (256, 2048, 1), (32, 2048, 1), (1024, 2048, 1),
              (8192, 512, 1), (16384, 512, 1), (768, 2048, 128), (4100, 2048, 1), (4096, 2000, 1), (4096, 8192, 1), (0, 2048, 1)]
    for (rows, K, n), engine, mode, expert, dfo in itertools.product(shapes, ("llama", "vllm"), ("hybrid", "huffman", "nibble"),
                                                                    (False, True), (False, True)):
        c = o.ref_choose(rows, K, n, engine=engine, mode=mode, expert=expert, dense_frag_order=dfo)
        pol.append([rows, K, n, engine, mode, int(expert), int(dfo), list(map(int, c)) if c else None])
    for rows in range(512 * 2 - 4, 512 * 16 * 3, 508):  # wave-model thresholds
        for engine in ("llama", "vllm"):
            c = o.ref_choose(rows, 4096, 1, engine=engine)
            pol.append([rows, 4096, 1, engine, "hybrid", 0, 0, list(map(int, c)) if c else None])
    with open(os.path.join(HERE, "policy_table.json"), "w") as f:
        json.dump(pol, f)
    print("wrote", len(meta), "encoder vectors and", len(pol), "policy rows")


if __name__ == "__main__":
    main()
