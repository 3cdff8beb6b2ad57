"""Host side of the library through the C ABI (no GPU): encoder bytes against the oracle and the golden vectors,
argument errors, header parse, shape policy, and the exported symbol list."""
import ctypes as C
import hashlib
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, bits_of, to_bf16_tensor
from oracle import cpu_oracle as o
from orin_qwen_lossless_b200 import _lib, ops


def enc(w, fmt, R, cm=False, fo=False):
    plane, aux, meta = ops.encode(to_bf16_tensor(w), fmt, R, cm, fo)
    return plane.numpy(), aux.numpy(), meta


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "bf16n_c.h")).read()
    declared = set(re.findall(r"\b(bf16n_[A-Za-z0-9_]+)\s*\(", hdr))
    lib = _lib.lib()
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name


def test_encoder_matches_golden_vectors(golden_vectors):
    meta, blobs = golden_vectors
    for rec in meta:
        w = blobs[rec["name"] + "__w"]
        plane, aux, m = enc(w, rec["format"], rec["R"], rec["cm"], rec["fo"])
        assert m.format == rec["format_out"]
        assert hashlib.sha256(plane.tobytes()).hexdigest() == rec["plane_sha256"], rec["name"]
        assert hashlib.sha256(aux.tobytes()).hexdigest() == rec["aux_sha256"], rec["name"]


@pytest.mark.parametrize("K", [512, 1024, 2048, 4096])
def test_encoder_byte_identical_to_oracle(K):
    rows = 48
    w = o.with_specials(o.weights_like(rows, K, 11 * K, outliers=True), K).reshape(rows, K)
    cases = [(1, 0, 0, 0)] + [(f, R, 0, 0) for f in (2, 3) for R in (1, 2, 4, 8, 16)]
    cases += [(3, R, 1, 0) for R in (4, 8, 16) if K > 512] + [(3, 16, 0, 1)]
    for fmt, R, cm, fo in cases:
        p0, a0, f0 = o.encode(w, fmt, R, cm, fo)
        p1, a1, m = enc(w, fmt, R, cm, fo)
        assert m.format == f0 and np.array_equal(p0, p1) and np.array_equal(a0, a1), (fmt, R, cm, fo)
        assert np.array_equal(o.decode(p1, a1), w)


def test_encoder_threads_large_tensor_round_trip():
    w = o.weights_like(2048, 2048, 77)
    p1, a1, m = enc(w, 3, 16)
    p0, a0, _ = o.encode(w, 3, 16)
    assert np.array_equal(a0, a1) and np.array_equal(p0, p1)
    assert (m.format, m.R, m.K, m.rows) == (3, 16, 2048, 2048)


@pytest.mark.parametrize("n", [4095, 4096, 4097])
def test_pair_fallback(n):
    w = o.with_pairs(16, 1024, n)
    for cm in (False, True):
        p, a, m = enc(w, 3, 4, cm)
        assert m.format == (3 if n <= 4096 else 2) and m.chunk_major == (cm and n <= 4096)
        assert np.array_equal(o.decode(p, a), w)


def test_argument_errors_and_messages():
    z = torch.zeros(64, 1024, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="multiple of R"):
        ops.encode(z[:15], 3, 4, False)
    with pytest.raises(ValueError, match="chunk-major"):
        ops.encode(z[:16, :512].contiguous(), 3, 4, True)
    with pytest.raises(ValueError, match="chunk-major"):
        ops.encode(z[:16], 2, 4, True)
    with pytest.raises(ValueError, match="fragment order|fragment-order"):
        ops.encode(z[:16], 3, 8, False, True)
    with pytest.raises(ValueError, match="NIBBLE"):
        ops.encode(z[:16], 1, 4, False)
    with pytest.raises(ValueError, match="unknown format"):
        ops.encode(z[:16], 4, 4, False)
    with pytest.raises(ValueError, match="K must be"):
        ops.encode(torch.zeros(16, 500, dtype=torch.bfloat16), 3, 4, False)
    with pytest.raises(RuntimeError):
        ops.encode(z.float(), 3, 4, False)


def test_parse_header_rejects_garbage():
    with pytest.raises(ValueError):
        ops.parse_header(torch.zeros(256, dtype=torch.uint8))
    with pytest.raises(ValueError):
        ops.parse_header(torch.zeros(16, dtype=torch.uint8))
    _, aux, meta = ops.encode(to_bf16_tensor(o.weights_like(16, 1024, 1)), 3, 8, True)
    h = o.parse_header(aux.numpy())
    assert (meta.format, meta.K, meta.rows, meta.R, meta.chunk_major, meta.frag_order) == (3, 1024, 16, 8, True, False)
    assert (meta.off_a, meta.off_b, meta.off_c, meta.off_d) == (h.off_a, h.off_b, h.off_c, h.off_d)
    aux[16] = 9  # unknown flag bits live at byte 72
    aux[72] = 4
    with pytest.raises(ValueError):
        ops.parse_header(aux)


def test_policy_matches_reference_table(policy_table):
    for rows, K, n, engine, mode, expert, dfo, want in policy_table:
        got = ops.choose(rows, K, n, engine=engine, mode=mode, expert=bool(expert), dense_frag_order=bool(dfo))
        assert (list(map(int, got)) if got else None) == want, (rows, K, n, engine, mode, expert, dfo)


def test_policy_of_the_benchmark_shapes():
    assert ops.choose(4096, 2048, engine="llama") == (3, 8, False, False)          # config 0
    assert ops.choose(248320, 2048, engine="llama") == (3, 16, False, False)       # config 1: vocabulary projection
    for rows, K in ((2048, 512), (512, 2048), (256, 2048)):                        # config 2: small matrices
        assert ops.choose(rows, K, engine="llama") == (1, 0, False, False)
    assert ops.choose(512, 2048, 256, engine="llama", expert=True) == (3, 8, True, False)    # expert gate / up
    assert ops.choose(2048, 512, 256, engine="llama", expert=True) == (3, 16, False, False)  # expert down


def test_cpp_wrapper_headers_compile_and_link(tmp_path):
    """include/bf16n/*.h give the reference's C++ surface (namespace, structs, exceptions) over the C ABI."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    src = tmp_path / "t.cpp"
    src.write_text('''
#include "bf16n/encode.h"
#include "bf16n/policy.h"
#include "bf16n/launch.h"
#include <cstdio>
int main() {
    std::vector<uint16_t> w(16 * 512, 0x3c00);
    const bf16n::encoded e = bf16n::encode(w.data(), 16, 512, bf16n::FMT_HUFPAIR, 4, false);
    const auto c = bf16n::choose(248320, 2048);
    bool threw = false;
    try { bf16n::encode(w.data(), 15, 512, bf16n::FMT_HUFPAIR, 4, false); } catch (const std::invalid_argument &) { threw = true; }
    bf16n::weight wv; bf16n::mmv_args a; (void) wv; (void) a;
    std::printf("%zu %d %d %d\\n", e.plane.size(), e.format, c ? c->R : -1, (int) threw);
    return 0;
}
''')
    lib = _lib._build.LIB
    exe = tmp_path / "t"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", str(src), "-o", str(exe),
                    lib, "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out == ["8192", "3", "16", "1"]


def test_adapter_choose_follows_the_llama_policy(policy_table):
    """ggml's conversion tags from the loader entry point of the llama.cpp adapter: 0 stays BF16, 1 NIBBLE, 2 Huffman
    (pairs with single-symbol fallback), for every llama row of the reference's policy table."""
    from orin_qwen_lossless_b200._lib import lib
    n_checked = 0
    for rows, K, n, engine, mode, expert, dfo, want in policy_table:
        if engine != "llama" or dfo:
            continue
        tag = lib().bf16n_adapter_choose(rows, K, n, mode.encode(), 8 << 20, expert)
        assert tag == (0 if want is None else 1 if want[0] == 1 else 2), (rows, K, n, mode, expert, want)
        n_checked += 1
    assert n_checked > 100
    assert lib().bf16n_adapter_count() == 0


def test_choose_for_machine_keeps_the_reference_table_at_512_units(policy_table):
    """The machine-size argument of the shape policy: 512 reproduces every row of the reference's table; a B200-sized
    machine (148 SMs x 24 warps) shortens the units of small dense shards only."""
    from orin_qwen_lossless_b200 import ops
    for rows, K, n, engine, mode, expert, dfo, want in policy_table:
        got = ops.choose(rows, K, n, engine=engine, mode=mode, expert=bool(expert), dense_frag_order=bool(dfo), min_units=512)
        assert (None if got is None else [got[0], got[1], int(got[2]), int(got[3])]) == want
    big = 148 * 24
    assert [ops.choose(r, 2048, engine="llama", mode="huffman", min_units=big)[1] for r in (248320, 124160, 62080, 31040)] == [16, 16, 16, 8]
    assert ops.choose(31040, 2048, engine="llama", mode="huffman")[1] == 16


def test_ep_layout_is_aligned_and_large_enough():
    import ctypes as C
    from orin_qwen_lossless_b200._lib import EpLayout, lib
    lay = EpLayout()
    lay.n_ranks, lay.rank, lay.cap, lay.K, lay.H, lay.n_pairs_max = 8, 3, 8192, 2048, 2048, 8192
    n = lib().bf16n_ep_layout_bytes(C.byref(lay))
    offs = [lay.off_counts, lay.off_expert, lay.off_pair, lay.off_rows, lay.off_back]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert lay.off_pair - lay.off_expert >= 4 * 8 * 8192 and lay.off_back - lay.off_rows >= 2 * 8 * 8192 * 2048
    assert n >= lay.off_back + 4 * 8192 * 2048


def test_workspace_size_and_registration_rules():
    """The two-pass batched product: workspace bytes follow from the matrix (rows x K x 2, twice for a gate/up pair;
    0 for layouts it does not take); registering needs a 1024-byte aligned buffer. No GPU work."""
    from orin_qwen_lossless_b200._lib import Weight, lib
    L = lib()

    def weight(rows, K, R, cm, fo=0, fmt=3):
        w = Weight()
        w.format, w.R, w.K, w.rows, w.cm, w.fo = fmt, R, K, rows, cm, fo
        return w

    gate, up, down = weight(256 * 512, 2048, 8, 1), weight(256 * 512, 2048, 8, 1), weight(256 * 2048, 512, 16, 0)
    assert L.bf16n_mm_ids_workspace_bytes(C.byref(gate), C.byref(up)) == 2 * 256 * 512 * 2048 * 2
    assert L.bf16n_mm_ids_workspace_bytes(C.byref(down), None) == 256 * 2048 * 512 * 2
    for other in (weight(4096, 2048, 16, 0, fo=1), weight(4096, 2048, 8, 0), weight(4096, 1024, 0, 0, fmt=1)):
        assert L.bf16n_mm_ids_workspace_bytes(C.byref(other), None) == 0
    assert L.bf16n_set_workspace(C.c_void_p(4096 + 16), 1 << 20) == 1      # EINVAL: not 1024-byte aligned
    assert b"1024" in L.bf16n_last_error()
    assert L.bf16n_set_workspace(None, 0) == 0
