"""The loader side of the llama.cpp adapter (csrc/adapter.cu): convert (encode, upload into the tensor's own storage,
aux allocation, registry, exhaustive device-side round trip, one log line), lookup of the tensor and of views that start
on later rows, products through the looked-up matrix, release by owner."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import bits_of, to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


def convert(lib, w_bits, n_matrices, tag, owner, name):
    rows, K = w_bits.shape
    plane = torch.empty(rows * K, dtype=torch.uint8, device="cuda")
    host = np.ascontiguousarray(w_bits)
    ok = C.c_int(-1)
    rc = lib.bf16n_adapter_convert(plane.data_ptr(), host.ctypes.data, K, rows // n_matrices, n_matrices, tag, owner, name.encode(), C.byref(ok))
    return rc, ok.value, plane


def test_convert_lookup_views_and_release(ops, capfd):
    from orin_qwen_lossless_b200._lib import MmvArgs, Weight, check, lib
    L = lib()
    base = L.bf16n_adapter_count()
    dense = o.weights_like(8192, 2048, 41, outliers=True)          # 16 M weights: pair Huffman, R = 16 by the llama policy
    small = o.weights_like(512, 2048, 42)                           # 1 M weights, format 1 requested: NIBBLE
    experts = o.weights_like(16 * 512, 2048, 43)                    # 16 experts of 512 x 2048: chunk-major R = 8
    rc, ok, p_dense = convert(L, dense, 1, 2, 0x1000, "blk.0.attn_q.weight")
    assert (rc, ok) == (0, 1)
    rc, ok, p_small = convert(L, small, 1, 1, 0x1000, "blk.0.ffn_gate_inp.weight")
    assert (rc, ok) == (0, 1)
    rc, ok, p_exp = convert(L, experts, 16, 2, 0x2000, "blk.0.ffn_gate_exps.weight")
    assert (rc, ok) == (0, 1)
    err = capfd.readouterr().err
    assert "bf16n: blk.0.attn_q.weight" in err and "hufpair K= 2048 rows=   8192 R=16" in err and "roundtrip=OK" in err
    assert "nibble  K= 2048 rows=    512 R= 0" in err
    assert L.bf16n_adapter_count() == base + 3

    w, row0 = Weight(), C.c_int64(-1)
    assert L.bf16n_adapter_lookup(p_dense.data_ptr(), C.byref(w), C.byref(row0)) == 1
    assert (w.format, w.R, w.K, w.rows, w.cm, row0.value) == (3, 16, 2048, 8192, 0, 0)
    assert L.bf16n_adapter_lookup(p_dense.data_ptr() + 4096 * 2048, C.byref(w), C.byref(row0)) == 1 and row0.value == 4096
    assert L.bf16n_adapter_lookup(p_dense.data_ptr() + 7, None, None) == 0                  # not on a row
    assert L.bf16n_adapter_lookup(p_dense.data_ptr() + 8192 * 2048, C.byref(w), C.byref(row0)) in (0, 1)  # past the end: another tensor or nothing
    we = Weight()
    assert L.bf16n_adapter_lookup(p_exp.data_ptr(), C.byref(we), C.byref(row0)) == 1 and (we.cm, we.R) == (1, 8)

    # a product through a looked-up view: rows [4096, 8192) of the dense tensor
    assert L.bf16n_adapter_lookup(p_dense.data_ptr() + 4096 * 2048, C.byref(w), C.byref(row0)) == 1
    xb = o.f32_to_bf16_bits(np.random.default_rng(1).standard_normal(2048).astype(np.float32))
    x = to_bf16_tensor(xb).view(1, 2048).cuda()
    y = torch.empty(1, 4096, device="cuda")
    a = MmvArgs()
    a.x, a.x_bf16, a.y, a.y_bf16, a.ncols, a.n_used, a.x_per_slot = x.data_ptr(), 1, y.data_ptr(), 0, 1, 1, 1
    a.x_tok, a.y_tok, a.rows_per_matrix, a.row0, a.nrows = 4096, 4096 * 4, 4096, row0.value, 4096
    check(L.bf16n_mmv(C.byref(w), C.byref(a), torch.cuda.current_stream().cuda_stream, 1))
    want = o.gemv_f32_order(dense[4096:], o.bf16_bits_to_f32(xb))
    assert np.array_equal(y.cpu().numpy()[0].view(np.uint32), want.view(np.uint32))
    # exact rows back out of the registry entry
    out = torch.empty(32, 2048, dtype=torch.bfloat16, device="cuda")
    check(L.bf16n_dequant(C.byref(w), 4096, 32, out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    assert np.array_equal(bits_of(out), dense[4096:4128])

    torch.cuda.synchronize()
    assert L.bf16n_adapter_release(0x1000) == 2
    assert L.bf16n_adapter_lookup(p_dense.data_ptr(), None, None) == 0
    assert L.bf16n_adapter_lookup(p_exp.data_ptr(), None, None) == 1
    assert L.bf16n_adapter_release(0x2000) == 1 and L.bf16n_adapter_count() == base


def test_convert_rejections(ops):
    from orin_qwen_lossless_b200._lib import EINVAL, lib
    L = lib()
    w = o.weights_like(16, 1000, 5)   # K is not a multiple of 512
    rc, ok, _ = convert(L, w, 1, 2, 0x3000, "odd")
    assert rc == EINVAL and L.bf16n_adapter_release(0x3000) == 0
    rc, ok, _ = convert(L, o.weights_like(16, 2048, 6), 1, 3, 0x3000, "tag")
    assert rc == EINVAL and b"format tag" in L.bf16n_last_error()
