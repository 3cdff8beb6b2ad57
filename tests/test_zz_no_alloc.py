"""bf16n_moe_decode_static: the MoE decode step for callers that cannot allocate device memory (its intermediate
buffers live in an array inside the library instead of a caller-provided scratch buffer).

Called here straight through the C ABI, twice in a row with different inputs: each result must equal, bit for bit, what
bf16n_moe_decode computes with a scratch buffer of the caller's own - the second call also shows that what the first
one left in the shared buffer does no harm. A step larger than the built-in buffer must be refused with a clear
message. This file sorts last on purpose, so a run that stops at the first failure has already run every other test;
it does not depend on them and also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
E, TOPK, H, N = 8, 4, 2048, 512


def _encode(ops, bits, R, cm):
    plane, aux, meta = ops.encode(to_bf16_tensor(bits), 3, R, cm)
    return ops.upload(plane, aux, meta, "cuda")


def test_static_scratch_entry_point_matches_the_allocating_one():
    from orin_qwen_lossless_b200 import _lib, ops
    assert torch.cuda.is_available()
    ops.init()
    lib = _lib.lib()
    gate, up, down = (_encode(ops, o.weights_like(E * N, H, 71), 8, True), _encode(ops, o.weights_like(E * N, H, 72), 8, True),
                      _encode(ops, o.weights_like(E * H, N, 73), 16, False))
    cg, cu, cd = gate.c(), up.c(), down.c()
    stream = torch.cuda.current_stream().cuda_stream
    for call, T in enumerate((4, 2)):  # two calls in a row, different shapes and data
        g = np.random.default_rng(100 + call)
        x = to_bf16_tensor(o.f32_to_bf16_bits(g.standard_normal((T, H)).astype(np.float32))).cuda()
        logits = torch.from_numpy(g.standard_normal((T, E)).astype(np.float32)).cuda()
        ids_a = torch.empty((T, TOPK), dtype=torch.int32, device="cuda")
        ids_b = torch.empty_like(ids_a)
        w_a = torch.empty((T, TOPK), dtype=torch.float32, device="cuda")
        w_b = torch.empty_like(w_a)
        y_a = torch.full((T, H), float("nan"), device="cuda")
        y_b = torch.full((T, H), float("nan"), device="cuda")
        nbytes = lib.bf16n_moe_decode_scratch_bytes(T, TOPK, N, H)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
        rc = lib.bf16n_moe_decode(C.byref(cg), C.byref(cu), C.byref(cd), x.data_ptr(), 1, x.stride(0) * 2, logits.data_ptr(), E,
                                  ids_a.data_ptr(), w_a.data_ptr(), T, TOPK, 0, E, scratch.data_ptr(), nbytes, y_a.data_ptr(), 0, stream)
        assert rc == 0, lib.bf16n_last_error()
        rc = lib.bf16n_moe_decode_static(C.byref(cg), C.byref(cu), C.byref(cd), x.data_ptr(), 1, x.stride(0) * 2, logits.data_ptr(), E,
                                         ids_b.data_ptr(), w_b.data_ptr(), T, TOPK, 0, E, y_b.data_ptr(), 0, stream)
        assert rc == 0, lib.bf16n_last_error()
        torch.cuda.synchronize()
        assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b)
        assert torch.isfinite(y_b).all() and torch.equal(y_a, y_b)  # same kernels, same order: equal bit for bit

    # a step that does not fit the built-in buffer is refused, and says so
    T = 64
    x = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
    logits = torch.zeros((T, E), dtype=torch.float32, device="cuda")
    ids = torch.empty((T, TOPK), dtype=torch.int32, device="cuda")
    wts = torch.empty((T, TOPK), dtype=torch.float32, device="cuda")
    y = torch.empty((T, H), device="cuda")
    rc = lib.bf16n_moe_decode_static(C.byref(cg), C.byref(cu), C.byref(cd), x.data_ptr(), 1, x.stride(0) * 2, logits.data_ptr(), E,
                                     ids.data_ptr(), wts.data_ptr(), T, TOPK, 0, E, y.data_ptr(), 0, stream)
    assert rc == _lib.EINVAL
    msg = lib.bf16n_last_error().decode()
    assert "built-in buffer" in msg and "196608" in msg
