"""Host-visible status of the bounded device waits: the read-and-clear fault word call, and a wait for a peer's
announcement that runs out (a flag nothing sets, polled in local memory, with a short host-set limit)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from orin_qwen_lossless_b200 import ops as m
    assert torch.cuda.is_available()
    m.init()
    return m


def test_fault_status_is_clear_after_normal_launches(ops):
    import numpy as np
    from conftest import to_bf16_tensor
    from oracle import cpu_oracle as o
    w = o.weights_like(8192, 2048, 3)
    plane, aux, meta = ops.encode(to_bf16_tensor(w), 3, 16, False)
    enc = ops.upload(plane, aux, meta, "cuda")
    x = torch.randn(1, 2048, device="cuda").to(torch.bfloat16)
    y = ops.mmv(x, enc)                      # the bulk-copy staged kernel
    assert ops.fault_status() == 0
    assert bool(torch.isfinite(y).all())
    assert ops.fault_status() == 0           # read-and-clear: still clear


def test_peer_wait_expires_and_reports(ops):
    from orin_qwen_lossless_b200._lib import check, lib
    base = C.c_void_p()
    handle = C.create_string_buffer(64)
    check(lib().bf16n_exchange_create(1024, C.byref(base), handle))
    try:
        ops.set_peer_wait_limit_ms(5)
        st = torch.cuda.current_stream().cuda_stream
        check(lib().bf16n_peer_wait(base, 0b10, st))       # rank 1 never announces anything
        v = C.c_int(-1)
        check(lib().bf16n_peer_expired(base, st, C.byref(v)))
        assert v.value == 1
        # the context is still usable and the next wait on an announced epoch passes: rank 1's flag word set by hand
        torch.cuda.synchronize()
    finally:
        ops.set_peer_wait_limit_ms(2000)
        check(lib().bf16n_exchange_destroy(base))
    with pytest.raises(ValueError, match="1..60000"):
        ops.set_peer_wait_limit_ms(0)


def test_null_arguments_are_rejected(ops):
    from orin_qwen_lossless_b200._lib import Weight, lib, EINVAL
    w = Weight()
    rc = lib().bf16n_moe_decode(C.byref(w), C.byref(w), None, None, 1, 0, None, 256, None, None, 1, 8, 0, 256, None, 0, None, 0, None)
    assert rc == EINVAL and b"null" in lib().bf16n_last_error()
    rc = lib().bf16n_fault_status(None, None)
    assert rc == EINVAL
