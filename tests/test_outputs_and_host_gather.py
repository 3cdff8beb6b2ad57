"""Host-side checks that need no GPU: validation of caller-supplied outputs in the Python layer, and the shared host
buffer exchange of a row-sharded projection between two gloo ranks (the GPU product replaced by a CPU stand-in)."""
import multiprocessing as mp
import os

import numpy as np
import pytest
import torch


def test_check_out_rejections():
    from orin_qwen_lossless_b200 import ops
    dev = torch.device("cpu")
    ok = torch.empty((2, 64), dtype=torch.float32)
    with pytest.raises(RuntimeError, match="shape"):
        ops._check_out(ok, (2, 32), torch.float32, dev, "mmv")
    with pytest.raises(RuntimeError, match="dtype"):
        ops._check_out(ok, (2, 64), torch.bfloat16, dev, "mmv")
    with pytest.raises(RuntimeError, match="pinned"):
        ops._check_out(ok, (2, 64), torch.float32, dev, "mmv")   # pageable host memory
    # the remaining rules do not depend on where the memory is: check them through a stand-in that claims to be pinned
    class Pinned(torch.Tensor):
        def is_pinned(self, *a, **k):
            return True
    t = torch.empty((2, 70), dtype=torch.float32).as_subclass(Pinned)
    with pytest.raises(RuntimeError, match="16-byte"):
        ops._check_out(t[:, 1:65], (2, 64), torch.float32, dev, "mmv")          # misaligned base
    with pytest.raises(RuntimeError, match="last dimension"):
        ops._check_out(torch.empty((64, 2)).as_subclass(Pinned).t(), (2, 64), torch.float32, dev, "mmv")
    t3 = torch.empty((2, 4, 80), dtype=torch.float32).as_subclass(Pinned)
    with pytest.raises(RuntimeError, match="dense below"):
        ops._check_out(t3[:, :, :64], (2, 4, 64), torch.float32, dev, "mmv")
    padded = torch.empty((2, 128), dtype=torch.float32).as_subclass(Pinned)[:, :64]
    assert ops._check_out(padded, (2, 64), torch.float32, dev, "mmv") == 512    # padded rows: the byte stride is passed on


def _rank(rank, world, port, rows, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from orin_qwen_lossless_b200 import sharded
    table = torch.arange(rows, dtype=torch.float32)

    def compute(x, out):           # stands in for the GEMV: row r of the projection "multiplies" to r * x[0, 0]
        a0 = sharded.unit_range(rank, world, rows, 16)[0]
        out.copy_(table[a0:a0 + out.shape[1]].view(1, -1) * x[0, 0])

    h = sharded.HostGatheredLinear(None, rows, 16, 1, compute=compute)
    got = []
    for s in range(1, 5):
        y = h.step(torch.full((1, 8), float(s)))
        got.append(bool(torch.equal(y[0], table * s)))   # every rank sees every shard of this step
    h.close()
    q.put((rank, got))
    dist.destroy_process_group()


def test_host_gathered_linear_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_rank, args=(r, 2, port, 16 * 37, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(timeout=60)
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(all(g) for _, g in res)
