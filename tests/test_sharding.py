"""Host logic of the multi-GPU paths, on CPU: slicing an encoded tensor into per-rank tensors, and the collectives'
bookkeeping with world_size 2 over gloo (row-sharded projection + all-gather, expert-parallel token dispatch)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o
from orin_qwen_lossless_b200 import ops, sharded


@pytest.mark.parametrize("fmt,R,cm", [(1, 0, False), (2, 8, False), (3, 16, False), (3, 8, True), (3, 1, False)])
def test_shard_rows_decodes_to_the_row_ranges(fmt, R, cm):
    rows, K = 96, 1024
    w = o.with_specials(o.weights_like(rows, K, fmt * 10 + R, outliers=True), 5).reshape(rows, K)
    plane, aux, meta = ops.encode(to_bf16_tensor(w), fmt, R, cm)
    unit = max(R, 1)
    for world in (1, 2, 3, 4):
        got = []
        for rank in range(world):
            r0, r1 = sharded.unit_range(rank, world, rows, unit)
            p, a, m = sharded.shard_rows(plane, aux, r0, r1)
            assert (m.format, m.K, m.rows, m.R, m.chunk_major) == (meta.format, K, r1 - r0, meta.R, meta.chunk_major)
            if r1 > r0:
                got.append(o.decode(p.numpy(), a.numpy()))
        assert np.array_equal(np.concatenate(got), w)
    with pytest.raises(ValueError):
        sharded.shard_rows(plane, aux, 1 if unit > 1 else -1, unit)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return [ret[r] for r in range(world)]


def _lm_head_job(rank, world):
    rows, K, R = 16 * 9, 512, 16   # 9 units: uneven shards (4 + 5)
    w = o.weights_like(rows, K, 3)
    dense = torch.from_numpy(o.bf16_bits_to_f32(w))
    r0, r1 = sharded.unit_range(rank, world, rows, R)
    ops.mmv = lambda x, wt, out=None: (out.copy_(x.float() @ wt.t()) if out is not None else x.float() @ wt.t())  # CPU stand-in
    lin = sharded.ShardedLinear(dense[r0:r1], rows, R)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((2, K)).astype(np.float32))
    g = lin(x, lin.buffers(2, "cpu"))
    y = lin.assemble(g)
    return bool(torch.allclose(y, x @ dense.t())) and y.shape == (2, rows)


def test_row_sharded_projection_all_gather_gloo():
    assert _run(_lm_head_job) == [True, True]


def _prefill_job(rank, world):
    E, k, H, T = 8, 3, 16, 5 + rank          # different token counts per rank
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    wts = torch.rand(T, k, generator=g)
    n_local = E // world

    def experts(rows, local_e):  # stand-in for the batched kernels: expert e scales by (e + 1)
        return rows * (local_e.to(rows.dtype) + 1 + rank * n_local).unsqueeze(1)

    y = sharded.moe_prefill_ep(x, wts, ids, None, None, None, E, experts_fn=experts)
    ref = sum(wts[:, s:s + 1] * x * (ids[:, s:s + 1].float() + 1) for s in range(k))
    return bool(torch.allclose(y, ref, atol=1e-5))


def test_expert_parallel_dispatch_all_to_all_gloo():
    assert _run(_prefill_job) == [True, True]


def test_dispatch_plan_orders_pairs_by_owner():
    ids = torch.tensor([[0, 5, 2], [7, 1, 4]])
    order, counts, local_e = sharded.dispatch_plan(ids, 8, 2)
    assert counts.tolist() == [3, 3]
    assert order.tolist() == [0, 2, 4, 1, 3, 5] and local_e.tolist() == [0, 2, 1, 1, 3, 0]
