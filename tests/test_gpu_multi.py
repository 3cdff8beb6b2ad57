"""Two-GPU runs of the sharded paths (skipped with fewer than two GPUs): row-sharded projection + NCCL all-gather, the same
projection with the gather fused into the GEMV kernel (stores to peer memory, epoch flags, bounded wait kernel),
expert-parallel MoE decode + all-reduce, expert-parallel MoE prefill + all-to-all, each against the single-GPU result."""
import os
import socket

import numpy as np
import pytest
import torch

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o

pytestmark = pytest.mark.gpu
E, TOPK, H, N = 8, 4, 2048, 512


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops, sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ops.init()
        dev = torch.device("cuda", rank)

        def enc(bits, R, cm):
            p, a, m = ops.encode(to_bf16_tensor(bits), 3, R, cm)
            return p, a, m

        # 1. projection: one encoded tensor, sliced on unit boundaries
        rows, K, R = 16 * 2049, 2048, 16
        wb = o.weights_like(rows, K, 7)
        p, a, m = enc(wb, R, False)
        r0, r1 = sharded.unit_range(rank, world, rows, R)
        sp, sa, sm = sharded.shard_rows(p, a, r0, r1)
        lin = sharded.ShardedLinear(ops.upload(sp, sa, sm, dev), rows, R)
        x = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(3).standard_normal((2, K)).astype(np.float32))).to(dev)
        y = lin.assemble(lin(x, lin.buffers(2, dev)))
        full = ops.mmv(x, ops.upload(p, a, m, dev))
        ok1 = bool(torch.equal(y, full))  # every row is computed by the same kernel code: bitwise

        # 1b. the same projection with the gather fused into the GEMV kernel: peer stores + epoch flags, no collective.
        # Several steps with changing activations, under a CUDA graph too (the epoch counters live on the device).
        ok1b = True
        for T1, big in ((2, 0), (1, 16), (1, 10)):  # units per SM and rank: general kernel, per-lane rings, bulk-copy staged
            if big:
                rows_b = 16 * 148 * big * world
                wb_b = o.weights_like(rows_b, K, 8)
                p_b, a_b, m_b = enc(wb_b, R, False)
                rb0, rb1 = sharded.unit_range(rank, world, rows_b, R)
                sh = ops.upload(*sharded.shard_rows(p_b, a_b, rb0, rb1), dev)
                whole, nrows = ops.upload(p_b, a_b, m_b, dev), rows_b
            else:
                sh, whole, nrows = ops.upload(sp, sa, sm, dev), ops.upload(p, a, m, dev), rows
            fused = sharded.FusedShardedLinear(sh, nrows, R, T1, wait_in_kernel=bool(big != 10))  # both forms of the wait
            xs = [to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(40 + i).standard_normal((T1, K)).astype(np.float32))).to(dev)
                  for i in range(4)]
            for i in range(4):
                got = fused.assemble(fused(xs[i]))
                ok1b = ok1b and bool(torch.equal(got, ops.mmv(xs[i], whole)))
            xg = xs[0].clone()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                outs = [fused.assemble(fused(xg)) for _ in range(2)]   # both buffers in turn
            for i in range(1, 4):
                xg.copy_(xs[i])
                gr.replay()
                torch.cuda.synchronize()
                want = ops.mmv(xs[i], whole)
                ok1b = ok1b and all(bool(torch.equal(t, want)) for t in outs)
            ok1b = ok1b and not fused.xchg.expired()
            fused.close()

        # 1c. the end-to-end form: every rank's kernel stores its shard into one pinned host buffer shared by the processes
        # and then its epoch word; eager, captured and replayed steps, one and two tokens
        hg = sharded.HostGatheredLinear(ops.upload(sp, sa, sm, dev), rows, R, 2)
        ok1c = True
        for T1 in (1, 2):
            xh = torch.empty((T1, K), dtype=torch.bfloat16).pin_memory()
            for i in range(6):
                xi = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(70 + i).standard_normal((T1, K)).astype(np.float32)))
                xh.copy_(xi)
                got = hg.step(xh).clone()
                ok1c = ok1c and bool(torch.equal(got, ops.mmv(xi.to(dev), ops.upload(p, a, m, dev)).cpu()))
        hg.close()
        ok1b = ok1b and ok1c

        # 2. MoE decode, experts split over the ranks
        bits = {"gate": o.weights_like(E * N, H, 11), "up": o.weights_like(E * N, H, 12), "down": o.weights_like(E * H, N, 13)}
        n_local = E // world

        def up_slice(name, R, cm, lo, n):
            rpe = bits[name].shape[0] // E
            return ops.upload(*enc(bits[name][lo * rpe:(lo + n) * rpe], R, cm), dev)

        g, u, d = (up_slice("gate", 8, True, 0, E), up_slice("up", 8, True, 0, E), up_slice("down", 16, False, 0, E))
        gl, ul, dl = (up_slice("gate", 8, True, rank * n_local, n_local), up_slice("up", 8, True, rank * n_local, n_local),
                      up_slice("down", 16, False, rank * n_local, n_local))
        T = 4
        xt = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(5).standard_normal((T, H)).astype(np.float32))).to(dev)
        logits = torch.from_numpy(np.random.default_rng(6).standard_normal((T, E)).astype(np.float32)).to(dev)
        y_ep, _, _ = sharded.moe_decode_ep(xt, gl, ul, dl, E, TOPK, logits)
        y_1, wts, ids = ops.moe_decode(xt, g, u, d, E, TOPK, router_logits=logits)
        ok2 = bool(torch.allclose(y_ep, y_1, rtol=0, atol=2.0 ** -17 * float(y_1.abs().max()) * TOPK))
        # 2b. the same step with the all-reduce fused away: the combine kernel stores the partial output into every rank,
        # a small kernel adds the partials in rank order (every rank gets the same bits), eager and from a CUDA graph
        fmd = sharded.FusedMoeDecode(gl, ul, dl, E, TOPK, T)
        extra = torch.from_numpy(np.random.default_rng(8).standard_normal((T, H)).astype(np.float32)).to(dev)
        y_f = torch.empty((T, H), device=dev)
        for _ in range(3):
            fmd(xt, logits, y_f, extra)
        tol = 2.0 ** -17 * float(y_1.abs().max()) * TOPK
        ok2 = ok2 and bool(torch.allclose(y_f - extra, y_1, rtol=0, atol=tol))
        both = [torch.empty_like(y_f) for _ in range(world)]
        dist.all_gather(both, y_f)
        ok2 = ok2 and all(bool(torch.equal(b_, y_f)) for b_ in both)
        torch.cuda.synchronize()
        gr2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr2):
            for _ in range(2):
                fmd(xt, logits, y_f, extra)
        want_f = y_f.clone()
        y_f.zero_()
        gr2.replay()
        torch.cuda.synchronize()
        ok2 = ok2 and bool(torch.equal(y_f, want_f)) and not fmd.xchg.expired()
        fmd.close()

        # 3. MoE prefill: tokens split over the ranks, all-to-all dispatch to the experts' ranks
        Tp = 40 + 8 * rank
        xp = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(20 + rank).standard_normal((Tp, H)).astype(np.float32))).to(dev)
        lg = torch.from_numpy(np.random.default_rng(30 + rank).standard_normal((Tp, E)).astype(np.float32)).to(dev)
        w_p, i_p = ops.moe_topk(lg, TOPK)
        y_a2a = sharded.moe_prefill_ep(xp, w_p, i_p, gl, ul, dl, E)
        y_loc = ops.moe_experts(xp, g, u, d, w_p, i_p, E)
        err = float((y_a2a.float() - y_loc.float()).abs().max())
        ok3 = err <= 2.0 ** -7 * float(y_loc.float().abs().max())
        # 3b. the same layer with the rows exchanged by peer stores on the device (no host round trip, no collective):
        # bit-equal to the all-to-all form, over several layers with different token counts and from a CUDA graph
        fmp = sharded.FusedMoePrefill(gl, ul, dl, E, TOPK, 64)
        ok3 = ok3 and bool(torch.equal(fmp(xp, w_p, i_p), y_a2a))
        for t2 in (9 + 3 * rank, 64):
            x2 = to_bf16_tensor(o.f32_to_bf16_bits(np.random.default_rng(50 + t2 + rank).standard_normal((t2, H)).astype(np.float32))).to(dev)
            w2, i2 = ops.moe_topk(torch.from_numpy(np.random.default_rng(60 + t2 + rank).standard_normal((t2, E)).astype(np.float32)).to(dev), TOPK)
            ok3 = ok3 and bool(torch.equal(fmp(x2, w2, i2), sharded.moe_prefill_ep(x2, w2, i2, gl, ul, dl, E)))
        want_g = fmp(xp, w_p, i_p).clone()
        torch.cuda.synchronize()
        gr3 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr3):
            y_g = fmp(xp, w_p, i_p)
        gr3.replay()
        gr3.replay()
        torch.cuda.synchronize()
        ok3 = ok3 and bool(torch.equal(y_g, want_g)) and not fmp.xchg.expired() and ops.fault_status() == 0
        fmp.close()
        ret[rank] = (ok1, ok1b, ok2, ok3)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_paths():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    assert [ret[r] for r in range(2)] == [(True, True, True, True)] * 2
