"""Benchmark of the BF16N hot path on B200: the vocabulary projection (lm_head) decode+GEMV, with the MoE layer and the
small-matrix graph of the same metric carried in the same line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-moe] [--no-cpu]

Workload of the headline number (the configuration the metric is quoted on): a 248320 x 2048 BF16 matrix, weights
N(0, 0.02) rounded to BF16 (seeded, synthetic), pair-Huffman coded with R = 16 as the shape policy chooses, multiplied by
one BF16 N(0,1) activation vector with FP32 accumulation and FP32 logits. With N > 1 ranks the rows are split into N
shards (one process per GPU); each rank's GEMV kernel stores its logits into every GPU itself (no collective).

A "block" is exactly --steps steps between barriers and device synchronisation, timed with CUDA events (max over
ranks); at least 30 blocks and one second of them are run and the line reports their median, minimum and maximum. A
shard smaller than 256 MB is multiplied from several copies at different addresses, used in turn, so that L2 cannot
serve it (config.l2 says what was done).

One JSON line on stdout (rank 0):
  value    GB/s of compressed bytes (plane + aux + x + y) per second with everything resident in HBM
  e2e      the same with the activation in pinned host memory and the logits back in host memory every step
           (sharded.HostGatheredLinear: one host buffer shared by the ranks, written by the GEMV kernels)
  roofline achieved / measured copy bandwidth for the GEMV kernel (one launch per step)
  cublas_bf16_gemv_us   the stock BF16 GEMV of the same (uncompressed) shard on the same GPU
  multi_token           the same matrix with 2 and 4 activation columns (one decode for all of them)
  moe      the MoE layer: decode at 1 / 2 / 4 tokens and prefill at 2048 / 8192 tokens (expert-parallel over the ranks),
           each with microseconds, bytes or flops, fraction of the roofline and a parity figure against the FP64 oracle
  small_matrices        the graph of 144 NIBBLE GEMVs (one GPU)
  cpu_baseline  the CPU oracle's decode+GEMV on this box's host threads (bounded sample)
`--impl reference` times the CPU arm only (the reference ships no CPU GEMV, so this is the oracle's port of its decoder
and summation; the encoder timed beside it is the reference's own when oracle/_ref is present).
`--workload small | moe_decode | moe_prefill | dense_mid` print those blocks on their own.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, K, R = 248320, 2048, 16
# DRAM bytes moved per algorithmic byte by the GEMV kernel: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture
# on a 65536-row case of the same matrix family (181.97 MB moved for 179.01 MB algorithmic, profiles/lm_head_gemv_ncu.md);
# traffic grows in proportion to the rows, so a full launch is this ratio times its algorithmic bytes.
DRAM_TRAFFIC_RATIO = 1.017
BLOCK_ROWS = 4096  # weights are generated in seeded blocks of rows so that every shard is reproducible on its own


def gen_rows(r0: int, r1: int):
    """BF16 weights of rows [r0, r1): N(0, 0.02) from torch's CPU generator, one seed per block of 4096 rows."""
    import torch
    out = torch.empty((r1 - r0, K), dtype=torch.bfloat16)
    b0 = r0 // BLOCK_ROWS
    for b in range(b0, (r1 + BLOCK_ROWS - 1) // BLOCK_ROWS):
        g = torch.Generator().manual_seed(0xB16 + b)
        blk = (torch.randn((BLOCK_ROWS, K), generator=g) * 0.02).to(torch.bfloat16)
        lo, hi = max(r0, b * BLOCK_ROWS), min(r1, (b + 1) * BLOCK_ROWS)
        out[lo - r0:hi - r0] = blk[lo - b * BLOCK_ROWS:hi - b * BLOCK_ROWS]
    return out


def gen_x():
    import torch
    g = torch.Generator().manual_seed(0xAC7)
    return torch.randn((1, K), generator=g).to(torch.bfloat16)


def shard_range(rank: int, world: int, rows: int):
    units = rows // R
    u0, u1 = units * rank // world, units * (rank + 1) // world
    return u0 * R, u1 * R


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.samples, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = [float(s[0]) for s in self.samples if len(s) >= 6 and s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples if len(s) >= 6 for n, v in zip(names, s[2:6]) if v.startswith("Active")})
        mx = [float(s[1]) for s in self.samples if len(s) >= 6 and s[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


CPU_SAMPLE_ROWS = 65536   # rows of the workload the CPU arm decodes and multiplies per pass (179 MB compressed)


METRIC = "lm_head_248320x2048_bf16n_decode_gemv_compressed_GBps"


def cpu_arm(rows_sample: int, reps: int, warmup: int = 1):
    """The CPU arm: encode (reference encoder when oracle/_ref is present, else the oracle's restatement) and the
    oracle's decode+GEMV on all host threads, on the first `rows_sample` rows of the workload."""
    from oracle import cpu_oracle as o
    import torch
    threads = os.cpu_count() or 1
    w = gen_rows(0, rows_sample)
    wb = w.view(torch.int16).numpy().view(np.uint16)
    t0 = time.perf_counter()
    plane, aux, _ = (o.ref_encode if o.have_ref() else o.encode)(wb, 3, R)
    t_enc = time.perf_counter() - t0
    x = o.bf16_bits_to_f32(gen_x().view(torch.int16).numpy().view(np.uint16)[0])
    units = rows_sample // R
    nbytes = plane.size + aux.size + K * 2 + rows_sample * 4
    t0 = time.perf_counter()
    o.decode_gemv_mt(plane, aux, x, 0, units, threads)       # first warm-up pass, also sizes the run: about 20 s of CPU work at most
    one = max(time.perf_counter() - t0, 1e-4)
    warmup = max(1, min(warmup, max(1, int(5.0 / one))))
    for _ in range(warmup - 1):
        o.decode_gemv_mt(plane, aux, x, 0, units, threads)
    reps = max(1, min(reps, max(3, int(20.0 / one))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        o.decode_gemv_mt(plane, aux, x, 0, units, threads)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"first {rows_sample} of {ROWS} rows ({nbytes / 1e6:.1f} MB compressed), median of {reps} passes of "
                      f"{dt:.3f} s; encoder ({'reference' if o.have_ref() else 'oracle'}) {rows_sample * K * 2 / t_enc / 1e9:.2f} GB/s of BF16 input",
            "ms_per_step": dt * 1e3, "encode_s": t_enc, "passes": reps, "warmup": warmup}, nbytes


def reference_kernels():
    """The reference's own CUDA kernels, recompiled for sm_100a (baseline/Makefile `ref`: its sources compiled where they
    lie, binary in baseline/_ref/), timed on this GPU on the same shape through the same C++ interface. None when the
    binary was not built."""
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "api_bench_ref")
    if not os.path.exists(exe):
        return None
    try:
        out = subprocess.run([exe, "lm_head", "30"], capture_output=True, text=True, timeout=300).stdout
        rec = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
        return {"us_per_step": rec["us"], "compressed_GBps": rec["compressed_GBps"], "what": rec["impl"] + ", " + rec["workload"]}
    except Exception as e:  # a missing CUDA runtime for the binary, a timeout: report, do not fail the bench
        return {"unavailable": str(e)[:200]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows_sample = CPU_SAMPLE_ROWS
    base, nbytes = cpu_arm(rows_sample, max(1, args.steps), max(0, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"],
            "unit": "GB/s", "n_gpus": args.gpus, "steps": base["passes"], "warmup": base["warmup"], "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "lm_head 248320x2048 HUFPAIR R=16, batch-1 decode GEMV (CPU arm: bounded row sample)",
                       "rows_sample": rows_sample},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


L2_ROTATE_BELOW = 256e6   # working sets smaller than this are served from rotating copies so that L2 cannot hold them
MIN_BLOCKS, MIN_TIMED_S = 30, 1.0


def run_ours(args):
    import torch
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the library has no CPU path; use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ops.init()
    rows = args.rows
    r0, r1 = shard_range(rank, world, rows)

    t0 = time.perf_counter()
    w = gen_rows(r0, r1)
    t_gen = time.perf_counter() - t0
    # rows per unit as the shape policy picks them for this rank's matrix on this machine (SMs x 24 warps must have a
    # unit each): 16 for the whole projection and its halves and quarters, 8 for an eighth
    shard_R = ops.choose(r1 - r0, K, engine="llama", mode="huffman", min_units=ops.sm_count() * 24)[1]
    t0 = time.perf_counter()
    plane, aux, meta = ops.encode(w, ops.FMT_HUFPAIR, shard_R, False)
    t_enc = time.perf_counter() - t0
    enc = ops.upload(plane, aux, meta, dev)
    ok = ops.roundtrip_equal(enc, w)  # verify at load: bit-exact decode of the whole shard on the GPU
    if not ok:
        raise SystemExit("bench.py: GPU decode of the encoded shard is not bit-exact")
    del w
    shard_bytes = plane.numel() + aux.numel()
    # a shard that L2 (126 MB) could serve is multiplied from rotating copies at different addresses
    n_copies = 1 if shard_bytes >= L2_ROTATE_BELOW else max(3, int(np.ceil(2 * L2_ROTATE_BELOW / shard_bytes)))
    copies = [enc] + [ops.upload(plane, aux, meta, dev) for _ in range(n_copies - 1)]
    counts = torch.tensor([shard_bytes], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(counts)
    total_weight_bytes = int(counts.item())
    algo_bytes = total_weight_bytes + K * 2 + rows * 4          # all ranks: compressed weights + x (BF16) + logits (FP32)
    shard_algo_bytes = shard_bytes + K * 2 + (r1 - r0) * 4      # one launch on this rank

    x_host = gen_x().pin_memory()
    x = x_host.to(dev)
    logits = torch.empty((1, rows), dtype=torch.float32, device=dev)
    # shards are padded to the widest one so that a single all-gather assembles the logits
    per = [shard_range(i, world, rows) for i in range(world)]
    width = max(b - a for a, b in per)
    gathered = torch.empty((world, width), dtype=torch.float32, device=dev)
    mine = gathered[rank, : r1 - r0].view(1, r1 - r0) if world > 1 else logits
    turn = [0]

    def next_copy():
        turn[0] = (turn[0] + 1) % n_copies
        return copies[turn[0]]

    def step_nccl():
        ops.mmv(x, next_copy(), out=mine)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), gathered[rank])

    # N > 1, the product: the GEMV kernel stores its logits into every GPU's gathered buffer itself (peer stores over
    # NVLink, epoch flags; the kernel ends when the peers' logits have arrived); no collective. A CUDA graph holds exactly
    # --steps steps (the two exchange buffers in turn, walking through the rotating copies); with an odd step count a second
    # graph that starts on the other buffer takes every other block, so that the buffers keep alternating across replays.
    fused = None
    graphs = []
    fused_note = None
    per_call = 1
    if world > 1:
        from orin_qwen_lossless_b200 import sharded
        try:
            fused = sharded.FusedShardedLinear(enc, rows, R, 1)
        except (RuntimeError, ValueError) as e:   # e.g. no peer access between these GPUs: say so and gather with NCCL
            fused_note = str(e)
        agree = torch.tensor([0 if fused else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(agree)
        if int(agree.item()) and fused:
            fused.close()
            fused, fused_note = None, "exchange buffers unavailable on another rank"
    if fused and args.steps <= 4096:
        per_call = args.steps
        last = [fused(x, next_copy()) for _ in range(2)]
        torch.cuda.synchronize()
        for _ in range(1 if per_call % 2 == 0 else 2):
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_):
                last = [fused(x, next_copy()) for _ in range(per_call)]
            graphs.append(g_)
    which = [0]

    def step():
        if graphs:
            graphs[which[0] % len(graphs)].replay()     # per_call steps
            which[0] += 1
        elif fused:
            fused(x, next_copy())
        else:
            step_nccl()

    # end to end: activation from pinned host memory, logits back in host memory, every step
    hosted = None
    y_host = None
    from orin_qwen_lossless_b200 import sharded
    try:   # every rank's kernel stores its shard into one pinned host buffer shared by the processes of the node
        hosted = sharded.HostGatheredLinear(enc, rows, R, 1)
    except (RuntimeError, OSError) as e:
        fused_note = (fused_note + "; " if fused_note else "") + f"shared host buffer unavailable: {e}"
    if world > 1:
        agree = torch.tensor([0 if hosted else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(agree)
        if int(agree.item()) and hosted:
            hosted.close()
            hosted = None
    if hosted is None:
        y_host = torch.empty((1, rows if world == 1 else world * (fused.width if fused else width)), dtype=torch.float32).pin_memory()

    def step_e2e():
        if hosted is not None:
            # one graph launch (activation copy from pinned memory + GEMV whose kernel stores the logits into the shared
            # host buffer and then this rank's epoch word), then a spin on every rank's epoch word
            hosted.w = next_copy()
            hosted.step(x_host)
            return
        if world == 1:
            # ops.linear_host without a device buffer for the logits: x is copied in (4 KB), the kernel stores the
            # logits into the pinned host buffer itself, so the D2H traffic is the kernel's own stores
            ops.linear_host(x_host, next_copy(), y_host, x)
            torch.cuda.current_stream().synchronize()  # a decode step consumes its logits on the host
            return
        x.copy_(x_host, non_blocking=True)
        if fused:
            y_dev_full = fused(x, next_copy()).view(1, -1)
        else:
            step_nccl()
            y_dev_full = gathered.view(1, -1)
        y_host.copy_(y_dev_full, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # a decode step consumes its logits on the host

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, calls):
        """One block: `calls` calls of fn between barriers and device synchronisation; CUDA-event milliseconds (this rank)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(calls):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    def blocks(fn, calls, steps_per_call=1):
        """At least MIN_BLOCKS blocks and MIN_TIMED_S seconds of them; per block the max over ranks. Returns the sorted
        per-step milliseconds of the blocks."""
        first = timed(fn, calls)
        n = max(MIN_BLOCKS, int(np.ceil(MIN_TIMED_S * 1e3 / max(first, 1e-3))))
        if world > 1:   # every rank must run the same number of blocks
            nb = torch.tensor([n], dtype=torch.int64, device=dev)
            dist.all_reduce(nb, op=dist.ReduceOp.MAX)
            n = int(nb.item())
        n = min(n, 2000)
        ms = torch.tensor([timed(fn, calls) for _ in range(n)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return sorted((ms / (calls * steps_per_call)).tolist())

    calls = max(1, args.steps // per_call)
    steps = calls * per_call                      # = --steps: a block is one graph of that many steps, or that many eager steps
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    per_step = blocks(step, calls, per_call)
    ms_step = statistics.median(per_step)
    nccl_us = None
    if world > 1:   # for comparison: the same shards with an NCCL all-gather behind the kernel (eager launches)
        for _ in range(3):
            step_nccl()
        nccl_us = statistics.median(blocks(step_nccl, args.steps)) * 1e3
    # the GEMV launch alone (no collective), per launch, on the launching stream: the roofline figure
    kernel_ms = ms_step if world == 1 else statistics.median(blocks(lambda: ops.mmv(x, next_copy(), out=mine), args.steps))
    for _ in range(6 * n_copies + 3):   # every (weight copy, logits buffer) pair reaches its captured graph
        step_e2e()
    e2e_steps = blocks(step_e2e, args.steps)
    ms_e2e = statistics.median(e2e_steps)
    clocks = sampler.stop() if sampler else None

    # multi-token batches on the same matrix (the verify batch of speculative decoding): 2 and 4 columns share one decode
    multi_tok = None
    if world == 1:
        multi_tok = {}
        g = torch.Generator().manual_seed(0xAC8)
        x4 = torch.randn((4, K), generator=g).to(torch.bfloat16).to(dev)
        singles = [ops.mmv(x4[i:i + 1], enc) for i in range(4)]
        for T in (2, 4):
            yT = torch.empty((T, rows), dtype=torch.float32, device=dev)
            for _ in range(3):
                ops.mmv(x4[:T], enc, out=yT)
            us = statistics.median(blocks(lambda: ops.mmv(x4[:T], next_copy(), out=yT), max(1, args.steps // 4))) * 1e3
            same = all(torch.equal(yT[i].view(torch.int32), singles[i][0].view(torch.int32)) for i in range(T))
            multi_tok[str(T)] = {"us_per_step": us, "ratio_to_one_token": us / (ms_step * 1e3), "bitwise_equal_to_single_token": bool(same)}
        del singles

    # comparator on the same GPU: a stock BF16 GEMV (cuBLAS through torch) over the uncompressed shard
    wd = gen_rows(r0, r1).to(dev)
    yb = torch.empty((1, r1 - r0), dtype=torch.bfloat16, device=dev)
    for _ in range(5):
        torch.mm(x, wd.t(), out=yb)
    cublas_us = statistics.median(blocks(lambda: torch.mm(x, wd.t(), out=yb), args.steps)) * 1e3
    del wd

    # parity of what was timed, on a sample of rows, against the FP64 oracle (rank 0, its own shard)
    parity = None
    if rank == 0:
        from oracle import cpu_oracle as o
        n = min(2048, r1 - r0)
        wb = gen_rows(r0, r0 + n).view(torch.int16).numpy().view(np.uint16)
        xf = o.bf16_bits_to_f32(x_host.view(torch.int16).numpy().view(np.uint16)[0])
        y64, s = o.gemv_f64(wb, xf)
        got = (last[-1][rank, 0, :n] if fused else mine[0, :n]).float().cpu().numpy()
        parity = {"rows_checked": n, "max_err_over_sum_abs": float((np.abs(got - y64) / s).max()), "roundtrip_bit_exact": bool(ok)}
        if hosted is not None or world == 1:
            got_h = (hosted._bufs[(hosted.epoch - 1) & 1][0, :n] if hosted is not None else y_host[0, :n]).numpy()
            parity["e2e_max_err_over_sum_abs"] = float((np.abs(got_h - y64) / s).max())

    expired = fused.xchg.expired() if fused else False
    exchange_timing = None
    if fused:
        mine_t = fused.xchg.timing()
        gathered_t = [None] * world
        dist.all_gather_object(gathered_t, mine_t)
        exchange_timing = gathered_t
    faults = ops.fault_status()
    fused_used, hosted_used = fused is not None, hosted is not None
    fused_width = fused.width if fused else width
    if hosted is not None:
        hosted.close()
    if fused:
        fused.close()
    del copies, enc
    torch.cuda.empty_cache()

    # the rest of the metric: the MoE layer (decode at 1 / 2 / 4 tokens, prefill at 2048 / 8192 tokens; expert-parallel
    # over the ranks) and the small-matrix graph (one GPU)
    moe = None
    small = None
    if not args.no_moe:
        moe = moe_block(args, torch, dist, ops, rank, world, dev)
        if world == 1:
            small = small_block(args, torch, ops, dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    if expired:
        raise SystemExit("bench.py: a wait for a peer's logits expired")
    if faults:
        raise SystemExit(f"bench.py: a bounded wait inside a kernel expired (fault status {faults})")
    peak, peak_src = measured_peak()
    achieved = shard_algo_bytes / (kernel_ms * 1e-3) / 1e9
    l2 = ("inputs larger than L2 (compressed matrix %.0f MB per GPU, one copy)" % (shard_bytes / 1e6) if n_copies == 1 else
          "%d copies of the %.0f MB shard at different addresses, used in turn (%.0f MB between reuses; L2 is 126 MB)"
          % (n_copies, shard_bytes / 1e6, n_copies * shard_bytes / 1e6))
    line = {
        "metric": METRIC,
        "value": algo_bytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"lm_head {rows}x{K} HUFPAIR R={shard_R}, batch-1 decode GEMV, BF16 activation, FP32 logits"
                               + (f", rows sharded over {world} GPUs, logits stored into every GPU's buffer by the GEMV kernel "
                                  "(peer stores + epoch flags, no collective)" if fused_used else
                                  f", rows sharded over {world} GPUs + NCCL all-gather ({fused_note})" if world > 1 else ""),
                   "l2": l2, "compressed_bytes": total_weight_bytes, "bf16_bytes": rows * K * 2,
                   "ratio": total_weight_bytes / (rows * K * 2)},
        "blocks": {"n": len(per_step), "steps_per_block": steps, "ms_per_step_min": per_step[0], "ms_per_step_median": ms_step,
                   "ms_per_step_max": per_step[-1], "timed_s": sum(per_step) * steps / 1e3},
        "us_per_step": ms_step * 1e3,
        "bf16_equivalent_GBps": (rows * K * 2 + K * 2 + rows * 4) / (ms_step * 1e-3) / 1e9,
        "frac_of_nominal_8TBps": algo_bytes / (ms_step * 1e-3) / 8e12 / world,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": DRAM_TRAFFIC_RATIO * shard_algo_bytes,
                     "traffic_source": "ncu capture of a 65536-row case scaled by rows (profiles/lm_head_gemv_ncu.md)", "peak_source": peak_src, "kernel_us": kernel_ms * 1e3,
                     "algorithmic_bytes_per_launch": shard_algo_bytes},
        "e2e": {"value": algo_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": K * 2, "d2h_bytes_per_step": int(rows * 4 if (hosted_used or world == 1) else world * fused_width * 4),
                "us_per_step": ms_e2e * 1e3, "us_per_step_min": e2e_steps[0] * 1e3, "us_per_step_max": e2e_steps[-1] * 1e3,
                "how": ("one graph launch per step: activation copied in from pinned host memory, logits stored by the GEMV kernel straight "
                        "into a pinned host buffer shared by the ranks of the node (every rank's kernel writes its shard and then its epoch "
                        "word); the step ends when the host has seen every rank's epoch word (no stream synchronise)" if hosted_used else
                        "activation copied in from pinned host memory, logits stored by the GEMV kernel straight into pinned host memory, "
                        "stream synchronised every step" if world == 1 else
                        "activation copied in, gathered logits copied out behind the kernel, stream synchronised every step")},
        "gpu_launches": steps,   # one kernel per step at every N
        "nccl_allgather_us_per_step": nccl_us,
        "kernel_alone_us": kernel_ms * 1e3,
        "exchange_timing_last_step_per_rank": exchange_timing,
        "cublas_bf16_gemv_us": cublas_us,
        "vs_cublas_bf16_gemv": cublas_us / (kernel_ms * 1e3),
        "multi_token": multi_tok,
        "moe": moe, "small_matrices": small,
        "clocks": clocks, "parity": parity,
        "host": {"gen_s": t_gen, "encode_s": t_enc, "encode_GBps_bf16": (r1 - r0) * K * 2 / t_enc / 1e9, "threads": os.cpu_count()},
    }
    if world == 1 and not args.no_cpu:
        base, _ = cpu_arm(CPU_SAMPLE_ROWS, 100, 1)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["reference_kernels_same_gpu"] = reference_kernels()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ the other configurations of the metric (MoE layer, small matrices)

def measured_tensor_peaks():
    """(burst, sustained) dense BF16 TFLOP/s of this pool's B200s from MEASURED_PEAKS.json, else the earlier measurement."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured (MEASURED_PEAKS.json)"
    return 1590.0, 1400.0, "fallback (earlier measurement on this pool)"


def _enc(ops, rows, K, fmt, R, cm, seed, dev, fo=False, keep=False):
    import torch
    g = torch.Generator().manual_seed(seed)
    w = torch.empty((rows, K), dtype=torch.bfloat16)
    step = 1 << 16
    for r0 in range(0, rows, step):
        n = min(step, rows - r0)
        w[r0:r0 + n] = (torch.randn((n, K), generator=g) * 0.02).to(torch.bfloat16)
    plane, aux, meta = ops.encode(w, fmt, R, cm, fo)
    enc = ops.upload(plane, aux, meta, dev)
    return (enc, w) if keep else enc


def _agree_max(torch, n: int) -> int:
    """The largest n over the ranks (ranks whose kernels wait for each other must replay the same number of times)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return n
    t = torch.tensor([n], dtype=torch.int64, device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())


def _time_graph(torch, fn, reps, inner=1, min_s=0.3):
    """A CUDA graph of `fn`, replayed back to back: every sample times enough replays to last about 5 ms (so that the
    launch of a replay overlaps the one before it, as in a decode loop), at least max(reps, 30) samples and about min_s
    seconds of them; the counts are agreed between the ranks. Returns (median, min, max) microseconds per inner step."""
    s = torch.cuda.Stream()
    fn()
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()

    def sample(m):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(m):
            g.replay()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / m

    one = sample(1)
    m = _agree_max(torch, max(1, int(np.ceil(5.0 / max(one, 1e-3)))))
    n = _agree_max(torch, min(2000, max(reps, 30, int(np.ceil(min_s * 1e3 / max(one * m, 1e-3))))))
    times = sorted(sample(m) for _ in range(n))
    k = 1e3 / inner
    return statistics.median(times) * k, times[0] * k, times[-1] * k


def expert_weights(e: int):
    """(gate [512, 2048], up [512, 2048], down [2048, 512]) of routed expert e: N(0, 0.02) rounded to BF16, one seed per
    expert, so that any rank (and the parity check) can regenerate any expert on its own."""
    import torch
    g = torch.Generator().manual_seed(0xE0000 + e)
    return tuple((torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16) for shape in ((512, 2048), (512, 2048), (2048, 512)))


def _moe_weights(ops, dev, e_lo, n_local, fo=False):
    """Routed experts [e_lo, e_lo + n_local) encoded as the policy lays them out. fo: 16-row fragment-order bands (the
    vLLM layout) instead of chunk-major R = 8 gate / up and row-major R = 16 down (the llama.cpp layout)."""
    import torch
    parts = [expert_weights(e) for e in range(e_lo, e_lo + n_local)]
    out = []
    for i, (R_, cm) in enumerate(((16 if fo else 8, not fo), (16 if fo else 8, not fo), (16, False))):
        w = torch.cat([p[i] for p in parts], dim=0)
        plane, aux, meta = ops.encode(w, 3, R_, cm, fo)
        out.append(ops.upload(plane, aux, meta, dev))
    return out


def _bits(t):
    import torch
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _routed_oracle(x_bits, wts, ids, e_lo, n_local, bf16_act):
    """FP64 output of the routed experts in [e_lo, e_lo + n_local) for the tokens given (x as BF16 bits [T, 2048];
    wts FP32 / ids int32 [T, k]); slots routed elsewhere contribute nothing. Only the experts these tokens use are
    generated."""
    from oracle import cpu_oracle as o
    used = sorted({int(e) for e in ids.reshape(-1) if e_lo <= int(e) < e_lo + n_local})
    if not used:
        return np.zeros((ids.shape[0], 2048))
    pos = {e: i for i, e in enumerate(used)}
    ws = [expert_weights(e) for e in used]
    gb, ub, db = (np.concatenate([_bits(w[i]) for w in ws], axis=0) for i in range(3))
    local = np.vectorize(lambda e: e_lo <= e < e_lo + n_local)(ids)
    ids_c = np.vectorize(lambda e: pos.get(int(e), 0))(ids).astype(np.int32)
    return o.moe_layer_f64(o.bf16_bits_to_f32(x_bits), gb, ub, db, np.where(local, wts, 0.0), ids_c, len(used), bf16_act=bf16_act)


def _dist_setup(torch):
    """(rank, world, device): one process per GPU under torchrun, NCCL process group when world > 1."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _max_over_ranks(torch, us, world, dev):
    if world == 1:
        return us
    import torch.distributed as dist
    t = torch.tensor([us], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def moe_decode_runs(args, torch, dist, ops, rank, world, dev, weights, shared):
    """Config 3: hidden 2048, 256 routed experts (gate|up 512x2048 each, down 2048x512) + shared expert (NIBBLE), softmax
    top-8 on the GPU, 1 / 2 / 4 tokens. A graph holds 16 steps with 16 different routings so that consecutive steps hit
    different experts (the 1.08 GB of expert weights do not fit L2; one step touches 34 MB per token)."""
    from oracle import cpu_oracle as o
    E, k = 256, 8
    n_local = E // world
    gate, up, down = weights
    sh_gu, sh_down = shared
    peak, _ = measured_peak()
    out = []
    for T in (1, 2, 4):
        steps = 16
        g = torch.Generator(device=dev).manual_seed(1234 + T)   # the same tokens and routing on every rank
        xs = [torch.randn(T, 2048, device=dev, generator=g).to(torch.bfloat16) for _ in range(steps)]
        logits = [torch.randn(T, E, device=dev, generator=g) for _ in range(steps)]
        if getattr(args, "shared_routing", False):   # a verify batch whose tokens agree on their experts
            logits = [l[:1].expand(T, E).contiguous() for l in logits]
        scratch = ops.moe_decode_scratch(T, k, gate, down, n_local, dev)
        ids = [torch.empty(T, k, dtype=torch.int32, device=dev) for _ in range(steps)]
        wts = [torch.empty(T, k, device=dev) for _ in range(steps)]
        y = torch.empty(T, 2048, device=dev)
        ysh = torch.empty(T, 2048, device=dev)
        a = torch.empty(T, 512, device=dev)

        side = torch.cuda.Stream()
        fmd = None
        if world > 1:
            from orin_qwen_lossless_b200 import sharded
            fmd = sharded.FusedMoeDecode(gate, up, down, E, k, T)

        def step():
            # the shared expert does not depend on the routed experts: it runs on a second stream (a parallel branch of
            # the captured graph) and joins before the final add
            for i in range(steps):
                main = torch.cuda.current_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ops._mmv_common(xs[i], sh_gu, None, 0, False, True, True, a)   # shared expert: merged gate|up GLU
                    ops.mmv(a, sh_down, out=ysh)
                if fmd and not args.nccl:
                    # expert-parallel, no collective: the combine kernel stores the partial output into every rank and
                    # waits for the peers'; one small kernel adds the partials and the shared expert
                    fmd(xs[i], logits[i], y, ysh, wts[i], ids[i], join=side)
                    continue
                ops.moe_decode(xs[i], gate, up, down, E, k, router_logits=logits[i], topk_weights=wts[i], topk_ids=ids[i],
                               scratch=scratch, out=y, expert_lo=rank * n_local, n_experts_local=n_local)
                main.wait_stream(side)
                if world > 1:
                    if rank == 0:
                        y.add_(ysh)
                    dist.all_reduce(y)      # the ranks' partial [T, 2048] outputs (NCCL over NVLink)
                else:
                    y.add_(ysh)

        med, lo, hi = _time_graph(torch, step, max(args.steps // 16, 5), inner=steps)
        us = _max_over_ranks(torch, med, world, dev)
        distinct = sum(len(torch.unique(i)) for i in ids) / steps
        per_expert = (gate.nbytes + up.nbytes + down.nbytes) / n_local
        nbytes = distinct * per_expert + sh_gu.nbytes + sh_down.nbytes
        # parity of the routed experts on step 0 (this rank's slice of them) against the FP64 oracle layer
        part, w0, i0 = ops.moe_decode(xs[0], gate, up, down, E, k, router_logits=logits[0], expert_lo=rank * n_local,
                                      n_experts_local=n_local)
        parity = None
        if rank == 0:
            ids_ref, w_ref = o.softmax_topk(logits[0].cpu().numpy(), k)
            ref = _routed_oracle(_bits(xs[0].cpu()), w0.cpu().numpy(), i0.cpu().numpy(), 0, n_local, False)
            parity = {"router_ids_equal_oracle": bool(np.array_equal(i0.cpu().numpy(), ids_ref)),
                      "router_weights_max_abs_diff": float(np.abs(w0.cpu().numpy() - w_ref).max()),
                      "max_err_over_max_abs": float(np.abs(part.cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30)),
                      "what": "routed experts held by rank 0, step 0, against the FP64 layer over the exact weights"}
        if rank == 0:
            out.append({"tokens": T, "n_gpus": world,
                        "parallelism": "1 GPU" if world == 1 else f"expert-parallel over {world} GPUs + NCCL all-reduce" if args.nccl
                        else f"expert-parallel over {world} GPUs, partial outputs stored into every GPU by the combine kernel, no collective",
                        "us_per_layer": us, "us_min": lo, "us_max": hi, "distinct_experts": distinct, "compressed_bytes": nbytes,
                        "GBps": nbytes / us / 1e3, "frac_of_measured_hbm": nbytes / us / 1e3 / peak / world,
                        "launches_per_layer": 7 + (world > 1), "parity": parity})
        if fmd:
            fmd.close()
    return out


def moe_prefill_runs(args, torch, dist, ops, rank, world, dev, weights, fo=False):
    """Config 4: the same expert weights with 2048 and 8192 tokens: routing sort, batched gate/up + SwiGLU (BF16 out),
    batched down (FP32 out), combine."""
    from orin_qwen_lossless_b200 import sharded
    E, k = 256, 8
    gate, up, down = weights
    hbm, _ = measured_peak()
    burst, sustained, _ = measured_tensor_peaks()
    out = []
    # two-pass form (decode into BF16 operand tiles in a workspace, then the tensor-core pass over the tiles) unless
    # --fused-prefill asks for the fused decode-and-multiply kernel; fragment-order experts have their own kernel
    two_pass = not fo and not args.fused_prefill
    ws_bytes = ops.ensure_workspace((gate, up), (down, None)) if two_pass else 0
    form = ("fragment-order kernel" if fo else "two-pass: decode into BF16 operand tiles (%.0f MB workspace), tcgen05 pass over the tiles" % (ws_bytes / 1e6)
            if two_pass else "fused decode-and-multiply kernel")
    for T in ((2048, 8192) if not args.tokens else (args.tokens,)):
        fused_us = None
        flops = 6.0 * 512 * 2048 * k * T
        nbytes = (gate.nbytes + up.nbytes + down.nbytes) * world
        g = torch.Generator(device=dev).manual_seed(4321 + T + rank)
        if world == 1:
            x = torch.randn(T, 2048, device=dev, generator=g).to(torch.bfloat16)
            wts, ids = ops.moe_topk(torch.randn(T, E, device=dev, generator=g), k)
            med, lo, hi = _time_graph(torch, lambda: ops.moe_experts(x, gate, up, down, wts, ids, E), max(args.steps // 100, 5))
            us = med
            y = ops.moe_experts(x, gate, up, down, wts, ids, E)
            par = "1 GPU"
            if two_pass:   # the fused kernel on the same inputs, for comparison
                ops.set_workspace(None)
                fused_us = _time_graph(torch, lambda: ops.moe_experts(x, gate, up, down, wts, ids, E), max(args.steps // 100, 5))[0]
                ops.ensure_workspace((gate, up), (down, None))
        elif not args.nccl:
            # tokens data-parallel (T / world per rank), experts sharded: every routed row is stored into the exchange
            # buffer of its expert's rank by a kernel (peer stores over NVLink), multiplied there by the batched kernels
            # and stored back; no host round trip, no collective: the layer is one CUDA graph per rank
            Tl = T // world
            x = torch.randn(Tl, 2048, device=dev, generator=g).to(torch.bfloat16)
            wts, ids = ops.moe_topk(torch.randn(Tl, E, device=dev, generator=g), k)
            fmp = sharded.FusedMoePrefill(gate, up, down, E, k, Tl)
            y = fmp(x, wts, ids)
            torch.cuda.synchronize(); dist.barrier()
            med, lo, hi = _time_graph(torch, lambda: fmp(x, wts, ids), max(args.steps // 100, 5))
            us = _max_over_ranks(torch, med, world, dev)
            lo, hi = _max_over_ranks(torch, lo, world, dev), _max_over_ranks(torch, hi, world, dev)
            y = fmp(x, wts, ids).clone()
            expired = fmp.xchg.expired()
            fmp.close()
            if expired:
                raise SystemExit("bench.py: a wait for a peer's rows expired")
            par = f"expert-parallel over {world} GPUs, routed rows exchanged by peer stores on the device (no host round trip, no collective)"
        else:
            # the NCCL form for comparison: all-to-all dispatch of the routed rows, batched kernels on the owner,
            # all-to-all back, combine. The exchange sizes come back to the host, so the layer is timed as eager launches
            # with CUDA events (max over ranks).
            Tl = T // world
            x = torch.randn(Tl, 2048, device=dev, generator=g).to(torch.bfloat16)
            wts, ids = ops.moe_topk(torch.randn(Tl, E, device=dev, generator=g), k)
            for _ in range(3):
                y = sharded.moe_prefill_ep(x, wts, ids, gate, up, down, E)
            reps = max(args.steps // 100, 10)
            times = []
            for _ in range(reps):
                torch.cuda.synchronize(); dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                sharded.moe_prefill_ep(x, wts, ids, gate, up, down, E)
                e1.record()
                torch.cuda.synchronize()
                times.append(_max_over_ranks(torch, e0.elapsed_time(e1) * 1e3, world, dev))
            times.sort()
            us, lo, hi = statistics.median(times), times[0], times[-1]
            par = f"expert-parallel over {world} GPUs, NCCL all-to-all dispatch and return"
        if rank == 0:
            n = 4   # tokens checked against the FP64 layer (BF16 SwiGLU activations, as the batched path stores them)
            ref = _routed_oracle(_bits(x[:n].cpu()), wts[:n].cpu().numpy(), ids[:n].cpu().numpy(), 0, E, True)
            got = y[:n].float().cpu().numpy()
            hbm_us, tensor_us = nbytes / world / hbm / 1e3, flops / world / burst / 1e6
            out.append({"tokens": T, "n_gpus": world, "parallelism": par, "layout": "fragment order" if fo else "lane-major (chunk-major R=8 gate/up, R=16 down)",
                        "form": form, "us_per_layer": us, "us_min": lo, "us_max": hi, "us_per_layer_fused_kernel": fused_us,
                        "TFLOPs": flops / us / 1e6, "weight_GBps": nbytes / us / 1e3,
                        "roofline": {"hbm_bound_us": hbm_us, "tensor_bound_us": tensor_us, "tensor_bound_us_sustained": flops / world / sustained / 1e6,
                                     "bound": "hbm" if hbm_us > tensor_us else "tensor", "frac": max(hbm_us, tensor_us) / us,
                                     "flops": flops, "compressed_bytes": nbytes},
                        "parity": {"tokens_checked": n, "max_err_over_max_abs": float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)),
                                   "what": "BF16 layer output of the first tokens of rank 0 against the FP64 layer (BF16 SwiGLU activations)"}})
    if two_pass:
        torch.cuda.synchronize()
        ops.set_workspace(None)
    return out


def moe_block(args, torch, dist, ops, rank, world, dev):
    """The MoE half of the metric for the contract line: decode layer at 1 / 2 / 4 tokens, prefill layer at 2048 / 8192
    tokens, expert-parallel over the ranks. Rank 0 returns the dict."""
    E = 256
    n_local = E // world
    t0 = time.perf_counter()
    weights = _moe_weights(ops, dev, rank * n_local, n_local)
    shared = (_enc(ops, 1024, 2048, 1, 0, False, 104, dev), _enc(ops, 2048, 512, 1, 0, False, 105, dev))
    t_w = time.perf_counter() - t0
    decode = moe_decode_runs(args, torch, dist, ops, rank, world, dev, weights, shared)
    prefill = moe_prefill_runs(args, torch, dist, ops, rank, world, dev, weights)
    faults = ops.fault_status()
    if world > 1:
        dist.barrier()
    if rank != 0:
        return None
    return {"experts": "256 routed experts (gate, up 512x2048; down 2048x512) + shared expert (NIBBLE 1024x2048, 2048x512), "
                       "N(0, 0.02) weights, one seed per expert; top-8 of N(0,1) router logits",
            "weights_gen_encode_s": t_w, "decode": decode, "prefill": prefill, "fault_status": faults}


def small_block(args, torch, ops, dev):
    """Config 2: 48 layers x {2048x512, 512x2048, 256x2048} NIBBLE, batch-1 GEMVs, one CUDA graph of 144 launches."""
    from oracle import cpu_oracle as o
    layers, nbytes, first = [], 0, None
    for l in range(48):
        made = [_enc(ops, 2048, 512, 1, 0, False, 3 * l, dev, keep=(l == 0)), _enc(ops, 512, 2048, 1, 0, False, 3 * l + 1, dev, keep=(l == 0)),
                _enc(ops, 256, 2048, 1, 0, False, 3 * l + 2, dev, keep=(l == 0))]
        if l == 0:
            first = [m[1] for m in made]
            made = [m[0] for m in made]
        nbytes += sum(w.nbytes for w in made)
        layers.append(made)
    x512 = torch.randn(1, 512, device=dev).to(torch.bfloat16)
    x2048 = torch.randn(1, 2048, device=dev).to(torch.bfloat16)
    outs = [[torch.empty(1, w.meta.rows, device=dev) for w in ws] for ws in layers]

    def step_one_by_one():
        for ws, ys in zip(layers, outs):
            ops.mmv(x512, ws[0], out=ys[0]); ops.mmv(x2048, ws[1], out=ys[1]); ops.mmv(x2048, ws[2], out=ys[2])

    xs3 = [x512, x2048, x2048]

    def step():   # the three products of a layer are independent: one grid serves them (48 launches per graph)
        for ws, ys in zip(layers, outs):
            ops.mmv_group(xs3, ws, ys)

    us1, _, _ = _time_graph(torch, step_one_by_one, args.steps // 10)
    torch.cuda.synchronize()
    singles = [[y.clone() for y in ys] for ys in outs]
    us, lo, hi = _time_graph(torch, step, args.steps // 10)
    torch.cuda.synchronize()
    same = all(torch.equal(a, b) for ya, yb in zip(singles, outs) for a, b in zip(ya, yb))
    peak, _ = measured_peak()
    worst = 0.0
    for wsrc, xv, yv in zip(first, (x512, x2048, x2048), outs[0]):   # FP64 check of the first layer's three products
        y64, sabs = o.gemv_f64(_bits(wsrc), o.bf16_bits_to_f32(_bits(xv.cpu())[0]))
        worst = max(worst, float((np.abs(yv[0].cpu().numpy() - y64) / sabs).max()))
    return {"workload": "small matrices: 48 layers x {2048x512, 512x2048, 256x2048} NIBBLE, batch-1, 144 GEMVs per CUDA graph, "
                        "the three independent products of a layer in one launch (bf16n_mmv_group)",
            "us_per_graph": us, "us_min": lo, "us_max": hi, "us_per_gemv": us / 144, "launches_per_graph": 48,
            "us_per_graph_one_launch_per_gemv": us1, "grouped_bitwise_equal_to_single_launches": bool(same), "compressed_bytes": nbytes, "GBps": nbytes / us / 1e3,
            "frac_of_measured_hbm": nbytes / us / 1e3 / peak, "l2": "191 MB of weights per replay > L2",
            "parity": {"max_err_over_sum_abs": worst, "what": "first layer's three GEMVs against FP64"}}


def run_small(args):
    import torch
    from orin_qwen_lossless_b200 import ops
    dev = torch.device("cuda", 0)
    ops.init()
    print(json.dumps(small_block(args, torch, ops, dev)), flush=True)


def run_moe_decode(args):
    import torch
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops
    rank, world, dev = _dist_setup(torch)
    ops.init()
    n_local = 256 // world
    weights = _moe_weights(ops, dev, rank * n_local, n_local, args.fo and world == 1)
    shared = (_enc(ops, 1024, 2048, 1, 0, False, 104, dev), _enc(ops, 2048, 512, 1, 0, False, 105, dev))
    for rec in moe_decode_runs(args, torch, dist, ops, rank, world, dev, weights, shared):
        rec["layout"] = "fragment order" if args.fo and world == 1 else "lane-major (chunk-major R=8 gate/up, R=16 down)"
        rec["routing"] = "every token of a step picks the same experts" if args.shared_routing else "independent N(0,1) router logits per token"
        print(json.dumps({"workload": f"MoE decode layer, {rec['tokens']} token(s), 256 experts top-8 + shared expert", **rec}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_moe_prefill(args):
    import torch
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops
    rank, world, dev = _dist_setup(torch)
    ops.init()
    n_local = 256 // world
    weights = _moe_weights(ops, dev, rank * n_local, n_local, args.fo)
    for rec in moe_prefill_runs(args, torch, dist, ops, rank, world, dev, weights, args.fo):
        print(json.dumps({"workload": f"MoE prefill layer, {rec['tokens']} tokens, 256 experts top-8", **rec}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_dense_mid(args):
    """Mid-size dense projections (8-32 M weights: what the policy gives HUFPAIR below the vocabulary projection), R as
    the policy picks it for the lane-major layout and 16-row bands for fragment order; 1, 4 and 8 BF16 tokens; every
    shape as a CUDA graph of 20 GEMVs over rotating copies so that weights come from HBM."""
    import torch
    from orin_qwen_lossless_b200 import ops
    dev = torch.device("cuda", 0)
    ops.init()
    for rows, K, R in ((4096, 2048, 8), (8192, 2048, 16), (16384, 2048, 16)):
        for fo in (False, True):
            copies = [_enc(ops, rows, K, 3, 16 if fo else R, False, 900 + c, dev, fo) for c in range(8)]  # 8 x >= 11 MB, rotated
            line = {"workload": f"dense {rows}x{K} HUFPAIR, " + ("fragment order" if fo else f"lane-major R={R}"),
                    "compressed_bytes": copies[0].nbytes}
            for T in (1, 4, 8):
                x = torch.randn(T, K, device=dev).to(torch.bfloat16)
                ys = [torch.empty(T, rows, device=dev) for _ in copies]

                def step():
                    for i in range(20):
                        ops.mmv(x, copies[i % 8], out=ys[i % 8])

                line[f"us_{T}_tok"] = round(_time_graph(torch, step, max(10, args.steps // 20), inner=20)[0], 2)
            print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="rows of the matrix (default: the vocabulary projection)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE layer and small-matrix blocks of the contract line")
    ap.add_argument("--tokens", type=int, default=0, help="--workload moe_prefill: this token count only (default: 2048 and 8192)")
    ap.add_argument("--fused-prefill", action="store_true", help="MoE prefill: the fused decode-and-multiply kernel instead of the two-pass form")
    ap.add_argument("--fo", action="store_true", help="moe_prefill / moe_decode (one GPU): experts in the fragment-order layout")
    ap.add_argument("--shared-routing", action="store_true", help="moe_decode: every token of a step picks the same experts")
    ap.add_argument("--nccl", action="store_true", help="N > 1, MoE workloads: NCCL collectives instead of the fused peer stores")
    ap.add_argument("--workload", default="lm_head", choices=["lm_head", "small", "moe_decode", "moe_prefill", "dense_mid"],
                    help="lm_head is the headline contract line; the others print extra lines for the other baseline configs "
                         "(small: 1 GPU; the MoE workloads run expert-parallel under torchrun)")
    args = ap.parse_args()
    if args.workload != "lm_head":
        return {"small": run_small, "moe_decode": run_moe_decode, "moe_prefill": run_moe_prefill,
                "dense_mid": run_dense_mid}[args.workload](args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
