"""Benchmark of the BF16N hot path on B200: the vocabulary projection (lm_head) decode+GEMV.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): a 248320 x 2048 BF16 matrix, weights N(0, 0.02) rounded
to BF16 (seeded, synthetic), pair-Huffman coded with R = 16 as the shape policy chooses, multiplied by one BF16 N(0,1)
activation vector with FP32 accumulation and FP32 logits. With N > 1 ranks the rows are split into N shards (one
process per GPU), each rank multiplies its shard and an NCCL all-gather assembles the logits.

One JSON line on stdout (rank 0):
  value    GB/s of compressed bytes (plane + aux + x + y) per second with everything resident in HBM
  e2e      the same through ops.linear_host: the activation comes from pinned host memory and the logits go back to it
           inside the timed region, every step
  roofline achieved / measured copy bandwidth for the GEMV kernel (one launch per step)
  cpu_baseline  the CPU oracle's decode+GEMV on this box's host threads (bounded sample)
`--impl reference` times the CPU arm only (the reference ships no CPU GEMV, so this is the oracle's port of its decoder
and summation; the encoder timed beside it is the reference's own when oracle/_ref is present).
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
# on a 65536-row case of the same matrix family (182.99 MB moved for 179.01 MB algorithmic, profiles/lm_head_gemv_ncu.md);
# traffic grows in proportion to the rows, so a full launch is this ratio times its algorithmic bytes.
DRAM_TRAFFIC_RATIO = 1.022
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


def cpu_arm(rows_sample: int, reps: int):
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
    o.decode_gemv_mt(plane, aux, x, 0, units, threads)       # warm-up pass, also sizes the run: about 20 s of CPU work at most
    reps = max(1, min(reps, max(3, int(20.0 / max(time.perf_counter() - t0, 1e-4)))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        o.decode_gemv_mt(plane, aux, x, 0, units, threads)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"first {rows_sample} of {ROWS} rows ({nbytes / 1e6:.1f} MB compressed), median of {reps} passes of "
                      f"{dt:.3f} s; encoder ({'reference' if o.have_ref() else 'oracle'}) {rows_sample * K * 2 / t_enc / 1e9:.2f} GB/s of BF16 input",
            "ms_per_step": dt * 1e3, "encode_s": t_enc, "passes": reps}, nbytes


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
    base, nbytes = cpu_arm(rows_sample, max(1, args.steps))
    line = {"impl": "reference", "metric": "lm_head_248320x2048_bf16n_decode_gemv_compressed_GBps", "value": base["value"],
            "unit": "GB/s", "n_gpus": args.gpus, "steps": base["passes"], "warmup": 1, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "lm_head 248320x2048 HUFPAIR R=16, batch-1 decode GEMV (CPU arm: bounded row sample)",
                       "rows_sample": rows_sample},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


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
    t0 = time.perf_counter()
    plane, aux, meta = ops.encode(w, ops.FMT_HUFPAIR, R, False)
    t_enc = time.perf_counter() - t0
    enc = ops.upload(plane, aux, meta, dev)
    ok = ops.roundtrip_equal(enc, w)  # verify at load: bit-exact decode of the whole shard on the GPU
    if not ok:
        raise SystemExit("bench.py: GPU decode of the encoded shard is not bit-exact")
    del w
    shard_bytes = plane.numel() + aux.numel()
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

    def step_nccl():
        ops.mmv(x, enc, out=mine)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), gathered[rank])

    # N > 1, the product: the GEMV kernel stores its logits into every GPU's gathered buffer itself (peer stores over
    # NVLink, epoch flags; the kernel ends when the peers' logits have arrived); no collective. Two steps (the two buffers in turn) form one CUDA graph.
    fused = graph2 = None
    fused_note = None
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
    if fused:
        last = [fused(x) for _ in range(2)]
        torch.cuda.synchronize()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2):
            last = [fused(x) for _ in range(2)]

    def step():
        if fused:
            graph2.replay()     # two steps
        else:
            step_nccl()

    per_call = 2 if fused else 1   # steps per call of step()
    y_host = torch.empty((1, rows if world == 1 else world * (fused.width if fused else width)), dtype=torch.float32).pin_memory()

    def step_e2e():
        if world == 1:
            # one GPU: ops.linear_host without a device buffer for the logits: x is copied in (4 KB), the kernel stores
            # the logits into the pinned host buffer itself, so the D2H traffic is the kernel's own stores
            ops.linear_host(x_host, enc, y_host, x)
            torch.cuda.current_stream().synchronize()  # a decode step consumes its logits on the host
            return
        x.copy_(x_host, non_blocking=True)
        if fused:
            y_dev_full = fused(x).view(1, -1)
        elif world > 1:
            step_nccl()
            y_dev_full = gathered.view(1, -1)
        else:
            step_nccl()
            y_dev_full = logits
        y_host.copy_(y_dev_full, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # a decode step consumes its logits on the host

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    ms_total = timed(step, args.steps // per_call) / (args.steps // per_call * per_call) * args.steps
    nccl_us = None
    if world > 1:   # for comparison: the same shards with an NCCL all-gather behind the kernel (eager launches)
        for _ in range(3):
            step_nccl()
        nccl_us = timed(step_nccl, args.steps) / args.steps * 1e3
    # the GEMV launch alone (no collective), per launch, on the launching stream: the roofline figure
    kernel_ms = ms_total / args.steps if world == 1 else timed(lambda: ops.mmv(x, enc, out=mine), args.steps) / args.steps
    for _ in range(3):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if sampler else None

    # comparator on the same GPU: a stock BF16 GEMV (cuBLAS through torch) over the uncompressed shard
    cublas_us = None
    if args.cublas:
        wd = gen_rows(r0, r1).to(dev)
        yb = torch.empty((1, r1 - r0), dtype=torch.bfloat16, device=dev)
        for _ in range(5):
            torch.mm(x, wd.t(), out=yb)
        cublas_us = timed(lambda: torch.mm(x, wd.t(), out=yb), args.steps) / args.steps * 1e3
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

    expired = fused.xchg.expired() if fused else False
    fused_used = fused is not None
    if fused:
        fused.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    if expired:
        raise SystemExit("bench.py: a wait for a peer's logits expired")
    ms_step = ms_total / args.steps
    peak, peak_src = measured_peak()
    achieved = shard_algo_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "lm_head_248320x2048_bf16n_decode_gemv_compressed_GBps",
        "value": algo_bytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"lm_head {rows}x{K} HUFPAIR R={R}, batch-1 decode GEMV, BF16 activation, FP32 logits"
                               + (f", rows sharded over {world} GPUs, logits stored into every GPU's buffer by the GEMV kernel "
                                  "(peer stores + epoch flags, no collective)" if fused_used else
                                  f", rows sharded over {world} GPUs + NCCL all-gather ({fused_note})" if world > 1 else ""),
                   "l2": "inputs larger than L2 (compressed matrix %.0f MB per GPU)" % (shard_bytes / 1e6),
                   "compressed_bytes": total_weight_bytes, "bf16_bytes": rows * K * 2,
                   "ratio": total_weight_bytes / (rows * K * 2)},
        "us_per_step": ms_step * 1e3,
        "bf16_equivalent_GBps": (rows * K * 2 + K * 2 + rows * 4) / (ms_step * 1e-3) / 1e9,
        "frac_of_nominal_8TBps": algo_bytes / (ms_step * 1e-3) / 8e12 / world,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": DRAM_TRAFFIC_RATIO * shard_algo_bytes,
                     "traffic_source": "ncu capture of a 65536-row case scaled by rows (profiles/lm_head_gemv_ncu.md)", "peak_source": peak_src, "kernel_us": kernel_ms * 1e3,
                     "algorithmic_bytes_per_launch": shard_algo_bytes},
        "e2e": {"value": algo_bytes / (ms_e2e / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": K * 2, "d2h_bytes_per_step": int(y_host.numel() * 4), "us_per_step": ms_e2e / args.steps * 1e3},
        "gpu_launches": args.steps,   # one kernel per step at every N
        "nccl_allgather_us_per_step": nccl_us,
        "cublas_bf16_gemv_us": cublas_us,
        "clocks": clocks, "parity": parity,
        "host": {"gen_s": t_gen, "encode_s": t_enc, "encode_GBps_bf16": (r1 - r0) * K * 2 / t_enc / 1e9, "threads": os.cpu_count()},
    }
    if world == 1 and not args.no_cpu:
        base, _ = cpu_arm(CPU_SAMPLE_ROWS, 100)
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["reference_kernels_same_gpu"] = reference_kernels()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ secondary workloads (configs 2, 3, 4 of the baseline)

def _enc(ops, rows, K, fmt, R, cm, seed, dev, fo=False):
    import torch
    g = torch.Generator().manual_seed(seed)
    w = torch.empty((rows, K), dtype=torch.bfloat16)
    step = 1 << 16
    for r0 in range(0, rows, step):
        n = min(step, rows - r0)
        w[r0:r0 + n] = (torch.randn((n, K), generator=g) * 0.02).to(torch.bfloat16)
    plane, aux, meta = ops.encode(w, fmt, R, cm, fo)
    return ops.upload(plane, aux, meta, dev)


def _time_graph(torch, fn, reps, inner=1):
    """Median-free mean over `reps` replays of a CUDA graph of `fn`; returns microseconds per inner step."""
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps / inner


def run_small(args):
    """Config 2: 48 layers x {2048x512, 512x2048, 256x2048} NIBBLE, batch-1 GEMVs, one CUDA graph of 144 launches."""
    import torch
    from orin_qwen_lossless_b200 import ops
    dev = torch.device("cuda", 0)
    ops.init()
    layers, nbytes = [], 0
    for l in range(48):
        ws = [_enc(ops, 2048, 512, 1, 0, False, 3 * l, dev), _enc(ops, 512, 2048, 1, 0, False, 3 * l + 1, dev),
              _enc(ops, 256, 2048, 1, 0, False, 3 * l + 2, dev)]
        nbytes += sum(w.nbytes for w in ws)
        layers.append(ws)
    x512 = torch.randn(1, 512, device=dev).to(torch.bfloat16)
    x2048 = torch.randn(1, 2048, device=dev).to(torch.bfloat16)
    outs = [[torch.empty(1, w.meta.rows, device=dev) for w in ws] for ws in layers]

    def step():
        for ws, ys in zip(layers, outs):
            ops.mmv(x512, ws[0], out=ys[0]); ops.mmv(x2048, ws[1], out=ys[1]); ops.mmv(x2048, ws[2], out=ys[2])

    us = _time_graph(torch, step, args.steps)
    peak, _ = measured_peak()
    print(json.dumps({"workload": "small matrices: 48 layers x {2048x512, 512x2048, 256x2048} NIBBLE, batch-1, one CUDA graph of 144 GEMVs",
                      "us_per_graph": us, "us_per_gemv": us / 144, "compressed_bytes": nbytes, "GBps": nbytes / us / 1e3,
                      "frac_of_measured_hbm": nbytes / us / 1e3 / peak, "l2": "191 MB of weights per replay > L2"}), flush=True)


def _moe_weights(ops, dev, n_experts, rank=0, fo=False):
    """Routed expert weights of one rank (every rank draws its own experts: seeds differ per rank). fo: 16-row
    fragment-order bands (the vLLM layout) instead of chunk-major R = 8 gate / up and row-major R = 16 down."""
    gate = _enc(ops, n_experts * 512, 2048, 3, 16 if fo else 8, not fo, 101 + 10 * rank, dev, fo)
    up = _enc(ops, n_experts * 512, 2048, 3, 16 if fo else 8, not fo, 102 + 10 * rank, dev, fo)
    down = _enc(ops, n_experts * 2048, 512, 3, 16, False, 103 + 10 * rank, dev, fo)
    return gate, up, down


def _dist_setup(torch):
    """(rank, world, device): one process per GPU under torchrun, NCCL process group when world > 1."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _max_over_ranks(torch, us, world, dev):
    if world == 1:
        return us
    import torch.distributed as dist
    t = torch.tensor([us], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_moe_decode(args):
    """Config 3: hidden 2048, 256 routed experts (gate|up 512x2048 each, down 2048x512) + shared expert (NIBBLE), softmax
    top-8 on the GPU, 1 / 2 / 4 tokens. A graph holds 16 steps with 16 different routings so that consecutive steps hit
    different experts (the 1.08 GB of expert weights do not fit L2; one step touches 34 MB per token)."""
    import torch
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops
    rank, world, dev = _dist_setup(torch)
    ops.init()
    E, k = 256, 8
    n_local = E // world                      # expert-parallel: rank r holds experts [r * n_local, (r + 1) * n_local)
    gate, up, down = _moe_weights(ops, dev, n_local, rank)
    sh_gu = _enc(ops, 1024, 2048, 1, 0, False, 104, dev)      # the shared expert is replicated; rank 0's result is used
    sh_down = _enc(ops, 2048, 512, 1, 0, False, 105, dev)
    peak, _ = measured_peak()
    for T in (1, 2, 4):
        steps = 16
        g = torch.Generator(device=dev).manual_seed(1234 + T)   # the same tokens and routing on every rank
        xs = [torch.randn(T, 2048, device=dev, generator=g).to(torch.bfloat16) for _ in range(steps)]
        logits = [torch.randn(T, E, device=dev, generator=g) for _ in range(steps)]
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

        us = _max_over_ranks(torch, _time_graph(torch, step, max(args.steps // 16, 5), inner=steps), world, dev)
        distinct = sum(len(torch.unique(i)) for i in ids) / steps
        per_expert = (gate.nbytes + up.nbytes + down.nbytes) / n_local
        nbytes = distinct * per_expert + sh_gu.nbytes + sh_down.nbytes
        if rank == 0:
            print(json.dumps({"workload": f"MoE decode layer, {T} token(s), 256 experts top-8 + shared expert", "n_gpus": world,
                              "parallelism": "1 GPU" if world == 1 else f"expert-parallel over {world} GPUs + NCCL all-reduce" if args.nccl
                              else f"expert-parallel over {world} GPUs, partial outputs stored into every GPU by the combine kernel, no collective",
                              "us_per_layer": us, "distinct_experts": distinct, "compressed_bytes": nbytes,
                              "GBps": nbytes / us / 1e3, "frac_of_measured_hbm": nbytes / us / 1e3 / peak / world,
                              "launches_per_layer": 7 + (world > 1)}), flush=True)
        if fmd:
            fmd.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_moe_prefill(args):
    """Config 4: the same expert weights with 2048 and 8192 tokens: routing sort, batched gate/up + SwiGLU (BF16 out),
    batched down (FP32 out), combine."""
    import torch
    import torch.distributed as dist
    from orin_qwen_lossless_b200 import ops, sharded
    rank, world, dev = _dist_setup(torch)
    ops.init()
    E, k = 256, 8
    n_local = E // world
    gate, up, down = _moe_weights(ops, dev, n_local, rank, args.fo)
    for T in (2048, 8192):
        flops = 6.0 * 512 * 2048 * k * T
        nbytes = (gate.nbytes + up.nbytes + down.nbytes) * world
        if world == 1:
            x = torch.randn(T, 2048, device=dev).to(torch.bfloat16)
            wts, ids = ops.moe_topk(torch.randn(T, E, device=dev), k)
            us = _time_graph(torch, lambda: ops.moe_experts(x, gate, up, down, wts, ids, E), max(args.steps // 100, 5))
            par = "1 GPU"
        else:
            # tokens data-parallel (T / world per rank), experts sharded: all-to-all dispatch of the routed rows, batched
            # kernels on the owner, all-to-all back, combine. The exchange sizes come back to the host, so the layer is
            # timed as eager launches with CUDA events (max over ranks).
            Tl = T // world
            x = torch.randn(Tl, 2048, device=dev).to(torch.bfloat16)
            wts, ids = ops.moe_topk(torch.randn(Tl, E, device=dev), k)
            for _ in range(3):
                sharded.moe_prefill_ep(x, wts, ids, gate, up, down, E)
            reps = max(args.steps // 100, 5)
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                sharded.moe_prefill_ep(x, wts, ids, gate, up, down, E)
            e1.record()
            torch.cuda.synchronize()
            us = _max_over_ranks(torch, e0.elapsed_time(e1) * 1e3 / reps, world, dev)
            par = f"expert-parallel over {world} GPUs, NCCL all-to-all dispatch and return"
        if rank == 0:
            print(json.dumps({"workload": f"MoE prefill layer, {T} tokens, 256 experts top-8" + (", fragment-order experts" if args.fo else ""),
                              "n_gpus": world, "parallelism": par,
                              "us_per_layer": us, "TFLOPs": flops / us / 1e6, "weight_GBps": nbytes / us / 1e3,
                              "frac_of_bf16_peak_1679": flops / us / 1e6 / 1679.3 / world}), flush=True)
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

                line[f"us_{T}_tok"] = round(_time_graph(torch, step, max(10, args.steps // 20), inner=20), 2)
            print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="rows of the matrix (default: the vocabulary projection)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cublas", action="store_true", help="also time a stock BF16 GEMV of the uncompressed matrix")
    ap.add_argument("--fo", action="store_true", help="moe_prefill: experts in the fragment-order layout (mma.sync batched kernel)")
    ap.add_argument("--nccl", action="store_true", help="N > 1, moe_decode: all-reduce with NCCL instead of the fused peer stores")
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
