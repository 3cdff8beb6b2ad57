"""Multi-GPU forms of the path (new: the reference is single-GPU). One process per GPU; torch.distributed carries the
collectives (NCCL over NVLink on the GPUs, gloo in the CPU tests).

* the vocabulary projection shards by rows on unit boundaries: `shard_rows` cuts one encoded tensor (one code for the
  whole tensor) into per-rank tensors with valid headers; `lm_head_allgather` multiplies the local shard and gathers
  the logits;
* the MoE decode step is expert-parallel: every rank routes all tokens (cheap, deterministic), multiplies only the
  slots whose expert it holds and the partial [T, H] outputs are all-reduced;
* the MoE prefill layer is expert-parallel with an all-to-all token dispatch: tokens are split over the ranks, each
  routed (token, slot) row travels to the rank that holds its expert and its result travels back.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import ops
from ._lib import EpLayout, MmvArgs, PeerOut, check, lib
from .ops import FLAG_CHUNK_MAJOR, FLAG_FRAG_ORDER, FMT_HUFFMAN, FMT_HUFPAIR, FMT_NIBBLE, HEADER, MAGIC, Meta

HP_TAIL_WORDS, HUF_TAIL_WORDS = 32, 16


def unit_range(rank: int, world: int, rows: int, unit_rows: int) -> tuple[int, int]:
    """Rows [r0, r1) of `rank`: whole units, sizes differing by at most one unit."""
    units = rows // unit_rows
    return units * rank // world * unit_rows, units * (rank + 1) // world * unit_rows


def _header(fmt, K, R, rows, off, n_a, n_b, flags) -> bytes:
    return HEADER.pack(MAGIC, fmt, K, R, rows, off[0], off[1], off[2], off[3], n_a, n_b, flags, 0).ljust(256, b"\0")


def shard_rows(plane: torch.Tensor, aux: torch.Tensor, r0: int, r1: int) -> tuple[torch.Tensor, torch.Tensor, Meta]:
    """Rows [r0, r1) of an encoded matrix (CPU tensors) as an encoded matrix of its own: same code tables, plane rows
    and per-unit / per-row arrays sliced, stream offsets rebased, a fresh header. r0 and r1 must be unit boundaries.
    Fragment-order tensors are not supported."""
    a = aux.numpy()
    magic, fmt, K, R, rows, oa, ob, oc, od, n_a, n_b, flags, _ = HEADER.unpack(bytes(a[:HEADER.size]))
    if magic != MAGIC or flags & FLAG_FRAG_ORDER:
        raise ValueError("bf16n shard_rows: bad header or fragment-order tensor")
    unit = 1 if fmt == FMT_NIBBLE else R
    if not (0 <= r0 <= r1 <= rows) or r0 % unit or r1 % unit:
        raise ValueError("bf16n shard_rows: rows must be a range of whole units")
    n = r1 - r0
    p = plane.reshape(rows, K)[r0:r1].contiguous()
    if fmt == FMT_NIBBLE:
        codes = a[oa + r0 * K // 2: oa + r1 * K // 2]
        luts = a[ob + r0 * 16: ob + r1 * 16]
        eo = a[oc: oc + 4 * (rows + 1)].view(np.uint32)
        esc = a[od: od + 4 * max(int(n_a), 1)].view(np.uint32)
        e0, e1 = int(eo[r0]), int(eo[r1])
        new_eo = (eo[r0:r1 + 1] - e0).astype(np.uint32)
        new_esc = esc[e0:e1] if e1 > e0 else np.zeros(1, np.uint32)
        off = [256, 256 + codes.size, 256 + codes.size + luts.size, 256 + codes.size + luts.size + new_eo.size * 4]
        body = [codes, luts, new_eo.view(np.uint8), new_esc.view(np.uint8)]
        hdr = _header(fmt, K, 0, n, off, e1 - e0, 0, 0)
    elif fmt == FMT_HUFPAIR:
        u0, u1 = r0 // R, r1 // R
        lut = a[oa: oa + 4 * 4096]
        ubase = a[ob: ob + 4 * n_a].view(np.uint32)
        lrel = a[oc: oc + 2 * 32 * n_a].view(np.uint16)
        w0 = int(ubase[u0]) if u0 < n_a else int(n_b)
        w1 = int(ubase[u1]) if u1 < n_a else int(n_b)
        new_ub = (ubase[u0:u1] - w0).astype(np.uint32)
        new_lr = lrel[32 * u0: 32 * u1]
        stream = a[od + 4 * w0: od + 4 * w1]
        o_b = 256 + lut.size
        o_c = o_b + new_ub.size * 4
        o_d = (o_c + new_lr.size * 2 + 15) & ~15
        off = [256, o_b, o_c, o_d]
        pad = np.zeros(o_d - (o_c + new_lr.size * 2), np.uint8)
        body = [lut, new_ub.view(np.uint8), new_lr.view(np.uint8), pad, stream, np.zeros(4 * HP_TAIL_WORDS, np.uint8)]
        hdr = _header(fmt, K, R, n, off, u1 - u0, w1 - w0, flags)
    else:
        u0, u1 = r0 // R, r1 // R
        lut = a[oa: oa + 4 * 1024]
        lane_off = a[ob: ob + 4 * 32 * n_a].view(np.uint32)
        w0 = int(lane_off[32 * u0]) if u0 < n_a else int(n_b)
        w1 = int(lane_off[32 * u1]) if u1 < n_a else int(n_b)
        new_lo = (lane_off[32 * u0: 32 * u1] - w0).astype(np.uint32)
        stream = a[oc + 4 * w0: oc + 4 * w1]
        o_b = 256 + lut.size
        o_c = o_b + new_lo.size * 4
        off = [256, o_b, o_c, 0]
        body = [lut, new_lo.view(np.uint8), stream, np.zeros(4 * HUF_TAIL_WORDS, np.uint8)]
        hdr = _header(fmt, K, R, n, off, u1 - u0, w1 - w0, 0)
    new_aux = torch.from_numpy(np.concatenate([np.frombuffer(hdr, np.uint8)] + [np.ascontiguousarray(b).view(np.uint8) for b in body]))
    return p, new_aux, ops.parse_header(new_aux)


# ------------------------------------------------------------------ exchange buffers between the GPUs of one node

HEADER_BYTES = 256          # BF16N_EXCHANGE_HEADER_BYTES
IPC_HANDLE_BYTES = 64


class PeerExchange:
    """One exchange buffer per rank ([256-byte header | payload], allocated by the library), every peer's buffer mapped
    into this process through CUDA IPC. Kernels launched with `peer_out()` store their output into all of them and
    announce it; `wait()` holds the stream until every peer has announced its next launch. One process per GPU, all on
    one node; the handles travel through the process group once, at construction."""

    def __init__(self, payload_bytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise ValueError("bf16n PeerExchange: 2..8 ranks on one node")
        self.payload_bytes = payload_bytes
        base = C.c_void_p()
        handle = C.create_string_buffer(IPC_HANDLE_BYTES)
        check(lib().bf16n_exchange_create(payload_bytes, C.byref(base), handle))
        self.base = base.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.bases = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.base)
                continue
            peer = C.c_void_p()
            check(lib().bf16n_exchange_open(h, C.byref(peer)))
            self.bases.append(peer.value)
        self.peers = [r for r in range(self.world) if r != self.rank]
        self.mask = sum(1 << r for r in self.peers)
        dist.barrier(group=group)  # every rank has mapped every buffer before anyone writes

    def payload(self, offset: int, shape, dtype) -> torch.Tensor:
        """A tensor over this rank's payload at `offset` bytes (a view of library-owned memory: keep `self` alive)."""
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + n > self.payload_bytes:
            raise ValueError("bf16n PeerExchange: payload range out of bounds or unaligned")
        buf = (C.c_char * n).from_address(self.base + HEADER_BYTES + offset)
        iface = {"shape": tuple(int(s) for s in shape), "typestr": {torch.float32: "<f4", torch.bfloat16: "<u2"}[dtype],
                 "data": (self.base + HEADER_BYTES + offset, False), "version": 3}
        holder = type("_Span", (), {"__cuda_array_interface__": iface, "_keep": buf})()
        t = torch.as_tensor(holder, device=torch.device("cuda", torch.cuda.current_device()))
        return t.view(dtype) if dtype == torch.bfloat16 else t

    def peer_out(self, offset: int, wait: bool = False) -> PeerOut:
        """Fan-out descriptor: the peers' payloads at `offset` and this rank's flag word in each peer's header.
        wait=True: the kernel also waits for the peers' outputs of the same epoch before it ends (no wait() call)."""
        o = PeerOut()
        o.wait_mask = self.mask if wait else 0
        o.n_peers = len(self.peers)
        for i, r in enumerate(self.peers):
            o.y[i] = self.bases[r] + HEADER_BYTES + offset
            o.flag[i] = self.bases[r] + 4 * self.rank
        o.local_header = self.base
        return o

    def wait(self) -> None:
        check(lib().bf16n_peer_wait(self.base, self.mask, ops._stream()))

    def timing(self) -> dict:
        """Diagnostics of the last fan-out launch on this rank, microseconds on this GPU's clock: from the launch's first
        block to the moment every block's stores were issued, from there to the epoch published in the peers' headers,
        and from there to every peer's epoch seen here (waiting for the slowest rank included)."""
        torch.cuda.synchronize()
        iface = {"shape": (4,), "typestr": "<i8", "data": (self.base + 4 * 20, False), "version": 3}  # header words 20..27
        holder = type("_Span", (), {"__cuda_array_interface__": iface})()
        t = torch.as_tensor(holder, device=torch.device("cuda", torch.cuda.current_device())).cpu().tolist()  # begin, stored, published, seen
        return {"begin_to_stored_us": (t[1] - t[0]) / 1e3, "stored_to_published_us": (t[2] - t[1]) / 1e3,
                "published_to_all_seen_us": (t[3] - t[2]) / 1e3}

    def expired(self) -> bool:
        v = C.c_int(0)
        check(lib().bf16n_peer_expired(self.base, ops._stream(), C.byref(v)))
        return bool(v.value)

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody still writes into a buffer that is about to go away
        for r in self.peers:
            check(lib().bf16n_exchange_close(self.bases[r]))
        check(lib().bf16n_exchange_destroy(self.base))
        self.bases, self.base = [], None


def mmv_peers(x: torch.Tensor, w: ops.Weight, y: torch.Tensor, peers: PeerOut) -> None:
    """y = W x for dense x [T, K] like ops.mmv, the same values stored into every peer's buffer by the same kernel."""
    cw = w.c()
    ops._check_x(x, w.meta.K)
    if x.dim() != 2 or y.dim() != 2 or y.shape != (x.shape[0], w.meta.rows) or y.stride(1) != 1:
        raise RuntimeError("bf16n.mmv_peers: x [T, K], y [T, rows] with unit column stride")
    a = MmvArgs()
    a.x, a.x_bf16, a.y, a.y_bf16 = x.data_ptr(), int(x.dtype == torch.bfloat16), y.data_ptr(), int(y.dtype == torch.bfloat16)
    a.ncols, a.n_used, a.x_per_slot = x.shape[0], 1, 1
    a.x_tok, a.y_tok = x.stride(0) * x.element_size(), y.stride(0) * y.element_size()
    a.rows_per_matrix, a.nrows = w.meta.rows, w.meta.rows
    with torch.cuda.device(w.plane.device):
        check(lib().bf16n_mmv_peers(C.byref(cw), C.byref(a), C.byref(peers), ops._stream()))


# ------------------------------------------------------------------ vocabulary projection: rows sharded + all-gather

class ShardedLinear:
    """Row shard of a projection on this rank plus the buffers of the gathered result."""

    def __init__(self, weight: ops.Weight, rows_total: int, unit_rows: int, group=None):
        self.w, self.group = weight, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ranges = [unit_range(r, self.world, rows_total, unit_rows) for r in range(self.world)]
        self.width = max(b - a for a, b in self.ranges)  # shards padded to the widest: one all-gather assembles them
        self.rows_total = rows_total

    def buffers(self, T: int, device) -> torch.Tensor:
        return torch.empty((self.world, T, self.width), dtype=torch.float32, device=device)

    def __call__(self, x: torch.Tensor, gathered: torch.Tensor) -> torch.Tensor:
        """x [T, K] (replicated) -> gathered[world, T, width] with rank r's logits in gathered[r, :, :rows_r]."""
        a, b = self.ranges[self.rank]
        mine = gathered[self.rank]
        if self.width == b - a:
            ops.mmv(x, self.w, out=mine)
        else:
            mine[:, : b - a].copy_(ops.mmv(x, self.w))
        if self.world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), mine.reshape(-1), group=self.group)
        return gathered

    def assemble(self, gathered: torch.Tensor) -> torch.Tensor:
        """[T, rows_total] logits from the gathered shards."""
        return torch.cat([gathered[r, :, : b - a] for r, (a, b) in enumerate(self.ranges)], dim=1)


class FusedShardedLinear:
    """Row shard of a projection whose GEMV kernel writes its logits into every rank's gathered buffer itself (peer
    stores over NVLink), announces them and (wait_in_kernel) ends only when the peers' logits have arrived: one kernel per
    step, no collective. With wait_in_kernel=False a separate small wait kernel follows instead. The gathered buffers live in a PeerExchange payload,
    two of them used in turn so that a step may start before every peer has read the previous one."""

    def __init__(self, weight: ops.Weight, rows_total: int, unit_rows: int, max_tokens: int, group=None, wait_in_kernel: bool = True):
        self.w = weight
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.ranges = [unit_range(r, self.world, rows_total, unit_rows) for r in range(self.world)]
        self.rows_total, self.T = rows_total, max_tokens
        # buffer b: [world][T][width] FP32, shards padded to the widest and placed at 256-byte aligned offsets
        self.width = (max(b - a for a, b in self.ranges) + 63) // 64 * 64
        self.area = self.world * max_tokens * self.width * 4
        self.xchg = PeerExchange(2 * self.area, group)
        self.step = 0
        self._views = [self.xchg.payload(b * self.area, (self.world, max_tokens, self.width), torch.float32) for b in range(2)]
        self.wait_in_kernel = wait_in_kernel
        self._outs = [self.xchg.peer_out(b * self.area + self.rank * max_tokens * self.width * 4, wait_in_kernel) for b in range(2)]

    def __call__(self, x: torch.Tensor, weight: ops.Weight | None = None) -> torch.Tensor:
        """x [T, K] (replicated, T == max_tokens) -> gathered [world, T, width]: rank r's logits in [r, :, :rows_r],
        complete on this stream when the call returns. weight: another copy of the same shard (benchmarks rotate copies
        so that a small shard is not served from L2)."""
        if x.shape[0] != self.T:
            raise RuntimeError("bf16n FusedShardedLinear: built for a fixed number of tokens")
        b = self.step & 1
        self.step += 1
        a0, a1 = self.ranges[self.rank]
        mmv_peers(x, weight or self.w, self._views[b][self.rank][:, : a1 - a0], self._outs[b])  # rows of the padded [T, width] slot
        if not self.wait_in_kernel:
            self.xchg.wait()
        return self._views[b]

    def assemble(self, gathered: torch.Tensor) -> torch.Tensor:
        return torch.cat([gathered[r, :, : b - a] for r, (a, b) in enumerate(self.ranges)], dim=1)

    def close(self) -> None:
        self.xchg.close()


class HostGatheredLinear:
    """Row-sharded projection whose logits land in HOST memory: one pinned buffer shared by the ranks of a node (POSIX
    shared memory, registered with CUDA in every process), into which every rank's GEMV kernel stores its shard
    directly, so the logits cross as many PCIe links as there are GPUs and no copy follows the kernels. The kernel treats
    the host buffer as its one "peer" (bf16n_mmv_peers): after its last block's stores it writes the step number into
    this rank's epoch word in the shared buffer, so a step is one graph launch (activation copy from pinned memory +
    GEMV) and a spin on the ranks' epoch words: no stream synchronise, and every process sees when all shards are there.
    Two logits buffers alternate: a rank cannot start step s + 2 before every rank has finished step s + 1, i.e. has
    consumed the logits of step s. compute(x, out) replaces the GPU product in the CPU tests of the exchange."""

    FLAG_STRIDE = 16  # int32 words between the ranks' epoch words (64 bytes: one cache line each)

    def __init__(self, weight, rows_total: int, unit_rows: int, max_tokens: int, group=None, compute=None):
        import mmap
        import os
        import uuid
        self.w, self.group, self.compute = weight, group, compute
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ranges = [unit_range(r, self.world, rows_total, unit_rows) for r in range(self.world)]
        self.rows_total, self.T = rows_total, max_tokens
        self.header = 4 * self.FLAG_STRIDE * 8
        area = (max_tokens * rows_total * 4 + 255) // 256 * 256
        nbytes = (self.header + 2 * area + 4095) // 4096 * 4096
        name = [f"/dev/shm/bf16n_logits_{uuid.uuid4().hex}"] if self.rank == 0 else [None]
        if self.rank == 0:
            with open(name[0], "wb") as f:
                f.truncate(nbytes)
        if self.world > 1:
            dist.broadcast_object_list(name, src=0, group=group)
        self._fd = os.open(name[0], os.O_RDWR)
        self._map = mmap.mmap(self._fd, nbytes)
        if self.world > 1:
            dist.barrier(group=group)  # every rank has the file open before its name goes away
        if self.rank == 0:
            os.unlink(name[0])
        self._np = np.frombuffer(self._map, dtype=np.uint8)
        self.flags = self._np[: self.header].view(np.int32)
        self._registered = False
        self._bufs = [torch.from_numpy(self._np[self.header + b * area: self.header + b * area + max_tokens * rows_total * 4]
                                       .view(np.float32)).view(max_tokens, rows_total) for b in range(2)]
        if compute is None:
            rc = torch.cuda.cudart().cudaHostRegister(self._np.ctypes.data, nbytes, 1 | 2)  # portable | mapped
            if int(rc) != 0:
                raise RuntimeError(f"bf16n HostGatheredLinear: cudaHostRegister failed ({rc})")
            self._registered = True
            dev = weight.plane.device
            self._hdr = torch.zeros(HEADER_BYTES // 4, dtype=torch.int32, device=dev)   # block counter and step number of the kernel
            self._y_dev = torch.empty(max_tokens, rows_total, dtype=torch.float32, device=dev)
            self._x_dev = torch.empty(max_tokens, weight.meta.K, dtype=torch.bfloat16, device=dev)
            a0 = self.ranges[self.rank][0]
            self._outs = []
            for b in range(2):
                o = PeerOut()
                o.n_peers, o.wait_mask = 1, 0
                o.y[0] = self._np.ctypes.data + self.header + b * area + 4 * a0
                o.flag[0] = self._np.ctypes.data + 4 * self.rank * self.FLAG_STRIDE
                o.local_header = self._hdr.data_ptr()
                self._outs.append(o)
            self._graphs = {}   # (activation address, tokens, buffer, weight address) -> None after the first eager step, then its graph
        self.epoch = 0

    def _launch(self, x_host: torch.Tensor, b: int) -> None:
        T = x_host.shape[0]
        a0, a1 = self.ranges[self.rank]
        x = self._x_dev[:T]
        x.copy_(x_host, non_blocking=True)
        mmv_peers(x, self.w, self._y_dev[:T, a0:a1], self._outs[b])

    def step(self, x_host: torch.Tensor, x_dev: torch.Tensor | None = None) -> torch.Tensor:
        """x_host [T, K] BF16 pinned -> logits [T, rows_total] (host; valid until the step after the next one), complete
        in every process when the call returns. The first step from a given activation buffer launches eagerly, the
        second captures a graph, later ones replay it."""
        b = self.epoch & 1
        logits = self._bufs[b][: x_host.shape[0]]
        if self.compute is not None:
            a0, a1 = self.ranges[self.rank]
            self.compute(x_host, logits[:, a0:a1])
            self.epoch += 1
            self.flags[self.rank * self.FLAG_STRIDE] = self.epoch
        else:
            if x_host.dtype != torch.bfloat16 or not x_host.is_pinned() or x_host.dim() != 2 or x_host.shape[0] > self.T:
                raise ValueError("bf16n HostGatheredLinear: x_host is a pinned BF16 [T <= max_tokens, K] tensor")
            key = (x_host.data_ptr(), x_host.shape[0], b, self.w.plane.data_ptr())
            g = self._graphs.get(key, False)
            if g is False:
                self._launch(x_host, b)
                self._graphs[key] = None
            else:
                if g is None:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self._launch(x_host, b)
                    self._graphs[key] = g
                g.replay()
            self.epoch += 1   # the kernel's last block writes the same number into this rank's epoch word
        for r in range(self.world):
            spins = 0
            while self.flags[r * self.FLAG_STRIDE] < self.epoch:
                spins += 1
                if spins > 50_000_000:
                    raise RuntimeError(f"bf16n HostGatheredLinear: rank {r} never announced step {self.epoch}")
        return logits

    def close(self) -> None:
        if self._registered:
            torch.cuda.synchronize()
            self._graphs = {}
            torch.cuda.cudart().cudaHostUnregister(self._np.ctypes.data)
            self._registered = False
        self._bufs = self.flags = self._np = None
        try:
            self._map.close()
        except BufferError:
            pass  # a view is still alive somewhere: the mapping goes with the process
        import os
        os.close(self._fd)


# ------------------------------------------------------------------ MoE decode: expert-parallel + all-reduce

def moe_decode_ep(x, gate, up, down, n_experts, top_k, router_logits, group=None, scratch=None):
    """Expert-parallel decode step: this rank's weights hold experts [rank*E/G, (rank+1)*E/G). Returns the full
    [T, H] FP32 output on every rank (sum of the ranks' partial outputs; the summation order differs from the
    single-GPU slot order, so results agree to FP32 rounding, not bitwise)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n_local = n_experts // world
    y, wts, ids = ops.moe_decode(x, gate, up, down, n_experts, top_k, router_logits=router_logits, expert_lo=rank * n_local,
                                 n_experts_local=n_local, scratch=scratch)
    if world > 1:
        dist.all_reduce(y, group=group)
    return y, wts, ids


class FusedMoeDecode:
    """Expert-parallel decode step without a collective: the step's last kernel (the slot-order combine) stores this
    rank's partial [T, H] output into every rank's exchange buffer, announces it and ends when the peers' partials have
    arrived; one small kernel then adds the partials in rank order (the same bits on every rank) plus an optional extra
    term (the shared expert). Two buffers alternate as in FusedShardedLinear."""

    def __init__(self, gate, up, down, n_experts: int, top_k: int, max_tokens: int, group=None):
        self.gate, self.up, self.down, self.E, self.k, self.T = gate, up, down, n_experts, top_k, max_tokens
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_local = n_experts // self.world
        self.H = down.meta.rows // self.n_local
        self.area = self.world * max_tokens * self.H * 4
        self.xchg = PeerExchange(2 * self.area, group)
        self.step = 0
        slot = self.rank * max_tokens * self.H * 4
        self._views = [self.xchg.payload(b * self.area, (self.world, max_tokens, self.H), torch.float32) for b in range(2)]
        self._outs = [self.xchg.peer_out(b * self.area + slot, wait=True) for b in range(2)]
        self.scratch = ops.moe_decode_scratch(max_tokens, top_k, gate, down, self.n_local, gate.plane.device)

    def __call__(self, x, router_logits, out, extra=None, topk_weights=None, topk_ids=None, join=None):
        """x [T, K], router_logits [T, E] (both replicated) -> out [T, H] = sum over ranks of the routed experts' output
        (+ extra [T, H] FP32). T == max_tokens. join: a stream the final sum waits for (the one that produces extra)."""
        if x.shape[0] != self.T:
            raise RuntimeError("bf16n FusedMoeDecode: built for a fixed number of tokens")
        b = self.step & 1
        self.step += 1
        _, wts, ids = ops.moe_decode(x, self.gate, self.up, self.down, self.E, self.k, router_logits=router_logits,
                                     topk_weights=topk_weights, topk_ids=topk_ids, expert_lo=self.rank * self.n_local,
                                     n_experts_local=self.n_local, scratch=self.scratch, out=self._views[b][self.rank],
                                     peers=self._outs[b])
        parts = self._views[b]
        if join is not None:
            torch.cuda.current_stream().wait_stream(join)
        check(lib().bf16n_peer_sum(parts.data_ptr(), self.world, self.T * self.H, extra.data_ptr() if extra is not None else None,
                                   out.data_ptr(), int(out.dtype == torch.bfloat16), ops._stream()))
        return out, wts, ids

    def close(self) -> None:
        self.xchg.close()


# ------------------------------------------------------------------ MoE prefill: expert-parallel + all-to-all dispatch

def dispatch_plan(topk_ids: torch.Tensor, n_experts: int, world: int):
    """For this rank's tokens: the routed (token, slot) pairs ordered by owner rank (then token, slot).
    Returns (order [P] indices into the flattened pairs, send_counts [world], local expert id of each ordered pair)."""
    n_local = n_experts // world
    flat = topk_ids.reshape(-1).to(torch.int64)
    owner = flat // n_local
    order = torch.argsort(owner, stable=True)
    send_counts = torch.bincount(owner, minlength=world)
    return order, send_counts, (flat - owner * n_local)[order]


def moe_prefill_ep(x, topk_weights, topk_ids, gate, up, down, n_experts, group=None, experts_fn=None):
    """Expert-parallel prefill layer. x [T_local, H] BF16 and its routing are this rank's tokens; gate/up/down hold this
    rank's experts. Every routed row is sent to its expert's rank (all-to-all), multiplied there with the batched
    kernels (as single-slot tokens), sent back and combined in slot order. `experts_fn(rows, local_ids)` -> [n, H]
    replaces the device kernels in the CPU tests of the exchange."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    T, k = topk_ids.shape
    H = x.shape[1]
    order, send_counts, local_e = dispatch_plan(topk_ids, n_experts, world)
    tok = torch.div(order, k, rounding_mode="floor")
    send_rows = x[tok]                                             # [P, H] ordered by owner
    if world > 1:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_rows = x.new_empty((sum(rc), H))
        dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=group)
        recv_e = local_e.new_empty(sum(rc))
        dist.all_to_all_single(recv_e, local_e, rc, sc, group=group)
    else:
        sc = rc = send_counts.tolist()
        recv_rows, recv_e = send_rows, local_e
    if experts_fn is None:
        n_local = n_experts // world
        ids1 = recv_e.to(torch.int32).view(-1, 1)
        if recv_rows.shape[0]:
            a = ops.moe_mm_ids(recv_rows.contiguous(), ids1, gate, n_local, up=up, out_dtype=torch.bfloat16)   # [n, 1, N]
            out_rows = ops.moe_mm_ids(a, ids1, down, n_local, out_dtype=torch.float32)[:, 0]                   # [n, H]
        else:
            out_rows = torch.empty((0, down.meta.rows // n_local), dtype=torch.float32, device=x.device)
    else:
        out_rows = experts_fn(recv_rows, recv_e)
    if world > 1:
        back = out_rows.new_empty((sum(sc), out_rows.shape[1]))
        dist.all_to_all_single(back, out_rows.contiguous(), sc, rc, group=group)
    else:
        back = out_rows
    ys = back.new_empty((T * k, back.shape[1]))
    ys[order] = back                                                # undo the owner ordering: [T*k, H] in (token, slot) order
    ys = ys.view(T, k, -1)
    if experts_fn is None:
        return ops.moe_combine(ys.contiguous(), topk_weights.contiguous(), torch.bfloat16)
    acc = torch.zeros((T, ys.shape[2]), dtype=ys.dtype)
    for s in range(k):
        acc = acc + topk_weights[:, s:s + 1].to(ys.dtype) * ys[:, s]
    return acc


class FusedMoePrefill:
    """Expert-parallel prefill layer without the host in the loop: this rank's tokens are routed on the device, every
    routed row is stored into the exchange buffer of the rank that owns its expert (peer stores over NVLink), multiplied
    there by the batched kernels and its result stored back; the slot-order combine finishes the layer. Only kernels on
    the current stream: no exchange of sizes through the host, no collective, capturable in a CUDA graph. Every rank
    calls it once per layer with at most `max_local_tokens` tokens (any rank's count may differ from call to call).
    Results equal moe_prefill_ep's bit for bit."""

    def __init__(self, gate, up, down, n_experts: int, top_k: int, max_local_tokens: int, group=None):
        self.gate, self.up, self.down, self.E, self.k = gate, up, down, n_experts, top_k
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_local = n_experts // self.world
        self.K, self.H = gate.meta.K, down.meta.rows // self.n_local
        self.dev = gate.plane.device
        self.P = max_local_tokens * top_k
        lay = EpLayout()
        lay.n_ranks, lay.rank, lay.cap, lay.K, lay.H, lay.n_pairs_max = self.world, self.rank, self.P, self.K, self.H, self.P
        nbytes = lib().bf16n_ep_layout_bytes(C.byref(lay))
        if self.world > 1:
            self.xchg = PeerExchange(nbytes, group)
            bases = self.xchg.bases
        else:
            self.xchg = None
            self._own = torch.zeros(HEADER_BYTES + nbytes, dtype=torch.uint8, device=self.dev)
            bases = [self._own.data_ptr()]
        for r, b in enumerate(bases):
            lay.base[r] = b
        self.lay = lay
        n_slots = self.world * self.P
        base = bases[self.rank] + HEADER_BYTES
        self.rows = _device_view(base + lay.off_rows, (n_slots, self.K), torch.bfloat16, self.dev)
        self.back = _device_view(base + lay.off_back, (self.P, self.H), torch.float32, self.dev)
        self.inbox_ids = torch.empty((n_slots, 1), dtype=torch.int32, device=self.dev)
        self.plan = torch.empty(self.P + 8, dtype=torch.int32, device=self.dev)

    def __call__(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """x [T, K] BF16 (this rank's tokens), topk_weights / topk_ids [T, k] -> [T, H] BF16."""
        T, k = topk_ids.shape
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] == T and x.stride(1) == 1):
            raise RuntimeError("bf16n FusedMoePrefill: x must be bf16 [tokens, K] on the GPU")
        if not (topk_ids.dtype == torch.int32 and topk_ids.is_contiguous() and k == self.k and 0 < T * k <= self.P):
            raise RuntimeError("bf16n FusedMoePrefill: topk_ids int32 [tokens, k] within the token limit it was built for")
        st = ops._stream()
        with torch.cuda.device(self.dev):
            check(lib().bf16n_ep_dispatch(C.byref(self.lay), x.data_ptr(), x.stride(0) * 2, topk_ids.data_ptr(), T, k, self.E,
                                          self.plan.data_ptr(), st))
            check(lib().bf16n_ep_inbox_ids(C.byref(self.lay), self.inbox_ids.data_ptr(), st))
        route = ops.moe_route(self.inbox_ids, self.n_local, False)
        a = ops.moe_mm_ids(self.rows, self.inbox_ids, self.gate, self.n_local, up=self.up, out_dtype=torch.bfloat16, route=route)
        ys = ops.moe_mm_ids(a, self.inbox_ids, self.down, self.n_local, out_dtype=torch.float32, route=(route[1], route[1], route[2]))
        with torch.cuda.device(self.dev):
            check(lib().bf16n_ep_give_back(C.byref(self.lay), ys.data_ptr(), st))
        return ops.moe_combine(self.back[: T * k].view(T, k, self.H), topk_weights.contiguous(), torch.bfloat16)

    def close(self) -> None:
        self.rows = self.back = None
        if self.xchg is not None:
            self.xchg.close()


def _device_view(ptr: int, shape, dtype, device) -> torch.Tensor:
    """A tensor over device memory the library owns (the caller keeps the owner alive)."""
    iface = {"shape": tuple(int(s) for s in shape), "typestr": {torch.float32: "<f4", torch.bfloat16: "<u2", torch.int32: "<i4"}[dtype],
             "data": (ptr, False), "version": 3}
    holder = type("_Span", (), {"__cuda_array_interface__": iface})()
    t = torch.as_tensor(holder, device=device)
    return t.view(dtype) if dtype == torch.bfloat16 else t
