"""Host-side mirror of the reference operator interface (engines/vllm/vllm_bf16n/ops.py:83-271 over
core/torch/torch_bindings.cpp:80-371) on top of the C ABI of libbf16n_b200.so.

Same names, argument meaning, output shapes and error behaviour (ValueError for invalid arguments, RuntimeError
otherwise). torch tensors carry device memory and the current CUDA stream; every product is computed by the library's
sm_100a kernels and there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import MmvArgs, check, lib
from ._lib import Weight as CWeight

FMT_NIBBLE, FMT_HUFFMAN, FMT_HUFPAIR = 1, 2, 3
FORMAT_NAMES = {FMT_NIBBLE: "nibble", FMT_HUFFMAN: "huffman", FMT_HUFPAIR: "hufpair"}
MAGIC = 0x4E363142
HEADER = struct.Struct("<IIIIQQQQQQQII")  # the 80 header bytes: magic, format, K, R, rows, off_a..d, n_a, n_b, flags, pad
FLAG_CHUNK_MAJOR, FLAG_FRAG_ORDER = 1, 2
GEMV_MAX_TOKENS = 8                      # up to 8 tokens through the GEMV kernels, more through the batched kernels
DEQUANT_CHUNK_BYTES = 64 << 20


@dataclass(frozen=True)
class Meta:
    """Host-side metadata of one encoded matrix, parsed once from its aux header."""
    format: int
    K: int
    rows: int
    R: int
    chunk_major: bool
    frag_order: bool
    off_a: int
    off_b: int
    off_c: int
    off_d: int

    def as_list(self) -> list[int]:
        flags = (FLAG_CHUNK_MAJOR if self.chunk_major else 0) | (FLAG_FRAG_ORDER if self.frag_order else 0)
        return [self.format, self.K, self.rows, self.R, flags, self.off_a, self.off_b, self.off_c, self.off_d]


def parse_header(aux: torch.Tensor) -> Meta:
    """Metadata from the first 256 bytes of a CPU aux tensor; raises ValueError on a malformed header."""
    if aux.device.type != "cpu" or aux.dtype != torch.uint8 or aux.numel() < 256:
        raise ValueError("bf16n: aux must be a CPU uint8 tensor of at least 256 bytes")
    aux = aux.contiguous()
    w = CWeight()
    check(lib().bf16n_parse_header(aux.data_ptr(), aux.numel(), C.byref(w)))
    return Meta(w.format, w.K, w.rows, w.R, bool(w.cm), bool(w.fo), w.off_a, w.off_b, w.off_c, w.off_d)


@dataclass
class Weight:
    """One encoded matrix on the device: plane (rows x K sign|mantissa bytes) + aux, and its metadata."""
    plane: torch.Tensor
    aux: torch.Tensor
    meta: Meta

    @property
    def m(self) -> list[int]:
        return self.meta.as_list()

    @property
    def nbytes(self) -> int:
        return self.plane.numel() + self.aux.numel()

    def c(self) -> CWeight:
        m = self.meta
        if not (self.plane.is_cuda and self.aux.is_cuda):
            raise RuntimeError("bf16n: plane and aux must be CUDA tensors")
        if self.plane.dtype != torch.uint8 or self.aux.dtype != torch.uint8:
            raise RuntimeError("bf16n: plane and aux must be uint8")
        if not (self.plane.is_contiguous() and self.aux.is_contiguous()):
            raise RuntimeError("bf16n: plane and aux must be contiguous")
        if self.plane.numel() != m.rows * m.K:
            raise RuntimeError(f"bf16n: plane has {self.plane.numel()} bytes, meta says {m.rows} x {m.K}")
        if max(m.off_a, m.off_b, m.off_c, m.off_d) >= self.aux.numel():
            raise RuntimeError(f"bf16n: aux ({self.aux.numel()} bytes) shorter than its offsets")
        return CWeight(self.plane.data_ptr(), self.aux.data_ptr(), m.format, m.R, m.K, m.rows, int(m.chunk_major),
                       int(m.frag_order), m.off_a, m.off_b, m.off_c, m.off_d)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def init() -> None:
    """Device attributes and kernel shared-memory limits; once per process, before any launch / graph capture."""
    check(lib().bf16n_init())


def fault_status() -> int:
    """Synchronises the current stream and returns (and clears) the bit mask of the kernels' bounded waits that ran out
    since the last call: 1 staged GEMV, 2 MoE decode units, 4 fragment-order kernels, 8 batched kernel. 0: all outputs
    complete; otherwise the outputs of the affected work items are NaN."""
    v = C.c_uint(0)
    check(lib().bf16n_fault_status(C.byref(v), _stream()))
    return int(v.value)


def set_peer_wait_limit_ms(ms: int) -> None:
    """How long a wait for the peers' announcements may take before it gives up and sets the exchange header's expired
    word (default 2000 ms); applies to launches made or captured after the call."""
    check(lib().bf16n_set_peer_wait_limit_ms(int(ms)))


def sm_count() -> int:
    n = C.c_int(0)
    check(lib().bf16n_sm_count(C.byref(n)))
    return n.value


# ------------------------------------------------------------------ host: encode, policy

def encode(w: torch.Tensor, fmt: int, R: int, chunk_major: bool, frag_order: bool = False
           ) -> tuple[torch.Tensor, torch.Tensor, Meta]:
    """Encode a BF16 CPU tensor (..., K) on all host cores: (plane uint8 [rows, K], aux uint8 [n], Meta). FMT_HUFPAIR
    falls back to FMT_HUFFMAN above 4096 distinct exponent pairs; Meta holds the format actually produced."""
    if w.device.type != "cpu":
        raise RuntimeError("bf16n.encode: weight must be on the CPU")
    if w.dtype != torch.bfloat16:
        raise RuntimeError("bf16n.encode: weight must be bfloat16")
    if w.dim() < 2:
        raise RuntimeError("bf16n.encode: weight must be at least 2-D (rows x K)")
    wc = w.contiguous()
    K = wc.shape[-1]
    rows = wc.numel() // max(K, 1)
    h = C.c_void_p()
    check(lib().bf16n_encode(wc.data_ptr(), rows, K, fmt, R, int(chunk_major), int(frag_order), C.byref(h)))
    try:
        n = C.c_size_t(0)
        p = lib().bf16n_encoded_plane(h, C.byref(n))
        plane = torch.empty((rows, K), dtype=torch.uint8)
        C.memmove(plane.data_ptr(), p, n.value)
        p = lib().bf16n_encoded_aux(h, C.byref(n))
        aux = torch.empty((n.value,), dtype=torch.uint8)
        C.memmove(aux.data_ptr(), p, n.value)
    finally:
        lib().bf16n_encoded_free(h)
    return plane, aux, parse_header(aux)


def choose(rows: int, K: int, n_matrices: int = 1, *, engine: str = "vllm", mode: str = "hybrid", dense_min: int = 8 << 20,
           expert: bool = False, dense_frag_order: bool = False, min_units: int = 512):
    """Shape policy: None (stays BF16) or (format, R, chunk_major, frag_order). min_units: the fewest units a dense
    pair-Huffman matrix may have (512 = the reference's constant; a loader that shards over several B200s passes about
    SMs x 24 so that small shards get shorter units)."""
    out = (C.c_int * 4)()
    ok = lib().bf16n_choose_for_machine(rows, K, n_matrices, int(engine == "vllm"), {"hybrid": 0, "huffman": 1, "nibble": 2}[mode],
                                        dense_min, int(expert), int(dense_frag_order), min_units, out)
    return (out[0], out[1], bool(out[2]), bool(out[3])) if ok else None


def upload(plane: torch.Tensor, aux: torch.Tensor, meta: Meta, device: torch.device | str) -> Weight:
    return Weight(plane.to(device), aux.to(device), meta)


# ------------------------------------------------------------------ device: dequant / verify

def dequant(w: Weight, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    nrows = w.meta.rows - row0 if nrows is None else nrows
    if row0 < 0 or nrows < 0 or row0 + nrows > w.meta.rows:
        raise RuntimeError("bf16n.dequant: rows out of range")
    cw = w.c()
    out = torch.empty((nrows, w.meta.K), dtype=torch.bfloat16, device=w.plane.device)
    with torch.cuda.device(w.plane.device):
        check(lib().bf16n_dequant(C.byref(cw), row0, nrows, out.data_ptr(), _stream()))
    return out


def mismatches(w: Weight, src: torch.Tensor, row0: int = 0, nrows: int | None = None) -> int:
    """Number of BF16 words of rows [row0, row0+nrows) that decode differently from src (a device BF16 tensor holding
    exactly those rows); the decode is compared in registers, nothing is materialised."""
    nrows = w.meta.rows - row0 if nrows is None else nrows
    cw = w.c()
    src = src.contiguous()
    if src.numel() != nrows * w.meta.K or src.dtype != torch.bfloat16 or src.device != w.plane.device:
        raise RuntimeError("bf16n.mismatches: src must be the bf16 rows on the weight's device")
    cnt = torch.zeros(1, dtype=torch.int64, device=w.plane.device)
    with torch.cuda.device(w.plane.device):
        check(lib().bf16n_verify(C.byref(cw), row0, nrows, src.data_ptr(), cnt.data_ptr(), _stream()))
    return int(cnt.item())


def roundtrip_equal(w: Weight, src: torch.Tensor, chunk_bytes: int = 64 << 20) -> bool:
    """Bitwise check of the GPU decode against the BF16 source (any device), in row chunks of whole units."""
    K, rows = w.meta.K, w.meta.rows
    unit = max(w.meta.R, 1)
    src2 = src.reshape(rows, K)
    step = max(chunk_bytes // (2 * K) // unit * unit, unit)
    for r0 in range(0, rows, step):
        nr = min(step, rows - r0)
        if mismatches(w, src2[r0:r0 + nr].to(w.plane.device), r0, nr) != 0:
            return False
    return True


# ------------------------------------------------------------------ device: GEMV family

def _check_x(x: torch.Tensor, K: int, what: str = "x") -> None:
    if not (x.is_cuda or x.is_pinned()):  # pinned host memory is mapped into the device's address space
        raise RuntimeError(f"bf16n: {what} must be a CUDA tensor (or pinned host memory)")
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError(f"bf16n: {what} must be bf16 or f32")
    if x.shape[-1] != K or x.stride(-1) != 1:
        raise RuntimeError(f"bf16n: {what} last dim must be K = {K} and contiguous")
    if x.data_ptr() % 16:
        raise RuntimeError(f"bf16n: {what} must be 16-byte aligned")
    for d in range(x.dim() - 1):
        if (x.stride(d) * x.element_size()) % 16:
            raise RuntimeError(f"bf16n: {what} row strides must be multiples of 16 bytes")


def _check_ids(ids: torch.Tensor) -> None:
    if not ids.is_cuda or ids.dim() != 2:
        raise RuntimeError("bf16n: ids must be a 2-D CUDA tensor [tokens, n_used]")
    if ids.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("bf16n: ids must be int32 or int64")
    if ids.stride(1) != 1:
        raise RuntimeError("bf16n: ids must be contiguous along the slot dimension")


def _check_out(out: torch.Tensor, shape: tuple, dtype: torch.dtype, device: torch.device, what: str) -> int:
    """A caller-supplied output: the result's shape and dtype, on the weight's device (or pinned host memory, which is
    mapped into the device's address space), last dimension contiguous, outer dimensions dense over the rows, 16-byte
    aligned base and row stride. Returns the byte stride between rows of the first dimension."""
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype:
        raise RuntimeError(f"bf16n.{what}: out must have shape {tuple(shape)} and dtype {dtype}, got {tuple(out.shape)} {out.dtype}")
    if out.device.type == "cpu":
        if not out.is_pinned():
            raise RuntimeError(f"bf16n.{what}: a host output must be pinned (page-locked and mapped into the device)")
    elif out.device != device:
        raise RuntimeError(f"bf16n.{what}: out is on {out.device}, the weight on {device}")
    if out.numel() and out.stride(-1) != 1:
        raise RuntimeError(f"bf16n.{what}: out must be contiguous along its last dimension")
    for d in range(1, out.dim() - 1):  # [tokens, slots, rows]: slots dense over the rows
        if out.stride(d) != out.shape[d + 1] * out.stride(d + 1):
            raise RuntimeError(f"bf16n.{what}: out must be dense below its first dimension")
    row = out.stride(0) * out.element_size() if out.dim() > 1 else 0
    if out.data_ptr() % 16 or row % 16:
        raise RuntimeError(f"bf16n.{what}: out and its row stride must be 16-byte aligned")
    if out.dim() > 1 and out.shape[0] > 1 and out.stride(0) < out.numel() // out.shape[0]:
        raise RuntimeError(f"bf16n.{what}: rows of out overlap")
    return row


def _mmv_common(x, w: Weight, ids, rows_per_matrix: int, out_bf16: bool, glu: bool, multi_col: bool = True,
                out: torch.Tensor | None = None) -> torch.Tensor:
    cw = w.c()
    m = w.meta
    _check_x(x, m.K)
    a = MmvArgs()
    a.x, a.x_bf16, a.y_bf16 = x.data_ptr(), int(x.dtype == torch.bfloat16), int(out_bf16)
    odt = torch.bfloat16 if out_bf16 else torch.float32
    osz = 2 if out_bf16 else 4
    if ids is None:
        if x.dim() != 2:
            raise RuntimeError("bf16n.mmv: dense x must be [tokens, K]")
        rpm = rows_per_matrix if rows_per_matrix > 0 else m.rows
        if rpm != m.rows:
            raise RuntimeError("bf16n.mmv: a dense product uses the whole matrix")
        if glu and rpm % 2:
            raise RuntimeError("bf16n.mmv_glu: odd row count")
        n_out = rpm // 2 if glu else rpm
        T = x.shape[0]
        y = torch.empty((T, n_out), dtype=odt, device=w.plane.device) if out is None else out
        y_row = n_out * osz if out is None else _check_out(out, (T, n_out), odt, w.plane.device, "mmv")
        if T == 0:
            return y
        a.y, a.ncols = y.data_ptr(), T
        a.x_tok, a.y_tok = x.stride(0) * x.element_size(), y_row
        a.n_used, a.x_per_slot = 1, 1
        a.rows_per_matrix, a.nrows = rpm, n_out
    else:
        _check_ids(ids)
        if ids.device != w.plane.device:
            raise RuntimeError("bf16n.mmv: ids on another device")
        T, n_used = ids.shape
        if rows_per_matrix <= 0 or m.rows % rows_per_matrix:
            raise RuntimeError("bf16n.mmv: rows_per_matrix must divide the rows")
        if glu and rows_per_matrix % 2:
            raise RuntimeError("bf16n.mmv_glu: odd rows per matrix")
        n_out = rows_per_matrix // 2 if glu else rows_per_matrix
        if not ((x.dim() == 2 and x.shape[0] == T) or (x.dim() == 3 and x.shape[0] == T and x.shape[1] == n_used)):
            raise RuntimeError("bf16n.mmv: x must be [tokens, K] or [tokens, n_used, K]")
        y = torch.empty((T, n_used, n_out), dtype=odt, device=w.plane.device) if out is None else out
        y_tok = n_used * n_out * osz if out is None else _check_out(out, (T, n_used, n_out), odt, w.plane.device, "mmv")
        if T == 0 or n_used == 0:
            return y
        a.y, a.ncols = y.data_ptr(), T * n_used
        a.ids, a.ids_s0, a.ids_s1 = ids.data_ptr(), ids.element_size(), ids.stride(0) * ids.element_size()
        a.n_used = n_used
        a.x_tok = x.stride(0) * x.element_size()
        a.x_per_slot = n_used if x.dim() == 3 else 1
        a.x_slot = x.stride(1) * x.element_size() if x.dim() == 3 else 0
        a.y_tok, a.y_slot = y_tok, n_out * osz
        a.rows_per_matrix, a.nrows = rows_per_matrix, n_out
    with torch.cuda.device(w.plane.device):
        if glu:
            check(lib().bf16n_mmv_glu_merged(C.byref(cw), C.byref(a), _stream()))
        else:
            check(lib().bf16n_mmv(C.byref(cw), C.byref(a), _stream(), int(multi_col)))
    return y


def mmv(x: torch.Tensor, w: Weight, ids: torch.Tensor | None = None, rows_per_matrix: int = 0,
        out_dtype: torch.dtype = torch.float32, multi_col: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    return _mmv_common(x, w, ids, rows_per_matrix, out_dtype == torch.bfloat16, False, multi_col, out)


def mmv_group(xs, ws, outs=None, out_dtype: torch.dtype = torch.float32):
    """Independent dense products ys[i] = ws[i] xs[i] in as few launches as possible: small NIBBLE matrices share one
    grid (eight products per launch), other formats are launched as mmv launches them. Same bits as mmv per product."""
    n = len(ws)
    if len(xs) != n or (outs is not None and len(outs) != n):
        raise RuntimeError("bf16n.mmv_group: one activation (and output) per matrix")
    if n == 0:
        return []
    out_bf16 = out_dtype == torch.bfloat16
    cws = (CWeight * n)()
    args = (MmvArgs * n)()
    ys = []
    dev = ws[0].plane.device
    for i, (x, w) in enumerate(zip(xs, ws)):
        cws[i] = w.c()
        m = w.meta
        _check_x(x, m.K)
        if x.dim() != 2 or w.plane.device != dev:
            raise RuntimeError("bf16n.mmv_group: dense x [tokens, K], all matrices on one device")
        T = x.shape[0]
        y = torch.empty((T, m.rows), dtype=out_dtype, device=dev) if outs is None else outs[i]
        y_row = m.rows * y.element_size() if outs is None else _check_out(y, (T, m.rows), out_dtype, dev, "mmv_group")
        a = args[i]
        a.x, a.x_bf16, a.y, a.y_bf16 = x.data_ptr(), int(x.dtype == torch.bfloat16), y.data_ptr(), int(out_bf16)
        a.ncols, a.n_used, a.x_per_slot = T, 1, 1
        a.x_tok, a.y_tok = x.stride(0) * x.element_size(), y_row
        a.rows_per_matrix, a.nrows = m.rows, m.rows if T else 0
        if T == 0:
            a.ncols = 1
        ys.append(y)
    with torch.cuda.device(dev):
        check(lib().bf16n_mmv_group(cws, args, n, _stream()))
    return ys


def mmv_glu(x: torch.Tensor, w: Weight, ids: torch.Tensor | None = None, rows_per_matrix: int = 0,
            out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """silu(gate x) * (up x) for a NIBBLE matrix whose rows per matrix are [gate; up]."""
    return _mmv_common(x, w, ids, rows_per_matrix or w.meta.rows, out_dtype == torch.bfloat16, True)


def mmv_glu2(x: torch.Tensor, gate: Weight, up: Weight, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """silu(gate x) * (up x) with separate dense gate / up matrices of one shape, format and R
    (bf16n::mmv_glu(gate, up, ...), core/include/bf16n/launch.h:54-60)."""
    cg, cu = gate.c(), up.c()
    _check_x(x, gate.meta.K)
    if x.dim() != 2:
        raise RuntimeError("bf16n.mmv_glu: dense x must be [tokens, K]")
    out_bf16 = out_dtype == torch.bfloat16
    T, n_out = x.shape[0], gate.meta.rows
    y = torch.empty((T, n_out), dtype=out_dtype, device=x.device)
    if T == 0:
        return y
    a = MmvArgs()
    a.x, a.x_bf16, a.y, a.y_bf16 = x.data_ptr(), int(x.dtype == torch.bfloat16), y.data_ptr(), int(out_bf16)
    a.ncols, a.n_used, a.x_per_slot = T, 1, 1
    a.x_tok, a.y_tok = x.stride(0) * x.element_size(), n_out * (2 if out_bf16 else 4)
    a.rows_per_matrix, a.nrows = n_out, n_out
    with torch.cuda.device(gate.plane.device):
        check(lib().bf16n_mmv_glu(C.byref(cg), C.byref(cu), C.byref(a), _stream()))
    return y


def linear(x: torch.Tensor, w: Weight, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ bias) in BF16: up to 8 tokens through the decode GEMV (FP32 accumulation; the bias is added in FP32
    before the single rounding), more through exact dequantisation in 64 MiB row chunks + a BF16 GEMM."""
    m = w.meta
    if x.dtype != torch.bfloat16:
        raise RuntimeError("bf16n.linear: x must be bf16")
    if x.shape[-1] != m.K:
        raise RuntimeError(f"bf16n.linear: x last dim must be K = {m.K}")
    oshape = (*x.shape[:-1], m.rows)
    x2 = x.reshape(-1, m.K)
    T = x2.shape[0]
    if T <= GEMV_MAX_TOKENS:
        ok = x2.stride(1) == 1 and (x2.stride(0) * 2) % 16 == 0 and x2.data_ptr() % 16 == 0
        xc = x2 if ok else x2.contiguous()
        if bias is not None:
            y = mmv(xc, w).add_(bias).to(torch.bfloat16)
        else:
            y = mmv(xc, w, out_dtype=torch.bfloat16)
    else:
        y = torch.empty((T, m.rows), dtype=x.dtype, device=x.device)
        unit = 1 if m.format == FMT_NIBBLE else m.R
        chunk = min(max(DEQUANT_CHUNK_BYTES // (m.K * 2) // unit * unit, unit), m.rows)
        for r0 in range(0, m.rows, chunk):
            nr = min(chunk, m.rows - r0)
            wc = dequant(w, r0, nr)
            ys = y.narrow(1, r0, nr)
            torch.mm(x2, wc.t(), out=ys) if ys.is_contiguous() else ys.copy_(x2 @ wc.t())
            if bias is not None:
                ys.add_(bias.narrow(0, r0, nr))
    return y.view(oshape)


def linear_host(x_host: torch.Tensor, w: Weight, y_host: torch.Tensor, x_dev: torch.Tensor, y_dev: torch.Tensor | None = None) -> None:
    """One decode step of a projection with HOST activations and logits: x_host (pinned, [T, K]) is copied to x_dev,
    multiplied on the GPU (FP32 out), and the result lands in y_host (pinned, [T, rows]). All on the current stream;
    the caller synchronises. The buffers are caller-owned so the call itself allocates nothing.
    With y_dev=None the kernel writes the logits straight into the pinned host buffer (the stores cross PCIe while the
    rest of the matrix is still being multiplied, so no copy follows the kernel); otherwise they go to y_dev and are
    copied. The activation is always copied first: every block reads all of it, which is slow across PCIe (measured:
    279 µs per step reading x from host memory against 225 µs with the 4 KB copy)."""
    x_dev.copy_(x_host, non_blocking=True)
    if y_dev is None:
        mmv(x_dev, w, out=y_host)
    else:
        mmv(x_dev, w, out=y_dev)
        y_host.copy_(y_dev, non_blocking=True)


def get_rows(ids: torch.Tensor, w: Weight, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    cw = w.c()
    if not ids.is_cuda or ids.dim() != 1:
        raise RuntimeError("bf16n.get_rows: ids must be a 1-D CUDA tensor")
    if ids.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("bf16n.get_rows: ids must be int32 or int64")
    n = ids.shape[0]
    out = torch.empty((n, w.meta.K), dtype=out_dtype, device=w.plane.device)
    with torch.cuda.device(w.plane.device):
        check(lib().bf16n_get_rows(C.byref(cw), ids.data_ptr(), ids.stride(0) * ids.element_size(), n, out.data_ptr(),
                                   int(out_dtype == torch.bfloat16), w.meta.K * out.element_size(), _stream(), 0))
    return out


def embedding(ids: torch.Tensor, w: Weight) -> torch.Tensor:
    return get_rows(ids.reshape(-1), w).view(*ids.shape, w.meta.K)


# ------------------------------------------------------------------ device: draft-only k-bit output head
# (engines/vllm/vllm_bf16n/ops.py:164-240 over core/torch/torch_bindings.cpp:241-295)

def _kbit_quantize(w: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor]:
    name = f"int{bits}_quantize"
    if not (w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()):
        raise RuntimeError(f"bf16n.{name}: w must be a contiguous 2-D CUDA bf16 tensor")
    rows, K = w.shape
    if K % 128:
        raise ValueError(f"bf16n.{name}: K must be a multiple of 128")
    q = torch.empty((rows, K * bits // 8), dtype=torch.uint8, device=w.device)
    s = torch.empty((rows, K // 128), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        check(getattr(lib(), f"bf16n_{name}")(w.data_ptr(), rows, K, q.data_ptr(), s.data_ptr(), _stream()))
    return q, s


def _kbit_gemv(x: torch.Tensor, q: torch.Tensor, s: torch.Tensor, bits: int) -> torch.Tensor:
    name = f"int{bits}_gemv"
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()):
        raise RuntimeError(f"bf16n.{name}: x must be contiguous bf16 [T, K]")
    T, K = x.shape
    if not (q.is_cuda and q.dtype == torch.uint8 and q.dim() == 2 and q.is_contiguous() and q.shape[1] == K * bits // 8):
        raise RuntimeError(f"bf16n.{name}: q must be uint8 [rows, K / {8 // bits}]")
    if not (s.is_cuda and s.dtype == torch.float32 and s.is_contiguous() and tuple(s.shape) == (q.shape[0], K // 128)):
        raise RuntimeError(f"bf16n.{name}: s must be f32 [rows, K / 128]")
    y = torch.empty((T, q.shape[0]), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(getattr(lib(), f"bf16n_{name}")(x.data_ptr(), T, q.data_ptr(), s.data_ptr(), q.shape[0], K, y.data_ptr(), _stream()))
    return y


def int4_quantize(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Draft-only 4-bit copy of a BF16 matrix (symmetric, FP32 scale per 128 weights): (q uint8 [R, K/2], s f32 [R, K/128])."""
    return _kbit_quantize(w, 4)


def int4_gemv(x: torch.Tensor, q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """Approximate y = x W^T (FP32 [T, R]) from the 4-bit copy; T <= 4."""
    return _kbit_gemv(x, q, s, 4)


def int2_quantize(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Draft-only 2-bit copy of a BF16 matrix: per 128 weights s = amax / 1.5 and each weight the nearest of
    -1.5 s, -0.5 s, 0.5 s, 1.5 s: (q uint8 [R, K/4], s f32 [R, K/128])."""
    return _kbit_quantize(w, 2)


def int2_gemv(x: torch.Tensor, q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """Approximate y = x W^T (FP32 [T, R]) from the 2-bit copy; T <= 4, K = 2048."""
    return _kbit_gemv(x, q, s, 2)


DRAFT_HEADS = {"int2": 2, "int4": 4}      # BF16N_DRAFT_HEAD values with a k-bit copy; "full" scores with the exact head
DEFAULT_CANDIDATES = {2: 128, 4: 32}      # candidates re-scored exactly (the reference's measured defaults, ops.py:187-191)


@dataclass(frozen=True)
class DraftHead:
    """Draft-only k-bit copy of an output head whose top `candidates` scores are re-scored exactly by draft_logits."""
    bits: int
    q: torch.Tensor
    s: torch.Tensor
    candidates: int

    def __post_init__(self):
        if self.bits not in DEFAULT_CANDIDATES:
            raise ValueError(f"draft head: {self.bits} bits (2 or 4)")
        if self.q.shape[1] * (8 // self.bits) != self.s.shape[1] * 128 or self.q.shape[0] != self.s.shape[0]:
            raise ValueError(f"draft head: q {tuple(self.q.shape)} and s {tuple(self.s.shape)} disagree for {self.bits} bits")
        if not 1 <= self.candidates <= self.q.shape[0]:
            raise ValueError(f"draft head: {self.candidates} candidates for {self.q.shape[0]} rows")

    def scores(self, h: torch.Tensor) -> torch.Tensor:
        return (int2_gemv if self.bits == 2 else int4_gemv)(h, self.q, self.s)


def draft_head_bits() -> int | None:
    """Bits of the draft head chosen by BF16N_DRAFT_HEAD (int2 by default, int4; full = the exact head, None). Read by
    the engine layer when it builds the head, never by a launch."""
    import os
    v = os.environ.get("BF16N_DRAFT_HEAD", "int2")
    if v == "full":
        return None
    if v not in DRAFT_HEADS:
        raise ValueError(f"BF16N_DRAFT_HEAD must be one of int2, int4, full; got {v!r}")
    return DRAFT_HEADS[v]


def make_draft_head(w: torch.Tensor, bits: int) -> DraftHead:
    """The k-bit draft copy of BF16 w with BF16N_DRAFT_CANDIDATES candidates (default per bits)."""
    import os
    q, s = (int2_quantize if bits == 2 else int4_quantize)(w)
    env = os.environ.get("BF16N_DRAFT_CANDIDATES")
    return DraftHead(bits, q, s, int(env) if env is not None else DEFAULT_CANDIDATES[bits])


def draft_logits(h: torch.Tensor, w: Weight, head: DraftHead, vocab: int) -> torch.Tensor:
    """Draft-token logits: the k-bit head selects candidates, the gathered lossless rows are re-scored in FP32, every
    other entry is -inf. A proposal path: candidate coverage does not guarantee the exact head's argmax."""
    n, K = h.shape
    h = h.contiguous()
    cand = head.scores(h).topk(head.candidates, dim=-1).indices                   # [n, C]
    rows = get_rows(cand.reshape(-1), w).view(n, head.candidates, K)              # exact BF16 rows
    exact = torch.einsum("nck,nk->nc", rows.float(), h.float())
    out = torch.full((n, vocab), float("-inf"), dtype=torch.float32, device=h.device)
    return out.scatter_(1, cand, exact)


# ------------------------------------------------------------------ device: MoE

def mm_ids_supported(w: Weight, up: Weight | None = None) -> bool:
    cw = w.c()
    cu = up.c() if up is not None else None
    return bool(lib().bf16n_mm_ids_supported(C.byref(cw), C.byref(cu) if cu is not None else None))


def mm_ids_workspace_bytes(w: Weight, up: Weight | None = None) -> int:
    """Bytes of workspace the two-pass batched product needs for this matrix (or gate/up pair); 0: not taken."""
    cw = w.c()
    cu = up.c() if up is not None else None
    return int(lib().bf16n_mm_ids_workspace_bytes(C.byref(cw), C.byref(cu) if cu is not None else None))


_workspace: torch.Tensor | None = None


def set_workspace(buf: torch.Tensor | None) -> None:
    """Registers a device buffer (uint8, kept alive here) for the two-pass form of the batched product: with it,
    moe_mm_ids / moe_experts on lane-major pair-Huffman experts decode into BF16 operand tiles first and multiply from
    them on the tensor cores. None withdraws it (the fused decode-and-multiply kernel runs again)."""
    global _workspace
    if buf is None:
        check(lib().bf16n_set_workspace(None, 0))
        _workspace = None
        return
    if not buf.is_cuda or buf.dtype != torch.uint8 or not buf.is_contiguous():
        raise RuntimeError("bf16n.set_workspace: a contiguous uint8 CUDA tensor")
    off = (-buf.data_ptr()) % 1024
    if buf.numel() <= off:
        raise RuntimeError("bf16n.set_workspace: buffer too small")
    check(lib().bf16n_set_workspace(buf.data_ptr() + off, buf.numel() - off))
    _workspace = buf


_auto_workspace = False


def set_auto_workspace(on: bool) -> None:
    """With on = True, moe_mm_ids (and so moe_experts and torch.ops.bf16n.moe_mm_ids) grows the registered workspace to
    what its matrices need before it launches, unless the stream is being captured (a capture never allocates: it uses
    the workspace registered before it, or the fused kernel). Off by default: the reference's operators allocate only
    their outputs."""
    global _auto_workspace
    _auto_workspace = bool(on)


def ensure_workspace(*pairs) -> int:
    """Grows the registered workspace to what the given (w, up) pairs need; returns its size in bytes."""
    need = max((mm_ids_workspace_bytes(w, up) for w, up in pairs), default=0)
    have = 0 if _workspace is None else _workspace.numel() - (-_workspace.data_ptr()) % 1024
    if need > have:
        dev = pairs[0][0].plane.device
        set_workspace(None)
        set_workspace(torch.empty(need + 1024, dtype=torch.uint8, device=dev))
        have = need
    return have


def moe_route(topk_ids: torch.Tensor, n_experts: int, per_slot: bool):
    """Routing sort on the GPU: (ids_src1, ids_dst, bounds) int32 device tensors."""
    _check_ids(topk_ids)
    T, n_used = topk_ids.shape
    dev = topk_ids.device
    src1 = torch.empty(T * n_used, dtype=torch.int32, device=dev)
    dst = torch.empty(T * n_used, dtype=torch.int32, device=dev)
    bounds = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    ny = n_used if per_slot else 1
    with torch.cuda.device(dev):
        check(lib().bf16n_mm_ids_route(topk_ids.data_ptr(), int(topk_ids.dtype == torch.int64), topk_ids.stride(0),
                                       src1.data_ptr(), dst.data_ptr(), bounds.data_ptr(), n_experts, T, n_used, ny, ny,
                                       _stream()))
    return src1, dst, bounds


def moe_mm_ids(x: torch.Tensor, topk_ids: torch.Tensor, w: Weight, n_experts: int, up: Weight | None = None,
               out_dtype: torch.dtype = torch.float32, route=None) -> torch.Tensor:
    """Batched routed product (more than 8 tokens). route: the (ids_src1, ids_dst, bounds) of moe_route for these ids and
    this activation layout, when the caller already has them (moe_experts sorts once for both of its products)."""
    cw = w.c()
    cu = up.c() if up is not None else None
    _check_ids(topk_ids)
    _check_x(x, w.meta.K)
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise RuntimeError("bf16n.moe_mm_ids: x must be contiguous bf16")
    if n_experts <= 0 or w.meta.rows % n_experts:
        raise RuntimeError("bf16n.moe_mm_ids: rows must split into n_experts")
    T, n_used = topk_ids.shape
    N = w.meta.rows // n_experts
    per_slot = x.dim() == 3
    if not ((x.dim() == 2 and x.shape[0] == T) or (per_slot and x.shape[0] == T and x.shape[1] == n_used)):
        raise RuntimeError("bf16n.moe_mm_ids: x must be [tokens, K] or [tokens, n_used, K]")
    y = torch.empty((T, n_used, N), dtype=out_dtype, device=x.device)
    if T == 0:
        return y
    if not lib().bf16n_mm_ids_supported(C.byref(cw), C.byref(cu) if cu is not None else None):
        raise ValueError("bf16n.moe_mm_ids: no batched kernel for this matrix (format/K/R/layout)")
    src1, dst, bounds = moe_route(topk_ids, n_experts, per_slot) if route is None else route
    if _auto_workspace and not torch.cuda.is_current_stream_capturing():
        ensure_workspace((w, up))
    with torch.cuda.device(x.device):
        check(lib().bf16n_mm_ids(C.byref(cw), C.byref(cu) if cu is not None else None, x.data_ptr(), w.meta.K,
                                 src1.data_ptr(), dst.data_ptr(), bounds.data_ptr(), y.data_ptr(),
                                 int(out_dtype == torch.bfloat16), N, n_experts, T, n_used, _stream()))
    return y


def moe_combine(ys: torch.Tensor, topk_weights: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    if not (ys.is_cuda and ys.dim() == 3 and ys.dtype == torch.float32 and ys.is_contiguous()):
        raise RuntimeError("bf16n.moe_combine: ys must be contiguous f32 [tokens, n_used, N]")
    if not (topk_weights.is_cuda and topk_weights.dim() == 2 and topk_weights.is_contiguous()
            and topk_weights.dtype in (torch.float32, torch.bfloat16)):
        raise RuntimeError("bf16n.moe_combine: topk_weights must be contiguous f32/bf16 [tokens, n_used]")
    T, n_used, N = ys.shape
    if tuple(topk_weights.shape) != (T, n_used):
        raise RuntimeError("bf16n.moe_combine: shape mismatch")
    y = torch.empty((T, N), dtype=out_dtype, device=ys.device)
    with torch.cuda.device(ys.device):
        check(lib().bf16n_moe_combine(ys.data_ptr(), topk_weights.data_ptr(), int(topk_weights.dtype == torch.bfloat16),
                                      y.data_ptr(), int(out_dtype == torch.bfloat16), T, n_used, N, _stream()))
    return y


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    if not (g.is_cuda and g.dtype == torch.float32 and g.is_contiguous() and u.shape == g.shape
            and u.dtype == torch.float32 and u.is_contiguous()):
        raise RuntimeError("bf16n.swiglu: g and u must be contiguous f32 of one shape")
    y = torch.empty_like(g)
    with torch.cuda.device(g.device):
        check(lib().bf16n_swiglu(g.data_ptr(), u.data_ptr(), y.data_ptr(), g.numel(), _stream()))
    return y


def moe_topk(router_logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Router on the GPU: softmax over the experts, the k largest per token (ties: lowest index), weights renormalised
    to sum 1. Returns (topk_weights f32 [T, k], topk_ids int32 [T, k])."""
    if not (router_logits.is_cuda and router_logits.dim() == 2 and router_logits.dtype == torch.float32
            and router_logits.is_contiguous()):
        raise RuntimeError("bf16n.moe_topk: router_logits must be contiguous f32 [tokens, n_experts]")
    T, E = router_logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=router_logits.device)
    wts = torch.empty((T, k), dtype=torch.float32, device=router_logits.device)
    with torch.cuda.device(router_logits.device):
        check(lib().bf16n_moe_topk(router_logits.data_ptr(), T, E, k, ids.data_ptr(), wts.data_ptr(), _stream()))
    return wts, ids


def moe_experts(x: torch.Tensor, gate: Weight, up: Weight, down: Weight, topk_weights: torch.Tensor,
                topk_ids: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Routed experts of one MoE layer: sum_k w_k * down(silu(gate x) * up x) over the top-k experts, BF16 out.
    Up to 8 tokens (or shapes without a batched kernel): expert GEMVs with FP32 activations between them; more: the
    batched kernels (fused gate/up + SwiGLU written as BF16, then down in FP32)."""
    T = x.shape[0]
    N = gate.meta.rows // n_experts
    H = down.meta.rows // n_experts
    x = x.contiguous()
    if T > GEMV_MAX_TOKENS and mm_ids_supported(gate, up) and mm_ids_supported(down):
        # one routing sort serves both products: with one activation row per (token, slot) a pair's source row is its
        # destination row, so the down product reads ids_dst in both roles
        src1, dst, bounds = moe_route(topk_ids, n_experts, False)
        a = moe_mm_ids(x, topk_ids, gate, n_experts, up=up, out_dtype=torch.bfloat16, route=(src1, dst, bounds))
        ys = moe_mm_ids(a, topk_ids, down, n_experts, out_dtype=torch.float32, route=(dst, dst, bounds))
    else:
        g = mmv(x, gate, topk_ids, N)
        u = mmv(x, up, topk_ids, N)
        ys = mmv(swiglu(g, u), down, topk_ids, H)
    return moe_combine(ys, topk_weights, torch.bfloat16)


def moe_decode_scratch(n_tok: int, n_used: int, gate: Weight, down: Weight, n_experts_local: int, device) -> torch.Tensor:
    """Scratch buffer for moe_decode (gate, up and per-slot down outputs, FP32)."""
    n = lib().bf16n_moe_decode_scratch_bytes(n_tok, n_used, gate.meta.rows // n_experts_local, down.meta.rows // n_experts_local)
    return torch.empty(max(n, 16) // 4, dtype=torch.float32, device=device)


def moe_decode(x: torch.Tensor, gate: Weight, up: Weight, down: Weight, n_experts: int, top_k: int, *,
               router_logits: torch.Tensor | None = None, topk_weights: torch.Tensor | None = None,
               topk_ids: torch.Tensor | None = None, expert_lo: int = 0, n_experts_local: int | None = None,
               scratch: torch.Tensor | None = None, out: torch.Tensor | None = None,
               out_dtype: torch.dtype = torch.float32, peers=None):
    """One MoE decode step of the routed experts in four launches (router, gate+up, down with SwiGLU on load,
    combine). Either router_logits (FP32 [T, n_experts]) or topk_weights / topk_ids (FP32 / int32 [T, top_k]) is given.
    The weights hold experts [expert_lo, expert_lo + n_experts_local); other slots add zeros (expert parallelism).
    peers (a bf16n_peer_out): the combine also stores y into the peers' exchange buffers and announces it.
    Returns (y [T, H], topk_weights, topk_ids)."""
    cg, cu, cd = gate.c(), up.c(), down.c()
    _check_x(x, gate.meta.K)
    if x.dim() != 2:
        raise RuntimeError("bf16n.moe_decode: x must be [tokens, K]")
    T = x.shape[0]
    n_local = n_experts if n_experts_local is None else n_experts_local
    H = down.meta.rows // n_local
    dev = x.device
    if router_logits is not None:
        if not (router_logits.is_cuda and router_logits.dtype == torch.float32 and router_logits.is_contiguous()
                and tuple(router_logits.shape) == (T, n_experts)):
            raise RuntimeError("bf16n.moe_decode: router_logits must be contiguous f32 [tokens, n_experts]")
        topk_ids = torch.empty((T, top_k), dtype=torch.int32, device=dev) if topk_ids is None else topk_ids
        topk_weights = torch.empty((T, top_k), dtype=torch.float32, device=dev) if topk_weights is None else topk_weights
    if not (topk_ids is not None and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
            and topk_weights is not None and topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()):
        raise RuntimeError("bf16n.moe_decode: topk_ids int32 / topk_weights f32, contiguous [tokens, top_k]")
    if scratch is None:
        scratch = moe_decode_scratch(T, top_k, gate, down, n_local, dev)
    elif not (scratch.is_cuda and scratch.device == dev and scratch.dtype == torch.float32 and scratch.is_contiguous()):
        raise RuntimeError("bf16n.moe_decode: scratch must be a contiguous f32 CUDA tensor on the weights' device")
    if topk_ids.device != dev or topk_weights.device != dev or tuple(topk_ids.shape) != (T, top_k) or tuple(topk_weights.shape) != (T, top_k):
        raise RuntimeError("bf16n.moe_decode: topk_ids / topk_weights must be [tokens, top_k] on the weights' device")
    if out is None:
        y = torch.empty((T, H), dtype=out_dtype, device=dev)
    else:
        y = out
        if _check_out(out, (T, H), out.dtype, dev, "moe_decode") != H * out.element_size() and T > 1:
            raise RuntimeError("bf16n.moe_decode: out must be contiguous")
        if out.dtype not in (torch.float32, torch.bfloat16) or out.device.type != "cuda":
            raise RuntimeError("bf16n.moe_decode: out must be an f32 or bf16 CUDA tensor")
    args = (C.byref(cg), C.byref(cu), C.byref(cd), x.data_ptr(), int(x.dtype == torch.bfloat16), x.stride(0) * x.element_size(),
            router_logits.data_ptr() if router_logits is not None else None, n_experts, topk_ids.data_ptr(), topk_weights.data_ptr(),
            T, top_k, expert_lo, n_local, scratch.data_ptr(), scratch.numel() * 4, y.data_ptr(), int(y.dtype == torch.bfloat16))
    with torch.cuda.device(dev):
        if peers is None:
            check(lib().bf16n_moe_decode(*args, _stream()))
        else:
            check(lib().bf16n_moe_decode_peers(*args, C.byref(peers), _stream()))
    return y, topk_weights, topk_ids
