"""numpy front end of the BF16N CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline / reference arm import this module; the library package
never does.  It loads

* ``libbf16n_oracle.so``  - the CPU restatement of the reference algorithm (bf16n_oracle.cpp), and
* ``_ref/libbf16n_ref.so`` - the reference project's own encoder and shape policy compiled from its sources
  (ref_shim.cpp + Makefile), when that build is present,

and adds the numpy-level oracles that need no C: the shape policy (core/src/policy.cpp:9-69), the routing helper
(core/src/mmid_helper.cu:49-136 semantics), softmax top-k, and the FP64 MoE layer
(engines/vllm/vllm_bf16n/ops.py:274-288 semantics).
"""
from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
FMT_NIBBLE, FMT_HUFFMAN, FMT_HUFPAIR = 1, 2, 3
FLAG_CHUNK_MAJOR, FLAG_FRAG_ORDER = 1, 2
HEADER = struct.Struct("<IIIIQQQQQQQII")  # core/include/bf16n/format.h:41-47
MAGIC = 0x4E363142

_u8p = C.POINTER(C.c_uint8)


def reference_checkout() -> str | None:
    """Where the reference project's sources lie: $BF16N_REFERENCE, else a directory named `reference` beside this
    repository; None when neither holds core/src/encode.cpp (then a prebuilt oracle/_ref is used if present)."""
    for cand in (os.environ.get("BF16N_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "core", "src", "encode.cpp")):
            return cand
    return None


def build() -> None:
    """Compile the oracle (and, where the reference checkout exists, oracle/_ref) with the Makefile beside this file."""
    ref = reference_checkout()
    subprocess.run(["make", "-s", "-C", HERE] + ([f"REF={ref}"] if ref else []), check=True, stdout=subprocess.DEVNULL)


def _load(path: str):
    return C.CDLL(path) if os.path.exists(path) else None


_orc = None
_ref = None


def orc():
    global _orc
    if _orc is None:
        p = os.path.join(HERE, "libbf16n_oracle.so")
        if not os.path.exists(p):
            build()
        _orc = C.CDLL(p)
        _orc.orc_encode.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                    C.POINTER(_u8p), C.POINTER(C.c_uint64), C.POINTER(C.c_int)]
        _orc.orc_free.argtypes = [C.c_void_p]
        _orc.orc_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        _orc.orc_gemv_f64.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        _orc.orc_gemv_f32_order.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int,
                                            C.c_void_p, C.c_void_p]
        _orc.orc_decode_gemv_mt.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int]
    return _orc


def ref():
    """The reference's own encoder/policy (None when oracle/_ref was not built)."""
    global _ref
    if _ref is None:
        _ref = _load(os.path.join(HERE, "_ref", "libbf16n_ref.so"))
        if _ref is not None:
            _ref.ref_encode.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                        C.POINTER(_u8p), C.POINTER(C.c_uint64), C.POINTER(C.c_int), C.POINTER(C.c_int)]
            _ref.ref_free.argtypes = [C.c_void_p]
            _ref.ref_choose.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int,
                                        C.POINTER(C.c_int)]
    return _ref


def have_ref() -> bool:
    return ref() is not None


# ------------------------------------------------------------------ data

def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns (uint16)."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def weights_like(rows: int, K: int, seed: int, outliers: bool = False) -> np.ndarray:
    """Seeded N(0, 0.02) weights rounded to BF16 (uint16 bits, rows x K). outliers: 1e-4 of entries x50, the
    reference's model-like fixture (tests/conftest.py:28-34)."""
    g = np.random.default_rng(seed)
    w = g.standard_normal((rows, K), dtype=np.float32) * np.float32(0.02)
    if outliers:
        m = g.random((rows, K)) < 1e-4
        w = np.where(m, w * np.float32(50.0), w).astype(np.float32)
    return f32_to_bf16_bits(w)


SPECIALS = np.array([0x0000, 0x8000, 0x0001, 0x807F, 0x7F7F, 0xFF7F, 0x7F80, 0xFF80, 0x7FC1, 0xFFFF, 0x3F80],
                    dtype=np.uint16)  # zeros, subnormals, max finite, infinities, NaNs, 1.0 (test_encode.cpp:181)


def with_specials(w: np.ndarray, seed: int, reps: int = 4) -> np.ndarray:
    g = np.random.default_rng(seed ^ 0x5EC1A1)
    w = w.copy().reshape(-1)
    for _ in range(reps):
        w[g.integers(0, w.size, SPECIALS.size)] = SPECIALS
    return w


def with_pairs(rows: int, K: int, n: int) -> np.ndarray:
    """rows x K weights whose (even, odd) exponent pairs take exactly n distinct values (test_encode.cpp:221-229)."""
    p = (np.arange(rows * K // 2) % n).astype(np.uint32)
    w = np.zeros(rows * K, dtype=np.uint16)
    w[0::2] = ((p & 0xFF) << 7).astype(np.uint16)
    w[1::2] = ((p >> 8) << 7).astype(np.uint16)
    return w.reshape(rows, K)


# ------------------------------------------------------------------ encode / decode

@dataclass(frozen=True)
class Hdr:
    magic: int
    format: int
    K: int
    R: int
    rows: int
    off_a: int
    off_b: int
    off_c: int
    off_d: int
    n_a: int
    n_b: int
    flags: int


def parse_header(aux: np.ndarray) -> Hdr:
    f = HEADER.unpack(bytes(aux[: HEADER.size]))
    return Hdr(*f[:12])


def _encode_with(fn, free, w, fmt, R, cm, fo, extra_out=False):
    w = np.ascontiguousarray(w, dtype=np.uint16)
    K = w.shape[-1]
    rows = w.size // K if K else 0
    plane = np.zeros(max(rows * K, 1), dtype=np.uint8)
    aux_p, aux_n, fmt_o, r_o = _u8p(), C.c_uint64(0), C.c_int(0), C.c_int(0)
    args = [w.ctypes.data, rows, K, fmt, R, int(cm), int(fo), plane.ctypes.data, C.byref(aux_p), C.byref(aux_n),
            C.byref(fmt_o)]
    if extra_out:
        args.append(C.byref(r_o))
    rc = fn(*args)
    if rc == 1:
        raise ValueError("bf16n encode: invalid argument")
    if rc != 0:
        raise RuntimeError("bf16n encode failed")
    aux = np.ctypeslib.as_array(aux_p, shape=(aux_n.value,)).copy()
    free(aux_p)
    return plane[: rows * K].reshape(rows, K), aux, fmt_o.value


def encode(w, fmt, R, cm=False, fo=False):
    """Oracle (restated) encoder: (plane u8 [rows,K], aux u8, format produced)."""
    return _encode_with(orc().orc_encode, orc().orc_free, w, fmt, R, cm, fo)


def ref_encode(w, fmt, R, cm=False, fo=False):
    """The reference's own encoder (requires oracle/_ref)."""
    return _encode_with(ref().ref_encode, ref().ref_free, w, fmt, R, cm, fo, extra_out=True)


def decode(plane: np.ndarray, aux: np.ndarray) -> np.ndarray:
    h = parse_header(aux)
    plane = np.ascontiguousarray(plane, dtype=np.uint8)
    aux = np.ascontiguousarray(aux, dtype=np.uint8)
    out = np.empty((h.rows, h.K), dtype=np.uint16)
    if orc().orc_decode(plane.ctypes.data, aux.ctypes.data, out.ctypes.data) != 0:
        raise ValueError("bf16n oracle decode: bad header")
    return out


# ------------------------------------------------------------------ products

def gemv_f64(w_bits: np.ndarray, x: np.ndarray, nthreads: int = 0):
    """y = W x in FP64 over the exact weights, and S = sum |w x| per row. x: FP32 values."""
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    rows, K = w_bits.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    y, s = np.empty(rows), np.empty(rows)
    orc().orc_gemv_f64(w_bits.ctypes.data, rows, K, x.ctypes.data, y.ctypes.data, s.ctypes.data,
                       nthreads or os.cpu_count() or 1)
    return y, s


def gemv_f32_order(w_bits: np.ndarray, x: np.ndarray, chunk_major: bool = False, esc=None) -> np.ndarray:
    """FP32 emulation of the reference kernels' summation order. esc: list of per-row escape-column lists (NIBBLE)."""
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    rows, K = w_bits.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(rows, dtype=np.float32)
    if esc is None:
        orc().orc_gemv_f32_order(w_bits.ctypes.data, rows, K, x.ctypes.data, y.ctypes.data, int(chunk_major), None, None)
    else:
        off = np.zeros(rows + 1, dtype=np.int64)
        off[1:] = np.cumsum([len(e) for e in esc])
        cols = np.ascontiguousarray(np.concatenate([np.asarray(e, dtype=np.int32) for e in esc] + [np.zeros(0, np.int32)]))
        orc().orc_gemv_f32_order(w_bits.ctypes.data, rows, K, x.ctypes.data, y.ctypes.data, int(chunk_major),
                                 cols.ctypes.data, off.ctypes.data)
    return y


def decode_gemv_mt(plane, aux, x, u0: int, u1: int, nthreads: int) -> np.ndarray:
    """The timed CPU arm: decode units [u0, u1) of a HUFPAIR matrix and multiply by x (FP32 accumulate)."""
    h = parse_header(aux)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty((u1 - u0) * h.R, dtype=np.float32)
    rc = orc().orc_decode_gemv_mt(plane.ctypes.data, aux.ctypes.data, u0, u1, x.ctypes.data, y.ctypes.data, nthreads)
    if rc:
        raise ValueError("oracle decode_gemv: unsupported header")
    return y


# ------------------------------------------------------------------ shape policy (core/src/policy.cpp:9-69)

def _dense_R(rows: int, engine: str) -> int:
    best, best_cost = 1, 0
    for r in (16, 8, 4, 2):
        if rows % r or rows // r < 512:
            continue
        units = rows // r
        cost = (units // 512 + (units % 512 != 0)) * r
        if best == 1:
            best, best_cost = r, cost
            if engine == "llama":
                break
        elif cost <= 0.95 * best_cost:
            best, best_cost = r, cost
    return best


def choose(rows, K, n_matrices=1, engine="vllm", mode="hybrid", dense_min=8 << 20, expert=False, dense_frag_order=False):
    """Restated policy: None (stays BF16) or (format, R, chunk_major, frag_order)."""
    if rows <= 0 or n_matrices <= 0 or K <= 0 or K % 512 or K > 4096:
        return None
    is_expert = expert if engine == "llama" else n_matrices > 1

    def at_least(threshold):
        if threshold <= 0:
            return True
        per = -(-threshold // n_matrices)
        return rows >= -(-per // K)

    if mode == "nibble" or (mode == "hybrid" and not is_expert and not at_least(dense_min)):
        return (FMT_NIBBLE, 0, False, False)
    fo_dense = engine == "vllm" and dense_frag_order and n_matrices == 1 and rows % 16 == 0
    fo_gate_up = engine == "vllm" and n_matrices > 1 and K == 2048 and rows % 16 == 0
    if n_matrices > 1:
        R = 16 if (fo_gate_up or (rows % 16 == 0 and rows >= 2048)) else 8 if rows % 8 == 0 else 4 if rows % 4 == 0 else 1
    else:
        R = 16 if fo_dense else _dense_R(rows, engine)
    fo_experts = fo_gate_up or (engine == "vllm" and n_matrices > 1 and K == 512 and R == 16)
    return (FMT_HUFPAIR, R, n_matrices > 1 and K > 512 and not fo_experts, fo_experts or fo_dense)


def ref_choose(rows, K, n_matrices=1, engine="vllm", mode="hybrid", dense_min=8 << 20, expert=False, dense_frag_order=False):
    out = (C.c_int * 4)()
    ok = ref().ref_choose(rows, K, n_matrices, int(engine == "vllm"), {"hybrid": 0, "huffman": 1, "nibble": 2}[mode],
                          dense_min, int(expert), int(dense_frag_order), out)
    return (out[0], out[1], bool(out[2]), bool(out[3])) if ok else None


# ------------------------------------------------------------------ MoE oracles (numpy)

def softmax_topk(logits: np.ndarray, k: int):
    """softmax over experts, the k largest (ties: lowest index first), weights renormalised to sum 1. FP64."""
    z = logits.astype(np.float64)
    p = np.exp(z - z.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    order = np.argsort(-p, axis=-1, kind="stable")[:, :k]
    w = np.take_along_axis(p, order, axis=-1)
    return order.astype(np.int32), w / w.sum(axis=-1, keepdims=True)


def route(ids: np.ndarray, n_experts: int, nchannels_y: int, sis1: int):
    """Routing helper semantics (core/src/mmid_helper.cu:4-8,117-135): (token, slot) pairs sorted by expert, then by
    token; ids_src1[j] = token*sis1 + slot % nchannels_y, ids_dst[j] = token*n_used + slot, bounds = prefix counts."""
    n_tok, n_used = ids.shape
    src1, dst, bounds = [], [], [0]
    for e in range(n_experts):
        for t in range(n_tok):
            for s in range(n_used):
                if ids[t, s] == e:
                    src1.append(t * sis1 + s % nchannels_y)
                    dst.append(t * n_used + s)
                    break  # one slot per (token, expert): experts of a token are distinct
        bounds.append(len(dst))
    return np.array(src1, np.int32), np.array(dst, np.int32), np.array(bounds, np.int32)


def silu(v):
    return v / (1.0 + np.exp(-v))


def moe_layer_f64(x, gate_bits, up_bits, down_bits, topk_w, topk_ids, n_experts, bf16_act=False):
    """sum_k w_k * down_e(silu(gate_e x) * up_e x) in FP64 over exact weights. x FP32 [T,H]; *_bits uint16
    [n_experts*rows, K]. bf16_act: round the SwiGLU activation to BF16 first (the batched path stores it as BF16,
    engines/vllm/vllm_bf16n/ops.py:264-266)."""
    T = x.shape[0]
    N = gate_bits.shape[0] // n_experts
    H = down_bits.shape[0] // n_experts
    out = np.zeros((T, H))
    xd = x.astype(np.float64)
    for t in range(T):
        for s in range(topk_ids.shape[1]):
            e = int(topk_ids[t, s])
            g = bf16_bits_to_f32(gate_bits[e * N:(e + 1) * N]).astype(np.float64) @ xd[t]
            u = bf16_bits_to_f32(up_bits[e * N:(e + 1) * N]).astype(np.float64) @ xd[t]
            a = silu(g) * u
            if bf16_act:
                a = bf16_bits_to_f32(f32_to_bf16_bits(a.astype(np.float32))).astype(np.float64)
            out[t] += float(topk_w[t, s]) * (bf16_bits_to_f32(down_bits[e * H:(e + 1) * H]).astype(np.float64) @ a)
    return out
