"""`torch.ops.bf16n.*`: the operator surface the reference registers from C++ (core/torch/torch_bindings.cpp:373-403),
registered here with `torch.library` on top of the C ABI, so that code written against the reference's ops (its vLLM
plugin, its tests) finds the same names, schemas, argument meaning and error types.

Schemas are the reference's, character for character, for all fourteen ops: init, encode, dequant, mmv, mmv_glu,
linear, get_rows, moe_mm_ids, moe_combine, swiglu and the draft-head ops int4_quantize, int4_gemv, int2_quantize,
int2_gemv. `int[] meta` is [format, K, rows, R, flags, off_a, off_b, off_c, off_d] (torch_bindings.cpp:7). Fake (meta)
implementations follow vllm_bf16n/ops.py:292-369 so that the ops trace under torch.compile.

Importing this module registers the library once per process; it does not initialise CUDA.
"""
from __future__ import annotations

import torch

from . import ops

_SCHEMAS = (
    "init() -> ()",
    "encode(Tensor w, int format, int R, bool chunk_major, bool frag_order=False) -> (Tensor, Tensor)",
    "dequant(Tensor plane, Tensor aux, int[] meta, int row0, int nrows) -> Tensor",
    "mmv(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? ids, int rows_per_matrix, bool out_bf16) -> Tensor",
    "mmv_glu(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? ids, int rows_per_matrix, bool out_bf16) -> Tensor",
    "linear(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? bias) -> Tensor",
    "get_rows(Tensor ids, Tensor plane, Tensor aux, int[] meta, bool out_bf16) -> Tensor",
    "moe_mm_ids(Tensor x, Tensor topk_ids, Tensor plane, Tensor aux, int[] meta, Tensor? up_plane, Tensor? up_aux, "
    "int[] up_meta, int n_experts, bool out_bf16) -> Tensor",
    "moe_combine(Tensor ys, Tensor topk_weights, bool out_bf16) -> Tensor",
    "swiglu(Tensor g, Tensor u) -> Tensor",
    "int4_quantize(Tensor w) -> (Tensor, Tensor)",
    "int4_gemv(Tensor x, Tensor q, Tensor s) -> Tensor",
    "int2_quantize(Tensor w) -> (Tensor, Tensor)",
    "int2_gemv(Tensor x, Tensor q, Tensor s) -> Tensor",
)

_lib = torch.library.Library("bf16n", "DEF")
for _s in _SCHEMAS:
    _lib.define(_s)


def _weight(plane: torch.Tensor, aux: torch.Tensor, meta) -> ops.Weight:
    """The (plane, aux, meta list) triple of the op schemas as a Weight (torch_bindings.cpp:31-56: nine integers)."""
    if len(meta) != 9:
        raise ValueError("bf16n: meta must be [format, K, rows, R, flags, off_a, off_b, off_c, off_d]")
    fmt, K, rows, R, flags, a, b, c, d = (int(v) for v in meta)
    return ops.Weight(plane, aux, ops.Meta(fmt, K, rows, R, bool(flags & ops.FLAG_CHUNK_MAJOR), bool(flags & ops.FLAG_FRAG_ORDER),
                                           a, b, c, d))


def _dt(out_bf16: bool) -> torch.dtype:
    return torch.bfloat16 if out_bf16 else torch.float32


# ------------------------------------------------------------------ implementations

def _init():
    ops.init()


def _encode_cpu(w, format, R, chunk_major, frag_order=False):
    plane, aux, _ = ops.encode(w, format, R, chunk_major, frag_order)
    return plane, aux


def _dequant(plane, aux, meta, row0, nrows):
    return ops.dequant(_weight(plane, aux, meta), row0, nrows)


def _mmv(x, plane, aux, meta, ids, rows_per_matrix, out_bf16):
    return ops.mmv(x, _weight(plane, aux, meta), ids, rows_per_matrix, _dt(out_bf16))


def _mmv_glu(x, plane, aux, meta, ids, rows_per_matrix, out_bf16):
    return ops.mmv_glu(x, _weight(plane, aux, meta), ids, rows_per_matrix, _dt(out_bf16))


def _linear(x, plane, aux, meta, bias):
    return ops.linear(x, _weight(plane, aux, meta), bias)


def _get_rows(ids, plane, aux, meta, out_bf16):
    return ops.get_rows(ids, _weight(plane, aux, meta), _dt(out_bf16))


def _moe_mm_ids(x, topk_ids, plane, aux, meta, up_plane, up_aux, up_meta, n_experts, out_bf16):
    up = _weight(up_plane, up_aux, up_meta) if up_plane is not None else None
    return ops.moe_mm_ids(x, topk_ids, _weight(plane, aux, meta), n_experts, up, _dt(out_bf16))


def _moe_combine(ys, topk_weights, out_bf16):
    return ops.moe_combine(ys, topk_weights, _dt(out_bf16))


def _swiglu(g, u):
    return ops.swiglu(g, u)


_lib.impl("init", _init, "CompositeExplicitAutograd")
_lib.impl("encode", _encode_cpu, "CPU")
for _name, _fn in (("dequant", _dequant), ("mmv", _mmv), ("mmv_glu", _mmv_glu), ("linear", _linear), ("get_rows", _get_rows),
                   ("moe_mm_ids", _moe_mm_ids), ("moe_combine", _moe_combine), ("swiglu", _swiglu),
                   ("int4_quantize", ops.int4_quantize), ("int4_gemv", ops.int4_gemv), ("int2_quantize", ops.int2_quantize),
                   ("int2_gemv", ops.int2_gemv)):
    _lib.impl(_name, _fn, "CUDA")


# ------------------------------------------------------------------ fake (meta) implementations

@torch.library.register_fake("bf16n::encode")
def _encode_fake(w, format, R, chunk_major, frag_order=False):
    ctx = torch.library.get_ctx()
    K = w.shape[-1]
    rows = w.numel() // K
    return w.new_empty((rows, K), dtype=torch.uint8), w.new_empty((ctx.new_dynamic_size(),), dtype=torch.uint8)


@torch.library.register_fake("bf16n::dequant")
def _dequant_fake(plane, aux, meta, row0, nrows):
    return plane.new_empty((nrows, meta[1]), dtype=torch.bfloat16)


def _mmv_shape(x, meta, ids, rows_per_matrix, glu):
    if ids is None:
        rows = meta[2]
        return (x.shape[0], rows // 2 if glu else rows)
    return (ids.shape[0], ids.shape[1], rows_per_matrix // 2 if glu else rows_per_matrix)


@torch.library.register_fake("bf16n::mmv")
def _mmv_fake(x, plane, aux, meta, ids, rows_per_matrix, out_bf16):
    return x.new_empty(_mmv_shape(x, meta, ids, rows_per_matrix, False), dtype=_dt(out_bf16))


@torch.library.register_fake("bf16n::mmv_glu")
def _mmv_glu_fake(x, plane, aux, meta, ids, rows_per_matrix, out_bf16):
    return x.new_empty(_mmv_shape(x, meta, ids, rows_per_matrix, True), dtype=_dt(out_bf16))


@torch.library.register_fake("bf16n::linear")
def _linear_fake(x, plane, aux, meta, bias):
    return x.new_empty((*x.shape[:-1], meta[2]))


@torch.library.register_fake("bf16n::get_rows")
def _get_rows_fake(ids, plane, aux, meta, out_bf16):
    return plane.new_empty((ids.shape[0], meta[1]), dtype=_dt(out_bf16))


@torch.library.register_fake("bf16n::moe_mm_ids")
def _moe_mm_ids_fake(x, topk_ids, plane, aux, meta, up_plane, up_aux, up_meta, n_experts, out_bf16):
    return x.new_empty((topk_ids.shape[0], topk_ids.shape[1], meta[2] // n_experts), dtype=_dt(out_bf16))


@torch.library.register_fake("bf16n::moe_combine")
def _moe_combine_fake(ys, topk_weights, out_bf16):
    return ys.new_empty((ys.shape[0], ys.shape[2]), dtype=_dt(out_bf16))


@torch.library.register_fake("bf16n::swiglu")
def _swiglu_fake(g, u):
    return torch.empty_like(g)


@torch.library.register_fake("bf16n::int4_quantize")
def _int4_quantize_fake(w):
    return w.new_empty((w.shape[0], w.shape[1] // 2), dtype=torch.uint8), w.new_empty((w.shape[0], w.shape[1] // 128), dtype=torch.float32)


@torch.library.register_fake("bf16n::int2_quantize")
def _int2_quantize_fake(w):
    return w.new_empty((w.shape[0], w.shape[1] // 4), dtype=torch.uint8), w.new_empty((w.shape[0], w.shape[1] // 128), dtype=torch.float32)


@torch.library.register_fake("bf16n::int4_gemv")
def _int4_gemv_fake(x, q, s):
    return x.new_empty((x.shape[0], q.shape[0]), dtype=torch.float32)


@torch.library.register_fake("bf16n::int2_gemv")
def _int2_gemv_fake(x, q, s):
    return x.new_empty((x.shape[0], q.shape[0]), dtype=torch.float32)
