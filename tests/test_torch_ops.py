"""`torch.ops.bf16n` on the CPU: the library registers the reference's schemas (core/torch/torch_bindings.cpp:373-388),
the CPU `encode` op returns the encoder's bytes, its fake implementation traces, and metadata lists round-trip."""
import pytest
import torch

from conftest import to_bf16_tensor
from oracle import cpu_oracle as o

HP = 3


@pytest.fixture(scope="module")
def b():
    from orin_qwen_lossless_b200 import torch_ops  # noqa: F401  (registers the library)
    return torch.ops.bf16n


def test_schemas_match_the_reference(b):
    want = {
        "init": "bf16n::init() -> ()",
        "encode": "bf16n::encode(Tensor w, int format, int R, bool chunk_major, bool frag_order=False) -> (Tensor, Tensor)",
        "dequant": "bf16n::dequant(Tensor plane, Tensor aux, int[] meta, int row0, int nrows) -> Tensor",
        "mmv": "bf16n::mmv(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? ids, int rows_per_matrix, bool out_bf16) -> Tensor",
        "mmv_glu": "bf16n::mmv_glu(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? ids, int rows_per_matrix, bool out_bf16) -> Tensor",
        "linear": "bf16n::linear(Tensor x, Tensor plane, Tensor aux, int[] meta, Tensor? bias) -> Tensor",
        "get_rows": "bf16n::get_rows(Tensor ids, Tensor plane, Tensor aux, int[] meta, bool out_bf16) -> Tensor",
        "moe_mm_ids": "bf16n::moe_mm_ids(Tensor x, Tensor topk_ids, Tensor plane, Tensor aux, int[] meta, Tensor? up_plane, "
                      "Tensor? up_aux, int[] up_meta, int n_experts, bool out_bf16) -> Tensor",
        "moe_combine": "bf16n::moe_combine(Tensor ys, Tensor topk_weights, bool out_bf16) -> Tensor",
        "swiglu": "bf16n::swiglu(Tensor g, Tensor u) -> Tensor",
        "int4_quantize": "bf16n::int4_quantize(Tensor w) -> (Tensor, Tensor)",
        "int4_gemv": "bf16n::int4_gemv(Tensor x, Tensor q, Tensor s) -> Tensor",
        "int2_quantize": "bf16n::int2_quantize(Tensor w) -> (Tensor, Tensor)",
        "int2_gemv": "bf16n::int2_gemv(Tensor x, Tensor q, Tensor s) -> Tensor",
    }
    for name, schema in want.items():
        assert str(getattr(b, name).default._schema) == schema


def test_encode_op_returns_the_encoder_bytes(b):
    from orin_qwen_lossless_b200 import ops
    w = to_bf16_tensor(o.weights_like(64, 1024, 5))
    plane, aux = b.encode(w, HP, 8, True)
    p2, a2, meta = ops.encode(w, HP, 8, True)
    assert torch.equal(plane, p2) and torch.equal(aux, a2)
    assert ops.parse_header(aux).as_list() == meta.as_list() and len(meta.as_list()) == 9


def test_encode_opcheck(b):
    w = to_bf16_tensor(o.weights_like(16, 512, 6))
    torch.library.opcheck(b.encode, (w, HP, 8, False), test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))


def test_encode_op_keeps_the_reference_errors(b):
    w = to_bf16_tensor(o.weights_like(16, 512, 7))
    with pytest.raises(ValueError, match="multiple of R"):
        b.encode(w[:12], HP, 8, False)
    with pytest.raises(RuntimeError, match="bfloat16"):
        b.encode(w.float(), HP, 8, False)
