"""B200 (sm_100a) implementation of the BF16N lossless weight path: host encoder and shape policy, decode-inside-GEMV
kernels, routed-MoE decode and batched-MoE prefill behind a C ABI (include/bf16n_c.h), with `ops` mirroring the
reference's Python operator interface on top of it. `import orin_qwen_lossless_b200.torch_ops` additionally registers
`torch.ops.bf16n.*` with the reference's schemas."""
from . import ops  # noqa: F401

__all__ = ["ops"]
