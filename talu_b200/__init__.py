"""talu_b200 - grouped-affine (gaf4 / gaf8) quantized matmul for NVIDIA B200.

Host-side mirror of the operator interface of talu's compute layer
(core/src/compute/cpu/matmul_primitives.zig:101-121, core/src/compute/cuda/
gaffine_u4_matvec.zig:19-97) on top of the C ABI in include/talu_gaf.h.
All arithmetic runs in hand-written CUDA kernels inside libtalu_gaf.so; there
is no CPU or PyTorch fallback, and importing `talu_b200.gaf` fails if the
library has not been built (`python -m talu_b200.build`).
"""
from .gaf import (  # noqa: F401
    SCALES_BF16,
    SCALES_F16,
    SHARD_COL,
    SHARD_NONE,
    SHARD_ROW,
    Context,
    GafError,
    Weight,
    dequant_f32,
    dequant_f32_host,
    embedding_lookup_f32,
    gaffine_matvec_f32,
    linear,
    linear_fixed_scratch,
    hint_next_weight,
    linear_allreduce,
    linear_bias,
    ACT_SILU,
    ACT_GELU,
    ffn_swiglu,
    linear_host,
    HostBatch,
    Batch,
    make_comm_id,
)

__all__ = [
    "Context", "Weight", "GafError", "linear", "linear_fixed_scratch", "hint_next_weight", "linear_allreduce", "linear_bias", "ACT_SILU", "ACT_GELU", "ffn_swiglu", "linear_host", "HostBatch", "Batch", "make_comm_id", "dequant_f32", "dequant_f32_host", "embedding_lookup_f32",
    "gaffine_matvec_f32", "SCALES_F16", "SCALES_BF16", "SHARD_NONE", "SHARD_COL", "SHARD_ROW",
]
