// TEST INFRASTRUCTURE ONLY.  Translation unit that compiles the reference's own grouped-affine CUDA kernels,
// UNCHANGED, from where they lie in a talu checkout: core/src/compute/cuda/kernels/ops/common_decode.cuh and
// ops/quant_ops.cu (talu_gaffine_u4_matvec_f32, :46-93; the fused _qkv_ :127-219 and _gate_up_ :221-286;
// talu_embedding_lookup_gaffine_u4_f32, :12-44), in the order and with the includes of the reference's own
// aggregation unit (kernels/kernels.cu:1-13).  Built by `make -C oracle ref REF=<talu checkout>` into
// oracle/_ref/talu_ref_quant_sm_100.cubin; the parity tests load that cubin and launch it under the
// reference's launch geometry, so outputs of the reference itself pin the random-data matmul, and the
// benchmark times it as the incumbent GPU kernel.  Nothing of the reference's source is copied here.
#include <cuda_fp16.h>
#include <stdint.h>

#include "ops/common_decode.cuh"
#include "ops/quant_ops.cu"
