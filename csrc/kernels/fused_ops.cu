// fp32 instantiation of the fused compute + communication kernels (fused_impl.cuh).
#define SP3_FUSED_T float
#define SP3_FUSED_NS fused_f32
#define SP3_FUSED_SUFFIX f32
#define SP3_FUSED_IS_F32 1
#include "fused_impl.cuh"
