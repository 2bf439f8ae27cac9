// fp64 instantiation of the fused compute + communication kernels (fused_impl.cuh): the reference's value type
// (real_t = double, src/basic.hpp:17).  Vectors are double2 (16 bytes), so a dense row of k/Z values is k/Z / 2
// vectors; the in-switch (multimem) Z reduction is built for fp32 only.
#define SP3_FUSED_T double
#define SP3_FUSED_NS fused_f64
#define SP3_FUSED_SUFFIX f64
#define SP3_FUSED_IS_F32 0
#include "fused_impl.cuh"
