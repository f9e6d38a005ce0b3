// Second build of the tensor-core intra-chunk kernels, for heads with at most 4 dimension groups
// (the calibrated assets of the reference use 2-5 groups per head): the same sources with the
// compiled group bound lowered, which shrinks the per-pair combine and the operand images.
#define OAL_IG 4
#define OAL_INTRA_NAME(name) name##_g4
#include "oal_intra.cu"
#include "oal_intra_bwd.cu"
