// p-norm / normalize kernel instantiations for f32 storage.
#define B200NORM_T float
#define B200NORM_GETTER pnorm_kernels_f32
#include "pnorm_kernels.inc"
