// p-norm / normalize kernel instantiations for f16 storage.
#define B200NORM_T __half
#define B200NORM_GETTER pnorm_kernels_f16
#include "pnorm_kernels.inc"
