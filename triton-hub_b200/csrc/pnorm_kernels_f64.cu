// p-norm / normalize kernel instantiations for f64 storage.
#define B200NORM_T double
#define B200NORM_GETTER pnorm_kernels_f64
#include "pnorm_kernels.inc"
