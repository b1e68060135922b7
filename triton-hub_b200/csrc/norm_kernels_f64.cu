// Kernel instantiations for f64 storage.
#define B200NORM_T double
#define B200NORM_GETTER kernels_f64
#include "norm_kernels.inc"
