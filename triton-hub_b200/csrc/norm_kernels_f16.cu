// Kernel instantiations for f16 storage.
#define B200NORM_T __half
#define B200NORM_GETTER kernels_f16
#include "norm_kernels.inc"
