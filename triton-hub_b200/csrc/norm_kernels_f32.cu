// Kernel instantiations for f32 storage.
#define B200NORM_T float
#define B200NORM_GETTER kernels_f32
#include "norm_kernels.inc"
