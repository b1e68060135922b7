// Kernel instantiations for f16 storage, fused activation 2 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T __half
#define B200NORM_ACT 2
#define B200NORM_GETTER kernels_f16_act2
#include "norm_kernels.inc"
