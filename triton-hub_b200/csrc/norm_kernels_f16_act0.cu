// Kernel instantiations for f16 storage, fused activation 0 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T __half
#define B200NORM_ACT 0
#define B200NORM_GETTER kernels_f16_act0
#include "norm_kernels.inc"
