// Kernel instantiations for f32 storage, fused activation 1 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T float
#define B200NORM_ACT 1
#define B200NORM_GETTER kernels_f32_act1
#include "norm_kernels.inc"
