// Kernel instantiations for f32 storage, fused activation 0 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T float
#define B200NORM_ACT 0
#define B200NORM_GETTER kernels_f32_act0
#include "norm_kernels.inc"
