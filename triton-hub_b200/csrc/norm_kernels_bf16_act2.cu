// Kernel instantiations for bf16 storage, fused activation 2 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T __nv_bfloat16
#define B200NORM_ACT 2
#define B200NORM_GETTER kernels_bf16_act2
#include "norm_kernels.inc"
