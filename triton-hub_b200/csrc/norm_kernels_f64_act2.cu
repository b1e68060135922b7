// Kernel instantiations for f64 storage, fused activation 2 (0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_T double
#define B200NORM_ACT 2
#define B200NORM_GETTER kernels_f64_act2
#include "norm_kernels.inc"
