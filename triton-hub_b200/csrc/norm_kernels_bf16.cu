// Kernel instantiations for bf16 storage.
#define B200NORM_T __nv_bfloat16
#define B200NORM_GETTER kernels_bf16
#include "norm_kernels.inc"
