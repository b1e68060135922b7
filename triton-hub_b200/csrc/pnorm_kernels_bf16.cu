// p-norm / normalize kernel instantiations for bf16 storage.
#define B200NORM_T __nv_bfloat16
#define B200NORM_GETTER pnorm_kernels_bf16
#include "pnorm_kernels.inc"
