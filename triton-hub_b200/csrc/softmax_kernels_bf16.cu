// Softmax / LogSoftmax kernel instantiations for bf16 storage.
#define B200NORM_T __nv_bfloat16
#define B200NORM_GETTER softmax_kernels_bf16
#include "softmax_kernels.inc"
