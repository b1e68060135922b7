// Softmax / LogSoftmax kernel instantiations for f16 storage.
#define B200NORM_T __half
#define B200NORM_GETTER softmax_kernels_f16
#include "softmax_kernels.inc"
