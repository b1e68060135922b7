// Softmax / LogSoftmax kernel instantiations for f32 storage.
#define B200NORM_T float
#define B200NORM_GETTER softmax_kernels_f32
#include "softmax_kernels.inc"
