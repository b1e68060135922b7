// Softmax / LogSoftmax kernel instantiations for f64 storage.
#define B200NORM_T double
#define B200NORM_GETTER softmax_kernels_f64
#include "softmax_kernels.inc"
