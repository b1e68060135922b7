// GeLU, exact (erf) and tanh forms, and its derivative -- the activation that follows the norm
// in the reference's Quick Start (README.md:44-48).  Formulas: TritonHub/Activations/gelu.py:20-28
// (forward) and :67-79 (derivative).  Used fused into the norm kernels' stores / loads and by the
// stand-alone element-wise kernels below.
#pragma once

#include "norm_common.cuh"

namespace b200norm {

enum : int { kActNone = 0, kActGeluErf = 1, kActGeluTanh = 2 };

// tanh(u) as 1 - 2 / (exp(2u) + 1): the reference's (e - 1) / (e + 1) (gelu.py:24) is inf / inf
// = NaN once exp(2u) overflows (x > ~10 in fp32); this form saturates to 1 instead and agrees
// with it wherever the reference is finite.
__device__ __forceinline__ float tanh_via_exp(float u) {
  const float e = ex2_fast(u * (2.f * kLog2e));
  return fmaf(-2.f, rcp_fast(e + 1.f), 1.f);  // e = inf gives 1
}

// erf(s) for s = x / sqrt(2), from e = exp(-s*s) which the caller also needs for the Gaussian density.
// Abramowitz & Stegun 7.1.26 (five-term rational-exponential fit): absolute error <= 1.5e-7 over the
// whole line, one reciprocal, five FMAs -- a third of the instructions of the library erff, which
// matters because these kernels are otherwise limited by HBM, not by arithmetic.
__device__ __forceinline__ float erf_from_exp(float s, float e) {
  const float t = rcp_fast(fmaf(0.3275911f, fabsf(s), 1.f));
  const float poly =
      t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f + t * (-1.453152027f + t * 1.061405429f))));
  return copysignf(1.f - poly * e, s);
}

template <int ACT>
__device__ __forceinline__ float act_fwd(float x) {
  if (ACT == kActGeluErf) {
    const float s = x * 0.70710678118654752f;
    return 0.5f * x * (1.f + erf_from_exp(s, ex2_fast(x * x * (-0.5f * kLog2e))));  // gelu.py:27
  } else if (ACT == kActGeluTanh) {
    const float inner = 0.79788456080286536f * (x + 0.044715f * x * x * x);  // gelu.py:22
    return 0.5f * x * (1.f + tanh_via_exp(inner));                           // gelu.py:25
  }
  return x;
}

// d act(x) / dx
template <int ACT>
__device__ __forceinline__ float act_grad(float x) {
  if (ACT == kActGeluErf) {
    const float s = x * 0.70710678118654752f;
    const float e = ex2_fast(x * x * (-0.5f * kLog2e));                    // exp(-x^2 / 2), used twice
    const float cdf = 0.5f * (1.f + erf_from_exp(s, e));                   // gelu.py:76
    const float pdf = e * 0.39894228040143268f;                            // gelu.py:77
    return cdf + x * pdf;                                                  // gelu.py:78
  } else if (ACT == kActGeluTanh) {
    const float k = 0.79788456080286536f;
    const float th = tanh_via_exp(k * (x + 0.044715f * x * x * x));       // gelu.py:69-71
    const float gp = k * (1.f + 3.f * 0.044715f * x * x);                  // gelu.py:72
    return 0.5f * (1.f + th + x * (1.f - th * th) * gp);                   // gelu.py:73
  }
  return 1.f;
}

// Stand-alone element-wise GeLU (gelu.py:12-29, 56-81): y = gelu(x), or dx = dout * gelu'(x).
struct ActParams {
  const void* x;
  const void* dout;  // backward only
  void* out;
  int64_t x_stride, dout_stride, out_stride;  // elements
  int64_t M;
  int N;
  int V;  // packets per row (packet kernel only)
};

template <typename T, int ACT, bool BWD>
__global__ void __launch_bounds__(256) act_kernel(const ActParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  grid_dependency_sync();
  trigger_dependents();
  const int64_t total = p.M * p.V;  // packets
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t row = i / p.V;
    const int v = static_cast<int>(i - row * p.V);
    float xf[VEC], o[VEC];
    Pack16<T>::unpack(ld_stream(reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.x_stride) + v), xf);
    if (BWD) {
      float gf[VEC];
      Pack16<T>::unpack(
          ld_stream(reinterpret_cast<const uint4*>(static_cast<const T*>(p.dout) + row * p.dout_stride) + v), gf);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = gf[e] * act_grad<ACT>(xf[e]);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = act_fwd<ACT>(xf[e]);
    }
    st_stream(reinterpret_cast<uint4*>(static_cast<T*>(p.out) + row * p.out_stride) + v, Pack16<T>::pack(o));
  }
}

// Any alignment, any row length.
template <typename T, int ACT, bool BWD>
__global__ void __launch_bounds__(256) act_any_kernel(const ActParams p) {
  const int64_t total = p.M * p.N;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t row = i / p.N;
    const int64_t c = i - row * p.N;
    const float xv = to_f32(static_cast<const T*>(p.x)[row * p.x_stride + c]);
    float o;
    if (BWD) o = to_f32(static_cast<const T*>(p.dout)[row * p.dout_stride + c]) * act_grad<ACT>(xv);
    else o = act_fwd<ACT>(xv);
    static_cast<T*>(p.out)[row * p.out_stride + c] = from_f32<T>(o);
  }
}

}  // namespace b200norm
