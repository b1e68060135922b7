// GeLU, exact (erf) and tanh forms, and its derivative -- the activation that follows the norm
// in the reference's Quick Start (README.md:44-48).  Formulas: TritonHub/Activations/gelu.py:20-28
// (forward) and :67-79 (derivative).  Used fused into the norm kernels' stores / loads and by the
// stand-alone element-wise kernels below.
#pragma once

#include "norm_common.cuh"

namespace b200norm {

enum : int { kActNone = 0, kActGeluErf = 1, kActGeluTanh = 2 };

// Both forms are evaluated through one quantity each, chosen so that an element costs as few
// instructions as the formulas allow (these kernels are issue-bound, not HBM-bound, once an
// activation is fused in):
//
// tanh form (gelu.py:20-25, 67-73).  With u = k (x + 0.044715 x^3) and r = 1 / (exp(2u) + 1):
//   tanh(u) = 1 - 2r,  gelu = 0.5 x (1 + tanh u) = x - x r,
//   gelu'   = 0.5 (1 + tanh u + x (1 - tanh^2 u) u') = s + x u' * 2 r s,   s = 1 - r.
// The reference's tanh, (e - 1) / (e + 1) (gelu.py:24), is inf / inf = NaN once exp(2u) overflows
// (x > ~10 in fp32); r simply becomes 0 there, and the two agree wherever the reference is finite.
//
// erf form (gelu.py:27, 75-78).  Abramowitz & Stegun 7.1.26 gives erfc(|s|) = poly(t) exp(-s^2),
// t = 1 / (1 + 0.3275911 |s|), absolute error <= 1.5e-7, one reciprocal and five FMAs -- a third of
// the instructions of the library erff.  With q = 0.5 erfc(|x| / sqrt 2):
//   Phi(x) = x >= 0 ? 1 - q : q,   gelu = x Phi(x) = max(x, 0) - |x| q,   gelu' = Phi(x) + x phi(x).
constexpr float kGeluK = 0.79788456080286536f;  // sqrt(2 / pi)

// r = 1 / (exp(2u) + 1) for the tanh form; x2 = x * x
__device__ __forceinline__ float gelu_tanh_r(float x, float x2) {
  const float arg = x * fmaf(x2, kGeluK * 0.044715f * 2.f * kLog2e, kGeluK * 2.f * kLog2e);  // 2u * log2(e)
  return rcp_fast(ex2_fast(arg) + 1.f);  // exp = inf gives 0, exp = 0 gives 1
}

// q = 0.5 * erfc(|x| / sqrt(2)) and e = exp(-x^2 / 2) for the erf form
__device__ __forceinline__ float gelu_erf_q(float x, float& e) {
  e = ex2_fast(x * x * (-0.5f * kLog2e));
  const float t = rcp_fast(fmaf(0.3275911f * 0.70710678118654752f, fabsf(x), 1.f));
  const float half_poly = t * (0.127414796f + t * (-0.142248368f + t * (0.7107068705f + t * (-0.7265760135f + t * 0.5307027145f))));
  return half_poly * e;
}

template <int ACT>
__device__ __forceinline__ float act_fwd(float x) {
  if (ACT == kActGeluErf) {
    float e;
    const float q = gelu_erf_q(x, e);
    return fmaf(-fabsf(x), q, fmaxf(x, 0.f));
  } else if (ACT == kActGeluTanh) {
    return fmaf(-x, gelu_tanh_r(x, x * x), x);
  }
  return x;
}

// d act(x) / dx
template <int ACT>
__device__ __forceinline__ float act_grad(float x) {
  if (ACT == kActGeluErf) {
    float e;
    const float q = gelu_erf_q(x, e);
    const float cdf = x >= 0.f ? 1.f - q : q;
    return fmaf(x, e * 0.39894228040143268f, cdf);  // Phi + x * phi
  } else if (ACT == kActGeluTanh) {
    const float x2 = x * x;
    const float r = gelu_tanh_r(x, x2);
    const float s = 1.f - r;
    const float xup2 = x * fmaf(x2, 2.f * 3.f * 0.044715f * kGeluK, 2.f * kGeluK);  // 2 x u'
    return fmaf(xup2, r * s, s);
  }
  return 1.f;
}

// ---------------------------------------------------------------------------------------
// The same, two elements per instruction (packed fp32 arithmetic, norm_common.cuh): every
// multiply-add of the formulas above is done on pairs; only the special-function calls (ex2, rcp)
// and the sign / select steps stay scalar.  Bit for bit the results of act_fwd / act_grad.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float2 gelu_tanh_r2(float2 x, float2 x2) {
  const float2 arg = mul2(x, fma2(x2, splat2(kGeluK * 0.044715f * 2.f * kLog2e), splat2(kGeluK * 2.f * kLog2e)));
  const float2 d = add2(make_float2(ex2_fast(arg.x), ex2_fast(arg.y)), splat2(1.f));
  return make_float2(rcp_fast(d.x), rcp_fast(d.y));
}

__device__ __forceinline__ float2 gelu_erf_q2(float2 x, float2& e) {
  const float2 arg = mul2(mul2(x, x), splat2(-0.5f * kLog2e));
  e = make_float2(ex2_fast(arg.x), ex2_fast(arg.y));
  const float2 d = fma2(splat2(0.3275911f * 0.70710678118654752f), make_float2(fabsf(x.x), fabsf(x.y)), splat2(1.f));
  const float2 t = make_float2(rcp_fast(d.x), rcp_fast(d.y));
  float2 poly = fma2(t, splat2(0.5307027145f), splat2(-0.7265760135f));
  poly = fma2(t, poly, splat2(0.7107068705f));
  poly = fma2(t, poly, splat2(-0.142248368f));
  poly = fma2(t, poly, splat2(0.127414796f));
  return mul2(mul2(t, poly), e);
}

template <int ACT>
__device__ __forceinline__ float2 act_fwd2(float2 x) {
  if (ACT == kActGeluErf) {
    float2 e;
    const float2 q = gelu_erf_q2(x, e);
    return fma2(make_float2(-fabsf(x.x), -fabsf(x.y)), q, make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f)));
  } else if (ACT == kActGeluTanh) {
    return fma2(mul2(x, splat2(-1.f)), gelu_tanh_r2(x, mul2(x, x)), x);
  }
  return x;
}

template <int ACT>
__device__ __forceinline__ float2 act_grad2(float2 x) {
  if (ACT == kActGeluErf) {
    float2 e;
    const float2 q = gelu_erf_q2(x, e);
    const float2 up = fma2(q, splat2(-1.f), splat2(1.f));  // 1 - q
    const float2 cdf = make_float2(x.x >= 0.f ? up.x : q.x, x.y >= 0.f ? up.y : q.y);
    return fma2(x, mul2(e, splat2(0.39894228040143268f)), cdf);  // Phi + x * phi
  } else if (ACT == kActGeluTanh) {
    const float2 x2 = mul2(x, x);
    const float2 r = gelu_tanh_r2(x, x2);
    const float2 s = fma2(r, splat2(-1.f), splat2(1.f));  // 1 - r
    const float2 xup2 = mul2(x, fma2(x2, splat2(2.f * 3.f * 0.044715f * kGeluK), splat2(2.f * kGeluK)));  // 2 x u'
    return fma2(xup2, mul2(r, s), s);
  }
  return splat2(1.f);
}

// y <- act(y) and g <- g * act'(y) over a packet's VEC values (VEC is even for every storage type).
template <int ACT, int VEC>
__device__ __forceinline__ void act_fwd_packet(float (&y)[VEC]) {
#pragma unroll
  for (int e = 0; e < VEC; e += 2) {
    const float2 r = act_fwd2<ACT>(make_float2(y[e], y[e + 1]));
    y[e] = r.x;
    y[e + 1] = r.y;
  }
}
template <int ACT, int VEC>
__device__ __forceinline__ void act_grad_mul_packet(const float (&y)[VEC], float (&g)[VEC]) {
#pragma unroll
  for (int e = 0; e < VEC; e += 2) {
    const float2 r = mul2(make_float2(g[e], g[e + 1]), act_grad2<ACT>(make_float2(y[e], y[e + 1])));
    g[e] = r.x;
    g[e + 1] = r.y;
  }
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
      act_grad_mul_packet<ACT, VEC>(xf, gf);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = gf[e];
    } else {
      act_fwd_packet<ACT, VEC>(xf);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = xf[e];
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
