// Row-wise p-norm and normalisation over the last dimension (TritonHub/Ops/norm.py:11-45, 66-101;
// Ops/normalize.py:11-33, 61-117), forward and backward.  Same skeleton as the norm and softmax
// kernels: a row in packed registers, one row reduction, rows staged through shared memory by bulk
// asynchronous copies.  Row passes: norm forward 1 (read only), norm backward 2 (element-wise, its
// own kernel), normalize forward 2, normalize backward 3 (4 for p other than 1 and 2).
//
//   norm      n = max((sum |x|^p)^(1/p), eps), stored in the storage type          norm.py:26-40
//   d norm    p = 1: g*sign(x);  p = 2: g*x/n;  else g*sign(x)*|x|^(p-1)/n^(p-1)    norm.py:92-99
//   normalize y = x / n, n the STORED (rounded) norm, as the reference's second kernel reads it
//                                                                               normalize.py:27-31
//   d normalize  p = 2: (g - y*proj)/n, proj = sum y*g;                          normalize.py:106-108
//                p = 1: g/n - sign(x)*proj/n^2, proj = sum x*g;                  normalize.py:101-105
//                else   g/n - sign(x)*|x|^(p-1)*proj/n^p, proj = sum y*g         normalize.py:109-113
// fp32 arithmetic throughout.  p = 2 is a compile-time case (P2); p = 1 and general p share the
// other instantiation and branch once per row pass.
#pragma once

#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

enum : int { kPnormFwd = 0, kNormalizeFwd = 1, kNormalizeBwd = 2 };

struct PnormParams {
  const void* a;     // forwards: x.  normalize backward: the saved output y (p != 1) or x (p == 1)
  const void* dout;  // normalize backward: gradient rows (M, N).  norm backward: gradient (M,)
  const void* x;     // normalize backward with p not in {1, 2}, and norm backward: the input
  void* out;         // normalize forward: y.  backwards: dx
  void* norms;       // (M,) in the storage type: written by the forwards, read by the backwards
  int64_t a_stride, dout_stride, x_stride, out_stride;  // elements
  int64_t M;
  int N;
  int V;  // packets per row (packet kernels)
  float p, eps;
  int lanes_log2;  // norm backward: log2 of the threads that share a row
  int* status;
};

__device__ __forceinline__ float sign_of(float x) { return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); }

// (sum |x|^p)^(1/p), clamped (norm.py:36-40)
template <bool P2>
__device__ __forceinline__ float finish_norm(float acc, float p, float eps) {
  const float n = P2 ? sqrtf(acc) : (p == 1.f ? acc : powf(acc, 1.f / p));
  return fmaxf(n, eps);
}

template <typename T, int LDGS, int WARPS_M, int WARPS_N, int STAGES, int MINB, int LANES, int MODE, bool P2>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, MINB) pnorm_kernel(const PnormParams p) {
  static_assert(LANES == 32 || (WARPS_N == 1 && STAGES == 0), "short rows: one warp, direct loads");
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int TPR = WARPS_N * LANES;
  constexpr int RPW = 32 / LANES;
  constexpr int NBAR = STAGES > 0 ? WARPS_M * STAGES : 1;
  constexpr bool BWD = MODE == kNormalizeBwd;
  constexpr int ROWS = BWD ? 2 : 1;  // rows per slot
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red_smem[WARPS_M][2 * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[NBAR];
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int t = warp_n * 32 + lane % LANES, sub = lane / LANES;
  int phase = 0;

  const T* ab = static_cast<const T*>(p.a);
  const T* gb = static_cast<const T*>(p.dout);
  const T* xb = static_cast<const T*>(p.x);
  T* ob = static_cast<T*>(p.out);
  T* nb = static_cast<T*>(p.norms);
  const int64_t first = ((int64_t)blockIdx.x * WARPS_M + warp_m) * RPW;
  const int64_t step = (int64_t)gridDim.x * WARPS_M * RPW;
  const uint32_t row_bytes = static_cast<uint32_t>(p.V) * 16u;
  unsigned char* slots = dyn_smem + (size_t)warp_m * STAGES * ROWS * row_bytes;
  uint64_t* bars = full_bar + (STAGES > 0 ? warp_m * STAGES : 0);
  const bool p_is_1 = !P2 && p.p == 1.f;

  auto fill = [&](int s, int64_t r) {
    unsigned char* dst = slots + (size_t)s * ROWS * row_bytes;
    mbar_expect_tx(&bars[s], ROWS * row_bytes);
    bulk_load(dst, ab + r * p.a_stride, row_bytes, &bars[s]);
    if (BWD) bulk_load(dst + row_bytes, gb + r * p.dout_stride, row_bytes, &bars[s]);
  };

  if (STAGES > 0) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < NBAR; ++i) mbar_init(&full_bar[i], 1);
      cta_abort = 0;
      mbar_init_fence();
    }
    __syncthreads();
  }
  grid_dependency_sync();
  trigger_dependents();
  if (STAGES > 0 && t == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const int64_t r = first + s * step;
      if (r < p.M) fill(s, r);
    }
  }
  int slot = 0;
  uint32_t parity = 0;

  for (int64_t base = first; base < p.M; base += step) {
    const int64_t row = base + sub;
    const bool valid = row < p.M;
    const int64_t r = valid ? row : 0;
    uint4 pa[LDGS], pg[BWD ? LDGS : 1];
    if (STAGES > 0) {
      mbar_wait(&bars[slot], parity, &cta_abort, p.status);
      const uint4* sa = reinterpret_cast<const uint4*>(slots + (size_t)slot * ROWS * row_bytes);
      const uint4* sg = reinterpret_cast<const uint4*>(slots + (size_t)slot * ROWS * row_bytes + row_bytes);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        pa[j] = make_uint4(0, 0, 0, 0);
        if (BWD) pg[j] = make_uint4(0, 0, 0, 0);
        if (v < p.V) {
          pa[j] = ld_shared16(sa + v);
          if (BWD) pg[j] = ld_shared16(sg + v);
        }
      }
    } else {
      const uint4* arow = reinterpret_cast<const uint4*>(ab + r * p.a_stride);
      const uint4* grow = reinterpret_cast<const uint4*>(gb + r * p.dout_stride);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        pa[j] = make_uint4(0, 0, 0, 0);
        if (BWD) pg[j] = make_uint4(0, 0, 0, 0);
        if (valid && v < p.V) {
          pa[j] = ld_stream(arow + v);
          if (BWD) pg[j] = ld_stream(grow + v);
        }
      }
    }

    // Pass 1: one row sum -- |x|^p (forwards) or the projection sum a*g (backward).  Masked packets
    // are zero and add nothing.
    float sacc[1] = {0.f};
    if (BWD) {
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float af[VEC], gf[VEC];
        Pack16<T>::unpack(pa[j], af);
        Pack16<T>::unpack(pg[j], gf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sacc[0] = fmaf(af[e], gf[e], sacc[0]);
      }
    } else if (P2) {
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float af[VEC];
        Pack16<T>::unpack(pa[j], af);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sacc[0] = fmaf(af[e], af[e], sacc[0]);
      }
    } else if (p_is_1) {
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float af[VEC];
        Pack16<T>::unpack(pa[j], af);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sacc[0] += fabsf(af[e]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float af[VEC];
        Pack16<T>::unpack(pa[j], af);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sacc[0] += powf(fabsf(af[e]), p.p);
      }
    }
    if (LANES == 32) {
      group_sum<WARPS_N, 1, 0>(sacc, red_smem[warp_m], phase, warp_m, warp_n, lane);
    } else {
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) sacc[0] += __shfl_xor_sync(0xffffffffu, sacc[0], o);
    }
    if (STAGES > 0) {
      // every thread of the group has its packets in registers (the reduction above needed them)
      if (t == 0) {
        const int64_t rn = row + STAGES * step;
        if (rn < p.M) fill(slot, rn);
      }
      if (++slot == STAGES) {
        slot = 0;
        parity ^= 1u;
      }
    }

    if (MODE != kNormalizeBwd) {
      // the norm, rounded to the storage type: the value a later kernel (and pass 2 here) reads
      const T n_t = from_f32<T>(finish_norm<P2>(sacc[0], p.p, p.eps));
      if (valid && t == 0) nb[row] = n_t;
      if (MODE == kPnormFwd) continue;
      const float inv = 1.f / to_f32(n_t);
      uint4* orow = reinterpret_cast<uint4*>(ob + r * p.out_stride);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float af[VEC], o[VEC];
        if (sizeof(T) < 4) forget(pa[j]);
        Pack16<T>::unpack(pa[j], af);
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = af[e] * inv;
        const int v = j * TPR + t;
        if (valid && v < p.V) st_stream(orow + v, Pack16<T>::pack(o));
      }
    } else {
      const float n = to_f32(nb[r]);
      const float inv = 1.f / n;
      const float proj = sacc[0];
      // p = 2: (g - y*proj)/n.  p = 1: g/n - sign(x)*proj/n^2.  else: g/n - sign(x)|x|^(p-1)*proj/n^p
      const float k = P2 ? proj * inv : (p_is_1 ? proj * inv * inv : proj / powf(n, p.p));
      uint4* orow = reinterpret_cast<uint4*>(ob + r * p.out_stride);
      const uint4* xrow = reinterpret_cast<const uint4*>(xb + r * p.x_stride);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        const bool live = valid && v < p.V;
        float af[VEC], gf[VEC], o[VEC];
        if (sizeof(T) < 4) {
          forget(pa[j]);
          forget(pg[j]);
        }
        Pack16<T>::unpack(pa[j], af);
        Pack16<T>::unpack(pg[j], gf);
        if (P2) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = fmaf(-af[e], k, gf[e] * inv);
        } else if (p_is_1) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = fmaf(-sign_of(af[e]), k, gf[e] * inv);
        } else {
          float xf[VEC];
          Pack16<T>::unpack(live ? ld_stream(xrow + v) : make_uint4(0, 0, 0, 0), xf);
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            o[e] = fmaf(-sign_of(xf[e]) * powf(fabsf(xf[e]), p.p - 1.f), k, gf[e] * inv);
        }
        if (live) st_stream(orow + v, Pack16<T>::pack(o));
      }
    }
  }
  if (STAGES > 0) {
    if (t == 0 && cta_abort) drain_ring<STAGES>(bars, first < p.M ? (p.M - first + step - 1) / step : 0);
  }
}

// Norm backward: element-wise once the row's norm and gradient are known, so no row is held and no
// reduction is made.  `LANES` (a power of two, at most 256) threads share a row and 256 / LANES rows
// are in flight per CTA.
template <typename T, bool P2>
__global__ void __launch_bounds__(256) pnorm_bwd_kernel(const PnormParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  grid_dependency_sync();
  trigger_dependents();
  const int lanes_log2 = p.lanes_log2;
  const int lanes = 1 << lanes_log2;
  const int rows_per_iter = 256 >> lanes_log2;
  const int v0 = threadIdx.x & (lanes - 1);
  const bool p_is_1 = !P2 && p.p == 1.f;
  const T* gb = static_cast<const T*>(p.dout);
  const T* nb = static_cast<const T*>(p.norms);
  for (int64_t row = (int64_t)blockIdx.x * rows_per_iter + (threadIdx.x >> lanes_log2); row < p.M;
       row += (int64_t)gridDim.x * rows_per_iter) {
    const float g = to_f32(gb[row]);
    // p = 1 needs no norm; p = 2: g/n; else g/n^(p-1)   (norm.py:84-87, 92-99)
    const float k = p_is_1 ? g : (P2 ? g / to_f32(nb[row]) : g / powf(to_f32(nb[row]), p.p - 1.f));
    const uint4* xrow = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + row * p.x_stride);
    uint4* orow = reinterpret_cast<uint4*>(static_cast<T*>(p.out) + row * p.out_stride);
    for (int v = v0; v < p.V; v += lanes) {
      float xf[VEC], o[VEC];
      Pack16<T>::unpack(ld_stream(xrow + v), xf);
      if (P2) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = xf[e] * k;
      } else if (p_is_1) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = sign_of(xf[e]) * k;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = sign_of(xf[e]) * powf(fabsf(xf[e]), p.p - 1.f) * k;
      }
      st_stream(orow + v, Pack16<T>::pack(o));
    }
  }
}

// Any alignment, any row length, any p: one CTA per row, scalar accesses (re-reads hit L1/L2).
// MODE as above, plus 3 = norm backward.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) pnorm_any_kernel(const PnormParams p) {
  __shared__ float red[2 * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int phase = 0;
  const bool p2 = p.p == 2.f, p1 = p.p == 1.f;
  T* nb = static_cast<T*>(p.norms);
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    const T* arow = static_cast<const T*>(p.a) + row * p.a_stride;
    const T* xrow = static_cast<const T*>(p.x) + row * p.x_stride;
    T* orow = static_cast<T*>(p.out) + row * p.out_stride;
    if (MODE == kPnormFwd || MODE == kNormalizeFwd) {
      float sacc[1] = {0.f};
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float v = to_f32(arow[c]);
        sacc[0] += p2 ? v * v : (p1 ? fabsf(v) : powf(fabsf(v), p.p));
      }
      group_sum<8, 1, 0>(sacc, red, phase, 0, warp, lane);
      const float n32 = p2 ? sqrtf(sacc[0]) : (p1 ? sacc[0] : powf(sacc[0], 1.f / p.p));
      const T n_t = from_f32<T>(fmaxf(n32, p.eps));
      if (threadIdx.x == 0) nb[row] = n_t;
      if (MODE == kNormalizeFwd) {
        const float inv = 1.f / to_f32(n_t);
        for (int c = threadIdx.x; c < p.N; c += 256) orow[c] = from_f32<T>(to_f32(arow[c]) * inv);
      }
    } else if (MODE == kNormalizeBwd) {
      const T* grow = static_cast<const T*>(p.dout) + row * p.dout_stride;
      float sacc[1] = {0.f};
      for (int c = threadIdx.x; c < p.N; c += 256) sacc[0] = fmaf(to_f32(arow[c]), to_f32(grow[c]), sacc[0]);
      group_sum<8, 1, 0>(sacc, red, phase, 0, warp, lane);
      const float n = to_f32(nb[row]), inv = 1.f / n, proj = sacc[0];
      const float k = p2 ? proj * inv : (p1 ? proj * inv * inv : proj / powf(n, p.p));
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float g = to_f32(grow[c]);
        float d;
        if (p2) {
          d = to_f32(arow[c]);
        } else if (p1) {
          d = sign_of(to_f32(arow[c]));
        } else {
          const float xv = to_f32(xrow[c]);
          d = sign_of(xv) * powf(fabsf(xv), p.p - 1.f);
        }
        orow[c] = from_f32<T>(fmaf(-d, k, g * inv));
      }
    } else {
      const float g = to_f32(static_cast<const T*>(p.dout)[row]);
      const float k = p1 ? g : (p2 ? g / to_f32(nb[row]) : g / powf(to_f32(nb[row]), p.p - 1.f));
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float xv = to_f32(xrow[c]);
        orow[c] = from_f32<T>((p2 ? xv : (p1 ? sign_of(xv) : sign_of(xv) * powf(fabsf(xv), p.p - 1.f))) * k);
      }
    }
  }
}

}  // namespace b200norm
