// Row-wise Softmax and LogSoftmax, forward and backward (TritonHub/Activations/softmax.py:11-62,
// logsoftmax.py:11-68; Softmin is Softmax of -x, softmin.py:103).  Same skeleton as the norm
// kernels -- a row in registers, one row reduction, rows staged through shared memory by bulk
// asynchronous copies -- and the same roofline: 2 row passes forward, 3 backward, no parameters.
//
// Forward: each thread forms the maximum m_t of its elements and s_t = sum exp(x - m_t); the row
// group merges the (m, s) pairs online, m = max(ma, mb), s = sa*exp(ma - m) + sb*exp(mb - m), in one
// reduction.  Softmax then scales the exponentials it already holds: y = exp(x - m_t) * exp(m_t - m) / s
// (softmax.py:19-22); LogSoftmax writes y = (x - m) - log s (logsoftmax.py:20-22).  fp32 throughout.
// Backward reads the saved OUTPUT y: Softmax dx = y * (dout - sum(dout * y)) (softmax.py:57-59);
// LogSoftmax dx = dout - exp(y) * sum(dout) (logsoftmax.py:63-65).
#pragma once

#include <math_constants.h>

#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

// Softmax forward keeps the exponentials of pass 1 in registers and scales them (16-bit types too:
// recomputing them from the packed row saved registers but cost an exponential per element).

struct SoftmaxParams {
  const void* x;     // forward: input; backward: the saved output y
  const void* dout;  // backward only
  void* out;         // forward: y; backward: dx
  int64_t x_stride, dout_stride, out_stride;  // elements
  int64_t M;
  int N;
  int V;  // packets per row (packet kernels)
  int* status;
};

// Maximum over the warp in one instruction (sm_100a: redux.sync on fp32).
__device__ __forceinline__ float warp_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// s counts exponentials relative to m; re-base it on M >= m.  m == M covers the empty pair
// (-inf, 0), whose difference would be NaN.
__device__ __forceinline__ float rebase(float s, float m, float M) {
  return (m == M) ? s : s * ex2_fast((m - M) * kLog2e);
}

// Online merge of (max, sum of exponentials relative to that max), for the short-row kernels.
__device__ __forceinline__ void maxsum_merge(float& m, float& s, float mb, float sb) {
  // One of the two scale factors is always exp(0) = 1: a single exponential of -|ma - mb| serves.
  // Two empty pairs (-inf, 0) give exp(NaN) * 0 on the scaled side, hence the guard.
  const bool a_is_max = m >= mb;
  const float d = a_is_max ? mb - m : m - mb;
  const float e = (d == d) ? ex2_fast(d * kLog2e) : 0.f;
  const float big = a_is_max ? s : sb, small = a_is_max ? sb : s;
  s = (m == mb) ? s + sb : fmaf(small, e, big);  // equal maxima: a commutative add on both sides
  m = a_is_max ? m : mb;
}

// (max, sum) of a row from per-thread pairs; every thread of the group gets the result.  The
// dependent chain is short on purpose -- a row waits on it with nothing else to do: the maximum
// first (one redux per warp), one re-basing exponential per thread, then a plain butterfly sum;
// across warps the same again with lane k holding warp k's pair.  All lanes add in the same
// order, so the result is identical across the group and from run to run.
template <int WARPS_N, int LANES>
__device__ __forceinline__ void group_maxsum(float& m, float& s, float* scratch, int& phase, int warp_m, int warp_n,
                                             int lane) {
  static_assert((WARPS_N & (WARPS_N - 1)) == 0 && WARPS_N <= 32, "lane k reads warp k's pair");
  if (LANES == 32) {
    const float mw = warp_max(m);
    s = warp_sum(rebase(s, m, mw));
    m = mw;
  } else {
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) {
      const float mb = __shfl_xor_sync(0xffffffffu, m, o);
      const float sb = __shfl_xor_sync(0xffffffffu, s, o);
      // symmetric down to the bits (both partners evaluate fma(smaller-side sum, e, larger-side
      // sum)), so no lane ordering and no divergent branch
      maxsum_merge(m, s, mb, sb);
    }
  }
  if (WARPS_N > 1) {
    float* buf = scratch + phase * (2 * WARPS_N);
    if (lane == 0) {
      buf[warp_n] = m;
      buf[WARPS_N + warp_n] = s;
    }
    group_sync<WARPS_N, 0>(warp_m);  // this file's kernels use no CTA-wide barrier after set-up
    const int k = lane & (WARPS_N - 1);
    const float mk = buf[k];
    float sk = buf[WARPS_N + k];
    m = warp_max(mk);
    sk = rebase(sk, mk, m);
#pragma unroll
    for (int o = WARPS_N / 2; o > 0; o >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
    s = sk;
    phase ^= 1;
  }
}

// Maximum of a packet's elements without leaving the packed form (16-bit types: four paired
// maxima per packet instead of eight conversions and eight scalar maxima).
template <typename T>
struct PackedMax {
  static constexpr bool kPacked = false;
};
template <>
struct PackedMax<__half> {
  static constexpr bool kPacked = true;
  static constexpr uint32_t kNegInf = 0xfc00fc00u;
  __device__ __forceinline__ static uint32_t max2(uint32_t a, uint32_t b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  __device__ __forceinline__ static float finish(uint32_t a) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&a));
    return fmaxf(f.x, f.y);
  }
};
template <>
struct PackedMax<__nv_bfloat16> {
  static constexpr bool kPacked = true;
  static constexpr uint32_t kNegInf = 0xff80ff80u;
  __device__ __forceinline__ static uint32_t max2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r =
        __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  __device__ __forceinline__ static float finish(uint32_t a) {
    return fmaxf(__uint_as_float(a << 16), __uint_as_float(a & 0xffff0000u));
  }
};

template <int LANES>
__device__ __forceinline__ float lanes_add(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One kernel for both directions and both functions.  BWD: rows of y and dout are staged side by
// side (two bulk copies per slot).  LANES < 32 (with WARPS_N == 1, STAGES == 0): short rows, 32 /
// LANES of them per warp, loaded straight from global memory.
template <typename T, int LDGS, int WARPS_M, int WARPS_N, int STAGES, int MINB, int LANES, bool LOG, bool BWD>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, MINB) softmax_kernel(const SoftmaxParams p) {
  static_assert(LANES == 32 || (WARPS_N == 1 && STAGES == 0), "short rows: one warp, direct loads");
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int TPR = WARPS_N * LANES;
  constexpr int RPW = 32 / LANES;
  constexpr int NBAR = STAGES > 0 ? WARPS_M * STAGES : 1;
  constexpr int ROWS = BWD ? 2 : 1;  // rows per slot
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red_smem[WARPS_M][2 * 2 * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[NBAR];
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int t = warp_n * 32 + lane % LANES, sub = lane / LANES;
  int phase = 0;

  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dout);
  T* ob = static_cast<T*>(p.out);
  const int64_t first = ((int64_t)blockIdx.x * WARPS_M + warp_m) * RPW;
  const int64_t step = (int64_t)gridDim.x * WARPS_M * RPW;
  const uint32_t row_bytes = static_cast<uint32_t>(p.V) * 16u;
  unsigned char* slots = dyn_smem + (size_t)warp_m * STAGES * ROWS * row_bytes;
  uint64_t* bars = full_bar + (STAGES > 0 ? warp_m * STAGES : 0);

  auto fill = [&](int s, int64_t r) {
    unsigned char* dst = slots + (size_t)s * ROWS * row_bytes;
    mbar_expect_tx(&bars[s], ROWS * row_bytes);
    bulk_load(dst, xb + r * p.x_stride, row_bytes, &bars[s]);
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
    // The row stays PACKED in registers and is unpacked where it is used: LogSoftmax needs x again
    // after the reduction, and holding it as fp32 next to the exponentials would halve occupancy.
    uint4 px[LDGS], pg[BWD ? LDGS : 1];
    if (STAGES > 0) {
      mbar_wait(&bars[slot], parity, &cta_abort, p.status);
      const uint4* sx = reinterpret_cast<const uint4*>(slots + (size_t)slot * ROWS * row_bytes);
      const uint4* sg = reinterpret_cast<const uint4*>(slots + (size_t)slot * ROWS * row_bytes + row_bytes);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        px[j] = make_uint4(0, 0, 0, 0);
        if (BWD) pg[j] = make_uint4(0, 0, 0, 0);
        if (v < p.V) {
          px[j] = ld_shared16(sx + v);
          if (BWD) pg[j] = ld_shared16(sg + v);
        }
      }
    } else {
      const uint4* xrow = reinterpret_cast<const uint4*>(xb + r * p.x_stride);
      const uint4* grow = reinterpret_cast<const uint4*>(gb + r * p.dout_stride);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        px[j] = make_uint4(0, 0, 0, 0);
        if (BWD) pg[j] = make_uint4(0, 0, 0, 0);
        if (valid && v < p.V) {
          px[j] = ld_stream(xrow + v);
          if (BWD) pg[j] = ld_stream(grow + v);
        }
      }
    }

    // Pass 1: the row reduction.  Forward: per-thread maximum m_t and s = sum exp(x - m_t), merged
    // over the group; backward: sum(dout) or sum(dout * y).
    constexpr bool HOLD = !BWD && !LOG;
    float held[HOLD ? LDGS : 1][VEC];  // Softmax forward: the exponentials, scaled in pass 2
    float m_t = 0.f, m_row = 0.f, s_row = 0.f;
    if (!BWD) {
      float m = -CUDART_INF_F;
      if constexpr (PackedMax<T>::kPacked) {
        uint32_t acc = PackedMax<T>::kNegInf;
#pragma unroll
        for (int j = 0; j < LDGS; ++j) {
          if ((j * TPR + t) < p.V) {
            using PM = PackedMax<T>;
            acc = PM::max2(acc, PM::max2(PM::max2(px[j].x, px[j].y), PM::max2(px[j].z, px[j].w)));
          }
        }
        m = PackedMax<T>::finish(acc);
      } else {
#pragma unroll
        for (int j = 0; j < LDGS; ++j) {
          if ((j * TPR + t) < p.V) {
            float xf[VEC];
            Pack16<T>::unpack(px[j], xf);
#pragma unroll
            for (int e = 0; e < VEC; ++e) m = fmaxf(m, xf[e]);
          }
        }
      }
      m_t = m;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const bool live = (j * TPR + t) < p.V;
        float xf[VEC];
        Pack16<T>::unpack(px[j], xf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float ex = live ? ex2_fast((xf[e] - m_t) * kLog2e) : 0.f;
          s += ex;
          if (HOLD) held[j][e] = ex;
        }
      }
      group_maxsum<WARPS_N, LANES>(m, s, red_smem[warp_m], phase, warp_m, warp_n, lane);
      m_row = m;
      s_row = s;
    } else {
      float sacc[1] = {0.f};
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        float xf[VEC], gf[VEC];
        Pack16<T>::unpack(px[j], xf);
        Pack16<T>::unpack(pg[j], gf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sacc[0] += LOG ? gf[e] : gf[e] * xf[e];  // masked packets are zero
      }
      if (LANES == 32) {
        group_sum<WARPS_N, 1, 0>(sacc, red_smem[warp_m], phase, warp_m, warp_n, lane);
      } else {
        sacc[0] = lanes_add<LANES>(sacc[0]);
      }
      s_row = sacc[0];
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

    // Pass 2: packet by packet from the packed registers, straight to the store.
    float f_scale = 0.f, shift = 0.f;
    if (!BWD) {
      if (LOG) {
        shift = m_row + __logf(s_row);  // y = (x - m) - log s
      } else if (HOLD) {
        f_scale = rebase(1.f, m_t, m_row) / s_row;  // exp(x - m) / s = exp(x - m_t) * f
      } else {
        shift = __log2f(s_row);  // y = 2^((x - m) * log2(e) - log2(s))
      }
    }
    uint4* orow = reinterpret_cast<uint4*>(ob + r * p.out_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      float xf[VEC], gf[VEC], o[VEC];
      if (sizeof(T) < 4) {
        forget(px[j]);
        if (BWD) forget(pg[j]);
      }
      Pack16<T>::unpack(px[j], xf);
      if (BWD) Pack16<T>::unpack(pg[j], gf);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        if (BWD) {
          o[e] = LOG ? (gf[e] - ex2_fast(xf[e] * kLog2e) * s_row) : xf[e] * (gf[e] - s_row);
        } else if (LOG) {
          o[e] = xf[e] - shift;
        } else if (HOLD) {
          o[e] = held[j][e] * f_scale;
        } else {
          o[e] = ex2_fast(fmaf(xf[e] - m_row, kLog2e, -shift));
        }
      }
      const int v = j * TPR + t;
      if (valid && v < p.V) st_stream(orow + v, Pack16<T>::pack(o));
    }
  }
  if (STAGES > 0) {
    if (t == 0 && cta_abort) drain_ring<STAGES>(bars, first < p.M ? (p.M - first + step - 1) / step : 0);
  }
}

// Any alignment, any row length: one CTA per row, scalar accesses (re-reads hit L1/L2).
template <typename T, bool LOG, bool BWD>
__global__ void __launch_bounds__(256) softmax_any_kernel(const SoftmaxParams p) {
  __shared__ float red[2 * 2 * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int phase = 0;
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    const T* xrow = static_cast<const T*>(p.x) + row * p.x_stride;
    T* orow = static_cast<T*>(p.out) + row * p.out_stride;
    if (!BWD) {
      float m = -CUDART_INF_F, s = 0.f;
      for (int c = threadIdx.x; c < p.N; c += 256) m = fmaxf(m, to_f32(xrow[c]));
      const float m_t = m;
      for (int c = threadIdx.x; c < p.N; c += 256) s += __expf(to_f32(xrow[c]) - m_t);
      group_maxsum<8, 32>(m, s, red, phase, 0, warp, lane);
      const float shift = m + __logf(s);
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float xv = to_f32(xrow[c]);
        orow[c] = from_f32<T>(LOG ? xv - shift : __expf(xv - m) / s);
      }
    } else {
      const T* grow = static_cast<const T*>(p.dout) + row * p.dout_stride;
      float sacc[1] = {0.f};
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float g = to_f32(grow[c]);
        sacc[0] += LOG ? g : g * to_f32(xrow[c]);
      }
      group_sum<8, 1, 0>(sacc, red, phase, 0, warp, lane);
      for (int c = threadIdx.x; c < p.N; c += 256) {
        const float y = to_f32(xrow[c]), g = to_f32(grow[c]);
        orow[c] = from_f32<T>(LOG ? g - __expf(y) * sacc[0] : y * (g - sacc[0]));
      }
    }
  }
}

}  // namespace b200norm
