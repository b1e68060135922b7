// Kernels for short rows (at most 32 packets, i.e. 512 bytes): a row is spread over LANES <= 16
// lanes of a warp, so one warp works on 32 / LANES rows at a time instead of leaving most of its
// lanes idle.  Same arithmetic as the wide-row kernels (the reference's two passes for the
// LayerNorm statistics, TritonHub/Normalization/layernorm.py:32-35); reductions are xor-shuffles
// that stay inside a row's lanes.  Rows are loaded straight from global memory: with contiguous
// rows a warp's access is still one contiguous segment.
#pragma once

#include "norm_bwd.cuh"
#include "norm_fwd.cuh"

namespace b200norm {

constexpr int kSmallWarps = 4;  // warps per CTA

template <int LANES>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, int LANES, int LDGS, int ACT, bool RMS>
__global__ void __launch_bounds__(kSmallWarps * 32) norm_fwd_small_kernel(const FwdParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int RPW = 32 / LANES;  // rows per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = lane % LANES, sub = lane / LANES;
  grid_dependency_sync();
  trigger_dependents();

  float wr[LDGS][VEC], br[LDGS][VEC];
#pragma unroll
  for (int j = 0; j < LDGS; ++j) {
    const int v = j * LANES + t;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wr[j][e] = 1.f;
      br[j][e] = 0.f;
    }
    if (v < p.V) {
      if (p.w != nullptr) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) wr[j][e] = load_param(p.w, p.w_dtype, (int64_t)v * VEC + e);
      }
      if (!RMS && p.b != nullptr) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) br[j][e] = load_param(p.b, p.w_dtype, (int64_t)v * VEC + e);
      }
    }
  }
  const float inv_n = 1.f / static_cast<float>(p.N);
  const T* xb = static_cast<const T*>(p.x);
  T* yb = static_cast<T*>(p.y);
  const int64_t step = (int64_t)gridDim.x * kSmallWarps * RPW;
  // every lane of a warp makes the same number of trips; rows past the end are masked
  for (int64_t base = ((int64_t)blockIdx.x * kSmallWarps + warp) * RPW; base < p.M; base += step) {
    const int64_t row = base + sub;
    const bool valid = row < p.M;
    const uint4* xrow = reinterpret_cast<const uint4*>(xb + (valid ? row : 0) * p.x_stride);
    float xf[LDGS][VEC];
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      uint4 pk = make_uint4(0, 0, 0, 0);
      if (valid && v < p.V) pk = ld_stream(xrow + v);
      Pack16<T>::unpack(pk, xf[j]);
    }
    float mean = 0.f;
    if (!RMS) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) s += xf[j][e];
      mean = lanes_sum<LANES>(s) * inv_n;
    }
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const bool live = (j * LANES + t) < p.V;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float d = live ? (xf[j][e] - mean) : 0.f;
        q += d * d;
      }
    }
    const float rstd = 1.f / sqrtf(lanes_sum<LANES>(q) * inv_n + p.eps);
    if (t == 0 && valid) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }
    uint4* yrow = reinterpret_cast<uint4*>(yb + (valid ? row : 0) * p.y_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      float yf[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        yf[e] = (xf[j][e] - mean) * rstd * wr[j][e] + br[j][e];
        if (ACT != kActNone) yf[e] = act_fwd<ACT>(yf[e]);
      }
      if (valid && v < p.V) st_stream(yrow + v, Pack16<T>::pack(yf));
    }
  }
}

template <typename T, int LANES, int LDGS, int ACT, bool RMS>
__global__ void __launch_bounds__(kSmallWarps * 32) norm_bwd_small_kernel(const BwdParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int RPW = 32 / LANES;
  constexpr int COLS = LANES * LDGS * VEC;  // columns a row group can hold
  __shared__ float acc[kSmallWarps][COLS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = lane % LANES, sub = lane / LANES;
  grid_dependency_sync();
  trigger_dependents();

  constexpr int BL = ACT != kActNone ? LDGS : 1;  // the bias is only needed to rebuild y for a fused activation
  float wr[LDGS][VEC], br[BL][VEC], dw[LDGS][VEC], db[LDGS][VEC];
#pragma unroll
  for (int j = 0; j < LDGS; ++j) {
    const int v = j * LANES + t;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wr[j][e] = 1.f;
      dw[j][e] = db[j][e] = 0.f;
      if (v < p.V && p.w != nullptr) wr[j][e] = load_param(p.w, p.w_dtype, (int64_t)v * VEC + e);
      if (ACT != kActNone) {
        br[j][e] = 0.f;
        if (!RMS && v < p.V && p.b != nullptr) br[j][e] = load_param(p.b, p.w_dtype, (int64_t)v * VEC + e);
      }
    }
  }
  const int shard = blockIdx.x / p.ctas_per_shard;
  const int cta_in_shard = blockIdx.x - shard * p.ctas_per_shard;
  const int64_t row_begin = (int64_t)shard * p.rows_per_shard;
  const int64_t row_end = min(row_begin + p.rows_per_shard, p.M);
  const int64_t step = (int64_t)p.ctas_per_shard * kSmallWarps * RPW;
  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dy);
  T* dxb = static_cast<T*>(p.dx);
  const float inv_n = 1.f / static_cast<float>(p.N);

  for (int64_t base = row_begin + ((int64_t)cta_in_shard * kSmallWarps + warp) * RPW; base < row_end; base += step) {
    const int64_t row = base + sub;
    const bool valid = row < row_end;
    const int64_t r = valid ? row : row_begin;
    const uint4* xrow = reinterpret_cast<const uint4*>(xb + r * p.x_stride);
    const uint4* grow = reinterpret_cast<const uint4*>(gb + r * p.dy_stride);
    float xh[LDGS][VEC], wdy[LDGS][VEC];
    const float mu = (RMS || !valid) ? 0.f : __ldg(p.mean + r);
    const float rs = valid ? __ldg(p.rstd + r) : 0.f;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      uint4 px = make_uint4(0, 0, 0, 0), pg = make_uint4(0, 0, 0, 0);
      if (valid && v < p.V) {
        px = ld_stream(xrow + v);
        pg = ld_stream(grow + v);
      }
      float xf[VEC], gf[VEC];
      Pack16<T>::unpack(px, xf);
      Pack16<T>::unpack(pg, gf);
      if (ACT != kActNone) {  // dy = dz * act'(y), rounded to the storage type like a separate kernel would
#pragma unroll
        for (int e = 0; e < VEC; ++e) gf[e] *= act_grad<ACT>((xf[e] - mu) * rs * wr[j][e] + br[j][e]);
        Pack16<T>::unpack(Pack16<T>::pack(gf), gf);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {  // masked packets and rows carry dy = 0: they add nothing
        xh[j][e] = (xf[e] - mu) * rs;
        wdy[j][e] = wr[j][e] * gf[e];
        dw[j][e] += gf[e] * xh[j][e];
        if (!RMS) db[j][e] += gf[e];
        s0 += xh[j][e] * wdy[j][e];
        if (!RMS) s1 += wdy[j][e];
      }
    }
    const float c1 = lanes_sum<LANES>(s0) * inv_n;
    const float c2 = RMS ? 0.f : lanes_sum<LANES>(s1) * inv_n;
    const float k1 = -c1 * rs, k2 = -c2 * rs;
    uint4* dxrow = reinterpret_cast<uint4*>(dxb + r * p.dx_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      float o[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = fmaf(xh[j][e], k1, fmaf(wdy[j][e], rs, k2));
      if (valid && v < p.V) st_stream(dxrow + v, Pack16<T>::pack(o));
    }
  }

  // One partial row per CTA: the warp's row groups first (lanes that own the same columns), then
  // the warps in order.
#pragma unroll
  for (int j = 0; j < LDGS; ++j)
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
#pragma unroll
      for (int o = LANES; o < 32; o <<= 1) {
        dw[j][e] += __shfl_xor_sync(0xffffffffu, dw[j][e], o);
        if (!RMS) db[j][e] += __shfl_xor_sync(0xffffffffu, db[j][e], o);
      }
    }
#pragma unroll
  for (int pass = 0; pass < (RMS ? 1 : 2); ++pass) {
    __syncthreads();
    if (sub == 0) {
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[warp][(j * LANES + t) * VEC + e] = (pass == 0) ? dw[j][e] : db[j][e];
    }
    __syncthreads();
    float* out = (pass == 0) ? p.dw_part : p.db_part;
    if (out != nullptr) {
      for (int c = threadIdx.x; c < p.N; c += kSmallWarps * 32) {
        float a = 0.f;
#pragma unroll
        for (int m = 0; m < kSmallWarps; ++m) a += acc[m][c];
        out[(size_t)blockIdx.x * p.N + c] = a;
      }
    }
  }
}

}  // namespace b200norm
