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

  constexpr int H = VEC / 2;  // per-element values as fp32 pairs, two per instruction (norm_common.cuh)
  float2 wr[LDGS][H], br[LDGS][H];
#pragma unroll
  for (int j = 0; j < LDGS; ++j) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      wr[j][h] = splat2(1.f);
      br[j][h] = splat2(0.f);
    }
  }
  load_param_packets<T, LDGS>(
      p.w, RMS ? nullptr : p.b, p.w_dtype, 0, t, LANES, p.V, [](int) { return true; }, []() {},
      [&](int which, int j, const float* f) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          if (which == 0) wr[j][h] = make_float2(f[2 * h], f[2 * h + 1]);
          else br[j][h] = make_float2(f[2 * h], f[2 * h + 1]);
        }
      });
  const float inv_n = 1.f / static_cast<float>(p.N);
  const T* xb = static_cast<const T*>(p.x);
  T* yb = static_cast<T*>(p.y);
  const int64_t step = (int64_t)gridDim.x * kSmallWarps * RPW;
  // every lane of a warp makes the same number of trips; rows past the end are masked
  for (int64_t base = ((int64_t)blockIdx.x * kSmallWarps + warp) * RPW; base < p.M; base += step) {
    const int64_t row = base + sub;
    const bool valid = row < p.M;
    const uint4* xrow = reinterpret_cast<const uint4*>(xb + (valid ? row : 0) * p.x_stride);
    float2 xf[LDGS][H];
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      uint4 pk = make_uint4(0, 0, 0, 0);
      if (valid && v < p.V) pk = ld_stream(xrow + v);
      Pack16<T>::unpack2(pk, xf[j]);
    }
    float mean = 0.f;
    if (!RMS) {
      float2 s2 = splat2(0.f);
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h) s2 = add2(s2, xf[j][h]);
      mean = lanes_sum<LANES>(s2.x + s2.y) * inv_n;
    }
    const float2 nm = splat2(-mean);
    float2 q2 = splat2(0.f);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      if ((j * LANES + t) < p.V) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 d = add2(xf[j][h], nm);
          q2 = fma2(d, d, q2);
        }
      }
    }
    const float rstd = 1.f / sqrtf(lanes_sum<LANES>(q2.x + q2.y) * inv_n + p.eps);
    if (t == 0 && valid) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }
    uint4* yrow = reinterpret_cast<uint4*>(yb + (valid ? row : 0) * p.y_stride);
    const float2 r2 = splat2(rstd);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      float2 yf[H];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        yf[h] = fma2(mul2(RMS ? xf[j][h] : add2(xf[j][h], nm), r2), wr[j][h], br[j][h]);
        if (ACT != kActNone) yf[h] = act_fwd2<ACT>(yf[h]);
      }
      if (valid && v < p.V) st_stream(yrow + v, Pack16<T>::pack2(yf));
    }
  }
}

template <typename T, int LANES, int LDGS, int ACT, bool RMS>
__global__ void __launch_bounds__(kSmallWarps * 32) norm_bwd_small_kernel(const BwdParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int RPW = 32 / LANES;
  constexpr int COLS = LANES * LDGS * VEC;  // columns a row group can hold
  __shared__ __align__(8) float acc[kSmallWarps][COLS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = lane % LANES, sub = lane / LANES;
  grid_dependency_sync();
  trigger_dependents();

  constexpr int H = VEC / 2;  // per-element values as fp32 pairs, two per instruction (norm_common.cuh)
  constexpr int BL = ACT != kActNone ? LDGS : 1;  // the bias is only needed to rebuild y for a fused activation
  float2 wr[LDGS][H], br[BL][H], dw[LDGS][H], db[LDGS][H];
#pragma unroll
  for (int j = 0; j < LDGS; ++j) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      wr[j][h] = splat2(1.f);
      dw[j][h] = db[j][h] = splat2(0.f);
      if (ACT != kActNone) br[j < BL ? j : 0][h] = splat2(0.f);
    }
  }
  load_param_packets<T, LDGS>(
      p.w, (ACT != kActNone && !RMS) ? p.b : nullptr, p.w_dtype, 0, t, LANES, p.V, [](int) { return true; }, []() {},
      [&](int which, int j, const float* f) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          if (which == 0) wr[j][h] = make_float2(f[2 * h], f[2 * h + 1]);
          else br[j < BL ? j : 0][h] = make_float2(f[2 * h], f[2 * h + 1]);
        }
      });
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
    float2 xh[LDGS][H], wdy[LDGS][H];
    const float mu = (RMS || !valid) ? 0.f : __ldg(p.mean + r);
    const float rs = valid ? __ldg(p.rstd + r) : 0.f;
    const float2 nmu2 = splat2(-mu), rs2 = splat2(rs);
    float2 s0 = splat2(0.f), s1 = splat2(0.f);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      uint4 px = make_uint4(0, 0, 0, 0), pg = make_uint4(0, 0, 0, 0);
      if (valid && v < p.V) {
        px = ld_stream(xrow + v);
        pg = ld_stream(grow + v);
      }
      float2 xf[H], gf[H];
      Pack16<T>::unpack2(px, xf);
      Pack16<T>::unpack2(pg, gf);
      if (ACT != kActNone) {  // dy = dz * act'(y), rounded to the storage type like a separate kernel would
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 y = fma2(mul2(RMS ? xf[h] : add2(xf[h], nmu2), rs2), wr[j][h], br[j < BL ? j : 0][h]);
          gf[h] = mul2(gf[h], act_grad2<ACT>(y));
        }
        Pack16<T>::unpack2(Pack16<T>::pack2(gf), gf);
      }
#pragma unroll
      for (int h = 0; h < H; ++h) {  // masked packets and rows carry dy = 0: they add nothing
        xh[j][h] = mul2(RMS ? xf[h] : add2(xf[h], nmu2), rs2);
        wdy[j][h] = mul2(wr[j][h], gf[h]);
        dw[j][h] = fma2(gf[h], xh[j][h], dw[j][h]);
        if (!RMS) db[j][h] = add2(db[j][h], gf[h]);
        s0 = fma2(xh[j][h], wdy[j][h], s0);
        if (!RMS) s1 = add2(s1, wdy[j][h]);
      }
    }
    const float c1 = lanes_sum<LANES>(s0.x + s0.y) * inv_n;
    const float c2 = RMS ? 0.f : lanes_sum<LANES>(s1.x + s1.y) * inv_n;
    const float2 k1 = splat2(-c1 * rs), k2 = splat2(-c2 * rs);
    uint4* dxrow = reinterpret_cast<uint4*>(dxb + r * p.dx_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * LANES + t;
      float2 o[H];
#pragma unroll
      for (int h = 0; h < H; ++h) o[h] = fma2(xh[j][h], k1, fma2(wdy[j][h], rs2, k2));
      if (valid && v < p.V) st_stream(dxrow + v, Pack16<T>::pack2(o));
    }
  }

  // One partial row per CTA: the warp's row groups first (lanes that own the same columns), then
  // the warps in order.
#pragma unroll
  for (int j = 0; j < LDGS; ++j)
#pragma unroll
    for (int h = 0; h < H; ++h) {
#pragma unroll
      for (int o = LANES; o < 32; o <<= 1) {
        dw[j][h].x += __shfl_xor_sync(0xffffffffu, dw[j][h].x, o);
        dw[j][h].y += __shfl_xor_sync(0xffffffffu, dw[j][h].y, o);
        if (!RMS) {
          db[j][h].x += __shfl_xor_sync(0xffffffffu, db[j][h].x, o);
          db[j][h].y += __shfl_xor_sync(0xffffffffu, db[j][h].y, o);
        }
      }
    }
#pragma unroll
  for (int pass = 0; pass < (RMS ? 1 : 2); ++pass) {
    __syncthreads();
    if (sub == 0) {
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h)
          *reinterpret_cast<float2*>(&acc[warp][(j * LANES + t) * VEC + 2 * h]) = (pass == 0) ? dw[j][h] : db[j][h];
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
