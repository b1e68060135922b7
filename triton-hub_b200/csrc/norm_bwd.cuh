// Backward kernels: LayerNorm (TritonHub/Normalization/layernorm.py:94-153) and RMSNorm
// (TritonHub/Normalization/rmsnorm.py:77-122).  Both leave fp32 dweight / dbias partial rows
// that the column reduce in norm_colreduce.cuh finishes.
#pragma once

#include "norm_common.cuh"

namespace b200norm {

struct BwdParams {
  const void* x;
  const void* dy;
  const void* w;      // may be null
  const float* mean;  // LayerNorm only
  const float* rstd;
  void* dx;
  float* dw_part;  // (P, N) fp32 partial rows, or null
  float* db_part;  // (P, N) fp32 partial rows, or null (always null for RMSNorm)
  int64_t x_stride;  // elements
  int64_t dy_stride;
  int64_t dx_stride;
  int64_t M;
  int64_t rows_per_shard;  // M / row_shards
  int ctas_per_shard;      // gridDim.x = row_shards * ctas_per_shard = P
  int N;
  int V;  // 16-byte packets per row (packet kernels only)
  int w_dtype;
};

// Packet kernel.  Same thread-to-column map as the forward kernel, so each thread owns a
// fixed set of columns and carries their dweight / dbias sums in fp32 registers across all
// the rows its row group visits.  x and dy stay packed in registers; xhat and w*dy are
// recomputed for the dx pass instead of being kept, which is what lets a 32 KB row fit.
// With PREFETCH the next row's packets are requested before the current row is reduced, so
// each row group always has loads in flight; the widest rows cannot spare those registers.
// The weight vector lives in shared memory as fp32.
//
// Row shards: CTA c serves shard c / ctas_per_shard and walks that shard's rows strided by
// ctas_per_shard * WARPS_M.  The rows a CTA sums, and their order, depend only on the shard's
// size -- not on how many shards this launch covers -- so one launch over 8 shards and 8
// launches (8 GPUs) over one shard each produce the same partial rows bit for bit.
template <typename T, int LDGS, int WARPS_M, int WARPS_N, bool PREFETCH, bool RMS>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32) norm_bwd_kernel(const BwdParams p) {
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int TPR = WARPS_N * 32;
  constexpr int NV = RMS ? 1 : 2;
  extern __shared__ __align__(16) float dyn_smem[];  // w as fp32 (N), later (WARPS_M, N) sums
  __shared__ float red_smem[WARPS_M][2 * NV * WARPS_N];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int t = warp_n * 32 + lane;
  int phase = 0;

  float* w_s = dyn_smem;
  for (int c = threadIdx.x; c < p.N; c += WARPS_M * TPR)
    w_s[c] = (p.w != nullptr) ? load_param(p.w, p.w_dtype, c) : 1.f;
  __syncthreads();

  const int shard = blockIdx.x / p.ctas_per_shard;
  const int cta_in_shard = blockIdx.x - shard * p.ctas_per_shard;
  const int64_t row_begin = (int64_t)shard * p.rows_per_shard;
  const int64_t row_end = min(row_begin + p.rows_per_shard, p.M);
  const int64_t step = (int64_t)p.ctas_per_shard * WARPS_M;
  int64_t row = row_begin + (int64_t)cta_in_shard * WARPS_M + warp_m;

  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dy);
  T* dxb = static_cast<T*>(p.dx);
  const float inv_n = 1.f / static_cast<float>(p.N);

  float dw[LDGS][VEC], db[LDGS][VEC];
#pragma unroll
  for (int j = 0; j < LDGS; ++j)
#pragma unroll
    for (int e = 0; e < VEC; ++e) dw[j][e] = db[j][e] = 0.f;

  uint4 xv[LDGS], gv[LDGS];
  float mu = 0.f, rs = 0.f;
  auto fetch = [&](int64_t r, uint4* xo, uint4* go, float& m_o, float& r_o) {
    const uint4* xrow = reinterpret_cast<const uint4*>(xb + r * p.x_stride);
    const uint4* grow = reinterpret_cast<const uint4*>(gb + r * p.dy_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      xo[j] = make_uint4(0, 0, 0, 0);
      go[j] = make_uint4(0, 0, 0, 0);
      if (v < p.V) {
        xo[j] = ld_stream(xrow + v);
        go[j] = ld_stream(grow + v);
      }
    }
    m_o = RMS ? 0.f : __ldg(p.mean + r);
    r_o = __ldg(p.rstd + r);
  };

  if (row < row_end) fetch(row, xv, gv, mu, rs);
  while (row < row_end) {
    const int64_t next = row + step;
    constexpr int NL = PREFETCH ? LDGS : 1;
    uint4 xn[NL], gn[NL];
    float mun = 0.f, rsn = 0.f;
    if (PREFETCH) {
      if (next < row_end) fetch(next, xn, gn, mun, rsn);
    }

    // Pass 1: dweight / dbias sums and the two row sums (layernorm.py:132-138).
    float s[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) s[i] = 0.f;
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      if (v < p.V) {
        float xf[VEC], gf[VEC];
        Pack16<T>::unpack(xv[j], xf);
        Pack16<T>::unpack(gv[j], gf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float xh = (xf[e] - mu) * rs;
          const float wdy = w_s[v * VEC + e] * gf[e];
          dw[j][e] += gf[e] * xh;
          if (!RMS) db[j][e] += gf[e];
          s[0] += xh * wdy;
          if (!RMS) s[NV - 1] += wdy;
        }
      }
    }
    group_sum<WARPS_N, NV>(s, red_smem[warp_m], phase, warp_m, warp_n, lane);
    const float c1 = s[0] * inv_n;
    const float c2 = RMS ? 0.f : s[NV - 1] * inv_n;

    // Pass 2: dx = (wdy - (xhat*c1 + c2)) * rstd (layernorm.py:139).
    uint4* dxrow = reinterpret_cast<uint4*>(dxb + row * p.dx_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      if (v < p.V) {
        float xf[VEC], gf[VEC], o[VEC];
        Pack16<T>::unpack(xv[j], xf);
        Pack16<T>::unpack(gv[j], gf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float xh = (xf[e] - mu) * rs;
          const float wdy = w_s[v * VEC + e] * gf[e];
          o[e] = (wdy - (xh * c1 + c2)) * rs;
        }
        st_stream(dxrow + v, Pack16<T>::pack(o));
      }
    }

    row = next;
    if (PREFETCH) {
#pragma unroll
      for (int j = 0; j < NL; ++j) {
        xv[j] = xn[j];
        gv[j] = gn[j];
      }
      mu = mun;
      rs = rsn;
    } else if (row < row_end) {
      fetch(row, xv, gv, mu, rs);
    }
  }

  // One partial row per CTA: add the row groups in order, then row group 0 stores.
  if (WARPS_M > 1) {
    float* acc = dyn_smem;  // (WARPS_M, N); the weights are no longer needed
#pragma unroll
    for (int pass = 0; pass < NV; ++pass) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        if (v < p.V) {
#pragma unroll
          for (int e = 0; e < VEC; ++e)
            acc[(size_t)warp_m * p.N + v * VEC + e] = (pass == 0) ? dw[j][e] : db[j][e];
        }
      }
      __syncthreads();
      if (warp_m == 0) {
#pragma unroll
        for (int j = 0; j < LDGS; ++j) {
          const int v = j * TPR + t;
          if (v < p.V) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
              float a = 0.f;
              for (int m = 0; m < WARPS_M; ++m) a += acc[(size_t)m * p.N + v * VEC + e];
              if (pass == 0) dw[j][e] = a;
              else db[j][e] = a;
            }
          }
        }
      }
    }
  }
  if (warp_m == 0) {
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      if (v < p.V) {
        const size_t o = (size_t)blockIdx.x * p.N + (size_t)v * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          if (p.dw_part != nullptr) p.dw_part[o + e] = dw[j][e];
          if (!RMS && p.db_part != nullptr) p.db_part[o + e] = db[j][e];
        }
      }
    }
  }
}

// Any-alignment dx kernel: one CTA per row, two scalar passes.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_bwd_dx_any_kernel(const BwdParams p) {
  constexpr int NV = RMS ? 1 : 2;
  __shared__ float red[2 * NV * 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int phase = 0;
  const float inv_n = 1.f / static_cast<float>(p.N);
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    const T* xrow = static_cast<const T*>(p.x) + row * p.x_stride;
    const T* grow = static_cast<const T*>(p.dy) + row * p.dy_stride;
    T* dxrow = static_cast<T*>(p.dx) + row * p.dx_stride;
    const float mu = RMS ? 0.f : p.mean[row];
    const float rs = p.rstd[row];
    float s[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) s[i] = 0.f;
    for (int c = threadIdx.x; c < p.N; c += 256) {
      const float xh = (to_f32(xrow[c]) - mu) * rs;
      const float wv = (p.w != nullptr) ? load_param(p.w, p.w_dtype, c) : 1.f;
      const float wdy = wv * to_f32(grow[c]);
      s[0] += xh * wdy;
      if (!RMS) s[NV - 1] += wdy;
    }
    group_sum<8, NV>(s, red, phase, -1, warp, lane);
    const float c1 = s[0] * inv_n;
    const float c2 = RMS ? 0.f : s[NV - 1] * inv_n;
    for (int c = threadIdx.x; c < p.N; c += 256) {
      const float xh = (to_f32(xrow[c]) - mu) * rs;
      const float wv = (p.w != nullptr) ? load_param(p.w, p.w_dtype, c) : 1.f;
      const float wdy = wv * to_f32(grow[c]);
      dxrow[c] = from_f32<T>((wdy - (xh * c1 + c2)) * rs);
    }
  }
}

// Any-alignment dweight / dbias kernel: one thread per column, blockIdx.y = partial row.
// Partial row q of shard s sums that shard's rows [q*chunk, (q+1)*chunk) in order.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_bwd_dwdb_any_kernel(const BwdParams p) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col >= p.N) return;
  const int shard = blockIdx.y / p.ctas_per_shard;
  const int q = blockIdx.y - shard * p.ctas_per_shard;
  const int64_t chunk = (p.rows_per_shard + p.ctas_per_shard - 1) / p.ctas_per_shard;
  const int64_t shard_begin = (int64_t)shard * p.rows_per_shard;
  const int64_t shard_end = min(shard_begin + p.rows_per_shard, p.M);
  const int64_t r0 = min(shard_begin + q * chunk, shard_end);
  const int64_t r1 = min(r0 + chunk, shard_end);
  float dw = 0.f, db = 0.f;
  for (int64_t r = r0; r < r1; ++r) {
    const float g = to_f32(static_cast<const T*>(p.dy)[r * p.dy_stride + col]);
    const float mu = RMS ? 0.f : p.mean[r];
    const float xh = (to_f32(static_cast<const T*>(p.x)[r * p.x_stride + col]) - mu) * p.rstd[r];
    dw += g * xh;
    db += g;
  }
  const size_t o = (size_t)blockIdx.y * p.N + col;
  if (p.dw_part != nullptr) p.dw_part[o] = dw;
  if (!RMS && p.db_part != nullptr) p.db_part[o] = db;
}

}  // namespace b200norm
