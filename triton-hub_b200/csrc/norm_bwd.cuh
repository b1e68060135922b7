// Backward kernels: LayerNorm (TritonHub/Normalization/layernorm.py:94-153) and RMSNorm
// (TritonHub/Normalization/rmsnorm.py:77-122).  Both leave fp32 dweight / dbias partial rows
// that the column reduce in norm_colreduce.cuh finishes.
#pragma once

#include "norm_act.cuh"
#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

struct BwdParams {
  const void* x;
  const void* dy;
  const void* w;      // may be null
  const void* b;      // bias: only read when an activation is fused (to rebuild y); may be null
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
  int* status;  // device status word for bounded waits that ran out
};

// Packet kernel.  Same thread-to-column map as the forward kernel, so each thread owns a
// fixed set of columns and carries their dweight / dbias sums in fp32 registers across all
// the rows its row group visits.  x and dy stay packed in registers; xhat and w*dy are
// recomputed for the dx pass instead of being kept, which is what lets a 32 KB row fit.
// The weight vector lives in shared memory as fp32.
//
// How rows arrive:
//   STAGES > 0   x and dy rows are staged through a ring of STAGES shared-memory slots per row
//                group by bulk asynchronous copies (norm_stage.cuh); the leader refills a slot
//                right after the row's reduction, which every thread passes only once its
//                shared-memory reads have returned.
//   PREFETCH     (STAGES == 0) the next row's packets are requested into registers before the
//                current row is reduced.
//   neither      plain streaming loads, one row at a time.
//
// Row shards: CTA c serves shard c / ctas_per_shard and walks that shard's rows strided by
// ctas_per_shard * WARPS_M.  The rows a CTA sums, and their order, depend only on the shard's
// size -- not on how many shards this launch covers -- so one launch over 8 shards and 8
// launches (8 GPUs) over one shard each produce the same partial rows bit for bit.
//
// KEEP: xhat and w*dy of the current row stay in fp32 registers between the two passes
// instead of being recomputed from the packed row (fewer instructions, more registers).
// MINB is the number of CTAs per SM the register allocation must leave room for.
//
// CL == 2: rows wider than one CTA's registers can carry (32 - 64 KB).  The kernel is launched
// in clusters of two CTAs; each CTA of a pair stages, reduces and writes one half of the columns
// of every row the pair owns, and the two halves of the row sums are swapped through distributed
// shared memory (one remote store + one cluster barrier per row).  Both CTAs add the halves in
// rank order, so they hold identical sums.  A "unit" below is the CTA (CL == 1) or the pair.
//
// ACT != 0: the incoming gradient is that of act(y), not of y.  y = xhat*w + b is rebuilt from the
// row (the forward did not store it) inside pass 1 and the gradient is multiplied by act'(y);
// the rest of the kernel runs unchanged on it.
template <typename T, int LDGS, int WARPS_M, int WARPS_N, bool PREFETCH, int STAGES, bool KEEP, int MINB, int CL,
          int ACT, bool RMS>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, MINB) norm_bwd_kernel(const BwdParams p) {
  static_assert(CL == 1 || (CL == 2 && WARPS_M == 1 && STAGES > 0), "cluster split: one row group, staged rows");
  constexpr int VEC = Pack16<T>::kElems;
  constexpr int TPR = WARPS_N * 32;
  constexpr int NV = RMS ? 1 : 2;
  constexpr int NBAR = STAGES > 0 ? WARPS_M * STAGES : 1;
  __shared__ __align__(8) PairBox<NV> pair_box[2];  // CL == 2: the partner's row sums, double-buffered
  // w as fp32 (N), later the (WARPS_M, N) sums; then, 128-byte aligned, the row slots
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red_smem[WARPS_M][2 * NV * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[NBAR];
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int t = warp_n * 32 + lane;
  int phase = 0;

  const uint32_t cr = (CL > 1) ? cluster_cta_rank() : 0u;
  const int unit = (CL > 1) ? static_cast<int>(blockIdx.x) / CL : static_cast<int>(blockIdx.x);
  const int Vl = p.V / CL;                       // packets of each row this CTA handles ...
  const int v0 = static_cast<int>(cr) * Vl;      // ... starting at this one
  const int Nl = Vl * VEC;                       // the same in elements
  int pair_buf = 0;
  uint32_t pair_seq = 0;  // exchanges with the partner so far
  const int shard = unit / p.ctas_per_shard;
  const int cta_in_shard = unit - shard * p.ctas_per_shard;
  const int64_t row_begin = (int64_t)shard * p.rows_per_shard;
  const int64_t row_end = min(row_begin + p.rows_per_shard, p.M);
  const int64_t step = (int64_t)p.ctas_per_shard * WARPS_M;
  const int64_t first = row_begin + (int64_t)cta_in_shard * WARPS_M + warp_m;

  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dy);
  T* dxb = static_cast<T*>(p.dx);
  const float inv_n = 1.f / static_cast<float>(p.N);

  float* w_s = reinterpret_cast<float*>(dyn_smem);
  const uint32_t row_bytes = static_cast<uint32_t>(Vl) * 16u;
  // (WARPS_M, Nl) floats for the weights / later the row-group sums, then Nl floats of bias if fused
  const size_t param_bytes = ((size_t)(WARPS_M + (ACT != kActNone ? 1 : 0)) * Nl * sizeof(float) + 127) & ~(size_t)127;
  float* b_s = w_s + (size_t)WARPS_M * Nl;
  unsigned char* slots = dyn_smem + param_bytes + (size_t)warp_m * STAGES * 2 * row_bytes;
  uint64_t* bars = full_bar + (STAGES > 0 ? warp_m * STAGES : 0);

  auto fill = [&](int s, int64_t r) {  // leader only: x row then dy row into slot s
    unsigned char* dst = slots + (size_t)s * 2 * row_bytes;
    mbar_expect_tx(&bars[s], 2 * row_bytes);
    bulk_load(dst, xb + r * p.x_stride + (size_t)v0 * VEC, row_bytes, &bars[s]);
    bulk_load(dst + row_bytes, gb + r * p.dy_stride + (size_t)v0 * VEC, row_bytes, &bars[s]);
  };

  if (STAGES > 0) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < NBAR; ++i) mbar_init(&full_bar[i], 1);
      cta_abort = 0;
      mbar_init_fence();
    }
    __syncthreads();
  }
  grid_dependency_sync();  // nothing above reads global memory
  trigger_dependents();
  // The first rows are requested right behind the (small) parameter loads and land while the
  // parameters are staged (a CTA with a few dozen rows spends a visible share of its life here).
  // The copies go to this CTA's own shared memory, so a pair's partner need not be running yet.
  auto first_fills = [&]() {
    if (STAGES > 0 && t == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const int64_t r = first + s * step;
        if (r < row_end) fill(s, r);
      }
    }
  };
  // Parameters as fp32 in shared memory.  Thread t of row group m fetches the packets j * TPR + t with
  // j % WARPS_M == m: between them the groups cover every column once.
  if (p.w == nullptr)
    for (int c = threadIdx.x; c < Nl; c += WARPS_M * TPR) w_s[c] = 1.f;
  if (ACT != kActNone && (RMS || p.b == nullptr))
    for (int c = threadIdx.x; c < Nl; c += WARPS_M * TPR) b_s[c] = 0.f;
  load_param_packets<T, LDGS>(
      p.w, (ACT != kActNone && !RMS) ? p.b : nullptr, p.w_dtype, v0, t, TPR, Vl,
      [&](int j) { return WARPS_M == 1 || (j % WARPS_M) == warp_m; }, first_fills,
      [&](int which, int j, const float* f) {
        float* dst = (which == 0 ? w_s : b_s) + (j * TPR + t) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) dst[e] = f[e];
      });
  if (CL > 1 && threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) pair_box[0].w[i] = pair_box[1].w[i] = 0ull;
  }
  __syncthreads();
  if (CL > 1) cluster_sync_all();  // the partner CTA is running and both boxes are clear: its shared memory may be written

  // Per-element values live as fp32 pairs (two per instruction, norm_common.cuh): H pairs per packet.
  constexpr int H = VEC / 2;
  float2 dw[LDGS][H], db[LDGS][H];
#pragma unroll
  for (int j = 0; j < LDGS; ++j)
#pragma unroll
    for (int h = 0; h < H; ++h) dw[j][h] = db[j][h] = splat2(0.f);

  uint4 xv[LDGS], gv[LDGS];
  auto fetch = [&](int64_t r, uint4* xo, uint4* go) {  // STAGES == 0: straight from global
    const uint4* xrow = reinterpret_cast<const uint4*>(xb + r * p.x_stride);
    const uint4* grow = reinterpret_cast<const uint4*>(gb + r * p.dy_stride);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      xo[j] = make_uint4(0, 0, 0, 0);
      go[j] = make_uint4(0, 0, 0, 0);
      if (v < Vl) {
        xo[j] = ld_stream(xrow + v);
        go[j] = ld_stream(grow + v);
      }
    }
  };

  int64_t row = first;
  float mu = 0.f, rs = 0.f;
  if (row < row_end) {
    if (STAGES == 0) fetch(row, xv, gv);
    mu = RMS ? 0.f : __ldg(p.mean + row);
    rs = __ldg(p.rstd + row);
  }
  int slot = 0;
  uint32_t parity = 0;

  while (row < row_end) {
    const int64_t next = row + step;
    constexpr int NL = (PREFETCH && STAGES == 0) ? LDGS : 1;
    uint4 xn[NL], gn[NL];
    float mun = 0.f, rsn = 0.f;
    if (next < row_end) {  // the next row's statistics are always requested one row ahead
      mun = RMS ? 0.f : __ldg(p.mean + next);
      rsn = __ldg(p.rstd + next);
      if (PREFETCH && STAGES == 0) fetch(next, xn, gn);
    }
    if (STAGES > 0) {
      mbar_wait(&bars[slot], parity, &cta_abort, p.status);
      const uint4* sx = reinterpret_cast<const uint4*>(slots + (size_t)slot * 2 * row_bytes);
      const uint4* sg = reinterpret_cast<const uint4*>(slots + (size_t)slot * 2 * row_bytes + row_bytes);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        xv[j] = make_uint4(0, 0, 0, 0);
        gv[j] = make_uint4(0, 0, 0, 0);
        if (v < Vl) {
          xv[j] = ld_shared16(sx + v);
          gv[j] = ld_shared16(sg + v);
        }
      }
    }

    // Pass 1: dweight / dbias sums and the two row sums (layernorm.py:132-138).  The row sums run as
    // two chains (the lanes of a pair), added at the end.
    float2 s0 = splat2(0.f), s1 = splat2(0.f);
    constexpr int KL = KEEP ? LDGS : 1;
    float2 xh_k[KL][H], wdy_k[KL][H];
    const float2 nmu2 = splat2(-mu), rs2 = splat2(rs);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      if (v < Vl) {
        float2 xf[H], gf[H];
        Pack16<T>::unpack2(xv[j], xf);
        Pack16<T>::unpack2(gv[j], gf);
        const float2* w2 = reinterpret_cast<const float2*>(&w_s[v * VEC]);
        if (ACT != kActNone) {
          // dy = dz * act'(y) with y = xhat*w + b rebuilt from the row.  When pass 2 reads the packed
          // row again, dy replaces dz there, rounded to the storage type as a separate activation
          // backward would have stored it; the kept form carries it on in fp32.
          const float2* b2 = reinterpret_cast<const float2*>(&b_s[v * VEC]);
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const float2 y = fma2(mul2(RMS ? xf[h] : add2(xf[h], nmu2), rs2), w2[h], b2[h]);
            gf[h] = mul2(gf[h], act_grad2<ACT>(y));
          }
          if (!KEEP) {
            gv[j] = Pack16<T>::pack2(gf);
            Pack16<T>::unpack2(gv[j], gf);
          }
        }
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 xh = mul2(RMS ? xf[h] : add2(xf[h], nmu2), rs2);  // RMSNorm: mean is zero
          const float2 wdy = mul2(w2[h], gf[h]);
          dw[j][h] = fma2(gf[h], xh, dw[j][h]);
          if (!RMS) db[j][h] = add2(db[j][h], gf[h]);
          s0 = fma2(xh, wdy, s0);
          if (!RMS) s1 = add2(s1, wdy);
          if (KEEP) {
            xh_k[j][h] = xh;
            wdy_k[j][h] = wdy;
          }
        }
      }
    }
    float s[NV];
    s[0] = s0.x + s0.y;
    if (!RMS) s[NV - 1] = s1.x + s1.y;
    // With a single row group its barrier is the CTA's barrier 0; several groups keep 1, 2, ... because
    // a group that has finished its rows waits on barrier 0 (the final sum) while the others still loop.
    group_sum<WARPS_N, NV, (WARPS_M == 1 ? 0 : 1)>(s, red_smem[warp_m], phase, warp_m, warp_n, lane);
    if (CL > 1) {
      // Swap this half's sums with the partner's and add them in rank order.
      float other[NV];
      pair_swap<NV>(s, other, pair_box, pair_buf, ++pair_seq, cr, &cta_abort, p.status);
#pragma unroll
      for (int i = 0; i < NV; ++i) s[i] = (cr == 0) ? s[i] + other[i] : other[i] + s[i];
    }
    if (STAGES > 0) {
      // Every thread of the group holds its packets in registers: the slot can be refilled.
      if (t == 0) {
        const int64_t r = row + STAGES * step;
        if (r < row_end) fill(slot, r);
      }
      if (++slot == STAGES) {
        slot = 0;
        parity ^= 1u;
      }
    }
    const float c1 = s[0] * inv_n;
    const float c2 = RMS ? 0.f : s[NV - 1] * inv_n;

    // Pass 2: dx = (wdy - (xhat*c1 + c2)) * rstd (layernorm.py:139), with the row's scalars folded
    // so that each element costs two FMAs:
    //   kept   : dx = xhat * (-c1*rstd) + (wdy * rstd + (-c2*rstd))
    //   packed : dx = (w*rstd) * dy + (x * (-c1*rstd^2) + (c1*rstd^2*mean - c2*rstd))
    uint4* dxrow = reinterpret_cast<uint4*>(dxb + row * p.dx_stride) + v0;
    const float k1 = -c1 * rs, k2 = -c2 * rs;
    const float kb = k1 * rs, kc = -kb * mu + k2;
    const float2 k1_2 = splat2(k1), k2_2 = splat2(k2), kb2 = splat2(kb), kc2 = splat2(kc);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      if (v < Vl) {
        float2 o[H];
        if (KEEP) {
#pragma unroll
          for (int h = 0; h < H; ++h) o[h] = fma2(xh_k[j][h], k1_2, fma2(wdy_k[j][h], rs2, k2_2));
        } else {
          float2 xf[H], gf[H];
          Pack16<T>::unpack2(xv[j], xf);
          Pack16<T>::unpack2(gv[j], gf);
          const float2* w2 = reinterpret_cast<const float2*>(&w_s[v * VEC]);
#pragma unroll
          for (int h = 0; h < H; ++h) o[h] = fma2(mul2(w2[h], rs2), gf[h], fma2(xf[h], kb2, kc2));
        }
        st_stream(dxrow + v, Pack16<T>::pack2(o));
      }
    }

    row = next;
    mu = mun;
    rs = rsn;
    if (STAGES == 0) {
      if (PREFETCH) {
#pragma unroll
        for (int j = 0; j < NL; ++j) {
          xv[j] = xn[j];
          gv[j] = gn[j];
        }
      } else if (row < row_end) {
        fetch(row, xv, gv);
      }
    }
  }
  if (STAGES > 0) {
    if (t == 0 && cta_abort) drain_ring<STAGES>(bars, first < row_end ? (row_end - first + step - 1) / step : 0);
  }

  if (CL > 1) cluster_sync_all();  // neither CTA of a pair leaves while the other may still store into it
  // One partial row per unit: add the row groups in order, then row group 0 stores.
  if (WARPS_M > 1) {
    float* acc = reinterpret_cast<float*>(dyn_smem);  // (WARPS_M, N); the weights are no longer needed
#pragma unroll
    for (int pass = 0; pass < NV; ++pass) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        if (v < Vl) {
          float2* dst = reinterpret_cast<float2*>(&acc[(size_t)warp_m * Nl + v * VEC]);
#pragma unroll
          for (int h = 0; h < H; ++h) dst[h] = (pass == 0) ? dw[j][h] : db[j][h];
        }
      }
      __syncthreads();
      if (warp_m == 0) {
#pragma unroll
        for (int j = 0; j < LDGS; ++j) {
          const int v = j * TPR + t;
          if (v < Vl) {
#pragma unroll
            for (int h = 0; h < H; ++h) {
              float2 a = splat2(0.f);
              for (int m = 0; m < WARPS_M; ++m)
                a = add2(a, *reinterpret_cast<const float2*>(&acc[(size_t)m * Nl + v * VEC + 2 * h]));
              if (pass == 0) dw[j][h] = a;
              else db[j][h] = a;
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
      if (v < Vl) {
        // partial rows start 256-byte aligned and N is a whole number of packets: vector stores
        const size_t o = (size_t)unit * p.N + (size_t)(v0 + v) * VEC;
        if (p.dw_part != nullptr) st_f32_pairs<H>(p.dw_part + o, dw[j]);
        if (!RMS && p.db_part != nullptr) st_f32_pairs<H>(p.db_part + o, db[j]);
      }
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
#pragma unroll 8
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
