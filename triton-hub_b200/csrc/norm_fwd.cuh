// Forward kernels: LayerNorm (TritonHub/Normalization/layernorm.py:14-46) and RMSNorm
// (TritonHub/Normalization/rmsnorm.py:14-38) with the whole row held in registers.
#pragma once

#include "norm_act.cuh"
#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

struct FwdParams {
  const void* x;
  void* y;
  const void* w;  // may be null
  const void* b;  // may be null (always null for RMSNorm)
  float* mean;    // (M,) LayerNorm only
  float* rstd;    // (M,)
  int64_t x_stride;  // elements
  int64_t y_stride;
  int64_t M;
  int N;        // elements per row
  int V;        // 16-byte packets per row (packet kernels only)
  int w_dtype;  // storage type of w and b
  float eps;
  int* status;  // device status word for bounded waits that ran out
};

// Packet kernel.  A CTA is WARPS_M row groups of WARPS_N warps; a row group owns one row at a
// time and walks the rows grid-strided.  Thread t of the group holds packets t, t+TPR, ... of
// the row (LDGS of them, predicated on the row length), so every warp-wide access is one
// contiguous 512-byte segment.
//
// PREG: weight and bias sit in fp32 registers for the life of the CTA; without it each row
// re-reads them through L1 as packets (needs 16-byte aligned parameter vectors when they are
// stored as T), which frees registers for occupancy.
//
// STAGES > 0: rows reach the registers through a ring of STAGES shared-memory slots per row
// group, filled by bulk asynchronous copies (norm_stage.cuh).  The group's leader refills a
// slot right after the row's first reduction, which every thread passes only once its
// shared-memory reads have returned.  STAGES == 0: plain streaming loads from global memory.
//
// Statistics: when every thread of a row group holds the same number of elements, each thread
// forms the mean and the centred sum of squares of its own elements (two passes over registers,
// as layernorm.py:32-35 does for the whole row) and the group merges them with Chan's update
// (norm_common.cuh) in ONE reduction; ragged rows take the reference's two reductions.  Never
// E[x^2]-E[x]^2.
//
// MINB is the number of CTAs per SM the register allocation must leave room for.
//
// CL == 2: rows of 32 - 64 KB.  Launched in clusters of two CTAs; each CTA of a pair holds one
// half of the columns of every row the pair owns (so weight and bias still fit in registers) and
// the halves' statistics are swapped through distributed shared memory and merged in rank order.
//
// ACT != 0: the activation that follows the norm (GeLU) is applied to y before the store, so the
// normalised tensor never goes to memory on its own.
template <typename T, int LDGS, int WARPS_M, int WARPS_N, bool PREG, int STAGES, int MINB, int CL, int ACT, bool RMS>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32, MINB) norm_fwd_kernel(const FwdParams p) {
  static_assert(CL == 1 || (CL == 2 && WARPS_M == 1 && STAGES > 0), "cluster split: one row group per CTA, staged rows");
  constexpr int VEC = Pack16<T>::kElems;
  __shared__ __align__(8) PairBox<2> pair_box[2];  // CL == 2: the partner's statistics, double-buffered
  const uint32_t cr = (CL > 1) ? cluster_cta_rank() : 0u;
  const int unit = (CL > 1) ? static_cast<int>(blockIdx.x) / CL : static_cast<int>(blockIdx.x);
  const int units = static_cast<int>(gridDim.x) / CL;
  const int Vl = p.V / CL;                   // packets of each row this CTA handles ...
  const int v0 = static_cast<int>(cr) * Vl;  // ... starting at this one
  int pair_buf = 0;
  uint32_t pair_seq = 0;  // exchanges with the partner so far
  constexpr int TPR = WARPS_N * 32;  // threads per row
  constexpr int NBAR = STAGES > 0 ? WARPS_M * STAGES : 1;
  extern __shared__ __align__(128) unsigned char dyn_smem[];  // (WARPS_M, STAGES, row bytes)
  __shared__ float red_smem[WARPS_M][2 * 3 * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[NBAR];
  __shared__ int cta_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int t = warp_n * 32 + lane;
  int phase = 0;

  const T* xb = static_cast<const T*>(p.x);
  T* yb = static_cast<T*>(p.y);
  const int64_t first = (int64_t)unit * WARPS_M + warp_m;
  const int64_t step = (int64_t)units * WARPS_M;
  const uint32_t row_bytes = static_cast<uint32_t>(Vl) * 16u;
  unsigned char* slots = dyn_smem + (size_t)warp_m * STAGES * row_bytes;
  uint64_t* bars = full_bar + (STAGES > 0 ? warp_m * STAGES : 0);

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
  if (CL > 1) {
    if (threadIdx.x == 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) pair_box[0].w[i] = pair_box[1].w[i] = 0ull;
    }
    cluster_sync_all();  // the partner CTA is running and both boxes are clear: its shared memory may be written
  }
  auto first_fills = [&]() {  // the group leader requests the first STAGES rows
    if (STAGES > 0 && t == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) {
        const int64_t r = first + s * step;
        if (r < p.M) {
          mbar_expect_tx(&bars[s], row_bytes);
          bulk_load(slots + (size_t)s * row_bytes, xb + r * p.x_stride + (size_t)v0 * VEC, row_bytes, &bars[s]);
        }
      }
    }
  };

  // Per-element values live as fp32 pairs (two per instruction, norm_common.cuh): H pairs per packet.
  constexpr int H = VEC / 2;
  constexpr int PL = PREG ? LDGS : 1;
  float2 wr[PL][H], br[PL][H];
#pragma unroll
  for (int j = 0; j < PL; ++j) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      wr[j][h] = splat2(1.f);
      br[j][h] = splat2(0.f);
    }
  }
  if (PREG) {
    // weight and bias are requested first, the rows right behind them (see load_param_packets)
    load_param_packets<T, PL>(
        p.w, RMS ? nullptr : p.b, p.w_dtype, v0, t, TPR, Vl, [](int) { return true; }, first_fills,
        [&](int which, int j, const float* f) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
            if (which == 0) wr[j][h] = make_float2(f[2 * h], f[2 * h + 1]);
            else br[j][h] = make_float2(f[2 * h], f[2 * h + 1]);
          }
        });
  } else {
    first_fills();
  }

  const float inv_n = 1.f / static_cast<float>(p.N);
  const bool uniform = (Vl % TPR) == 0 && Vl >= TPR;  // every thread of a row group holds the same element count
  // uniform rows: each thread holds V / TPR packets
  const float thread_cnt = static_cast<float>((Vl / TPR) * VEC);
  const float thread_inv_cnt = 1.f / (thread_cnt > 0.f ? thread_cnt : 1.f);
  int slot = 0;
  uint32_t parity = 0;

  for (int64_t row = first; row < p.M; row += step) {
    float2 xf[LDGS][H];
    if (STAGES > 0) {
      mbar_wait(&bars[slot], parity, &cta_abort, p.status);
      const uint4* srow = reinterpret_cast<const uint4*>(slots + (size_t)slot * row_bytes);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        uint4 pk = make_uint4(0, 0, 0, 0);
        if (v < Vl) pk = ld_shared16(srow + v);
        Pack16<T>::unpack2(pk, xf[j]);
      }
    } else {
      const uint4* xrow = reinterpret_cast<const uint4*>(xb + row * p.x_stride) + v0;
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * TPR + t;
        uint4 pk = make_uint4(0, 0, 0, 0);
        if (v < Vl) pk = ld_stream(xrow + v);
        Pack16<T>::unpack2(pk, xf[j]);
      }
    }

    // Per-thread sums run as two chains (the lanes of a pair), added at the end.
    float mean = 0.f;
    float q[1] = {0.f};
    float2 q2 = splat2(0.f);
    if (!RMS) {
      float2 s2 = splat2(0.f);
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h) s2 = add2(s2, xf[j][h]);
      float s[1] = {s2.x + s2.y};
      if (uniform) {
        // One reduction: per-thread mean and centred squares, merged with Chan's update.
        float cnt = thread_cnt;
        mean = s[0] * thread_inv_cnt;
        const float2 nm = splat2(-mean);
#pragma unroll
        for (int j = 0; j < LDGS; ++j) {
          if ((j * TPR + t) < Vl) {
#pragma unroll
            for (int h = 0; h < H; ++h) {
              const float2 d = add2(xf[j][h], nm);
              q2 = fma2(d, d, q2);
            }
          }
        }
        q[0] = q2.x + q2.y;
        group_moments<WARPS_N, 0>(cnt, mean, q[0], red_smem[warp_m], phase, warp_m, warp_n, lane);
        if (CL > 1) {  // merge the two halves (equal counts), rank 0's first
          const float mine[2] = {mean, q[0]};
          float theirs[2];
          pair_swap<2>(mine, theirs, pair_box, pair_buf, ++pair_seq, cr, &cta_abort, p.status);
          const float m0 = cr == 0 ? mine[0] : theirs[0], m1 = cr == 0 ? theirs[0] : mine[0];
          const float q0 = cr == 0 ? mine[1] : theirs[1], q1 = cr == 0 ? theirs[1] : mine[1];
          const float d = m1 - m0;
          mean = 0.5f * (m0 + m1);
          q[0] = (q0 + q1) + d * d * (0.5f * cnt);
        }
      } else {
        // Ragged rows (threads hold different element counts): the reference's two passes,
        // mean first, then the centred sum of squares (layernorm.py:32-35).
        group_sum<WARPS_N, 1, 0>(s, red_smem[warp_m], phase, warp_m, warp_n, lane);
        if (CL > 1) {
          const float mine[2] = {s[0], 0.f};
          float theirs[2];
          pair_swap<2>(mine, theirs, pair_box, pair_buf, ++pair_seq, cr, &cta_abort, p.status);
          s[0] = cr == 0 ? mine[0] + theirs[0] : theirs[0] + mine[0];
        }
        mean = s[0] * inv_n;
      }
    } else {
#pragma unroll
      for (int j = 0; j < LDGS; ++j)
#pragma unroll
        for (int h = 0; h < H; ++h) q2 = fma2(xf[j][h], xf[j][h], q2);
      q[0] = q2.x + q2.y;
      group_sum<WARPS_N, 1, 0>(q, red_smem[warp_m], phase, warp_m, warp_n, lane);
      if (CL > 1) {
        const float mine[2] = {q[0], 0.f};
        float theirs[2];
        pair_swap<2>(mine, theirs, pair_box, pair_buf, ++pair_seq, cr, &cta_abort, p.status);
        q[0] = cr == 0 ? mine[0] + theirs[0] : theirs[0] + mine[0];
      }
    }
    if (STAGES > 0) {
      // Every thread of the group has its packets in registers: the slot can be refilled.
      if (t == 0) {
        const int64_t r = row + STAGES * step;
        if (r < p.M) {
          mbar_expect_tx(&bars[slot], row_bytes);
          bulk_load(slots + (size_t)slot * row_bytes, xb + r * p.x_stride + (size_t)v0 * VEC, row_bytes, &bars[slot]);
        }
      }
      if (++slot == STAGES) {
        slot = 0;
        parity ^= 1u;
      }
    }
    if (!RMS && !uniform) {
      const float2 nm = splat2(-mean);
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        if ((j * TPR + t) < Vl) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const float2 d = add2(xf[j][h], nm);
            q2 = fma2(d, d, q2);
          }
        }
      }
      q[0] = q2.x + q2.y;
      group_sum<WARPS_N, 1, 0>(q, red_smem[warp_m], phase, warp_m, warp_n, lane);
      if (CL > 1) {
        const float mine[2] = {q[0], 0.f};
        float theirs[2];
        pair_swap<2>(mine, theirs, pair_box, pair_buf, ++pair_seq, cr, &cta_abort, p.status);
        q[0] = cr == 0 ? mine[0] + theirs[0] : theirs[0] + mine[0];
      }
    }
    const float rstd = 1.f / sqrtf(q[0] * inv_n + p.eps);
    if (t == 0 && cr == 0) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }

    // y = (x - mean) * rstd * w + b (layernorm.py:38-45)
    uint4* yrow = reinterpret_cast<uint4*>(yb + row * p.y_stride) + v0;
    const float2 nm = splat2(-mean), r2 = splat2(rstd);
#pragma unroll
    for (int j = 0; j < LDGS; ++j) {
      const int v = j * TPR + t;
      float2 yf[H];
      if (PREG) {
#pragma unroll
        for (int h = 0; h < H; ++h) yf[h] = fma2(mul2(RMS ? xf[j][h] : add2(xf[j][h], nm), r2), wr[j][h], br[j][h]);
      } else if (v < Vl) {
        float wf[VEC], bf[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          wf[e] = 1.f;
          bf[e] = 0.f;
        }
        if (p.w != nullptr) load_param_packet<T>(p.w, p.w_dtype, v0 + v, wf);
        if (!RMS && p.b != nullptr) load_param_packet<T>(p.b, p.w_dtype, v0 + v, bf);
#pragma unroll
        for (int h = 0; h < H; ++h)
          yf[h] = fma2(mul2(RMS ? xf[j][h] : add2(xf[j][h], nm), r2), make_float2(wf[2 * h], wf[2 * h + 1]),
                       make_float2(bf[2 * h], bf[2 * h + 1]));
      }
      if (ACT != kActNone && v < Vl) {
#pragma unroll
        for (int h = 0; h < H; ++h) yf[h] = act_fwd2<ACT>(yf[h]);
      }
      if (v < Vl) st_stream(yrow + v, Pack16<T>::pack2(yf));
    }
  }
  if (STAGES > 0) {
    if (t == 0 && cta_abort) drain_ring<STAGES>(bars, first < p.M ? (p.M - first + step - 1) / step : 0);
  }
  if (CL > 1) cluster_sync_all();  // neither CTA of a pair leaves while the other may still store into it
}

}  // namespace b200norm
