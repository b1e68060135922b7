// LayerNorm / RMSNorm for rows of ANY alignment: a base address, row stride or row length that is
// not a multiple of 16 bytes (odd lengths, offset views).  The reference runs such rows at full
// speed through masked vector loads (TritonHub/Normalization/layernorm.py:28-46, `cols < N`); the
// packet kernels cannot (their threads own fixed 16-byte packets), so these kernels stage each
// row through shared memory instead:
//
//   global -> shared : the row's aligned 16-byte interior by ONE bulk asynchronous copy completed
//                      on an mbarrier (norm_stage.cuh), the few elements before and after it one
//                      by one; the row lands at the same offset within a 16-byte line as in global
//                      memory, so element i sits at a fixed place whatever the row's alignment.
//                      A ring of up to four such slots per CTA keeps that many rows in flight;
//   shared -> shared : every pass (sum, centred squares, output) streams the row out of shared
//                      memory, thread t taking elements t, t + THREADS, ...: one trip to global
//                      memory per row, no element kept in a register across a reduction;
//   shared -> global : the result row is laid out at ITS alignment and written back with 128-bit
//                      stores for the interior.
//
// One CTA works on one row at a time and walks the rows grid-strided.  Forward: statistics by the
// reference's two passes (mean, then centred squares).  Backward: dx here, dweight / dbias by the
// column kernel in norm_bwd.cuh.  Every mbarrier wait is bounded like in the packet kernels.
#pragma once

#include "norm_bwd.cuh"
#include "norm_fwd.cuh"

namespace b200norm {

constexpr int kRowStagesMax = 4;

__device__ __forceinline__ uint32_t dynamic_smem_bytes() {
  uint32_t n;
  asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(n));
  return n;
}

// How a row of `n` elements of T at `ptr` (any alignment) splits into the elements before the first
// 16-byte boundary, the aligned interior and the elements after it.  In a slot, element i lives at
// slot + phase + i * sizeof(T); a slot is 16-byte aligned and holds n * sizeof(T) + 16 bytes.
// Last step of a CTA whose bounded wait ran out: copies it issued may still be in flight, so the
// leader lingers 10 ms before the CTA's shared memory is released (the packet kernels wait on
// their ring's barriers instead; here the number of slots is a run-time value).
__device__ __forceinline__ void linger_after_abort() {
  const unsigned long long t0 = global_ns();
  while (global_ns() - t0 < 10000000ull) {
  }
}

template <typename T>
struct RowSpan {
  int phase, head, body_bytes, tail0;
  __device__ __forceinline__ RowSpan(const T* ptr, int n) {
    constexpr int ES = static_cast<int>(sizeof(T));
    phase = static_cast<int>(reinterpret_cast<uintptr_t>(ptr) & 15u);
    head = min(n, ((16 - phase) & 15) / ES);   // elements before the first 16-byte boundary
    const int body = (n - head) * ES / 16;     // whole 16-byte packets after them
    body_bytes = body * 16;
    tail0 = head + body * (16 / ES);           // first element after the packets
  }
};

template <typename T>
__device__ __forceinline__ void copy_row_edges(unsigned char* shm, const T* src, int n, const RowSpan<T>& sp, int tid,
                                               int nthreads) {
  T* dst = reinterpret_cast<T*>(shm + sp.phase);
  if (tid < sp.head) dst[tid] = src[tid];
  for (int i = sp.tail0 + tid; i < n; i += nthreads) dst[i] = src[i];
}

// The mirror image: `n` elements laid out in shared memory at the phase of `dst` go to global memory.
template <typename T>
__device__ __forceinline__ void stage_row_out(const unsigned char* shm, T* dst, int n, int tid, int nthreads) {
  constexpr int ES = static_cast<int>(sizeof(T));
  const uintptr_t start = reinterpret_cast<uintptr_t>(dst);
  const int phase = static_cast<int>(start & 15u);
  const int head = min(n, ((16 - phase) & 15) / ES);
  const int body = (n - head) * ES / 16;
  const int tail0 = head + body * (16 / ES);
  const T* src = reinterpret_cast<const T*>(shm + phase);
  uint4* gdst = reinterpret_cast<uint4*>(dst + head);
  const uint4* ssrc = reinterpret_cast<const uint4*>(shm + phase + head * ES);
  for (int v = tid; v < body; v += nthreads) st_stream(gdst + v, ssrc[v]);
  if (tid < head) dst[tid] = src[tid];
  for (int i = tail0 + tid; i < n; i += nthreads) dst[i] = src[i];
}

// Parameter values of the columns tid, tid + nthreads, ... (K of them), `fill` past the end or
// without a parameter vector.  The storage type is switched on once, outside the loop, so that the
// K loads are issued together.
template <int K>
__device__ __forceinline__ void load_param_columns(const void* p, int dtype, int tid, int nthreads, int n, float fill,
                                                   float (&out)[K]) {
#pragma unroll
  for (int k = 0; k < K; ++k) out[k] = fill;
  if (p == nullptr) return;
  switch (dtype) {
    case kF32:
#pragma unroll
      for (int k = 0; k < K; ++k)
        if (tid + k * nthreads < n) out[k] = __ldg(static_cast<const float*>(p) + tid + k * nthreads);
      break;
    case kF16:
#pragma unroll
      for (int k = 0; k < K; ++k)
        if (tid + k * nthreads < n) out[k] = __half2float(__ldg(static_cast<const __half*>(p) + tid + k * nthreads));
      break;
    case kBF16:
#pragma unroll
      for (int k = 0; k < K; ++k)
        if (tid + k * nthreads < n)
          out[k] = __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(p) + tid + k * nthreads));
      break;
    default:
#pragma unroll
      for (int k = 0; k < K; ++k)
        if (tid + k * nthreads < n) out[k] = static_cast<float>(__ldg(static_cast<const double*>(p) + tid + k * nthreads));
      break;
  }
}

// Dynamic shared memory of these kernels: `rows` row buffers of row_buffer_bytes(N, sizeof(T)) each.
__host__ __device__ inline size_t row_buffer_bytes(int64_t N, int es) {
  return (static_cast<size_t>(N) * es + 16 + 15) & ~static_cast<size_t>(15);
}

// One parameter element of storage type P as fp32.
template <typename P>
__device__ __forceinline__ float param_at(const void* p, int c) {
  return to_f32(__ldg(static_cast<const P*>(p) + c));
}

// Calls body(tag) with a value of the parameter vectors' storage type, switched on ONCE outside the
// element loops.
template <typename Body>
__device__ __forceinline__ void with_param_type(int dtype, Body body) {
  switch (dtype) {
    case kF32: body(float{}); break;
    case kF16: body(__half{}); break;
    case kBF16: body(__nv_bfloat16{}); break;
    default: body(double{}); break;
  }
}

// Forward.  The staged row is streamed out of shared memory once per pass (sum, centred squares,
// output): no element lives in a register across a reduction, so one kernel shape serves every row
// length, nothing is predicated off for short rows and the register count stays low enough for
// several CTAs per SM.  Weight and bias are read through L1 as the output is formed.
// Dynamic shared memory: (stages + 1) row buffers -- the ring, then the output row.
template <typename T, int THREADS, bool RMS>
__global__ void __launch_bounds__(THREADS) norm_fwd_row_kernel(const FwdParams p) {
  constexpr int WARPS = THREADS / 32;
  constexpr int ES = static_cast<int>(sizeof(T));
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red[2 * WARPS];
  __shared__ __align__(8) uint64_t full_bar[kRowStagesMax];
  __shared__ int cta_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t buf = row_buffer_bytes(p.N, ES);
  const int stages = min(kRowStagesMax, static_cast<int>(dynamic_smem_bytes() / buf) - 1);
  unsigned char* s_out = dyn_smem + (size_t)stages * buf;
  int phase_bit = 0;
  const T* xb = static_cast<const T*>(p.x);
  const int N = p.N;

  auto fill = [&](int slot, int64_t row) {  // every thread calls it; the leader arms the barrier and copies
    const T* xrow = xb + row * p.x_stride;
    const RowSpan<T> sp(xrow, N);
    unsigned char* shm = dyn_smem + (size_t)slot * buf;
    if (tid == 0) {
      mbar_expect_tx(&full_bar[slot], static_cast<uint32_t>(sp.body_bytes));
      if (sp.body_bytes > 0)
        bulk_load(shm + sp.phase + sp.head * ES, xrow + sp.head, static_cast<uint32_t>(sp.body_bytes), &full_bar[slot]);
    }
    copy_row_edges<T>(shm, xrow, N, sp, tid, THREADS);
  };

  if (tid == 0) {
    for (int i = 0; i < kRowStagesMax; ++i) mbar_init(&full_bar[i], 1);
    cta_abort = 0;
    mbar_init_fence();
  }
  __syncthreads();
  for (int s = 0; s < stages; ++s) {
    const int64_t r = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
    if (r < p.M) fill(s, r);
  }
  __syncthreads();  // the edge elements of the first rows are in place
  const float inv_n = 1.f / static_cast<float>(N);
  int slot = 0;
  uint32_t parity = 0;
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    T* yrow = static_cast<T*>(p.y) + row * p.y_stride;
    mbar_wait(&full_bar[slot], parity, &cta_abort, p.status);
    const T* xs = reinterpret_cast<const T*>(dyn_smem + (size_t)slot * buf +
                                             (reinterpret_cast<uintptr_t>(xb + row * p.x_stride) & 15u));
    float mean = 0.f;
    if (!RMS) {
      float s[1] = {0.f};
#pragma unroll 4
      for (int c = tid; c < N; c += THREADS) s[0] += to_f32(xs[c]);
      group_sum<WARPS, 1, 0>(s, red, phase_bit, 0, warp, lane);
      mean = s[0] * inv_n;
    }
    float q[1] = {0.f};
#pragma unroll 4
    for (int c = tid; c < N; c += THREADS) {
      const float d = to_f32(xs[c]) - mean;
      q[0] += d * d;
    }
    group_sum<WARPS, 1, 0>(q, red, phase_bit, 0, warp, lane);
    const float rstd = 1.f / sqrtf(q[0] * inv_n + p.eps);
    if (tid == 0) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }
    // s_out is free: every thread passed the reductions above after its part of the previous copy-out
    T* ys = reinterpret_cast<T*>(s_out + static_cast<int>(reinterpret_cast<uintptr_t>(yrow) & 15u));
    with_param_type(p.w_dtype, [&](auto tag) {
      using P = decltype(tag);
      if (p.w != nullptr && !RMS && p.b != nullptr) {
#pragma unroll 4
        for (int c = tid; c < N; c += THREADS)
          ys[c] = from_f32<T>((to_f32(xs[c]) - mean) * rstd * param_at<P>(p.w, c) + param_at<P>(p.b, c));
      } else if (p.w != nullptr) {
#pragma unroll 4
        for (int c = tid; c < N; c += THREADS) ys[c] = from_f32<T>((to_f32(xs[c]) - mean) * rstd * param_at<P>(p.w, c));
      } else if (!RMS && p.b != nullptr) {
#pragma unroll 4
        for (int c = tid; c < N; c += THREADS) ys[c] = from_f32<T>((to_f32(xs[c]) - mean) * rstd + param_at<P>(p.b, c));
      } else {
#pragma unroll 4
        for (int c = tid; c < N; c += THREADS) ys[c] = from_f32<T>((to_f32(xs[c]) - mean) * rstd);
      }
    });
    __syncthreads();  // the output row is complete, and every thread is done reading the slot
    {
      const int64_t r = row + (int64_t)stages * gridDim.x;
      if (r < p.M) fill(slot, r);
      if (++slot == stages) {
        slot = 0;
        parity ^= 1u;
      }
    }
    stage_row_out<T>(s_out, yrow, N, tid, THREADS);
  }
  if (tid == 0 && cta_abort) linger_after_abort();
}

// Backward, dx only, streamed out of shared memory the same way (two passes over the staged x and dy
// rows).  Dynamic shared memory: (2 * stages + 1) row buffers -- the ring of (x, dy) pairs, then the
// output row.
template <typename T, int THREADS, bool RMS>
__global__ void __launch_bounds__(THREADS) norm_bwd_dx_row_kernel(const BwdParams p) {
  constexpr int WARPS = THREADS / 32;
  constexpr int NV = RMS ? 1 : 2;
  constexpr int ES = static_cast<int>(sizeof(T));
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red[2 * NV * WARPS];
  __shared__ __align__(8) uint64_t full_bar[kRowStagesMax];
  __shared__ int cta_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t buf = row_buffer_bytes(p.N, ES);
  const int stages = min(kRowStagesMax, (static_cast<int>(dynamic_smem_bytes() / buf) - 1) / 2);
  unsigned char* s_out = dyn_smem + (size_t)2 * stages * buf;
  int phase_bit = 0;
  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dy);
  const int N = p.N;

  auto fill = [&](int slot, int64_t row) {
    const T* xrow = xb + row * p.x_stride;
    const T* grow = gb + row * p.dy_stride;
    const RowSpan<T> sx(xrow, N), sg(grow, N);
    unsigned char* shx = dyn_smem + (size_t)(2 * slot) * buf;
    unsigned char* shg = shx + buf;
    if (tid == 0) {
      mbar_expect_tx(&full_bar[slot], static_cast<uint32_t>(sx.body_bytes + sg.body_bytes));
      if (sx.body_bytes > 0)
        bulk_load(shx + sx.phase + sx.head * ES, xrow + sx.head, static_cast<uint32_t>(sx.body_bytes), &full_bar[slot]);
      if (sg.body_bytes > 0)
        bulk_load(shg + sg.phase + sg.head * ES, grow + sg.head, static_cast<uint32_t>(sg.body_bytes), &full_bar[slot]);
    }
    copy_row_edges<T>(shx, xrow, N, sx, tid, THREADS);
    copy_row_edges<T>(shg, grow, N, sg, tid, THREADS);
  };

  if (tid == 0) {
    for (int i = 0; i < kRowStagesMax; ++i) mbar_init(&full_bar[i], 1);
    cta_abort = 0;
    mbar_init_fence();
  }
  __syncthreads();
  for (int s = 0; s < stages; ++s) {
    const int64_t r = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
    if (r < p.M) fill(s, r);
  }
  __syncthreads();
  const float inv_n = 1.f / static_cast<float>(N);
  int slot = 0;
  uint32_t parity = 0;
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    T* dxrow = static_cast<T*>(p.dx) + row * p.dx_stride;
    const float mu = RMS ? 0.f : __ldg(p.mean + row);
    const float rs = __ldg(p.rstd + row);
    mbar_wait(&full_bar[slot], parity, &cta_abort, p.status);
    const T* xs = reinterpret_cast<const T*>(dyn_smem + (size_t)(2 * slot) * buf +
                                             (reinterpret_cast<uintptr_t>(xb + row * p.x_stride) & 15u));
    const T* gs = reinterpret_cast<const T*>(dyn_smem + (size_t)(2 * slot + 1) * buf +
                                             (reinterpret_cast<uintptr_t>(gb + row * p.dy_stride) & 15u));
    T* os = reinterpret_cast<T*>(s_out + static_cast<int>(reinterpret_cast<uintptr_t>(dxrow) & 15u));
    with_param_type(p.w_dtype, [&](auto tag) {
      using P = decltype(tag);
      const bool has_w = p.w != nullptr;
      float s[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) s[i] = 0.f;
#pragma unroll 4
      for (int c = tid; c < N; c += THREADS) {
        const float xh = (to_f32(xs[c]) - mu) * rs;
        const float wdy = (has_w ? param_at<P>(p.w, c) : 1.f) * to_f32(gs[c]);
        s[0] += xh * wdy;
        if (!RMS) s[NV - 1] += wdy;
      }
      group_sum<WARPS, NV, 0>(s, red, phase_bit, 0, warp, lane);
      const float c1 = s[0] * inv_n;
      const float c2 = RMS ? 0.f : s[NV - 1] * inv_n;
      // s_out is free: every thread passed the reduction after its part of the previous copy-out
#pragma unroll 4
      for (int c = tid; c < N; c += THREADS) {
        const float xh = (to_f32(xs[c]) - mu) * rs;
        const float wdy = (has_w ? param_at<P>(p.w, c) : 1.f) * to_f32(gs[c]);
        os[c] = from_f32<T>((wdy - (xh * c1 + c2)) * rs);
      }
    });
    __syncthreads();  // the output row is complete, and every thread is done reading the slot
    {
      const int64_t r = row + (int64_t)stages * gridDim.x;
      if (r < p.M) fill(slot, r);
      if (++slot == stages) {
        slot = 0;
        parity ^= 1u;
      }
    }
    stage_row_out<T>(s_out, dxrow, N, tid, THREADS);
  }
  if (tid == 0 && cta_abort) linger_after_abort();
}

// ---------------------------------------------------------------------------------------
// Short rows of any alignment (at most 32 * K elements): one WARP per row, no shared memory.
// Lane l takes elements l, l + 32, ...: a warp's access is one contiguous run of the row, the
// K loads of a lane are all in flight at once, and the reductions are shuffles.  A CTA of eight
// warps works on eight rows at a time, so short rows no longer cost a whole CTA each.
// ---------------------------------------------------------------------------------------
constexpr int kWarpRowWarps = 8;

template <typename T, int K, bool RMS>
__global__ void __launch_bounds__(kWarpRowWarps * 32) norm_fwd_warp_row_kernel(const FwdParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kWarpRowWarps;
  float wr[K], br[K];
  load_param_columns<K>(p.w, p.w_dtype, lane, 32, p.N, 1.f, wr);
  load_param_columns<K>(RMS ? nullptr : p.b, p.w_dtype, lane, 32, p.N, 0.f, br);
  const float inv_n = 1.f / static_cast<float>(p.N);
  for (int64_t row = (int64_t)blockIdx.x * kWarpRowWarps + (threadIdx.x >> 5); row < p.M; row += warps) {
    const T* xrow = static_cast<const T*>(p.x) + row * p.x_stride;
    T* yrow = static_cast<T*>(p.y) + row * p.y_stride;
    T xraw[K];  // all loads first, then the conversions
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      xraw[k] = c < p.N ? xrow[c] : from_f32<T>(0.f);
    }
    float xv[K];
#pragma unroll
    for (int k = 0; k < K; ++k) xv[k] = to_f32(xraw[k]);
    float mean = 0.f;
    if (!RMS) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) s += xv[k];
      mean = warp_sum(s) * inv_n;
    }
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float d = (lane + 32 * k) < p.N ? xv[k] - mean : 0.f;
      q += d * d;
    }
    const float rstd = 1.f / sqrtf(warp_sum(q) * inv_n + p.eps);
    if (lane == 0) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      if (c < p.N) yrow[c] = from_f32<T>((xv[k] - mean) * rstd * wr[k] + br[k]);
    }
  }
}

template <typename T, int K, bool RMS>
__global__ void __launch_bounds__(kWarpRowWarps * 32) norm_bwd_dx_warp_row_kernel(const BwdParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kWarpRowWarps;
  float wr[K];
  load_param_columns<K>(p.w, p.w_dtype, lane, 32, p.N, 1.f, wr);
  const float inv_n = 1.f / static_cast<float>(p.N);
  for (int64_t row = (int64_t)blockIdx.x * kWarpRowWarps + (threadIdx.x >> 5); row < p.M; row += warps) {
    const T* xrow = static_cast<const T*>(p.x) + row * p.x_stride;
    const T* grow = static_cast<const T*>(p.dy) + row * p.dy_stride;
    T* dxrow = static_cast<T*>(p.dx) + row * p.dx_stride;
    const float mu = RMS ? 0.f : __ldg(p.mean + row);
    const float rs = __ldg(p.rstd + row);
    T xraw[K], graw[K];  // all loads first, then their uses
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      xraw[k] = c < p.N ? xrow[c] : from_f32<T>(0.f);
      graw[k] = c < p.N ? grow[c] : from_f32<T>(0.f);
    }
    // x and dy stay as loaded; xhat and w*dy are formed twice (three flops) instead of being kept, which
    // leaves the registers for having every load of the row in flight at once.
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const bool live = (lane + 32 * k) < p.N;
      const float xh = live ? (to_f32(xraw[k]) - mu) * rs : 0.f;
      const float wdy = live ? wr[k] * to_f32(graw[k]) : 0.f;
      s0 += xh * wdy;
      if (!RMS) s1 += wdy;
    }
    const float c1 = warp_sum(s0) * inv_n;
    const float c2 = RMS ? 0.f : warp_sum(s1) * inv_n;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      const float xh = (to_f32(xraw[k]) - mu) * rs;
      const float wdy = wr[k] * to_f32(graw[k]);
      if (c < p.N) dxrow[c] = from_f32<T>((wdy - (xh * c1 + c2)) * rs);
    }
  }
}

}  // namespace b200norm
