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
    if (stages == 1) __syncthreads();  // the edge elements other threads just wrote into the only slot
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
    if (stages == 1) __syncthreads();  // the edge elements other threads just wrote into the only slot
  }
  if (tid == 0 && cta_abort) linger_after_abort();
}

// ---------------------------------------------------------------------------------------
// Vector kernels for rows whose buffers SHARE one alignment: x and y (forward), or x, dy and dx
// (backward), start every row at the same offset within a 16-byte line -- rows of an odd length in
// contiguous tensors from one allocator, offset views of such tensors.  Then a row's 16-byte
// interior is made of the same columns in every buffer, and the packet arithmetic of the aligned
// kernels applies to it:
//
//   * the interior of each row is staged by one bulk asynchronous copy into a ring of shared-memory
//     slots and read from there with 128-bit loads; results go to global memory with 128-bit
//     stores straight from registers;
//   * the up to 2 * (16 / sizeof(T) - 1) elements before and after the interior belong to one thread
//     each of the CTA's last warp, which reads them from global memory a row ahead;
//   * the host sizes the grid so that all rows of a CTA have the same alignment (the alignment of
//     rows repeats with a period of at most 16 / sizeof(T) rows); the parameter vectors are copied
//     once per CTA into shared memory, shifted so that they line up with the interior's packets;
//   * backward: the CTA carries dweight / dbias of its columns in registers across its rows and
//     writes one partial row, like the packet kernels -- x and dy are read once.
//
// p.V carries the number of ring slots.  Dynamic shared memory: slots * (1 or 2) row interiors of
// (N * sizeof(T) / 16) * 16 bytes, then one (backward) or two (forward) parameter vectors of
// vrow_param_bytes() each.
// ---------------------------------------------------------------------------------------
__host__ __device__ inline size_t vrow_interior_bytes(int64_t N, int es) { return static_cast<size_t>(N * es / 16) * 16; }
__host__ __device__ inline int param_elem_size(int dtype) { return dtype == kF32 ? 4 : dtype == kF64 ? 8 : 2; }
__host__ __device__ inline size_t vrow_param_bytes(int64_t N, int w_dtype) {
  return (static_cast<size_t>(N) * param_elem_size(w_dtype) + 15) & ~static_cast<size_t>(15);
}

// EPP parameter values of storage type P, packet v of the shifted copy in shared memory.
template <typename P, int EPP>
__device__ __forceinline__ void ld_param_chunk(const unsigned char* base, int v, float2 (&out)[EPP / 2]) {
  struct alignas((sizeof(P) * EPP > 16) ? 16 : sizeof(P) * EPP) Chunk {
    P e[EPP];
  };
  const Chunk c = reinterpret_cast<const Chunk*>(base)[v];
#pragma unroll
  for (int i = 0; i < EPP / 2; ++i) out[i] = make_float2(to_f32(c.e[2 * i]), to_f32(c.e[2 * i + 1]));
}

// dst[i] = src[i], i < n, element by element (the source has no alignment to speak of).
template <typename U>
__device__ __forceinline__ void copy_elements(void* dst, const void* src, int n, int tid, int nthreads) {
#pragma unroll 8
  for (int i = tid; i < n; i += nthreads) static_cast<U*>(dst)[i] = __ldg(static_cast<const U*>(src) + i);
}
__device__ __forceinline__ void stage_params(unsigned char* dst, const void* src, int first, int n, int dtype, int tid,
                                             int nthreads) {
  const unsigned char* from = static_cast<const unsigned char*>(src) + (size_t)first * param_elem_size(dtype);
  if (dtype == kF32) copy_elements<uint32_t>(dst, from, n, tid, nthreads);
  else if (dtype == kF64) copy_elements<unsigned long long>(dst, from, n, tid, nthreads);
  else copy_elements<unsigned short>(dst, from, n, tid, nthreads);
}
__device__ __forceinline__ float param_scalar(const void* p, int dtype, int c, float fill) {
  if (p == nullptr) return fill;
  switch (dtype) {
    case kF32: return param_at<float>(p, c);
    case kF16: return param_at<__half>(p, c);
    case kBF16: return param_at<__nv_bfloat16>(p, c);
    default: return param_at<double>(p, c);
  }
}

// A pair of copies of a row-wide scalar in ordinary registers.  Row statistics are the same in every
// thread, and a compiler that notices keeps them in warp-uniform registers, from where every packed
// instruction that uses them first has to fetch them; the opaque statement pins them per thread.
__device__ __forceinline__ float2 splat2_pinned(float v) {
  asm volatile("" : "+f"(v));
  return make_float2(v, v);
}

// The output pass of the forward kernel over the interior packets of one row.
template <typename T, typename P, int GT, bool HAS_W, bool HAS_B>
__device__ __forceinline__ void vrow_fwd_out(const uint4* xs4, const unsigned char* s_w, const unsigned char* s_b,
                                             uint4* ybody, int VB, int gtid, float mean, float rstd) {
  constexpr int EPP = Pack16<T>::kElems, H = EPP / 2;
  const float2 nm = splat2_pinned(-mean), rs = splat2_pinned(rstd);
#pragma unroll 2
  for (int v = gtid; v < VB; v += GT) {
    float2 f[H], w[H], b[H];
    Pack16<T>::unpack2(xs4[v], f);
    if (HAS_W) ld_param_chunk<P, EPP>(s_w, v, w);
    if (HAS_B) ld_param_chunk<P, EPP>(s_b, v, b);
#pragma unroll
    for (int h = 0; h < H; ++h) {
      float2 t = mul2(add2(f[h], nm), rs);
      if (HAS_W && HAS_B) t = fma2(t, w[h], b[h]);
      else if (HAS_W) t = mul2(t, w[h]);
      else if (HAS_B) t = add2(t, b[h]);
      f[h] = t;
    }
    st_stream(ybody + v, Pack16<T>::pack2(f));
  }
}
template <typename T, typename P, int GT>
__device__ __forceinline__ void vrow_fwd_out_any(bool has_w, bool has_b, const uint4* xs4, const unsigned char* s_w,
                                                 const unsigned char* s_b, uint4* ybody, int VB, int gtid, float mean,
                                                 float rstd) {
  if (has_w && has_b) vrow_fwd_out<T, P, GT, true, true>(xs4, s_w, s_b, ybody, VB, gtid, mean, rstd);
  else if (has_w) vrow_fwd_out<T, P, GT, true, false>(xs4, s_w, s_b, ybody, VB, gtid, mean, rstd);
  else if (has_b) vrow_fwd_out<T, P, GT, false, true>(xs4, s_w, s_b, ybody, VB, gtid, mean, rstd);
  else vrow_fwd_out<T, P, GT, false, false>(xs4, s_w, s_b, ybody, VB, gtid, mean, rstd);
}

// A CTA is WARPS_M row groups of WARPS_N warps; each group works on a row of its own, with its own
// ring of slots, and the groups share the CTA's copy of the parameter vectors.  Group g of CTA c
// takes rows c + (g + i * WARPS_M) * gridDim.x, i = 0, 1, ...
template <typename T, int WARPS_M, int WARPS_N, bool RMS>
__global__ void __launch_bounds__(32 * WARPS_M * WARPS_N) norm_fwd_vrow_kernel(const FwdParams p) {
  constexpr int GT = 32 * WARPS_N, THREADS = GT * WARPS_M;
  constexpr int ES = static_cast<int>(sizeof(T)), EPP = Pack16<T>::kElems, H = EPP / 2;
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red[WARPS_M][2 * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[WARPS_M][kRowStagesMax];
  __shared__ int cta_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp - warp_m * WARPS_N, gtid = tid - warp_m * GT;
  const int N = p.N, stages = p.V;
  const size_t slot_bytes = vrow_interior_bytes(N, ES);
  const T* xb = static_cast<const T*>(p.x);
  T* yb = static_cast<T*>(p.y);
  const int64_t row0 = blockIdx.x + (int64_t)warp_m * gridDim.x, step = (int64_t)WARPS_M * gridDim.x;
  // the same for every row of this CTA
  const RowSpan<T> sp(xb + (int64_t)blockIdx.x * p.x_stride, N);
  const int VB = sp.body_bytes / 16;
  const int edges = sp.head + (N - sp.tail0);
  unsigned char* ring = dyn_smem + (size_t)warp_m * stages * slot_bytes;
  unsigned char* s_w = dyn_smem + (size_t)WARPS_M * stages * slot_bytes;
  unsigned char* s_b = s_w + vrow_param_bytes(N, p.w_dtype);
  const bool has_w = p.w != nullptr, has_b = !RMS && p.b != nullptr;
  int phase_bit = 0;

  auto fill = [&](int slot, int64_t row) {  // the group's leader only
    mbar_expect_tx(&full_bar[warp_m][slot], static_cast<uint32_t>(sp.body_bytes));
    bulk_load(ring + (size_t)slot * slot_bytes, xb + row * p.x_stride + sp.head, static_cast<uint32_t>(sp.body_bytes),
              &full_bar[warp_m][slot]);
  };

  if (tid == 0) cta_abort = 0;
  if (gtid == 0) {
    for (int i = 0; i < kRowStagesMax; ++i) mbar_init(&full_bar[warp_m][i], 1);
    mbar_init_fence();
    for (int s = 0; s < stages; ++s) {
      const int64_t r = row0 + (int64_t)s * step;
      if (r < p.M) fill(s, r);
    }
  }
  // this thread's edge element, if it has one: the group's last warp holds them
  const int ej = gtid - (GT - 32);
  const bool is_edge = ej >= 0 && ej < edges && row0 < p.M;
  const int ecol = is_edge ? (ej < sp.head ? ej : sp.tail0 + (ej - sp.head)) : 0;
  float xe_next = 0.f, we = 1.f, be = 0.f;
  const T* xe_ptr = xb + row0 * p.x_stride + ecol;
  if (is_edge) {
    xe_next = to_f32(*xe_ptr);
    we = param_scalar(p.w, p.w_dtype, ecol, 1.f);
    be = RMS ? 0.f : param_scalar(p.b, p.w_dtype, ecol, 0.f);
  }
  if (has_w) stage_params(s_w, p.w, sp.head, VB * EPP, p.w_dtype, tid, THREADS);
  if (has_b) stage_params(s_b, p.b, sp.head, VB * EPP, p.w_dtype, tid, THREADS);
  __syncthreads();  // barriers initialised, parameters in place

  const float inv_n = 1.f / static_cast<float>(N);
  const int64_t xe_step = step * p.x_stride;
  int slot = 0, prev_slot = -1;
  uint32_t parity = 0;
  for (int64_t row = row0; row < p.M; row += step) {
    const float xe = xe_next;
    xe_ptr += xe_step;
    if (is_edge && row + step < p.M) xe_next = to_f32(*xe_ptr);
    mbar_wait(&full_bar[warp_m][slot], parity, &cta_abort, p.status);
    const uint4* xs4 = reinterpret_cast<const uint4*>(ring + (size_t)slot * slot_bytes);
    float mean = 0.f;
    if (!RMS) {
      float2 a = splat2(0.f);
#pragma unroll 4
      for (int v = gtid; v < VB; v += GT) {
        float2 f[H];
        Pack16<T>::unpack2(xs4[v], f);
#pragma unroll
        for (int h = 0; h < H; ++h) a = add2(a, f[h]);
      }
      float s[1] = {a.x + a.y + (is_edge ? xe : 0.f)};
      group_sum<WARPS_N, 1>(s, red[warp_m], phase_bit, warp_m, warp_n, lane);
      mean = s[0] * inv_n;
    }
    float2 q2 = splat2(0.f);
    {
      const float2 nm = splat2_pinned(-mean);
#pragma unroll 4
      for (int v = gtid; v < VB; v += GT) {
        float2 f[H];
        Pack16<T>::unpack2(xs4[v], f);
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 d = RMS ? f[h] : add2(f[h], nm);
          q2 = fma2(d, d, q2);
        }
      }
    }
    float q[1] = {q2.x + q2.y + (is_edge ? (xe - mean) * (xe - mean) : 0.f)};
    group_sum<WARPS_N, 1>(q, red[warp_m], phase_bit, warp_m, warp_n, lane);
    // every thread of the group is past the previous row's output pass: its slot can take the row
    // `stages` on
    if (gtid == 0 && prev_slot >= 0) {
      const int64_t r = row + (int64_t)(stages - 1) * step;
      if (r < p.M) fill(prev_slot, r);
    }
    const float rstd = 1.f / sqrtf(q[0] * inv_n + p.eps);
    if (gtid == 0) {
      if (!RMS) p.mean[row] = mean;
      p.rstd[row] = rstd;
    }
    T* yrow = yb + row * p.y_stride;
    uint4* ybody = reinterpret_cast<uint4*>(yrow + sp.head);
    switch (p.w_dtype) {
      case kF32: vrow_fwd_out_any<T, float, GT>(has_w, has_b, xs4, s_w, s_b, ybody, VB, gtid, mean, rstd); break;
      case kF16: vrow_fwd_out_any<T, __half, GT>(has_w, has_b, xs4, s_w, s_b, ybody, VB, gtid, mean, rstd); break;
      case kBF16: vrow_fwd_out_any<T, __nv_bfloat16, GT>(has_w, has_b, xs4, s_w, s_b, ybody, VB, gtid, mean, rstd); break;
      default: vrow_fwd_out_any<T, double, GT>(has_w, has_b, xs4, s_w, s_b, ybody, VB, gtid, mean, rstd); break;
    }
    if (is_edge) yrow[ecol] = from_f32<T>((xe - mean) * rstd * we + be);
    if (WARPS_N == 1) __syncwarp();  // the refill above relies on the group having finished this row
    prev_slot = slot;
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  if (tid == 0 && cta_abort) linger_after_abort();
}

// The two passes of the backward kernel over the interior packets of one row.
template <typename T, typename P, int GT, int K, bool RMS, bool HAS_W, bool KEEP>
__device__ __forceinline__ void vrow_bwd_sums(const uint4* xs4, const uint4* gs4, const unsigned char* s_w, int VB, int gtid,
                                              float mu, float rs, float2 (&acc_w)[K][Pack16<T>::kElems / 2],
                                              float2 (&acc_b)[K][Pack16<T>::kElems / 2], float2& s0, float2& s1,
                                              float2 (&kept_xh)[KEEP ? K : 1][Pack16<T>::kElems / 2],
                                              float2 (&kept_wdy)[KEEP ? K : 1][Pack16<T>::kElems / 2]) {
  constexpr int EPP = Pack16<T>::kElems, H = EPP / 2;
  const float2 nm = splat2_pinned(-mu), r2 = splat2_pinned(rs);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = gtid + k * GT;
    if (v < VB) {
      float2 x[H], g[H], w[H];
      Pack16<T>::unpack2(xs4[v], x);
      Pack16<T>::unpack2(gs4[v], g);
      if (HAS_W) ld_param_chunk<P, EPP>(s_w, v, w);
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const float2 xh = RMS ? mul2(x[h], r2) : mul2(add2(x[h], nm), r2);
        const float2 wdy = HAS_W ? mul2(w[h], g[h]) : g[h];
        s0 = fma2(xh, wdy, s0);
        if (!RMS) s1 = add2(s1, wdy);
        acc_w[k][h] = fma2(g[h], xh, acc_w[k][h]);
        if (!RMS) acc_b[k][h] = add2(acc_b[k][h], g[h]);
        if (KEEP) {
          kept_xh[k][h] = xh;
          kept_wdy[k][h] = wdy;
        }
      }
    }
  }
}
// The dx pass from xhat and w * dy kept in registers by the pass above.
template <typename T, int GT, int K, bool RMS>
__device__ __forceinline__ void vrow_bwd_dx_kept(uint4* dxbody, int VB, int gtid, float rs, float c1, float c2,
                                                 const float2 (&kept_xh)[K][Pack16<T>::kElems / 2],
                                                 const float2 (&kept_wdy)[K][Pack16<T>::kElems / 2]) {
  constexpr int H = Pack16<T>::kElems / 2;
  const float2 r2 = splat2_pinned(rs), nc1 = splat2_pinned(-c1), nc2 = splat2_pinned(-c2);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = gtid + k * GT;
    if (v < VB) {
      float2 o[H];
#pragma unroll
      for (int h = 0; h < H; ++h) o[h] = mul2(add2(kept_wdy[k][h], fma2(kept_xh[k][h], nc1, nc2)), r2);
      st_stream(dxbody + v, Pack16<T>::pack2(o));
    }
  }
}
template <typename T, typename P, int GT, int K, bool RMS, bool HAS_W>
__device__ __forceinline__ void vrow_bwd_dx(const uint4* xs4, const uint4* gs4, const unsigned char* s_w, uint4* dxbody,
                                            int VB, int gtid, float mu, float rs, float c1, float c2) {
  constexpr int EPP = Pack16<T>::kElems, H = EPP / 2;
  const float2 nm = splat2_pinned(-mu), r2 = splat2_pinned(rs), nc1 = splat2_pinned(-c1), nc2 = splat2_pinned(-c2);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = gtid + k * GT;
    if (v < VB) {
      float2 x[H], g[H], w[H];
      Pack16<T>::unpack2(xs4[v], x);
      Pack16<T>::unpack2(gs4[v], g);
      if (HAS_W) ld_param_chunk<P, EPP>(s_w, v, w);
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const float2 xh = RMS ? mul2(x[h], r2) : mul2(add2(x[h], nm), r2);
        const float2 wdy = HAS_W ? mul2(w[h], g[h]) : g[h];
        x[h] = mul2(add2(wdy, fma2(xh, nc1, nc2)), r2);  // (wdy - (xh * c1 + c2)) * rstd
      }
      st_stream(dxbody + v, Pack16<T>::pack2(x));
    }
  }
}

// Backward: row groups as in the forward kernel, within a row shard -- CTA c of the shard's
// p.ctas_per_shard / WARPS_M serves rows c + (g + i * WARPS_M) * that count of the shard -- and one
// partial row of dweight / dbias per group (p.ctas_per_shard counts partial rows), each thread
// carrying the sums of its K interior packets (and its edge element) across the group's rows.
// KEEP: xhat and w * dy of the row stay in fp32 registers between the two passes (2 * K * 16 / sizeof(T)
// registers) instead of being formed again from shared memory: a third fewer instructions per row.
template <typename T, int WARPS_M, int WARPS_N, int K, bool KEEP, bool RMS>
__global__ void __launch_bounds__(32 * WARPS_M * WARPS_N, 512 / (32 * WARPS_M * WARPS_N)) norm_bwd_vrow_kernel(const BwdParams p) {
  constexpr int GT = 32 * WARPS_N, THREADS = GT * WARPS_M;
  constexpr int NV = RMS ? 1 : 2;
  constexpr int ES = static_cast<int>(sizeof(T)), EPP = Pack16<T>::kElems, H = EPP / 2;
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ float red[WARPS_M][2 * NV * WARPS_N];
  __shared__ __align__(8) uint64_t full_bar[WARPS_M][kRowStagesMax];
  __shared__ int cta_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp / WARPS_N, warp_n = warp - warp_m * WARPS_N, gtid = tid - warp_m * GT;
  const int N = p.N, stages = p.V;
  const size_t slot_bytes = vrow_interior_bytes(N, ES);
  const T* xb = static_cast<const T*>(p.x);
  const T* gb = static_cast<const T*>(p.dy);
  T* db = static_cast<T*>(p.dx);
  const int ctas = p.ctas_per_shard / WARPS_M;  // per shard
  const int shard = blockIdx.x / ctas, cta = blockIdx.x - shard * ctas;
  const int64_t shard_begin = (int64_t)shard * p.rows_per_shard;
  const int64_t shard_end = min(shard_begin + p.rows_per_shard, p.M);
  const int64_t row0 = shard_begin + cta + (int64_t)warp_m * ctas, step = (int64_t)WARPS_M * ctas;
  const size_t part = ((size_t)shard * p.ctas_per_shard + (size_t)cta * WARPS_M + warp_m) * N;
  float* dw_row = p.dw_part != nullptr ? p.dw_part + part : nullptr;
  float* db_row = (!RMS && p.db_part != nullptr) ? p.db_part + part : nullptr;
  const bool has_rows = row0 < shard_end;
  if (shard_begin + cta >= shard_end) {  // no row for this CTA: its partial rows are zero
    for (int c = gtid; c < N; c += GT) {
      if (dw_row != nullptr) dw_row[c] = 0.f;
      if (db_row != nullptr) db_row[c] = 0.f;
    }
    return;
  }
  // the same for every row of this CTA
  const RowSpan<T> sp(xb + (shard_begin + cta) * p.x_stride, N);
  const int VB = sp.body_bytes / 16;
  const int edges = sp.head + (N - sp.tail0);
  unsigned char* ring = dyn_smem + (size_t)warp_m * 2 * stages * slot_bytes;
  unsigned char* s_w = dyn_smem + (size_t)WARPS_M * 2 * stages * slot_bytes;
  const bool has_w = p.w != nullptr;
  int phase_bit = 0;

  auto fill = [&](int slot, int64_t row) {  // the group's leader only
    mbar_expect_tx(&full_bar[warp_m][slot], static_cast<uint32_t>(2 * sp.body_bytes));
    unsigned char* shx = ring + (size_t)(2 * slot) * slot_bytes;
    bulk_load(shx, xb + row * p.x_stride + sp.head, static_cast<uint32_t>(sp.body_bytes), &full_bar[warp_m][slot]);
    bulk_load(shx + slot_bytes, gb + row * p.dy_stride + sp.head, static_cast<uint32_t>(sp.body_bytes),
              &full_bar[warp_m][slot]);
  };

  if (tid == 0) cta_abort = 0;
  if (gtid == 0) {
    for (int i = 0; i < kRowStagesMax; ++i) mbar_init(&full_bar[warp_m][i], 1);
    mbar_init_fence();
    for (int s = 0; s < stages; ++s) {
      const int64_t r = row0 + (int64_t)s * step;
      if (r < shard_end) fill(s, r);
    }
  }
  const int ej = gtid - (GT - 32);
  const bool is_edge = ej >= 0 && ej < edges;
  const int ecol = is_edge ? (ej < sp.head ? ej : sp.tail0 + (ej - sp.head)) : 0;
  float xe_next = 0.f, ge_next = 0.f, we = 1.f, mu_next = 0.f, rs_next = 0.f;
  const T* xe_ptr = xb + row0 * p.x_stride + ecol;
  const T* ge_ptr = gb + row0 * p.dy_stride + ecol;
  if (has_rows) {
    if (is_edge) {
      xe_next = to_f32(*xe_ptr);
      ge_next = to_f32(*ge_ptr);
      we = param_scalar(p.w, p.w_dtype, ecol, 1.f);
    }
    if (!RMS) mu_next = __ldg(p.mean + row0);
    rs_next = __ldg(p.rstd + row0);
  }
  if (has_w) stage_params(s_w, p.w, sp.head, VB * EPP, p.w_dtype, tid, THREADS);
  __syncthreads();  // barriers initialised, weight in place

  float2 acc_w[K][H], acc_b[K][H];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int h = 0; h < H; ++h) acc_w[k][h] = acc_b[k][h] = splat2(0.f);
  float ew_acc = 0.f, eb_acc = 0.f;
  const float inv_n = 1.f / static_cast<float>(N);
  const int64_t xe_step = step * p.x_stride, ge_step = step * p.dy_stride;
  int slot = 0, prev_slot = -1;
  uint32_t parity = 0;
  for (int64_t row = row0; row < shard_end; row += step) {
    const float xe = xe_next, ge = ge_next, mu = mu_next, rs = rs_next;
    xe_ptr += xe_step;
    ge_ptr += ge_step;
    if (row + step < shard_end) {
      if (is_edge) {
        xe_next = to_f32(*xe_ptr);
        ge_next = to_f32(*ge_ptr);
      }
      if (!RMS) mu_next = __ldg(p.mean + row + step);
      rs_next = __ldg(p.rstd + row + step);
    }
    mbar_wait(&full_bar[warp_m][slot], parity, &cta_abort, p.status);
    const uint4* xs4 = reinterpret_cast<const uint4*>(ring + (size_t)(2 * slot) * slot_bytes);
    const uint4* gs4 = reinterpret_cast<const uint4*>(ring + (size_t)(2 * slot + 1) * slot_bytes);
    float2 s0 = splat2(0.f), s1 = splat2(0.f);
    float2 kept_xh[KEEP ? K : 1][H], kept_wdy[KEEP ? K : 1][H];
#define B200NORM_VROW_SUMS(P)                                                                                        \
  if (has_w)                                                                                                         \
    vrow_bwd_sums<T, P, GT, K, RMS, true, KEEP>(xs4, gs4, s_w, VB, gtid, mu, rs, acc_w, acc_b, s0, s1, kept_xh,      \
                                                kept_wdy);                                                           \
  else                                                                                                               \
    vrow_bwd_sums<T, P, GT, K, RMS, false, KEEP>(xs4, gs4, s_w, VB, gtid, mu, rs, acc_w, acc_b, s0, s1, kept_xh,     \
                                                 kept_wdy)
    switch (p.w_dtype) {
      case kF32: B200NORM_VROW_SUMS(float); break;
      case kF16: B200NORM_VROW_SUMS(__half); break;
      case kBF16: B200NORM_VROW_SUMS(__nv_bfloat16); break;
      default: B200NORM_VROW_SUMS(double); break;
    }
#undef B200NORM_VROW_SUMS
    float s[NV];
    s[0] = s0.x + s0.y;
    if (!RMS) s[NV - 1] = s1.x + s1.y;
    float xh_e = 0.f, wdy_e = 0.f;
    if (is_edge) {
      xh_e = (xe - mu) * rs;
      wdy_e = we * ge;
      s[0] += xh_e * wdy_e;
      if (!RMS) s[NV - 1] += wdy_e;
      ew_acc += ge * xh_e;
      eb_acc += ge;
    }
    group_sum<WARPS_N, NV>(s, red[warp_m], phase_bit, warp_m, warp_n, lane);
    // every thread of the group is past the previous row's dx pass: its slot can take the row
    // `stages` on
    if (gtid == 0 && prev_slot >= 0) {
      const int64_t r = row + (int64_t)(stages - 1) * step;
      if (r < shard_end) fill(prev_slot, r);
    }
    const float c1 = s[0] * inv_n;
    const float c2 = RMS ? 0.f : s[NV - 1] * inv_n;
    T* dxrow = db + row * p.dx_stride;
    uint4* dxbody = reinterpret_cast<uint4*>(dxrow + sp.head);
#define B200NORM_VROW_DX(P)                                                                            \
  if (has_w) vrow_bwd_dx<T, P, GT, K, RMS, true>(xs4, gs4, s_w, dxbody, VB, gtid, mu, rs, c1, c2);       \
  else vrow_bwd_dx<T, P, GT, K, RMS, false>(xs4, gs4, s_w, dxbody, VB, gtid, mu, rs, c1, c2)
    if constexpr (KEEP) {
      vrow_bwd_dx_kept<T, GT, K, RMS>(dxbody, VB, gtid, rs, c1, c2, kept_xh, kept_wdy);
    } else {
      switch (p.w_dtype) {
        case kF32: B200NORM_VROW_DX(float); break;
        case kF16: B200NORM_VROW_DX(__half); break;
        case kBF16: B200NORM_VROW_DX(__nv_bfloat16); break;
        default: B200NORM_VROW_DX(double); break;
      }
    }
#undef B200NORM_VROW_DX
    if (is_edge) dxrow[ecol] = from_f32<T>((wdy_e - (xh_e * c1 + c2)) * rs);
    if (WARPS_N == 1) __syncwarp();  // the refill above relies on the group having finished this row
    prev_slot = slot;
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  // this group's partial rows (all zeros for a group without rows)
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = gtid + k * GT;
    if (v < VB) {
      const int c = sp.head + v * EPP;
#pragma unroll
      for (int h = 0; h < H; ++h) {
        if (dw_row != nullptr) {
          dw_row[c + 2 * h] = acc_w[k][h].x;
          dw_row[c + 2 * h + 1] = acc_w[k][h].y;
        }
        if (db_row != nullptr) {
          db_row[c + 2 * h] = acc_b[k][h].x;
          db_row[c + 2 * h + 1] = acc_b[k][h].y;
        }
      }
    }
  }
  if (is_edge) {
    if (dw_row != nullptr) dw_row[ecol] = ew_acc;
    if (db_row != nullptr) db_row[ecol] = eb_acc;
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
