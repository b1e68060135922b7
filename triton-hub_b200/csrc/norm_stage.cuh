// Shared-memory row staging with bulk asynchronous copies (the TMA engine's 1-D form,
// cp.async.bulk) completed on mbarriers.  Each row group owns a ring of STAGES slots; its
// leader thread keeps the ring full, so STAGES rows per group are always in flight no matter
// how few registers the consumers can spare.
//
// Every wait is bounded: a wait that runs out raises the CTA's abort flag and the device's
// status word, after which all further waits in the CTA return at once.  The kernel then runs
// to its normal end on whatever the slots hold (indices stay in range, so nothing faults) and
// the host reports B200NORM_ERR_TIMEOUT from the status word.
#pragma once

#include "norm_common.cuh"

namespace b200norm {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait, far beyond any copy

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bulk copy global -> this CTA's shared memory; both addresses and the size are multiples of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Wait for `parity` of `bar`, giving up after kWaitLimitNs.  Returns false (and poisons the
// CTA) on timeout or if the CTA is already poisoned.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* cta_abort, int* status) {
  if (*cta_abort) return false;
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*cta_abort) return false;
    if (global_ns() - t0 > kWaitLimitNs) {
      *cta_abort = 1;
      if (status != nullptr) *reinterpret_cast<volatile int*>(status) = 4;  // B200NORM_ERR_TIMEOUT
      return false;
    }
  }
}

// Last step of a poisoned CTA: the leader of a row group gives the copies it issued (`count`
// rows over STAGES slots) a bounded chance to land before the CTA's shared memory is released.
template <int STAGES>
__device__ __forceinline__ void drain_ring(uint64_t* bars, int64_t count) {
  constexpr int kSlots = STAGES > 0 ? STAGES : 1;  // instantiated (never called) with STAGES == 0
  const unsigned long long t0 = global_ns();
#pragma unroll
  for (int s = 0; s < STAGES; ++s) {
    if (count <= s) continue;
    const int64_t fills = (count - s + kSlots - 1) / kSlots;
    const uint32_t parity = static_cast<uint32_t>((fills - 1) & 1);
    while (!mbar_try_wait(&bars[s], parity)) {
      if (global_ns() - t0 > 10000000ull) return;  // 10 ms for the whole ring
    }
  }
}

// ---------------------------------------------------------------------------------------
// Thread-block clusters: a row too wide for one CTA's registers is split over a pair of CTAs on
// neighbouring SMs, which exchange their partial row sums through distributed shared memory.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `local` (a shared-memory address of this CTA) in CTA `cta` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(cta));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Hardware barrier over every thread of the cluster (release / acquire: remote shared-memory
// stores made before it are visible after it).  Like __syncthreads, it relies on the hardware
// co-scheduling all CTAs of a cluster; it is not a software spin.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Exchange of NV floats with the partner CTA of a pair, point to point and without any fence.
// Thread 0 stores each value together with the exchange's sequence number as ONE 8-byte word into
// the partner's `box`; every thread polls its own CTA's box until the words carry that number.  A
// word is never torn, so a matching number vouches for its value and nothing has to be ordered.
// That matters: a cluster barrier (or any release / acquire at cluster scope) makes the warp wait
// until its earlier GLOBAL stores -- the previous row's output -- are acknowledged, once per row
// (`membar` was the top stall of the pair kernels: 3.2 per issued instruction, 0.77-0.86 of the copy
// bandwidth whatever the launch shape).  The wait is bounded like mbar_wait.  `box` is
// double-buffered by the caller (`buf` flips per call): the partner can be at most one exchange
// ahead, because its next-but-one exchange needs this CTA's answer to its next, which thread 0
// sends only after every thread of this CTA has read the current values (a CTA-wide barrier -- the
// next row's reduction -- lies in between).
template <int NV>
struct PairBox {
  unsigned long long w[NV];  // {fp32 value (low word), sequence number (high word)}
};

__device__ __forceinline__ void st_cluster_u64(uint32_t addr, unsigned long long v) {
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_volatile_shared_u64(const void* p) {
  unsigned long long v;
  asm volatile("ld.volatile.shared.u64 %0, [%1];" : "=l"(v) : "r"(smem_addr(p)) : "memory");
  return v;
}

template <int NV>
__device__ __forceinline__ void pair_swap(const float (&mine)[NV], float (&theirs)[NV], PairBox<NV>* box, int& buf,
                                          uint32_t seq, uint32_t cr, volatile int* cta_abort, int* status) {
  PairBox<NV>* b = box + buf;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      st_cluster_u64(cluster_map(smem_addr(&b->w[i]), cr ^ 1u),
                     (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(mine[i]));
  }
  unsigned long long got[NV];
  auto arrived = [&]() {
    bool ok = true;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      got[i] = ld_volatile_shared_u64(&b->w[i]);
      ok = ok && static_cast<uint32_t>(got[i] >> 32) == seq;
    }
    return ok;
  };
  if (!arrived() && !*cta_abort) {
    const unsigned long long t0 = global_ns();
    for (;;) {
      bool ok = false;
#pragma unroll 1
      for (int i = 0; i < 256 && !ok; ++i) ok = arrived();
      if (ok || *cta_abort) break;
      if (global_ns() - t0 > kWaitLimitNs) {
        *cta_abort = 1;
        if (status != nullptr) *reinterpret_cast<volatile int*>(status) = 4;  // B200NORM_ERR_TIMEOUT
        break;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) theirs[i] = __uint_as_float(static_cast<uint32_t>(got[i]));
  buf ^= 1;
}

__device__ __forceinline__ uint4 ld_shared16(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(smem_addr(p)));
  return v;
}

}  // namespace b200norm
