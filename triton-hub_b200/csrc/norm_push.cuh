// Column reduce fused with a one-shot push all-gather over NVLink peer memory, and the kernel
// that finishes dweight / dbias from what the peers pushed.
//
// Every rank owns an "inbox" of `depth` equal slots, each holding (total_shards, slots, N) fp32
// at its start whatever the exchange's slots and N, and a flag array
// (depth, world) of 64-bit sequence numbers, both mapped into every peer.  The column-reduce
// kernel of exchange number `seq` writes each of its shard sums straight into slot
// seq % depth of EVERY rank's inbox with plain remote stores -- the transfer happens tile by
// tile as the sums are produced -- and the last CTA to finish raises this rank's flag on every
// peer.  No kernel of one GPU ever needs a kernel of another GPU to be resident at the same
// time (unlike a collective library's kernel), so the persistent forward / backward grids
// cannot be stalled by a late peer.  Only plain stores cross NVLink; all loads are local.
//
// The finish kernel waits (bounded) for the world's flags of that slot, then adds the
// total_shards sums left to right and casts: the same arithmetic on every rank and the same as
// a single GPU summing the same shards, so the result is bit-identical across ranks, runs and
// GPU counts.
#pragma once

#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

constexpr int kMaxPeers = 8;

// This rank's private bookkeeping (the `counter` buffer of b200norm_peers, 128 bytes, zeroed once).
// Keeping the sequence numbers on the device lets a captured CUDA graph be replayed: with seq == 0
// the kernels number the exchanges themselves instead of taking the number from the host.
struct LocalState {
  unsigned int push_ctas[8];      // CTAs of the current push kernel that are done, per inbox slot
  unsigned long long push_seq;    // last exchange pushed
  unsigned long long fin_seq;     // last exchange finished
  unsigned int fin_ctas;          // CTAs of the current finish kernel that are done
};

struct PeerTargets {
  float* inbox[kMaxPeers];                // peer r's inbox, mapped here
  unsigned long long* flags[kMaxPeers];   // peer r's flags (depth, world)
  LocalState* local;                      // this rank's bookkeeping
  int world, rank, depth, total_shards;
  size_t slot_floats;  // fp32 capacity of one of the `depth` inbox slots (the same for every exchange)
};

struct ColReducePushParams {
  const float* part[2];  // (P, N) partial rows of dweight / dbias
  PeerTargets peers;
  unsigned long long seq;
  int per_shard;   // partial rows per local row shard
  int row_shards;  // local row shards; this rank fills shards [rank*row_shards, (rank+1)*row_shards)
  int slots;
  int N;
};

// A flag store with no ordering of its own: the caller has already fenced at system scope.  (A
// st.release per peer would repeat that fence world times, one NVLink round trip each.)
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Same reduction order as colreduce_kernel (rows ty, ty+16, ... then the 16 running sums in ty
// order), so a pushed shard sum equals the group_sums value of the unfused path bit for bit.
__global__ void __launch_bounds__(512) colreduce_push_kernel(const ColReducePushParams p) {
  __shared__ float tile[16][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * 32 + tx;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  const float* part = p.part[slot];
  const bool live = col < p.N && part != nullptr;
  // seq == 0: number the exchange from the device-side counter (read before any CTA can advance it)
  const unsigned long long seq = p.seq != 0 ? p.seq : p.peers.local->push_seq + 1;
  const int buf = static_cast<int>(seq % static_cast<unsigned long long>(p.peers.depth));
  const size_t buf_off = (size_t)buf * p.peers.slot_floats;
  for (int g = 0; g < p.row_shards; ++g) {
    float s = 0.f;
    if (live) {
      const float* base = part + (size_t)g * p.per_shard * p.N + col;
      for (int r = ty; r < p.per_shard; r += 16) s += base[(size_t)r * p.N];
    }
    tile[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && live) {
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) a += tile[k][tx];
      const size_t off = buf_off + ((size_t)(p.peers.rank * p.row_shards + g) * p.slots + slot) * p.N + col;
      for (int r = 0; r < p.peers.world; ++r) p.peers.inbox[r][off] = a;  // remote (NVLink) or local store
    }
    __syncthreads();
  }
  // Publish: the storing threads make their stores visible system-wide, then the last CTA to
  // get here raises the flags.
  if (ty == 0) __threadfence_system();
  __syncthreads();
  if (tx == 0 && ty == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    const unsigned int prev = atomicAdd(&p.peers.local->push_ctas[buf], 1u);
    if (prev == total - 1) {
      p.peers.local->push_ctas[buf] = 0;  // ready for this slot's next use
      p.peers.local->push_seq = seq;      // every CTA of this launch has read the old value by now
      // One fence for all flags: it takes in the other CTAs' fenced stores (seen through the counter)
      // and this CTA's own, and orders them before the flag stores below.
      __threadfence_system();
      for (int r = 0; r < p.peers.world; ++r)
        st_relaxed_sys(&p.peers.flags[r][(size_t)buf * p.peers.world + p.peers.rank], seq);
    }
  }
}

// Four columns at a time (N a multiple of 4): 128-bit loads of the partial rows and 128-bit remote
// stores, a quarter of the CTAs (and of the fences and flag traffic).  Same per-column order.
__global__ void __launch_bounds__(512) colreduce4_push_kernel(const ColReducePushParams p) {
  __shared__ float4 tile[16][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = (blockIdx.x * 32 + tx) * 4;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  const float* part = p.part[slot];
  const bool live = col < p.N && part != nullptr;
  const unsigned long long seq = p.seq != 0 ? p.seq : p.peers.local->push_seq + 1;
  const int buf = static_cast<int>(seq % static_cast<unsigned long long>(p.peers.depth));
  const size_t buf_off = (size_t)buf * p.peers.slot_floats;
  for (int g = 0; g < p.row_shards; ++g) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
      const float* base = part + (size_t)g * p.per_shard * p.N + col;
      for (int r = ty; r < p.per_shard; r += 16) {
        const float4 v = *reinterpret_cast<const float4*>(base + (size_t)r * p.N);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    tile[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && live) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float4 v = tile[k][tx];
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      const size_t off = buf_off + ((size_t)(p.peers.rank * p.row_shards + g) * p.slots + slot) * p.N + col;
      for (int r = 0; r < p.peers.world; ++r) *reinterpret_cast<float4*>(p.peers.inbox[r] + off) = a;
    }
    __syncthreads();
  }
  if (ty == 0) __threadfence_system();
  __syncthreads();
  if (tx == 0 && ty == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    const unsigned int prev = atomicAdd(&p.peers.local->push_ctas[buf], 1u);
    if (prev == total - 1) {
      p.peers.local->push_ctas[buf] = 0;
      p.peers.local->push_seq = seq;
      __threadfence_system();
      for (int r = 0; r < p.peers.world; ++r)
        st_relaxed_sys(&p.peers.flags[r][(size_t)buf * p.peers.world + p.peers.rank], seq);
    }
  }
}

struct FinalizePushedParams {
  const float* inbox;               // this rank's inbox
  const unsigned long long* flags;  // this rank's flags
  void* out[2];
  int* status;
  LocalState* local;
  unsigned long long seq;
  size_t slot_floats;
  int world, depth, total_shards, slots, N, w_dtype;
};

// blockIdx.x = tile of 256 columns, blockIdx.y = slot.  Thread r < world waits for rank r's
// flag; the wait is bounded (2 s): on expiry the device status word is set and the kernel goes
// on with whatever the inbox holds, so the stream never hangs.
__global__ void __launch_bounds__(256) finalize_pushed_kernel(const FinalizePushedParams p) {
  grid_dependency_sync();
  trigger_dependents();
  const unsigned long long seq = p.seq != 0 ? p.seq : p.local->fin_seq + 1;  // 0: device-side numbering
  const int buf = static_cast<int>(seq % static_cast<unsigned long long>(p.depth));
  if (threadIdx.x < p.world) {
    const unsigned long long* f = p.flags + (size_t)buf * p.world + threadIdx.x;
    if (ld_acquire_sys(f) < seq) {
      const unsigned long long t0 = global_ns();
      bool ok = false;
      while (!ok) {
#pragma unroll 1
        for (int i = 0; i < 64 && !ok; ++i) ok = ld_acquire_sys(f) >= seq;
        if (!ok && global_ns() - t0 > kWaitLimitNs) {
          if (p.status != nullptr) *reinterpret_cast<volatile int*>(p.status) = 4;  // B200NORM_ERR_TIMEOUT
          break;
        }
      }
    }
  }
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  const int slot = blockIdx.y;
  if (col < p.N && p.out[slot] != nullptr) {
    const float* base = p.inbox + (size_t)buf * p.slot_floats + (size_t)slot * p.N + col;
    float total = 0.f;
    for (int g = 0; g < p.total_shards; ++g) total += __ldcg(base + (size_t)g * p.slots * p.N);  // L2: peers wrote it
    store_param(p.out[slot], p.w_dtype, col, total);
  }
  // The last CTA to finish records the exchange as done (every CTA has read fin_seq by then).
  if (threadIdx.x == 0) {
    const unsigned int total_ctas = gridDim.x * gridDim.y;
    if (atomicAdd(&p.local->fin_ctas, 1u) == total_ctas - 1) {
      p.local->fin_ctas = 0;
      p.local->fin_seq = seq;
    }
  }
}

}  // namespace b200norm
