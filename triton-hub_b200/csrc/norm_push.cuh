// Column reduce fused with a one-shot push all-gather over NVLink peer memory, and the code
// that finishes dweight / dbias from what the peers pushed.
//
// Every rank owns an "inbox" of `depth` equal slots mapped into every peer.  A slot holds one
// exchange's (total_shards, slots, N) shard sums as 8-byte ENTRIES: the fp32 value in the low
// word and a 32-bit tag derived from the exchange number in the high word.  The column-reduce
// kernel of exchange `seq` writes each shard sum it produces straight into slot seq % depth of
// EVERY rank's inbox with plain remote stores -- the transfer happens tile by tile as the sums
// are produced.  Value and tag travel in one 8-byte store, which is never torn, so an entry
// whose tag matches carries its value: there are no flags to raise, no fences and no counters on
// the data path (the scheme of the "low latency" protocol of collective libraries).  No kernel of
// one GPU ever needs a kernel of another GPU to be resident at the same time, so the persistent
// forward / backward grids cannot be stalled by a late peer.  Only plain stores cross NVLink;
// all loads are local.
//
// Finishing exchange f: poll (bounded) the entries of slot f % depth until their tags match,
// add the total_shards values of a column left to right and cast.  The same arithmetic on every
// rank and the same as a single GPU summing the same shards, so the result is bit-identical
// across ranks, runs and GPU counts.  A finish can run as a kernel of its own
// (finalize_pushed_kernel) or as the second phase of a later -- or the same -- exchange's push
// kernel, which saves a launch per step.
//
// An entry overwritten by exchange f + depth before a slow rank has read exchange f makes that
// rank's wait run out (status word set) instead of handing it another exchange's numbers.
#pragma once

#include "norm_common.cuh"
#include "norm_stage.cuh"

namespace b200norm {

constexpr int kMaxPeers = 8;

// This rank's private bookkeeping (the `counter` buffer of b200norm_peers, 128 bytes, zeroed once).
// Keeping the sequence numbers on the device lets a captured CUDA graph be replayed: with seq == 0
// the kernels number the exchanges themselves instead of taking the number from the host.
struct LocalState {
  unsigned int push_ctas;         // CTAs of the current push kernel that are done
  unsigned int fin_ctas;          // CTAs of the current finish kernel that are done
  unsigned long long push_seq;    // last exchange pushed
  unsigned long long fin_seq;     // last exchange finished
};

struct PeerTargets {
  unsigned char* inbox[kMaxPeers];  // peer r's inbox, mapped here
  LocalState* local;                // this rank's bookkeeping
  int world, rank, depth, total_shards;
  size_t slot_bytes;  // size of one of the `depth` inbox slots (the same for every exchange)
};

// What to finish, and where the result goes.  N == 0: nothing.
struct FinishSpec {
  void* out[2];             // dweight, dbias (either may be null)
  unsigned long long seq;   // 0: the exchange after the last finished one (device-side numbering)
  int* status;              // device status word for a wait that ran out
  int slots, N, w_dtype;
};

struct ColReducePushParams {
  const float* part[2];  // (P, N) partial rows of dweight / dbias
  PeerTargets peers;
  FinishSpec fin;
  unsigned long long seq;
  int per_shard;   // partial rows per local row shard
  int row_shards;  // local row shards; this rank fills shards [rank*row_shards, (rank+1)*row_shards)
  int slots;
  int N;
};

// The 32-bit tag of an exchange: never 0 (what a fresh inbox holds), and different for two
// exchanges that share a slot.
__device__ __forceinline__ unsigned int exchange_tag(unsigned long long seq) {
  return static_cast<unsigned int>(seq % 0xFFFFFFFFull) + 1u;
}
__device__ __forceinline__ unsigned long long make_entry(float v, unsigned int tag) {
  return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
}
// Entries are written and polled with volatile accesses whose elements are 64 bits wide: each
// entry is one indivisible access at the memory system (system scope), two entries per instruction.
__device__ __forceinline__ void st_entry(void* p, unsigned long long e) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(e) : "memory");
}
__device__ __forceinline__ void st_entry2(void* p, unsigned long long e0, unsigned long long e1) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(e0), "l"(e1) : "memory");
}
__device__ __forceinline__ unsigned long long ld_entry(const void* p) {
  unsigned long long e;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(e) : "l"(p) : "memory");
  return e;
}
__device__ __forceinline__ void ld_entry2(const void* p, unsigned long long& e0, unsigned long long& e1) {
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(e0), "=l"(e1) : "l"(p) : "memory");
}

// Finish exchange `seq` on this rank: thread `tid` of `nthreads` takes column pairs (single
// columns when N is odd) of the `slots` result vectors.  The entries of up to eight shards are
// requested at once and checked afterwards, so a column costs one trip to memory, not one per
// shard.  Each wait is bounded (2 s); a thread whose wait runs out sets the status word and stops
// waiting, so the kernel always ends.
template <int PAIR>  // 2: two columns per thread (N even), 1: one
__device__ __forceinline__ void finish_columns_impl(const unsigned char* inbox, const PeerTargets& peers,
                                                    const FinishSpec& f, unsigned long long seq, unsigned int tid,
                                                    unsigned int nthreads) {
  constexpr int kChunk = 8;
  const unsigned int tag = exchange_tag(seq);
  const unsigned char* base = inbox + (size_t)(seq % static_cast<unsigned long long>(peers.depth)) * peers.slot_bytes;
  bool gave_up = false;
  const unsigned int per_slot = static_cast<unsigned int>(f.N) / PAIR;
  const size_t shard_stride = (size_t)f.slots * f.N * 8;
  auto fetch = [&](const unsigned char* p, unsigned long long& e0, unsigned long long& e1) {
    if (PAIR == 2) {
      ld_entry2(p, e0, e1);
    } else {
      e0 = ld_entry(p);
      e1 = e0;
    }
  };
  for (unsigned int it = tid; it < per_slot * f.slots; it += nthreads) {
    const int slot = static_cast<int>(it / per_slot);
    const int col = static_cast<int>(it - slot * per_slot) * PAIR;
    if (f.out[slot] == nullptr) continue;
    const unsigned char* p0 = base + ((size_t)slot * f.N + col) * 8;
    float t0 = 0.f, t1 = 0.f;
    for (int g0 = 0; g0 < peers.total_shards; g0 += kChunk) {
      unsigned long long e0[kChunk], e1[kChunk];
#pragma unroll
      for (int k = 0; k < kChunk; ++k)
        if (g0 + k < peers.total_shards) fetch(p0 + (size_t)(g0 + k) * shard_stride, e0[k], e1[k]);
#pragma unroll
      for (int k = 0; k < kChunk; ++k) {
        if (g0 + k >= peers.total_shards) break;
        if (!gave_up && ((e0[k] >> 32) != tag || (e1[k] >> 32) != tag)) {  // not there yet: poll this one
          const unsigned char* p = p0 + (size_t)(g0 + k) * shard_stride;
          const unsigned long long start = global_ns();
          for (;;) {
            bool ok = false;
#pragma unroll 1
            for (int i = 0; i < 64 && !ok; ++i) {
              fetch(p, e0[k], e1[k]);
              ok = (e0[k] >> 32) == tag && (e1[k] >> 32) == tag;
            }
            if (ok) break;
            if (global_ns() - start > kWaitLimitNs) {
              if (f.status != nullptr) *reinterpret_cast<volatile int*>(f.status) = 4;  // B200NORM_ERR_TIMEOUT
              gave_up = true;
              break;
            }
          }
        }
        t0 += __uint_as_float(static_cast<unsigned int>(e0[k]));  // shards left to right
        t1 += __uint_as_float(static_cast<unsigned int>(e1[k]));
      }
    }
    store_param(f.out[slot], f.w_dtype, col, t0);
    if (PAIR == 2) store_param(f.out[slot], f.w_dtype, col + 1, t1);
  }
}

__device__ __forceinline__ void finish_columns(const unsigned char* inbox, const PeerTargets& peers,
                                               const FinishSpec& f, unsigned long long seq, unsigned int tid,
                                               unsigned int nthreads) {
  if ((f.N & 1) == 0) finish_columns_impl<2>(inbox, peers, f, seq, tid, nthreads);
  else finish_columns_impl<1>(inbox, peers, f, seq, tid, nthreads);
}

// W = 4 (N a multiple of 4: 128-bit loads of the partial rows, two entries per remote store) or
// W = 1 (any N).  blockIdx.x walks tiles of 32 * W columns, blockIdx.y = slot.  Same reduction
// order as colreduce_kernel (rows ty, ty+16, ... then the 16 running sums in ty order), so a
// pushed shard sum equals the group_sums value of the unfused path bit for bit.
//
// Phase 1 pushes this rank's shard sums of exchange `seq`; phase 2 (fin.N > 0) finishes an
// exchange -- an earlier one, whose entries arrived long ago, or this very one, in which case the
// kernel ends once every peer's push has arrived.  The push goes first so that a late peer holds
// up nobody but the finishing rank.  The grid never exceeds what the device keeps resident (the
// host caps it), so a CTA waiting in phase 2 for entries of another CTA of this grid always gets them.
template <int W>
__global__ void __launch_bounds__(512) colreduce_push_kernel(const ColReducePushParams p) {
  __shared__ float tile[16][32 * W + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  volatile LocalState* local = p.peers.local;
  // seq == 0: number the exchange from the device-side counter (read before any CTA can advance it)
  const unsigned long long seq = p.seq != 0 ? p.seq : local->push_seq + 1;
  const unsigned long long fseq = p.fin.seq != 0 ? p.fin.seq : local->fin_seq + 1;
  const unsigned int tag = exchange_tag(seq);
  const size_t buf_off = (size_t)(seq % static_cast<unsigned long long>(p.peers.depth)) * p.peers.slot_bytes;
  const float* part = p.part[slot];
  const int tiles = (p.N + 32 * W - 1) / (32 * W);
  for (int tile_i = blockIdx.x; tile_i < tiles; tile_i += gridDim.x) {
    const int col = (tile_i * 32 + tx) * W;
    const bool live = col < p.N && part != nullptr;
    for (int g = 0; g < p.row_shards; ++g) {
      float s[W];
#pragma unroll
      for (int e = 0; e < W; ++e) s[e] = 0.f;
      if (live) {
        const float* base = part + (size_t)g * p.per_shard * p.N + col;
        // four rows requested at a time, added in row order
        for (int r = ty; r < p.per_shard; r += 64) {
          if constexpr (W == 4) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              v[k] = (r + 16 * k < p.per_shard) ? *reinterpret_cast<const float4*>(base + (size_t)(r + 16 * k) * p.N)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (r + 16 * k < p.per_shard) { s[0] += v[k].x; s[1] += v[k].y; s[2] += v[k].z; s[3] += v[k].w; }
          } else {
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = (r + 16 * k < p.per_shard) ? base[(size_t)(r + 16 * k) * p.N] : 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (r + 16 * k < p.per_shard) s[0] += v[k];
          }
        }
      }
#pragma unroll
      for (int e = 0; e < W; ++e) tile[ty][e * 32 + tx] = s[e];
      __syncthreads();
      if (ty == 0 && live) {
        float a[W];
#pragma unroll
        for (int e = 0; e < W; ++e) a[e] = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k)
#pragma unroll
          for (int e = 0; e < W; ++e) a[e] += tile[k][e * 32 + tx];
        const size_t off = buf_off + (((size_t)(p.peers.rank * p.row_shards + g) * p.slots + slot) * p.N + col) * 8;
        for (int r = 0; r < p.peers.world; ++r) {  // remote (NVLink) or local stores
          unsigned char* dst = p.peers.inbox[r] + off;
          if constexpr (W == 4) {
            st_entry2(dst, make_entry(a[0], tag), make_entry(a[1], tag));
            st_entry2(dst + 16, make_entry(a[2], tag), make_entry(a[3], tag));
          } else {
            st_entry(dst, make_entry(a[0], tag));
          }
        }
      }
      __syncthreads();
    }
  }
  if (p.fin.N > 0) {
    const unsigned int cta = blockIdx.y * gridDim.x + blockIdx.x;
    finish_columns(p.peers.inbox[p.peers.rank], p.peers, p.fin, fseq, cta * 512u + ty * 32u + tx,
                   gridDim.x * gridDim.y * 512u);
  }
  // The last CTA to finish records the exchange numbers (every CTA has read them by then).
  __syncthreads();
  if (tx == 0 && ty == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    if (atomicAdd(&p.peers.local->push_ctas, 1u) == total - 1) {
      p.peers.local->push_ctas = 0;
      local->push_seq = seq;
      if (p.fin.N > 0) local->fin_seq = fseq;
    }
  }
}

struct FinalizePushedParams {
  PeerTargets peers;
  FinishSpec fin;
};

// Stand-alone finish of one exchange.
__global__ void __launch_bounds__(256) finalize_pushed_kernel(const FinalizePushedParams p) {
  grid_dependency_sync();
  trigger_dependents();
  volatile LocalState* local = p.peers.local;
  const unsigned long long seq = p.fin.seq != 0 ? p.fin.seq : local->fin_seq + 1;  // 0: device-side numbering
  finish_columns(p.peers.inbox[p.peers.rank], p.peers, p.fin, seq, blockIdx.x * 256u + threadIdx.x, gridDim.x * 256u);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&p.peers.local->fin_ctas, 1u) == gridDim.x - 1) {
      p.peers.local->fin_ctas = 0;
      local->fin_seq = seq;
    }
  }
}

}  // namespace b200norm
