// Deterministic column reduce of the backward kernels' fp32 partial rows, and the finish
// step for gathered shard sums.  Together they replace `_dw.sum(0).to(dtype)`
// (TritonHub/Normalization/layernorm.py:207-208, rmsnorm.py:166).
#pragma once

#include "norm_common.cuh"

namespace b200norm {

// Column reduce of the partial rows.  blockIdx.x = tile of 32 columns, blockIdx.y = slot
// (0 dweight, 1 dbias).  A block is 32 x 16 threads: thread (tx, ty) adds rows ty, ty+16, ...
// of one shard's partials, the 16 running sums are added in ty order, and the shard sums are
// added left to right.  The order is a function of (partial rows per shard, shards) only.
struct ColReduceParams {
  const float* part[2];  // (P, N) each
  void* out[2];          // (N,) in w_dtype, or null
  float* group_sums;     // (row_shards, slots, N) fp32 or null
  int per_shard;         // partial rows per shard
  int row_shards;
  int slots;
  int N;
  int w_dtype;
};

__global__ void __launch_bounds__(512) colreduce_kernel(const ColReduceParams p) {
  __shared__ float tile[16][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * 32 + tx;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  const float* part = p.part[slot];
  const bool live = col < p.N && part != nullptr;
  float total = 0.f;
  for (int g = 0; g < p.row_shards; ++g) {
    float s = 0.f;
    if (live) {
      const float* base = part + (size_t)g * p.per_shard * p.N + col;
      // four rows requested at a time, added in row order
      for (int r = ty; r < p.per_shard; r += 64) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = (r + 16 * k < p.per_shard) ? base[(size_t)(r + 16 * k) * p.N] : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (r + 16 * k < p.per_shard) s += v[k];
      }
    }
    tile[ty][tx] = s;
    __syncthreads();
    if (ty == 0) {
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) a += tile[k][tx];
      if (live && p.group_sums != nullptr) p.group_sums[((size_t)g * p.slots + slot) * p.N + col] = a;
      total += a;
    }
    __syncthreads();
  }
  if (ty == 0 && live && p.out[slot] != nullptr) store_param(p.out[slot], p.w_dtype, col, total);
}

// The same reduction four columns at a time (N a multiple of 4: every partial row is then 16-byte
// aligned).  A CTA covers 128 columns with 128-bit loads; per column the additions happen in exactly
// the order of colreduce_kernel, so both produce the same bits.
__global__ void __launch_bounds__(512) colreduce4_kernel(const ColReduceParams p) {
  __shared__ float4 tile[16][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = (blockIdx.x * 32 + tx) * 4;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  const float* part = p.part[slot];
  const bool live = col < p.N && part != nullptr;
  float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < p.row_shards; ++g) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
      const float* base = part + (size_t)g * p.per_shard * p.N + col;
      // four rows requested at a time, added in row order
      for (int r = ty; r < p.per_shard; r += 64) {
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          v[k] = (r + 16 * k < p.per_shard) ? *reinterpret_cast<const float4*>(base + (size_t)(r + 16 * k) * p.N)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (r + 16 * k < p.per_shard) { s.x += v[k].x; s.y += v[k].y; s.z += v[k].z; s.w += v[k].w; }
      }
    }
    tile[ty][tx] = s;
    __syncthreads();
    if (ty == 0) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float4 v = tile[k][tx];
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      if (live && p.group_sums != nullptr)
        *reinterpret_cast<float4*>(p.group_sums + ((size_t)g * p.slots + slot) * p.N + col) = a;
      total.x += a.x; total.y += a.y; total.z += a.z; total.w += a.w;
    }
    __syncthreads();
  }
  if (ty == 0 && live && p.out[slot] != nullptr) {
    store_param(p.out[slot], p.w_dtype, col, total.x);
    store_param(p.out[slot], p.w_dtype, col + 1, total.y);
    store_param(p.out[slot], p.w_dtype, col + 2, total.z);
    store_param(p.out[slot], p.w_dtype, col + 3, total.w);
  }
}

// dweight / dbias from gathered shard sums (groups, slots, N): left-to-right add, then cast.
struct FinalizeParams {
  const float* group_sums;
  void* out[2];
  int groups;
  int slots;
  int N;
  int w_dtype;
};

__global__ void __launch_bounds__(256) finalize_kernel(const FinalizeParams p) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  const int slot = blockIdx.y;
  grid_dependency_sync();
  trigger_dependents();
  if (col >= p.N || p.out[slot] == nullptr) return;
  float total = 0.f;
  for (int g = 0; g < p.groups; ++g) total += p.group_sums[((size_t)g * p.slots + slot) * p.N + col];
  store_param(p.out[slot], p.w_dtype, col, total);
}

}  // namespace b200norm
