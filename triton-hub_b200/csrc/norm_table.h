// Host-side description of the compiled kernels: one table per storage type, filled in by
// the per-type translation units and consulted by the launch code.  This fixed table is
// what stands in for the reference's run-time autotuner (TritonHub/autotune.py:61-65).
#pragma once

namespace b200norm {

// A packet kernel instantiation: each thread holds `ldgs` 16-byte packets of the row, a row
// is spread over `warps_n` warps, and a CTA runs `warps_m` such row groups side by side.
struct PacketKernel {
  int ldgs, warps_m, warps_n;
  int stages;          // shared-memory slots per row group filled by bulk copies (0: none)
  int cluster;         // CTAs that share one row (1, or 2: column halves on a CTA pair)
  int lanes;           // lanes of a warp that share one row (32, or fewer: short rows, several per warp)
  bool packet_params;  // re-reads weight / bias per row as 16-byte packets: they must be aligned
  const void* fn;
  int capacity() const { return ldgs * lanes * warps_n * cluster; }  // packets per row it can hold
  int rows_per_cta() const { return warps_m * (32 / lanes); }       // rows a CTA works on at a time
  int threads() const { return 32 * warps_m * warps_n; }
};

// The any-alignment row kernels: rows of up to kWarpRowSizes[2] elements take the warp-per-row
// kernels, longer ones the kernels that stage a row through shared memory, with kRowThreads[i]
// threads per row ([0] up to kRowSplit elements, [1] beyond).
constexpr int kWarpRowSizes[3] = {256, 512, 1024};  // 32 lanes x 8 / 16 / 32 elements
constexpr int kRowShapeCount = 2;
constexpr int kRowThreads[kRowShapeCount] = {256, 512};
constexpr int kRowSplit = 8192;
// The vector kernels for rows whose buffers share one alignment: CTAs of `groups` row groups of `warps`
// warps each.  Forward: a shape serves rows of up to 32 * warps * kVRowFwdPackets interior packets.
// Backward: every thread carries dweight / dbias of `packets` interior packets; per storage type and op a
// shape either keeps xhat and w * dy in registers between its two passes, or forms them twice, or does
// not exist (too many registers), see vrow_bwd_variant().
struct VRowShape {
  int groups, warps, packets;
  constexpr int threads() const { return 32 * groups * warps; }
  constexpr int capacity() const { return 32 * warps * packets; }
};
constexpr int kVRowFwdPackets = 8;
constexpr int kVRowFwdCount = 5;
constexpr VRowShape kVRowFwd[kVRowFwdCount] = {{8, 1, 8}, {4, 2, 8}, {2, 4, 8}, {1, 8, 8}, {1, 16, 8}};
constexpr int kVRowBwdCount = 15;
constexpr VRowShape kVRowBwd[kVRowBwdCount] = {{8, 1, 2},  {8, 1, 4},  {8, 1, 8},  {4, 2, 2},  {4, 2, 4},
                                               {4, 2, 8},  {2, 4, 2},  {2, 4, 4},  {2, 4, 8},  {1, 8, 2},
                                               {1, 8, 4},  {1, 8, 8},  {1, 16, 2}, {1, 16, 4}, {1, 16, 8}};
// 2: keeps xhat and w * dy (registers for the sums and the kept values: packets * elements per packet *
// (1 or 2 sums + 2) <= 64: beyond that the 128 registers of a thread spill); 1: forms them twice (sums alone
// <= 64 registers); 0: no kernel.
constexpr int vrow_bwd_variant(int packets, int elems_per_packet, bool rms) {
  const int sums = packets * elems_per_packet * (rms ? 1 : 2);
  if (sums + packets * elems_per_packet * 2 <= 64) return 2;
  return sums <= 64 ? 1 : 0;
}

struct DTypeKernels {
  int elem_size;
  // [0] LayerNorm, [1] RMSNorm; each table in ascending capacity
  const PacketKernel* fwd[2];
  int n_fwd[2];
  const PacketKernel* bwd[2];
  int n_bwd[2];
  // any-alignment norm kernels (tables without a fused activation only): rows staged through shared
  // memory, [op][shape] with the shapes of kRowShapes below; dweight / dbias by a column kernel
  const void* fwd_rows[2][kRowShapeCount];
  const void* bwd_dx_rows[2][kRowShapeCount];
  // the same for short rows, one warp per row: [op][i] for rows of up to kWarpRowSizes[i] elements
  const void* fwd_warp_rows[2][3];
  const void* bwd_dx_warp_rows[2][3];
  const void* bwd_dwdb_any[2];
  const void* fwd_vrows[2][kVRowFwdCount];
  const void* bwd_vrows[2][kVRowBwdCount];
  int bwd_vrow_variant[2][kVRowBwdCount];  // vrow_bwd_variant() of each entry
  const void* act_packet[2];    // stand-alone activation, [0] forward [1] backward (tables of an activation only)
  const void* act_any[2];
};

// Softmax / LogSoftmax: one shape list per storage type; fn[log][bwd].
struct SoftmaxKernel {
  int ldgs, warps_m, warps_n;
  int stages_fwd, stages_bwd;  // bulk-copy slots per row group (0: direct loads)
  int lanes;                   // lanes of a warp per row (32, or fewer for short rows)
  const void* fn[2][2];
  int capacity() const { return ldgs * lanes * warps_n; }
  int threads() const { return 32 * warps_m * warps_n; }
  int rows_per_cta() const { return warps_m * (32 / lanes); }
};
struct SoftmaxTable {
  int elem_size;
  const SoftmaxKernel* kernels;  // ascending capacity
  int n;
  const void* any[2][2];  // any-alignment kernels, [log][bwd]
};
const SoftmaxTable* softmax_kernels_f32();
const SoftmaxTable* softmax_kernels_f16();
const SoftmaxTable* softmax_kernels_bf16();
const SoftmaxTable* softmax_kernels_f64();

// p-norm / normalize over the last dimension: fn[mode][p == 2], mode 0 norm forward, 1 normalize
// forward, 2 normalize backward; the element-wise norm backward and the any-alignment kernels apart.
struct PnormKernel {
  int ldgs, warps_m, warps_n;
  int stages_fwd, stages_bwd;
  int lanes;
  const void* fn[3][2];
  int capacity() const { return ldgs * lanes * warps_n; }
  int threads() const { return 32 * warps_m * warps_n; }
  int rows_per_cta() const { return warps_m * (32 / lanes); }
};
struct PnormTable {
  int elem_size;
  const PnormKernel* kernels;  // ascending capacity
  int n;
  const void* norm_bwd[2];  // [p == 2]
  const void* any[4];       // modes 0-2 as above, 3 norm backward
};
const PnormTable* pnorm_kernels_f32();
const PnormTable* pnorm_kernels_f16();
const PnormTable* pnorm_kernels_bf16();
const PnormTable* pnorm_kernels_f64();

// One table per (storage type, fused activation: 0 none, 1 GeLU erf, 2 GeLU tanh).
#define B200NORM_DECLARE_TABLES(name)      \
  const DTypeKernels* kernels_##name##_act0(); \
  const DTypeKernels* kernels_##name##_act1(); \
  const DTypeKernels* kernels_##name##_act2();
B200NORM_DECLARE_TABLES(f32)
B200NORM_DECLARE_TABLES(f16)
B200NORM_DECLARE_TABLES(bf16)
B200NORM_DECLARE_TABLES(f64)

}  // namespace b200norm
