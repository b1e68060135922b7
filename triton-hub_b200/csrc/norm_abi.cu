// C ABI of libb200norm.so (declared in include/b200norm.h): argument checks, the fixed launch
// table and the kernel launches.  Nothing here synchronises or, after a device's first call,
// allocates.
#include <cuda_runtime.h>

#include <algorithm>
#include <numeric>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "b200norm.h"
#include "norm_bwd.cuh"
#include "norm_colreduce.cuh"
#include "norm_fwd.cuh"
#include "norm_push.cuh"
#include "norm_rows_any.cuh"
#include "norm_table.h"
#include "pnorm.cuh"
#include "softmax.cuh"

namespace b200norm {
namespace {

constexpr int kMaxDevices = 64;
constexpr int64_t kMaxRowBytes = 65536;  // the reference's limit (layernorm.py:69-72)
constexpr int kLN = 0, kRMS = 1;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

struct DeviceState {
  // Launch planning: SM count, occupancies, shared-memory allowances.  Set up without allocating
  // anything, and shared by every entry point -- a kernel's shared-memory allowance is a property
  // of the device, so there must be exactly one record of it per device.
  std::once_flag once;
  cudaError_t init_err = cudaSuccess;
  int sm_count = 0;
  std::mutex mu;
  std::unordered_map<unsigned long long, int> occupancy;  // (kernel, dyn smem) -> CTAs per SM
  std::unordered_map<const void*, size_t> smem_limit;     // kernel -> dynamic shared memory it has been allowed
  // Status word: pinned, mapped host memory where kernels report a timed-out wait.  Allocated by the
  // first call of an entry point that reports through it (never by b200norm_rms_bwd_static).
  std::once_flag status_once;
  cudaError_t status_err = cudaSuccess;
  int* status_host = nullptr;
  int* status_dev = nullptr;
};
DeviceState g_dev[kMaxDevices];

// The launch-planning part of the current device's state; allocates nothing.
int device_caches(DeviceState** out) {
  int d = -1;
  cudaError_t e = cudaGetDevice(&d);
  if (e != cudaSuccess) return fail(B200NORM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (d < 0 || d >= kMaxDevices) return fail(B200NORM_ERR_CUDA, "device index %d out of range", d);
  DeviceState& s = g_dev[d];
  std::call_once(s.once, [&]() {
    s.init_err = cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, d);
  });
  if (s.init_err != cudaSuccess)
    return fail(B200NORM_ERR_CUDA, "device set-up: %s", cudaGetErrorString(s.init_err));
  *out = &s;
  return B200NORM_OK;
}

// Per-device set-up, run by the first call on each device: the above plus the status word.
int device_state(DeviceState** out) {
  DeviceState* s = nullptr;
  if (int rc = device_caches(&s)) return rc;
  std::call_once(s->status_once, [&]() {
    s->status_err = cudaHostAlloc(reinterpret_cast<void**>(&s->status_host), 64, cudaHostAllocMapped);
    if (s->status_err != cudaSuccess) return;
    std::memset(s->status_host, 0, 64);
    s->status_err = cudaHostGetDevicePointer(reinterpret_cast<void**>(&s->status_dev), s->status_host, 0);
  });
  if (s->status_err != cudaSuccess)
    return fail(B200NORM_ERR_CUDA, "device set-up: %s", cudaGetErrorString(s->status_err));
  *out = s;
  return B200NORM_OK;
}

// Resident CTAs per SM of `fn` at this block size and dynamic shared memory (cluster == 1), or
// resident clusters on the whole device (cluster > 1); cached.
int occupancy(DeviceState& s, const void* fn, int threads, size_t smem, int* out, int cluster = 1) {
  const unsigned long long key =
      (reinterpret_cast<unsigned long long>(fn) * 0x9E3779B97F4A7C15ull) ^ (unsigned long long)smem;
  std::lock_guard<std::mutex> lock(s.mu);
  auto it = s.occupancy.find(key);
  if (it != s.occupancy.end()) {
    *out = it->second;
    return B200NORM_OK;
  }
  cudaError_t e;
  // Static shared memory counts toward the 48 KB default limit too, hence 32 KB.  The limit is only
  // ever raised: one kernel serves a range of row lengths, and a shorter row after a longer one must
  // not take the allowance away from a launch shape whose occupancy is already cached.
  size_t& allowed = s.smem_limit[fn];
  if (smem > 32 * 1024 && smem > allowed) {
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess)
      return fail(B200NORM_ERR_CUDA, "cudaFuncSetAttribute(%zu B): %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  int n = 0;
  if (cluster > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(cluster * s.sm_count));
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaOccupancyMaxActiveClusters(&n, fn, &cfg);
  } else {
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, smem);
  }
  if (e != cudaSuccess) return fail(B200NORM_ERR_CUDA, "occupancy query: %s", cudaGetErrorString(e));
  if (n < 1) return fail(B200NORM_ERR_CUDA, "kernel does not fit on an SM (%d threads, %zu B smem)", threads, smem);
  s.occupancy.emplace(key, n);
  *out = n;
  return B200NORM_OK;
}

// The kernel table of a storage type and a fused activation (0 none, 1 GeLU erf, 2 GeLU tanh).
const DTypeKernels* kernels_for(int dtype, int act = 0) {
#define B200NORM_PICK(name) \
  return act == 0 ? kernels_##name##_act0() : act == 1 ? kernels_##name##_act1() : kernels_##name##_act2();
  switch (dtype) {
    case B200NORM_F32: B200NORM_PICK(f32)
    case B200NORM_F16: B200NORM_PICK(f16)
    case B200NORM_BF16: B200NORM_PICK(bf16)
    case B200NORM_F64: B200NORM_PICK(f64)
    default: return nullptr;
  }
#undef B200NORM_PICK
}

bool valid_act(int act) { return act >= B200NORM_ACT_NONE && act <= B200NORM_ACT_GELU_TANH; }

// Tuning builds only (-DB200NORM_TUNING, which the shipped library is not built with): an environment
// variable, read once, that overrides a launch decision -- the index of the table entry to use
// whenever it can hold the row (B200NORM_FORCE_FWD / _BWD / _SOFTMAX / _PNORM), or B200NORM_PDL=0 to
// launch without programmatic dependent launch.  Without the flag these return `fallback`.
int tuning_env(const char* name, int fallback) {
#ifdef B200NORM_TUNING
  const char* v = std::getenv(name);
  return v != nullptr ? std::atoi(v) : fallback;
#else
  (void)name;
  return fallback;
#endif
}

constexpr size_t kMaxSmemPerCta = 227 * 1024;  // opt-in dynamic + static shared memory of one sm_100 CTA

bool valid_dtype(int d) { return d >= B200NORM_F32 && d <= B200NORM_F64; }

bool aligned16(const void* p, int64_t stride_elems, int es) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && ((stride_elems * es) & 15) == 0;
}

// Dynamic shared memory of a backward launch, per CTA: (warps_m [+1 with a fused activation: the
// bias]) x columns fp32 for the weights and the row-group sums, padded to 128 bytes, then the
// x + dy row slots.  A CTA of a pair holds half of the columns.
size_t bwd_smem_bytes(const PacketKernel& pk, int64_t N, int es, int act) {
  if (pk.lanes < 32) return 0;  // the short-row kernels keep their sums in static shared memory
  const int64_t Nl = N / pk.cluster;
  return ((static_cast<size_t>(pk.warps_m + (act != 0 ? 1 : 0)) * Nl * sizeof(float) + 127) & ~static_cast<size_t>(127)) +
         static_cast<size_t>(pk.warps_m) * pk.stages * 2 * (Nl * es);
}

// First table entry whose capacity covers a row of V packets (and, for a backward table, whose
// shared memory fits), or null.
const PacketKernel* pick(const PacketKernel* tab, int n, int64_t V, bool bwd = false, int64_t N = 0, int es = 0,
                         int act = 0) {
  static const int forced[2] = {tuning_env("B200NORM_FORCE_FWD", -1), tuning_env("B200NORM_FORCE_BWD", -1)};
  const int f = forced[bwd ? 1 : 0];
  if (f >= 0 && f < n && tab[f].capacity() >= V && V % tab[f].cluster == 0) return &tab[f];
  for (int i = 0; i < n; ++i) {
    if (tab[i].capacity() < V || V % tab[i].cluster != 0) continue;
    if (bwd && bwd_smem_bytes(tab[i], N, es, act) + 2048 > kMaxSmemPerCta) continue;
    return &tab[i];
  }
  return nullptr;
}

// `pdl`: launch with programmatic stream serialization (the kernel calls grid_dependency_sync()
// before its first global access); the any-alignment kernels do not and are launched plainly.
int launch(const void* fn, dim3 grid, dim3 block, size_t smem, void* params, cudaStream_t stream, bool pdl = true,
           int cluster = 1) {
  void* args[1] = {params};
  cudaError_t e;
  static const bool pdl_enabled = tuning_env("B200NORM_PDL", 1) != 0;
  if ((pdl && pdl_enabled) || cluster > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl && pdl_enabled) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    if (cluster > 1) {
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = static_cast<unsigned>(cluster);
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    e = cudaLaunchKernelExC(&cfg, fn, args);
  } else {
    e = cudaLaunchKernel(fn, grid, block, args, smem, stream);
  }
  if (e != cudaSuccess) return fail(B200NORM_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return B200NORM_OK;
}

// Launches an any-alignment row kernel (forward: one staged row per ring slot, backward dx: two).
// Shared memory per CTA = (rows_per_slot * slots + 1) row buffers; four slots when that leaves room
// for a second CTA on the SM, else as many as fit.
int launch_row_kernel(DeviceState& dev, const void* const (&fns)[kRowShapeCount], const void* const (&warp_fns)[3], int64_t M, int64_t N, int es, int rows_per_slot,
                      void* params, cudaStream_t stream) {
  if (N <= kWarpRowSizes[2]) {  // short rows: one warp per row, eight rows per CTA, no shared memory
    const void* fn = warp_fns[N <= kWarpRowSizes[0] ? 0 : N <= kWarpRowSizes[1] ? 1 : 2];
    int occ;
    if (int rc = occupancy(dev, fn, kWarpRowWarps * 32, 0, &occ)) return rc;
    const int64_t want = (M + kWarpRowWarps - 1) / kWarpRowWarps;
    const int grid = static_cast<int>(std::min<int64_t>(want, (int64_t)dev.sm_count * occ));
    return launch(fn, dim3(grid), dim3(kWarpRowWarps * 32), 0, params, stream, false);
  }
  const int shape = N <= kRowSplit ? 0 : 1;
  const void* fn = fns[shape];
  const int threads = kRowThreads[shape];
  const size_t buf = row_buffer_bytes(N, es);
  auto bytes = [&](int slots) { return (static_cast<size_t>(rows_per_slot) * slots + 1) * buf; };
  int slots = 4;
  while (slots > 2 && bytes(slots) > 112 * 1024) --slots;
  if (bytes(slots) > 112 * 1024) {  // wide rows: one CTA per SM, as many slots as its shared memory holds
    slots = 4;
    while (slots > 1 && bytes(slots) > kMaxSmemPerCta - 4096) --slots;
  }
  const size_t smem = bytes(slots);
  int occ;
  if (int rc = occupancy(dev, fn, threads, smem, &occ)) return rc;
  const int grid = static_cast<int>(std::min<int64_t>(M, (int64_t)dev.sm_count * occ));
  return launch(fn, dim3(grid), dim3(threads), smem, params, stream, false);
}

// Whether two buffers start every row at the same offset within a 16-byte line.
bool same_phase(const void* a, int64_t sa, const void* b, int64_t sb, int es) {
  return ((reinterpret_cast<uintptr_t>(a) ^ reinterpret_cast<uintptr_t>(b)) & 15u) == 0 && ((sa - sb) * es) % 16 == 0;
}

// After how many rows the offset of a row within a 16-byte line repeats.
int phase_period(int64_t stride, int es) {
  const int r = static_cast<int>((stride * es) % 16);
  return r == 0 ? 1 : 16 / std::gcd(16, r);
}

// Ring slots of a vector row kernel (norm_rows_any.cuh) and its dynamic shared memory; 0 when two
// slots do not fit.  Small footprints first: several CTAs per SM hide the per-row reductions.
int vrow_slots(int64_t N, int es, int rows_per_slot, int param_vectors, int w_dtype, size_t* smem) {
  const size_t interior = vrow_interior_bytes(N, es) * rows_per_slot;  // of all the CTA's row groups
  const size_t params = vrow_param_bytes(N, w_dtype) * param_vectors;
  // three, two or one CTA per SM (228 KB, 1 KB of it reserved per CTA, a little static shared memory)
  const size_t caps[3] = {74 * 1024, 112 * 1024 + 512, kMaxSmemPerCta - 4096};
  for (size_t cap : caps)
    for (int slots = 4; slots >= 2; --slots)
      if (slots * interior + params <= cap) {
        *smem = slots * interior + params;
        return slots;
      }
  return 0;
}

// CTAs (per shard) of a vector row kernel whose CTAs take `groups` rows at a time: enough for every
// row while they are all resident, else the resident count; a multiple of the period of the rows'
// alignment either way, so that all rows of a CTA are aligned alike.  Never more than
// kVRowPartialsPerSm partial rows (one per group) per SM.
constexpr int kVRowPartialsPerSm = 16;
// Shorter rows go to the warp-per-row kernels: the vector kernels' per-row bookkeeping outweighs their
// packets there (measured: 16-bit forward at 1.5 KB per row 0.45 against 0.55 of the copy bandwidth,
// 32-bit forward at 1.2 KB 0.82).  The backward switches earlier, because the warp-per-row path pays
// for a separate dweight / dbias pass over x and dy (514-byte rows: 0.33 against 0.18).
constexpr int64_t kVRowMinBytesFwd16 = 2049, kVRowMinBytesFwd32 = 1024, kVRowMinBytesBwd = 512;
int64_t vrow_ctas(const DeviceState& dev, int64_t rows, int groups, int64_t resident, int period) {
  resident = std::min<int64_t>(resident, (int64_t)dev.sm_count * kVRowPartialsPerSm / groups);
  const int64_t want = (rows + groups - 1) / groups;
  if (want <= resident / period * period) return (want + period - 1) / period * period;
  return resident / period * period;
}

// Forward through the vector row kernel when x and y share their rows' alignment; *done says whether
// it was launched.
int launch_vrow_fwd(DeviceState& dev, const DTypeKernels* k, int op, FwdParams& p, int es, cudaStream_t stream, bool* done) {
  *done = false;
  if ((int64_t)p.N * es < (es >= 4 ? kVRowMinBytesFwd32 : kVRowMinBytesFwd16) || !same_phase(p.x, p.x_stride, p.y, p.y_stride, es)) return B200NORM_OK;
  int shape = 0;
  while (shape < kVRowFwdCount && kVRowFwd[shape].capacity() < (int64_t)p.N * es / 16) ++shape;
  if (shape == kVRowFwdCount || k->fwd_vrows[op][shape] == nullptr) return B200NORM_OK;
  const VRowShape& sh = kVRowFwd[shape];
  const void* fn = k->fwd_vrows[op][shape];
  size_t smem;
  const int slots = vrow_slots(p.N, es, sh.groups, 2, p.w_dtype, &smem);
  if (slots == 0) return B200NORM_OK;
  int occ;
  if (int rc = occupancy(dev, fn, sh.threads(), smem, &occ)) return rc;
  const int64_t grid = vrow_ctas(dev, p.M, sh.groups, (int64_t)dev.sm_count * occ, phase_period(p.x_stride, es));
  if (grid < 1) return B200NORM_OK;
  p.V = slots;
  *done = true;
  return launch(fn, dim3(static_cast<unsigned>(grid)), dim3(sh.threads()), smem, &p, stream, false);
}

int check_common(int64_t M, int64_t N, int io_dtype, int w_dtype) {
  if (!valid_dtype(io_dtype) || !valid_dtype(w_dtype))
    return fail(B200NORM_ERR_ARG, "unknown dtype code (io %d, w %d)", io_dtype, w_dtype);
  if (M < 0 || N < 1) return fail(B200NORM_ERR_ARG, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
  if (N * kernels_for(io_dtype)->elem_size > kMaxRowBytes)
    return fail(B200NORM_ERR_UNSUPPORTED, "This layer norm doesn't support feature dim >= 64KB.");
  return B200NORM_OK;
}

int fwd_impl(int op, const void* x, int64_t xs, const void* w, const void* b, void* y, int64_t ys, float* mean,
             float* rstd, int64_t M, int64_t N, float eps, int io_dtype, int w_dtype, void* stream, int act = 0) {
  if (int rc = check_common(M, N, io_dtype, w_dtype)) return rc;
  if (!valid_act(act)) return fail(B200NORM_ERR_ARG, "unknown activation code %d", act);
  if (M == 0) return B200NORM_OK;
  if (!x || !y || !rstd || (op == kLN && !mean)) return fail(B200NORM_ERR_ARG, "null x / y / mean / rstd");
  if (xs < N || ys < N) return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  const DTypeKernels* k = kernels_for(io_dtype, act);
  const int es = k->elem_size;

  FwdParams p;
  p.x = x; p.y = y; p.w = w; p.b = (op == kLN) ? b : nullptr;
  p.mean = mean; p.rstd = rstd;
  p.x_stride = xs; p.y_stride = ys;
  p.M = M; p.N = static_cast<int>(N); p.V = 0;
  p.w_dtype = w_dtype; p.eps = eps; p.status = dev->status_dev;

  const bool packets = (N * es) % 16 == 0 && aligned16(x, xs, es) && aligned16(y, ys, es);
  const PacketKernel* pk = packets ? pick(k->fwd[op], k->n_fwd[op], N * es / 16) : nullptr;
  if (pk != nullptr && pk->packet_params && w_dtype == io_dtype &&
      (((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b)) & 15u) != 0))
    pk = nullptr;
  if (pk != nullptr) {
    p.V = static_cast<int>(N * es / 16);
    // the row slots (half a row each on a CTA pair)
    const size_t smem = static_cast<size_t>(pk->warps_m) * pk->stages * (p.V / pk->cluster) * 16;  // 0 unstaged
    int occ;  // resident CTAs per SM, or resident clusters per device
    if (int rc = occupancy(*dev, pk->fn, pk->threads(), smem, &occ, pk->cluster)) return rc;
    const int64_t resident = (pk->cluster > 1) ? occ : (int64_t)dev->sm_count * occ;
    const int64_t want = (M + pk->rows_per_cta() - 1) / pk->rows_per_cta();
    const int units = static_cast<int>(std::min<int64_t>(want, resident));
    return launch(pk->fn, dim3(units * pk->cluster), dim3(pk->threads()), smem, &p, static_cast<cudaStream_t>(stream),
                  true, pk->cluster);
  }
  if (act != 0)
    return fail(B200NORM_ERR_UNSUPPORTED,
                "a fused activation needs rows whose base, stride and length are multiples of 16 bytes; run the norm "
                "and b200norm_gelu_fwd separately");
  bool done;
  if (int rc = launch_vrow_fwd(*dev, k, op, p, es, static_cast<cudaStream_t>(stream), &done)) return rc;
  if (done) return B200NORM_OK;
  return launch_row_kernel(*dev, k->fwd_rows[op], k->fwd_warp_rows[op], M, N, es, 1, &p, static_cast<cudaStream_t>(stream));
}

// How a backward call is laid out: which kernel, how many partial rows.
struct BwdPlan {
  const PacketKernel* pk;  // null: any-alignment kernels
  int ctas_per_shard;
  size_t smem;
  const void* vrow;  // any alignment: the vector row kernel (dx and partial rows in one), or null
  int vrow_threads, vrow_groups, vrow_slots;
};

// The buffers of a backward call, for the choice among the any-alignment kernels.
struct BwdBuffers {
  const void *x, *dy, *dx;
  int64_t xs, dys, dxs;
  int w_dtype;
};

// Upper bound of the partial rows per shard of a vector row kernel: one per row group, the CTA count
// rounded up to at most 8 more (the period of the rows' alignment).
int64_t vrow_partials_bound(const DeviceState& dev, int64_t rows_per_shard) {
  return std::min<int64_t>(rows_per_shard + 64, (int64_t)dev.sm_count * kVRowPartialsPerSm);
}

// Partial rows per shard of the any-alignment dweight / dbias kernel (one thread per column, one CTA
// per 256 columns and partial row): enough CTAs to fill the GPU twice over whatever the row length,
// at least 32 rows each.  A function of the shard's shape only, so the order of additions is fixed.
int any_ctas_per_shard(int64_t rows_per_shard, int64_t N) {
  const int64_t column_blocks = (N + 255) / 256;
  const int64_t want = (2368 + column_blocks - 1) / column_blocks;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, 2048), (rows_per_shard + 31) / 32)));
}

int plan_bwd(DeviceState& dev, const DTypeKernels* k, int op, int64_t rows_per_shard, int64_t N, bool packets,
             BwdPlan* plan, int act = 0, const BwdBuffers* bufs = nullptr) {
  const int es = k->elem_size;
  plan->pk = packets ? pick(k->bwd[op], k->n_bwd[op], N * es / 16, true, N, es, act) : nullptr;
  plan->vrow = nullptr;
  if (plan->pk == nullptr) {
    plan->ctas_per_shard = any_ctas_per_shard(rows_per_shard, N);
    plan->smem = 0;
    if (bufs == nullptr || act != 0 || rows_per_shard < 1 || N * es < kVRowMinBytesBwd ||
        !same_phase(bufs->x, bufs->xs, bufs->dy, bufs->dys, es) || !same_phase(bufs->x, bufs->xs, bufs->dx, bufs->dxs, es))
      return B200NORM_OK;
    // The smallest capacity that holds the row.  Among equals, as measured: 16-bit rows of 512 packets or
    // more do best on eight warps per row (two packets per thread with xhat and w * dy kept beat four
    // packets on four warps by 15 %, and four packets on eight warps beat two on sixteen by 11 %), shorter
    // 16-bit rows on fewer warps with more packets each; 32-bit rows do equally well either way and take
    // the kernel that keeps xhat and w * dy, then more packets per thread.
    auto better = [&](int i, int b) {
      const VRowShape &si = kVRowBwd[i], &sb = kVRowBwd[b];
      if (si.capacity() != sb.capacity()) return si.capacity() < sb.capacity();
      if (es == 2) {
        if (si.capacity() >= 512 && (si.warps == 8) != (sb.warps == 8)) return si.warps == 8;
        return si.packets > sb.packets;
      }
      const int vi = k->bwd_vrow_variant[op][i], vb = k->bwd_vrow_variant[op][b];
      return vi != vb ? vi > vb : si.packets > sb.packets;
    };
    int best = -1;
    for (int i = 0; i < kVRowBwdCount; ++i) {
      if (k->bwd_vrows[op][i] == nullptr || kVRowBwd[i].capacity() < N * es / 16) continue;
      if (best < 0 || better(i, best)) best = i;
    }
    if (best >= 0) {
      const VRowShape& sh = kVRowBwd[best];
      const void* fn = k->bwd_vrows[op][best];
      size_t smem;
      const int slots = vrow_slots(N, es, 2 * sh.groups, 1, bufs->w_dtype, &smem);
      if (slots == 0) return B200NORM_OK;
      int occ;
      if (int rc = occupancy(dev, fn, sh.threads(), smem, &occ)) return rc;
      const int64_t ctas =
          vrow_ctas(dev, rows_per_shard, sh.groups, (int64_t)dev.sm_count * occ, phase_period(bufs->xs, es));
      if (ctas < 1) return B200NORM_OK;
      plan->vrow = fn;
      plan->vrow_threads = sh.threads();
      plan->vrow_groups = sh.groups;
      plan->vrow_slots = slots;
      plan->smem = smem;
      plan->ctas_per_shard = static_cast<int>(ctas * sh.groups);  // partial rows: one per row group
    }
    return B200NORM_OK;
  }
  const PacketKernel* pk = plan->pk;
  plan->smem = bwd_smem_bytes(*pk, N, es, act);
  int occ;  // resident CTAs per SM, or resident clusters per device
  if (int rc = occupancy(dev, pk->fn, pk->threads(), plan->smem, &occ, pk->cluster)) return rc;
  const int64_t resident = (pk->cluster > 1) ? occ : (int64_t)dev.sm_count * occ;
  const int64_t want = std::max<int64_t>(1, (rows_per_shard + pk->rows_per_cta() - 1) / pk->rows_per_cta());
  plan->ctas_per_shard = static_cast<int>(std::min<int64_t>(want, resident));  // units: CTAs or CTA pairs
  return B200NORM_OK;
}

size_t partial_bytes(int64_t P, int64_t N) {
  // one (P, N) fp32 block, rounded so the dbias block that follows stays 256-byte aligned
  return (static_cast<size_t>(P) * N * sizeof(float) + 255) & ~static_cast<size_t>(255);
}

int check_peers(const b200norm_peers* peers, int slots, int64_t N, int row_shards) {
  if (peers->world < 1 || peers->world > B200NORM_MAX_PEERS || peers->rank < 0 || peers->rank >= peers->world)
    return fail(B200NORM_ERR_ARG, "peers: bad world / rank (%d / %d)", peers->world, peers->rank);
  if (peers->depth < 3 || peers->depth > 8)
    return fail(B200NORM_ERR_ARG, "peers: depth must be 3..8 (got %d)", peers->depth);
  if (row_shards >= 1 && peers->world * row_shards != peers->total_shards)
    return fail(B200NORM_ERR_ARG, "peers: world %d x row_shards %d != total_shards %d", peers->world, row_shards,
                peers->total_shards);
  // each of the `depth` slots is inbox_bytes / depth and must hold (total_shards, slots, N) 8-byte entries
  const size_t need = static_cast<size_t>(peers->depth) * peers->total_shards * slots * N * 8;
  if (need > peers->inbox_bytes || peers->inbox_bytes % (16 * static_cast<size_t>(peers->depth)) != 0)
    return fail(B200NORM_ERR_ARG, "peers: inbox holds %zu bytes (must be a multiple of 16 x depth), this exchange needs %zu",
                peers->inbox_bytes, need);
  if (peers->counter == nullptr) return fail(B200NORM_ERR_ARG, "peers: null counter");
  for (int r = 0; r < peers->world; ++r)
    if (peers->inbox[r] == nullptr || (reinterpret_cast<uintptr_t>(peers->inbox[r]) & 15u) != 0)
      return fail(B200NORM_ERR_ARG, "peers: null or misaligned inbox for rank %d", r);
  return B200NORM_OK;
}

PeerTargets peer_targets(const b200norm_peers* peers) {
  PeerTargets t;
  for (int r = 0; r < kMaxPeers; ++r)
    t.inbox[r] = (r < peers->world) ? static_cast<unsigned char*>(peers->inbox[r]) : nullptr;
  t.local = static_cast<LocalState*>(peers->counter);
  t.world = peers->world; t.rank = peers->rank; t.depth = peers->depth; t.total_shards = peers->total_shards;
  t.slot_bytes = peers->inbox_bytes / peers->depth;
  return t;
}

// Checks a finish request against the inbox and turns it into the kernels' form.
int finish_spec(const b200norm_peers* peers, const b200norm_finish* fin, int* status, FinishSpec* out) {
  out->out[0] = out->out[1] = nullptr;
  out->seq = 0; out->status = status; out->slots = 0; out->N = 0; out->w_dtype = B200NORM_F32;
  if (fin == nullptr) return B200NORM_OK;
  if ((fin->slots != 1 && fin->slots != 2) || fin->N < 1 || !valid_dtype(fin->w_dtype))
    return fail(B200NORM_ERR_ARG, "bad finish request (slots=%d N=%lld w_dtype=%d)", fin->slots, (long long)fin->N,
                fin->w_dtype);
  if (int rc = check_peers(peers, fin->slots, fin->N, 0)) return rc;
  out->out[0] = fin->dw;
  out->out[1] = (fin->slots == 2) ? fin->db : nullptr;
  out->seq = fin->seq; out->slots = fin->slots; out->N = static_cast<int>(fin->N); out->w_dtype = fin->w_dtype;
  return B200NORM_OK;
}

int bwd_impl(int op, const void* x, int64_t xs, const void* dy, int64_t dys, const void* w, const float* mean,
             const float* rstd, void* dx, int64_t dxs, void* dw, void* db, float* group_sums, int row_shards,
             void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int io_dtype, int w_dtype,
             void* stream_v, const b200norm_peers* peers = nullptr, uint64_t seq = 0, int act = 0,
             const void* bias = nullptr, const b200norm_finish* finish = nullptr) {
  if (int rc = check_common(M, N, io_dtype, w_dtype)) return rc;
  if (!valid_act(act)) return fail(B200NORM_ERR_ARG, "unknown activation code %d", act);
  if (peers != nullptr) {
    if (int rc = check_peers(peers, (op == kLN) ? 2 : 1, N, row_shards)) return rc;
  }
  if (row_shards < 1 || M % row_shards != 0)
    return fail(B200NORM_ERR_ARG, "row_shards=%d must be >= 1 and divide M=%lld", row_shards, (long long)M);
  if (M > 0 && (!x || !dy || !dx || !rstd || (op == kLN && !mean)))
    return fail(B200NORM_ERR_ARG, "null x / dy / dx / mean / rstd");
  if (xs < N || dys < N || dxs < N) return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  if (op == kRMS) db = nullptr;
  const bool want_params = dw != nullptr || db != nullptr || group_sums != nullptr || peers != nullptr;
  if (M == 0 && !want_params) return B200NORM_OK;
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  const DTypeKernels* k = kernels_for(io_dtype, act);
  const int es = k->elem_size;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const bool packets =
      (N * es) % 16 == 0 && aligned16(x, xs, es) && aligned16(dy, dys, es) && aligned16(dx, dxs, es);
  BwdPlan plan;
  const BwdBuffers bufs = {x, dy, dx, xs, dys, dxs, w_dtype};
  if (int rc = plan_bwd(*dev, k, op, M / row_shards, N, packets, &plan, act, &bufs)) return rc;
  if (act != 0 && plan.pk == nullptr)
    return fail(B200NORM_ERR_UNSUPPORTED,
                "a fused activation needs rows whose base, stride and length are multiples of 16 bytes; run "
                "b200norm_gelu_bwd and the norm's backward separately");
  const int64_t P = (int64_t)plan.ctas_per_shard * row_shards;
  const int slots = (op == kLN) ? 2 : 1;

  BwdParams p;
  p.x = x; p.dy = dy; p.w = w; p.b = bias; p.mean = mean; p.rstd = rstd; p.dx = dx;
  p.dw_part = nullptr; p.db_part = nullptr;
  p.x_stride = xs; p.dy_stride = dys; p.dx_stride = dxs;
  p.M = M; p.rows_per_shard = M / row_shards; p.ctas_per_shard = plan.ctas_per_shard;
  p.N = static_cast<int>(N); p.V = static_cast<int>(N * es / 16); p.w_dtype = w_dtype;
  p.status = dev->status_dev;

  if (want_params) {
    const size_t need = partial_bytes(P, N) * slots;
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
      return fail(B200NORM_ERR_ARG, "workspace needs %zu bytes, 256-byte aligned (got %zu)", need, workspace_bytes);
    const bool want_dw = dw != nullptr || group_sums != nullptr || peers != nullptr;
    const bool want_db = op == kLN && (db != nullptr || group_sums != nullptr || peers != nullptr);
    if (want_dw) p.dw_part = static_cast<float*>(workspace);
    if (want_db) p.db_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + partial_bytes(P, N));
  }

  if (plan.pk != nullptr) {
    if (int rc = launch(plan.pk->fn, dim3(static_cast<unsigned>(P * plan.pk->cluster)), dim3(plan.pk->threads()),
                        plan.smem, &p, stream, true, plan.pk->cluster))
      return rc;
  } else if (plan.vrow != nullptr) {
    p.V = plan.vrow_slots;
    if (int rc = launch(plan.vrow, dim3(static_cast<unsigned>(P / plan.vrow_groups)), dim3(plan.vrow_threads), plan.smem, &p,
                        stream, false))
      return rc;
  } else {
    if (M > 0) {
      if (int rc = launch_row_kernel(*dev, k->bwd_dx_rows[op], k->bwd_dx_warp_rows[op], M, N, es, 2, &p, stream)) return rc;
    }
    if (want_params) {
      const dim3 grid(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(P));
      if (int rc = launch(k->bwd_dwdb_any[op], grid, dim3(256), 0, &p, stream, false)) return rc;
    }
  }
  if (!want_params) return B200NORM_OK;

  if (peers != nullptr) {  // column reduce fused with the push to every rank's inbox [and a finish]
    ColReducePushParams c;
    c.part[0] = p.dw_part; c.part[1] = p.db_part;
    c.peers = peer_targets(peers);
    if (int rc = finish_spec(peers, finish, dev->status_dev, &c.fin)) return rc;
    c.seq = seq;
    c.per_shard = plan.ctas_per_shard; c.row_shards = row_shards; c.slots = slots; c.N = static_cast<int>(N);
    // At most 256 CTAs of 512 threads: all resident at once on any device this library runs on, which
    // the finish phase relies on when it waits for entries other CTAs of the same grid push.
    const bool wide = N % 4 == 0;
    const int tiles = static_cast<int>((N + (wide ? 127 : 31)) / (wide ? 128 : 32));
    const dim3 grid(static_cast<unsigned>(std::min(tiles, 256 / slots)), slots);
    return launch(wide ? reinterpret_cast<const void*>(&colreduce_push_kernel<4>)
                       : reinterpret_cast<const void*>(&colreduce_push_kernel<1>),
                  grid, dim3(32, 16), 0, &c, stream);
  }

  ColReduceParams c;
  c.part[0] = p.dw_part; c.part[1] = p.db_part;
  c.out[0] = dw; c.out[1] = db;
  c.group_sums = group_sums;
  c.per_shard = plan.ctas_per_shard; c.row_shards = row_shards; c.slots = slots;
  c.N = static_cast<int>(N); c.w_dtype = w_dtype;
  if (N % 4 == 0 && (group_sums == nullptr || (reinterpret_cast<uintptr_t>(group_sums) & 15u) == 0))
    return launch(reinterpret_cast<const void*>(&colreduce4_kernel), dim3(static_cast<unsigned>((N + 127) / 128), slots),
                  dim3(32, 16), 0, &c, stream);
  return launch(reinterpret_cast<const void*>(&colreduce_kernel), dim3(static_cast<unsigned>((N + 31) / 32), slots),
                dim3(32, 16), 0, &c, stream);
}

// Stand-alone GeLU (TritonHub/Activations/gelu.py:31-49, 83-105): approximate 0 = erf form, 1 = tanh form.
int act_impl(bool bwd, const void* x, int64_t xs, const void* dout, int64_t ds, void* out, int64_t os, int64_t M,
             int64_t N, int approximate, int io_dtype, void* stream) {
  if (!valid_dtype(io_dtype)) return fail(B200NORM_ERR_ARG, "unknown dtype code %d", io_dtype);
  if (approximate != 0 && approximate != 1) return fail(B200NORM_ERR_ARG, "approximate must be 0 (erf) or 1 (tanh)");
  if (M < 0 || N < 1) return fail(B200NORM_ERR_ARG, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
  if (M == 0) return B200NORM_OK;
  if (!x || !out || (bwd && !dout)) return fail(B200NORM_ERR_ARG, "null x / dout / output");
  if (xs < N || os < N || (bwd && ds < N)) return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  const DTypeKernels* k = kernels_for(io_dtype, approximate == 0 ? B200NORM_ACT_GELU_ERF : B200NORM_ACT_GELU_TANH);
  const int es = k->elem_size;
  ActParams p;
  p.x = x; p.dout = dout; p.out = out;
  p.x_stride = xs; p.dout_stride = ds; p.out_stride = os;
  p.M = M; p.N = static_cast<int>(N); p.V = static_cast<int>(N * es / 16);
  const bool packets = (N * es) % 16 == 0 && aligned16(x, xs, es) && aligned16(out, os, es) &&
                       (!bwd || aligned16(dout, ds, es));
  const void* fn = packets ? k->act_packet[bwd ? 1 : 0] : k->act_any[bwd ? 1 : 0];
  const int64_t work = packets ? M * p.V : M * N;  // threads' worth of items
  int occ;
  if (int rc = occupancy(*dev, fn, 256, 0, &occ)) return rc;
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, (int64_t)dev->sm_count * occ)));
  return launch(fn, dim3(grid), dim3(256), 0, &p, static_cast<cudaStream_t>(stream), packets);
}

// Row-wise Softmax / LogSoftmax (TritonHub/Activations/softmax.py:24-41, 64-84; logsoftmax.py:26-48, 69-91).
// Forward: x -> y.  Backward: the saved output y and dout -> dx.
int softmax_impl(bool bwd, const void* x, int64_t xs, const void* dout, int64_t ds, void* out, int64_t os, int64_t M,
                 int64_t N, int log_softmax, int io_dtype, void* stream) {
  if (!valid_dtype(io_dtype)) return fail(B200NORM_ERR_ARG, "unknown dtype code %d", io_dtype);
  if (log_softmax != 0 && log_softmax != 1) return fail(B200NORM_ERR_ARG, "log_softmax must be 0 or 1");
  if (M < 0 || N < 1) return fail(B200NORM_ERR_ARG, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
  const SoftmaxTable* k = io_dtype == B200NORM_F32   ? softmax_kernels_f32()
                          : io_dtype == B200NORM_F16 ? softmax_kernels_f16()
                          : io_dtype == B200NORM_BF16 ? softmax_kernels_bf16()
                                                      : softmax_kernels_f64();
  const int es = k->elem_size;
  if (N * es > kMaxRowBytes)
    return fail(B200NORM_ERR_UNSUPPORTED, "softmax rows wider than 64KB are not supported (N=%lld)", (long long)N);
  if (M == 0) return B200NORM_OK;
  if (!x || !out || (bwd && !dout)) return fail(B200NORM_ERR_ARG, "null x / dout / output");
  if (xs < N || os < N || (bwd && ds < N)) return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  SoftmaxParams p;
  p.x = x; p.dout = dout; p.out = out;
  p.x_stride = xs; p.dout_stride = ds; p.out_stride = os;
  p.M = M; p.N = static_cast<int>(N); p.V = static_cast<int>(N * es / 16); p.status = dev->status_dev;
  const bool packets = (N * es) % 16 == 0 && aligned16(x, xs, es) && aligned16(out, os, es) &&
                       (!bwd || aligned16(dout, ds, es));
  const SoftmaxKernel* pk = nullptr;
  static const int forced = tuning_env("B200NORM_FORCE_SOFTMAX", -1);
  if (packets && forced >= 0 && forced < k->n && k->kernels[forced].capacity() >= p.V) pk = &k->kernels[forced];
  if (packets)
    for (int i = 0; i < k->n && pk == nullptr; ++i)
      if (k->kernels[i].capacity() >= p.V) pk = &k->kernels[i];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pk != nullptr) {
    const void* fn = pk->fn[log_softmax][bwd ? 1 : 0];
    const int stages = bwd ? pk->stages_bwd : pk->stages_fwd;
    const size_t smem = static_cast<size_t>(pk->warps_m) * stages * (bwd ? 2 : 1) * p.V * 16;
    int occ;
    if (int rc = occupancy(*dev, fn, pk->threads(), smem, &occ)) return rc;
    const int64_t want = (M + pk->rows_per_cta() - 1) / pk->rows_per_cta();
    const int grid = static_cast<int>(std::min<int64_t>(want, (int64_t)dev->sm_count * occ));
    return launch(fn, dim3(grid), dim3(pk->threads()), smem, &p, s);
  }
  const void* fn = k->any[log_softmax][bwd ? 1 : 0];
  int occ;
  if (int rc = occupancy(*dev, fn, 256, 0, &occ)) return rc;
  const int grid = static_cast<int>(std::min<int64_t>(M, (int64_t)dev->sm_count * occ));
  return launch(fn, dim3(grid), dim3(256), 0, &p, s, false);
}

// p-norm and normalisation over the last dimension (TritonHub/Ops/norm.py:47-60, 103-126;
// Ops/normalize.py:35-59, 119-144).  mode: 0 norm forward, 1 normalize forward, 2 normalize backward,
// 3 norm backward.  `a` is the staged input of the row kernels (x, or the saved y), `x` the input where a
// backward needs it besides.
int pnorm_impl(int mode, const void* a, int64_t as, const void* x, int64_t xs, const void* dout, int64_t ds,
               void* out, int64_t os, void* norms, int64_t M, int64_t N, float pw, float eps, int io_dtype,
               void* stream) {
  if (!valid_dtype(io_dtype)) return fail(B200NORM_ERR_ARG, "unknown dtype code %d", io_dtype);
  if (M < 0 || N < 1) return fail(B200NORM_ERR_ARG, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
  if (!(pw >= 1.f) || !(pw <= 6.f)) return fail(B200NORM_ERR_ARG, "p must be in [1, 6] (p=%g)", (double)pw);
  if (!(eps >= 0.f)) return fail(B200NORM_ERR_ARG, "eps must be non-negative");
  const PnormTable* k = io_dtype == B200NORM_F32   ? pnorm_kernels_f32()
                        : io_dtype == B200NORM_F16 ? pnorm_kernels_f16()
                        : io_dtype == B200NORM_BF16 ? pnorm_kernels_bf16()
                                                    : pnorm_kernels_f64();
  const int es = k->elem_size;
  if (N * es > kMaxRowBytes)
    return fail(B200NORM_ERR_UNSUPPORTED, "rows wider than 64KB are not supported (N=%lld)", (long long)N);
  if (M == 0) return B200NORM_OK;
  const bool has_out = mode != 0, has_dout = mode >= 2;
  const bool needs_x = mode == 3 || (mode == 2 && pw != 1.f && pw != 2.f);
  if (!norms || (mode != 3 && !a) || (has_out && !out) || (has_dout && !dout) || (needs_x && !x))
    return fail(B200NORM_ERR_ARG, "null input / output");
  if ((mode != 3 && as < N) || (has_out && os < N) || (mode == 2 && ds < N) || (needs_x && xs < N))
    return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  PnormParams p;
  p.a = a; p.dout = dout; p.x = x; p.out = out; p.norms = norms;
  p.a_stride = as; p.dout_stride = ds; p.x_stride = xs; p.out_stride = os;
  p.M = M; p.N = static_cast<int>(N); p.V = static_cast<int>(N * es / 16); p.p = pw; p.eps = eps;
  p.lanes_log2 = 0; p.status = dev->status_dev;
  const bool p2 = pw == 2.f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool packets = (N * es) % 16 == 0 && (mode == 3 || aligned16(a, as, es)) && (!has_out || aligned16(out, os, es)) &&
                       (mode != 2 || aligned16(dout, ds, es)) && (!needs_x || aligned16(x, xs, es));
  if (packets && mode == 3) {
    while ((1 << p.lanes_log2) < p.V && p.lanes_log2 < 8) ++p.lanes_log2;
    const void* fn = k->norm_bwd[p2 ? 1 : 0];
    const int rows_per_cta = 256 >> p.lanes_log2;
    int occ;
    if (int rc = occupancy(*dev, fn, 256, 0, &occ)) return rc;
    const int64_t want = (M + rows_per_cta - 1) / rows_per_cta;
    const int grid = static_cast<int>(std::min<int64_t>(want, (int64_t)dev->sm_count * occ));
    return launch(fn, dim3(grid), dim3(256), 0, &p, s);
  }
  if (packets) {
    const PnormKernel* pk = nullptr;
    static const int forced = tuning_env("B200NORM_FORCE_PNORM", -1);
    if (forced >= 0 && forced < k->n && k->kernels[forced].capacity() >= p.V) pk = &k->kernels[forced];
    for (int i = 0; i < k->n && pk == nullptr; ++i)
      if (k->kernels[i].capacity() >= p.V) pk = &k->kernels[i];
    if (pk != nullptr) {
      const void* fn = pk->fn[mode][p2 ? 1 : 0];
      const int stages = mode == 2 ? pk->stages_bwd : pk->stages_fwd;
      const size_t smem = static_cast<size_t>(pk->warps_m) * stages * (mode == 2 ? 2 : 1) * p.V * 16;
      int occ;
      if (int rc = occupancy(*dev, fn, pk->threads(), smem, &occ)) return rc;
      const int64_t want = (M + pk->rows_per_cta() - 1) / pk->rows_per_cta();
      const int grid = static_cast<int>(std::min<int64_t>(want, (int64_t)dev->sm_count * occ));
      return launch(fn, dim3(grid), dim3(pk->threads()), smem, &p, s);
    }
  }
  const void* fn = k->any[mode];
  int occ;
  if (int rc = occupancy(*dev, fn, 256, 0, &occ)) return rc;
  const int grid = static_cast<int>(std::min<int64_t>(M, (int64_t)dev->sm_count * occ));
  return launch(fn, dim3(grid), dim3(256), 0, &p, s, false);
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward with built-in scratch (b200norm_rms_bwd_static): for hosts that plan their
// device memory once and cannot hand over, or allocate, a workspace per call.
//
// The dweight partial rows live in this file-scope device array instead of a caller buffer.
// Every GPU that loads the library holds it until the process exits.  All calls on a device
// share it and it keeps the last call's contents; nothing in it has to start at zero, because
// each launch writes every partial row (all P of them, zero-row CTAs included) before the
// column reduce reads them.  Calls that overlap on the GPU race on it.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = B200NORM_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_status;  // where this variant's kernels report an expired wait

struct StaticState {
  std::once_flag once;
  cudaError_t init_err = cudaSuccess;
  void* scratch = nullptr;     // device address of g_static_scratch
  int* status_dev = nullptr;   // device address of g_static_status
};
StaticState g_static[kMaxDevices];

// Per-device set-up of the static variant, run by its first call on each device with that
// device current.  In host code `g_static_scratch` names a host-side stand-in for the device
// array, not a device address -- handing it to a kernel would fault, or quietly use the wrong
// memory where the GPU can reach host memory -- so the address is asked for here, once.
// Launch planning (SM count, occupancies, shared-memory allowances) is the device's one shared
// record, `dev`: a private copy here once let this path lower an allowance under a launch shape
// that the other entry points had already cached.
int static_state(StaticState** out, DeviceState** dev) {
  if (int rc = device_caches(dev)) return rc;
  int d = -1;
  cudaError_t e = cudaGetDevice(&d);
  if (e != cudaSuccess) return fail(B200NORM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  StaticState& s = g_static[d];
  std::call_once(s.once, [&]() {
    s.init_err = cudaGetSymbolAddress(&s.scratch, g_static_scratch);
    if (s.init_err != cudaSuccess) return;
    s.init_err = cudaGetSymbolAddress(reinterpret_cast<void**>(&s.status_dev), g_static_status);
  });
  if (s.init_err != cudaSuccess)
    return fail(B200NORM_ERR_CUDA, "static scratch set-up: %s", cudaGetErrorString(s.init_err));
  *out = &s;
  return B200NORM_OK;
}

int rms_bwd_static_impl(const void* x, int64_t xs, const void* dy, int64_t dys, const void* w, const float* rstd,
                        void* dx, int64_t dxs, void* dw, int64_t M, int64_t N, int io_dtype, int w_dtype,
                        void* stream_v) {
  if (int rc = check_common(M, N, io_dtype, w_dtype)) return rc;
  if (M > 0 && (!x || !dy || !dx || !rstd)) return fail(B200NORM_ERR_ARG, "null x / dy / dx / rstd");
  if (xs < N || dys < N || dxs < N) return fail(B200NORM_ERR_ARG, "row stride smaller than N");
  if (M == 0 && dw == nullptr) return B200NORM_OK;
  StaticState* st = nullptr;
  DeviceState* dev = nullptr;
  if (int rc = static_state(&st, &dev)) return rc;
  const DTypeKernels* k = kernels_for(io_dtype);
  const int es = k->elem_size;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const bool packets =
      (N * es) % 16 == 0 && aligned16(x, xs, es) && aligned16(dy, dys, es) && aligned16(dx, dxs, es);
  BwdPlan plan;
  if (int rc = plan_bwd(*dev, k, kRMS, M, N, packets, &plan)) return rc;
  const int64_t P = plan.ctas_per_shard;
  if (dw != nullptr && partial_bytes(P, N) > kStaticScratchBytes)
    return fail(B200NORM_ERR_UNSUPPORTED,
                "b200norm_rms_bwd_static: %zu bytes of dweight partial rows needed (%lld rows x N=%lld), the built-in "
                "scratch holds %zu; use b200norm_rms_bwd with a caller workspace",
                partial_bytes(P, N), (long long)P, (long long)N, kStaticScratchBytes);

  BwdParams p;
  p.x = x; p.dy = dy; p.w = w; p.b = nullptr; p.mean = nullptr; p.rstd = rstd; p.dx = dx;
  p.dw_part = (dw != nullptr) ? static_cast<float*>(st->scratch) : nullptr;
  p.db_part = nullptr;
  p.x_stride = xs; p.dy_stride = dys; p.dx_stride = dxs;
  p.M = M; p.rows_per_shard = M; p.ctas_per_shard = plan.ctas_per_shard;
  p.N = static_cast<int>(N); p.V = static_cast<int>(N * es / 16); p.w_dtype = w_dtype;
  p.status = st->status_dev;

  if (plan.pk != nullptr) {
    if (int rc = launch(plan.pk->fn, dim3(static_cast<unsigned>(P * plan.pk->cluster)), dim3(plan.pk->threads()),
                        plan.smem, &p, stream, true, plan.pk->cluster))
      return rc;
  } else {
    if (M > 0) {
      if (int rc = launch_row_kernel(*dev, k->bwd_dx_rows[kRMS], k->bwd_dx_warp_rows[kRMS], M, N, es, 2, &p, stream)) return rc;
    }
    if (dw != nullptr) {
      const dim3 grid(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(P));
      if (int rc = launch(k->bwd_dwdb_any[kRMS], grid, dim3(256), 0, &p, stream, false)) return rc;
    }
  }
  if (dw == nullptr) return B200NORM_OK;

  ColReduceParams c;
  c.part[0] = p.dw_part; c.part[1] = nullptr;
  c.out[0] = dw; c.out[1] = nullptr;
  c.group_sums = nullptr;
  c.per_shard = plan.ctas_per_shard; c.row_shards = 1; c.slots = 1;
  c.N = static_cast<int>(N); c.w_dtype = w_dtype;
  return launch(reinterpret_cast<const void*>(&colreduce_kernel), dim3(static_cast<unsigned>((N + 31) / 32), 1),
                dim3(32, 16), 0, &c, stream);
}

}  // namespace
}  // namespace b200norm

using namespace b200norm;

extern "C" {

int b200norm_version(void) { return B200NORM_VERSION; }

const char* b200norm_last_error(void) { return g_err; }

int b200norm_query(int* sm_count, int* max_partials) {
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  if (sm_count) *sm_count = dev->sm_count;
  if (max_partials) *max_partials = std::max(256, dev->sm_count * 16);
  return B200NORM_OK;
}

int b200norm_device_status(int clear) {
  DeviceState* dev = nullptr;
  if (device_state(&dev)) return -1;
  const int v = *static_cast<volatile int*>(dev->status_host);
  if (clear) *static_cast<volatile int*>(dev->status_host) = 0;
  return v;
}

size_t b200norm_bwd_workspace_bytes(int64_t M, int64_t N, int io_dtype, int row_shards) {
  if (check_common(M, N, io_dtype, B200NORM_F32) || row_shards < 1 || M % row_shards != 0) return 0;
  DeviceState* dev = nullptr;
  if (device_state(&dev)) return 0;
  const DTypeKernels* k = kernels_for(io_dtype);
  const int64_t rps = M / row_shards;
  int64_t per_shard = any_ctas_per_shard(rps, N);
  if (N * k->elem_size >= kVRowMinBytesBwd) per_shard = std::max(per_shard, vrow_partials_bound(*dev, rps));  // misaligned views of any N
  if ((N * k->elem_size) % 16 == 0) {
    // LayerNorm and RMSNorm instantiations may differ in occupancy: take the larger.
    // and with or without a fused activation
    for (int act = 0; act < 3; ++act)
      for (int op = 0; op < 2; ++op) {
        BwdPlan plan;
        if (plan_bwd(*dev, kernels_for(io_dtype, act), op, rps, N, true, &plan, act)) return 0;
        if (plan.pk != nullptr) per_shard = std::max<int64_t>(per_shard, plan.ctas_per_shard);
      }
  }
  return 2 * partial_bytes(per_shard * row_shards, N);
}

int b200norm_ln_fwd(const void* x, int64_t x_row_stride, const void* w, const void* b, void* y,
                    int64_t y_row_stride, float* mean, float* rstd, int64_t M, int64_t N, float eps,
                    int io_dtype, int w_dtype, void* stream) {
  return fwd_impl(kLN, x, x_row_stride, w, b, y, y_row_stride, mean, rstd, M, N, eps, io_dtype, w_dtype, stream);
}

int b200norm_rms_fwd(const void* x, int64_t x_row_stride, const void* w, void* y, int64_t y_row_stride,
                     float* rstd, int64_t M, int64_t N, float eps, int io_dtype, int w_dtype, void* stream) {
  return fwd_impl(kRMS, x, x_row_stride, w, nullptr, y, y_row_stride, nullptr, rstd, M, N, eps, io_dtype, w_dtype,
                  stream);
}

int b200norm_ln_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                    const void* w, const float* mean, const float* rstd, void* dx, int64_t dx_row_stride,
                    void* dw, void* db, float* group_sums, int row_shards, void* workspace,
                    size_t workspace_bytes, int64_t M, int64_t N, int io_dtype, int w_dtype, void* stream) {
  return bwd_impl(kLN, x, x_row_stride, dy, dy_row_stride, w, mean, rstd, dx, dx_row_stride, dw, db, group_sums,
                  row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream);
}

int b200norm_rms_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                     const void* w, const float* rstd, void* dx, int64_t dx_row_stride, void* dw,
                     float* group_sums, int row_shards, void* workspace, size_t workspace_bytes, int64_t M,
                     int64_t N, int io_dtype, int w_dtype, void* stream) {
  return bwd_impl(kRMS, x, x_row_stride, dy, dy_row_stride, w, nullptr, rstd, dx, dx_row_stride, dw, nullptr,
                  group_sums, row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream);
}

int b200norm_finalize_dwdb(const float* group_sums, int groups, int slots, void* dw, void* db, int64_t N,
                           int w_dtype, void* stream) {
  if (!group_sums || groups < 1 || (slots != 1 && slots != 2) || N < 1 || !valid_dtype(w_dtype))
    return fail(B200NORM_ERR_ARG, "bad finalize arguments (groups=%d slots=%d N=%lld)", groups, slots, (long long)N);
  FinalizeParams p;
  p.group_sums = group_sums;
  p.out[0] = dw;
  p.out[1] = (slots == 2) ? db : nullptr;
  p.groups = groups; p.slots = slots; p.N = static_cast<int>(N); p.w_dtype = w_dtype;
  return launch(reinterpret_cast<const void*>(&finalize_kernel), dim3(static_cast<unsigned>((N + 255) / 256), slots),
                dim3(256), 0, &p, static_cast<cudaStream_t>(stream));
}

int b200norm_ln_bwd_push(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride, const void* w,
                         const float* mean, const float* rstd, void* dx, int64_t dx_row_stride, int row_shards,
                         void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int io_dtype, int w_dtype,
                         const b200norm_peers* peers, uint64_t seq, const b200norm_finish* finish, void* stream) {
  if (peers == nullptr) return fail(B200NORM_ERR_ARG, "null peers");
  return bwd_impl(kLN, x, x_row_stride, dy, dy_row_stride, w, mean, rstd, dx, dx_row_stride, nullptr, nullptr,
                  nullptr, row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream, peers, seq, 0,
                  nullptr, finish);
}

int b200norm_rms_bwd_push(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride, const void* w,
                          const float* rstd, void* dx, int64_t dx_row_stride, int row_shards, void* workspace,
                          size_t workspace_bytes, int64_t M, int64_t N, int io_dtype, int w_dtype,
                          const b200norm_peers* peers, uint64_t seq, const b200norm_finish* finish, void* stream) {
  if (peers == nullptr) return fail(B200NORM_ERR_ARG, "null peers");
  return bwd_impl(kRMS, x, x_row_stride, dy, dy_row_stride, w, nullptr, rstd, dx, dx_row_stride, nullptr, nullptr,
                  nullptr, row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream, peers, seq, 0,
                  nullptr, finish);
}

int b200norm_finalize_pushed(const b200norm_peers* peers, uint64_t seq, int slots, void* dw, void* db, int64_t N,
                             int w_dtype, void* stream) {
  if (peers == nullptr) return fail(B200NORM_ERR_ARG, "null peers");
  DeviceState* dev = nullptr;
  if (int rc = device_state(&dev)) return rc;
  b200norm_finish fin;
  fin.seq = seq; fin.slots = slots; fin.w_dtype = w_dtype; fin.N = N; fin.dw = dw; fin.db = db;
  FinalizePushedParams p;
  p.peers = peer_targets(peers);
  if (int rc = finish_spec(peers, &fin, dev->status_dev, &p.fin)) return rc;
  const int64_t items = (N % 2 == 0 ? N / 2 : N) * slots;
  return launch(reinterpret_cast<const void*>(&finalize_pushed_kernel),
                dim3(static_cast<unsigned>(std::min<int64_t>((items + 255) / 256, 256))), dim3(256), 0, &p,
                static_cast<cudaStream_t>(stream));
}

int b200norm_ln_act_fwd(const void* x, int64_t x_row_stride, const void* w, const void* b, void* z,
                        int64_t z_row_stride, float* mean, float* rstd, int64_t M, int64_t N, float eps, int act,
                        int io_dtype, int w_dtype, void* stream) {
  return fwd_impl(kLN, x, x_row_stride, w, b, z, z_row_stride, mean, rstd, M, N, eps, io_dtype, w_dtype, stream, act);
}

int b200norm_rms_act_fwd(const void* x, int64_t x_row_stride, const void* w, void* z, int64_t z_row_stride,
                         float* rstd, int64_t M, int64_t N, float eps, int act, int io_dtype, int w_dtype,
                         void* stream) {
  return fwd_impl(kRMS, x, x_row_stride, w, nullptr, z, z_row_stride, nullptr, rstd, M, N, eps, io_dtype, w_dtype,
                  stream, act);
}

int b200norm_ln_act_bwd(const void* x, int64_t x_row_stride, const void* dz, int64_t dz_row_stride, const void* w,
                        const void* b, const float* mean, const float* rstd, void* dx, int64_t dx_row_stride,
                        void* dw, void* db, float* group_sums, int row_shards, void* workspace,
                        size_t workspace_bytes, int64_t M, int64_t N, int act, int io_dtype, int w_dtype,
                        void* stream) {
  return bwd_impl(kLN, x, x_row_stride, dz, dz_row_stride, w, mean, rstd, dx, dx_row_stride, dw, db, group_sums,
                  row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream, nullptr, 0, act, b);
}

int b200norm_rms_act_bwd(const void* x, int64_t x_row_stride, const void* dz, int64_t dz_row_stride, const void* w,
                         const float* rstd, void* dx, int64_t dx_row_stride, void* dw, float* group_sums,
                         int row_shards, void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int act,
                         int io_dtype, int w_dtype, void* stream) {
  return bwd_impl(kRMS, x, x_row_stride, dz, dz_row_stride, w, nullptr, rstd, dx, dx_row_stride, dw, nullptr,
                  group_sums, row_shards, workspace, workspace_bytes, M, N, io_dtype, w_dtype, stream, nullptr, 0, act,
                  nullptr);
}

int b200norm_gelu_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int64_t M, int64_t N,
                      int approximate, int io_dtype, void* stream) {
  return act_impl(false, x, x_row_stride, nullptr, 0, y, y_row_stride, M, N, approximate, io_dtype, stream);
}

int b200norm_gelu_bwd(const void* x, int64_t x_row_stride, const void* dout, int64_t dout_row_stride, void* dx,
                      int64_t dx_row_stride, int64_t M, int64_t N, int approximate, int io_dtype, void* stream) {
  return act_impl(true, x, x_row_stride, dout, dout_row_stride, dx, dx_row_stride, M, N, approximate, io_dtype,
                  stream);
}

int b200norm_pnorm_fwd(const void* x, int64_t x_row_stride, void* norms, int64_t M, int64_t N, float p, float eps,
                       int io_dtype, void* stream) {
  return pnorm_impl(0, x, x_row_stride, nullptr, 0, nullptr, 0, nullptr, 0, norms, M, N, p, eps, io_dtype, stream);
}

int b200norm_pnorm_bwd(const void* x, int64_t x_row_stride, const void* norms, const void* dout, void* dx,
                       int64_t dx_row_stride, int64_t M, int64_t N, float p, int io_dtype, void* stream) {
  return pnorm_impl(3, nullptr, 0, x, x_row_stride, dout, 0, dx, dx_row_stride, const_cast<void*>(norms), M, N, p, 0.f,
                    io_dtype, stream);
}

int b200norm_normalize_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, void* norms, int64_t M,
                           int64_t N, float p, float eps, int io_dtype, void* stream) {
  return pnorm_impl(1, x, x_row_stride, nullptr, 0, nullptr, 0, y, y_row_stride, norms, M, N, p, eps, io_dtype, stream);
}

int b200norm_normalize_bwd(const void* x, int64_t x_row_stride, const void* y, int64_t y_row_stride, const void* norms,
                           const void* dout, int64_t dout_row_stride, void* dx, int64_t dx_row_stride, int64_t M,
                           int64_t N, float p, int io_dtype, void* stream) {
  // the projection sum runs over x for p = 1 and over the saved output otherwise (normalize.py:87-95)
  const bool p1 = p == 1.f;
  return pnorm_impl(2, p1 ? x : y, p1 ? x_row_stride : y_row_stride, x, x_row_stride, dout, dout_row_stride, dx,
                    dx_row_stride, const_cast<void*>(norms), M, N, p, 0.f, io_dtype, stream);
}

int b200norm_softmax_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int64_t M, int64_t N,
                         int log_softmax, int io_dtype, void* stream) {
  return softmax_impl(false, x, x_row_stride, nullptr, 0, y, y_row_stride, M, N, log_softmax, io_dtype, stream);
}

int b200norm_softmax_bwd(const void* y, int64_t y_row_stride, const void* dout, int64_t dout_row_stride, void* dx,
                         int64_t dx_row_stride, int64_t M, int64_t N, int log_softmax, int io_dtype, void* stream) {
  return softmax_impl(true, y, y_row_stride, dout, dout_row_stride, dx, dx_row_stride, M, N, log_softmax, io_dtype,
                      stream);
}

int b200norm_rms_bwd_static(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                            const void* w, const float* rstd, void* dx, int64_t dx_row_stride, void* dw, int64_t M,
                            int64_t N, int io_dtype, int w_dtype, void* stream) {
  return rms_bwd_static_impl(x, x_row_stride, dy, dy_row_stride, w, rstd, dx, dx_row_stride, dw, M, N, io_dtype,
                             w_dtype, stream);
}

}  // extern "C"
