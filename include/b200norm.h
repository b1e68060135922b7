/*
 * b200norm.h -- C ABI of libb200norm.so: LayerNorm / RMSNorm forward and backward for
 * NVIDIA B200 (sm_100a), written as hand-tuned CUDA kernels.
 *
 * The library stands where the host wrappers of TritonHub's Normalization package stand:
 *
 *   b200norm_ln_fwd   replaces  _layernorm_fwd   TritonHub/Normalization/layernorm.py:48-87
 *                               (+ kernel        TritonHub/Normalization/layernorm.py:14-46)
 *   b200norm_ln_bwd   replaces  _layernorm_bwd   TritonHub/Normalization/layernorm.py:155-209
 *                               (+ kernel        TritonHub/Normalization/layernorm.py:94-153,
 *                                 + the `_dw.sum(0).to(dtype)` finish at :207-208)
 *   b200norm_rms_fwd  replaces  _rmsnorm_fwd     TritonHub/Normalization/rmsnorm.py:40-70
 *   b200norm_rms_bwd  replaces  _rmsnorm_bwd     TritonHub/Normalization/rmsnorm.py:124-167
 *   the launch table behind them replaces get_cuda_autotune_config(block_keys=None)
 *                                                TritonHub/autotune.py:61-65
 *
 * and, for the steps either side of the norm, where these stand (each documented at its declaration):
 *
 *   b200norm_gelu_fwd/_bwd, b200norm_{ln,rms}_act_fwd/_bwd     TritonHub/Activations/gelu.py
 *   b200norm_softmax_fwd/_bwd                                  TritonHub/Activations/softmax.py, logsoftmax.py, softmin.py
 *   b200norm_pnorm_fwd/_bwd, b200norm_normalize_fwd/_bwd       TritonHub/Ops/norm.py, normalize.py
 *
 * Conventions shared by every entry point
 *   - Rows are the flattened leading dimensions: x is (M, N) with unit column stride and a
 *     row stride given in ELEMENTS (>= N).  y, dy and dx likewise.
 *   - All pointers are device pointers of the CUDA device that is current on the calling
 *     thread; the caller owns every buffer.  The library only enqueues work on `stream`
 *     (a cudaStream_t passed as void*; NULL = legacy default stream).  It never
 *     synchronises, never changes the current device and, after the first call on a device,
 *     never allocates.  The first call on a device caches the device's SM count, the
 *     occupancy of each kernel and maps a small pinned status word; make that call before
 *     any stream capture.
 *   - Alignment.  Any base address, row stride and row length are accepted, like the reference's
 *     masked loads (layernorm.py:28-46, `cols < N`).  Fastest: every row of every buffer starts on
 *     a 16-byte boundary and is a multiple of 16 bytes long.  Next: rows of at least 0.5 - 2 KB
 *     whose buffers are misaligned ALIKE (x, y -- and dy, dx -- start each row at the same offset
 *     within a 16-byte line: contiguous tensors of an odd row length, views offset by the same
 *     number of elements); their 16-byte interiors still move and compute as 16-byte packets.
 *     Everything else runs element by element at a fraction of the bandwidth.
 *   - Arithmetic is fp32 whatever the storage type (the reference promotes every load to
 *     fp32, layernorm.py:31,41); results are rounded once on store.
 *   - Return value: B200NORM_OK or one of the error codes below.  Nothing throws or aborts.
 *     b200norm_last_error() returns a thread-local description of the last failure.
 *   - Re-entrant and thread-safe (autograd calls backward from its own worker thread).
 */
#ifndef B200NORM_H_
#define B200NORM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200NORM_VERSION 101 /* major*10000 + minor*100 + patch */

#if defined(__GNUC__)
#define B200NORM_API __attribute__((visibility("default")))
#else
#define B200NORM_API
#endif

/* Storage types of x / y / dy / dx (io_dtype) and of weight / bias / dweight / dbias (w_dtype). */
enum b200norm_dtype {
  B200NORM_F32 = 0,
  B200NORM_F16 = 1,
  B200NORM_BF16 = 2,
  B200NORM_F64 = 3 /* accepted like the reference does: loaded, then computed in fp32 */
};

enum b200norm_status {
  B200NORM_OK = 0,
  B200NORM_ERR_ARG = 1,         /* null pointer, bad stride, negative size, bad enum, small workspace */
  B200NORM_ERR_UNSUPPORTED = 2, /* row wider than 64 KB (the reference's limit, layernorm.py:69-72) */
  B200NORM_ERR_CUDA = 3,        /* a CUDA runtime call failed; text in b200norm_last_error() */
  B200NORM_ERR_TIMEOUT = 4      /* a bounded device-side wait gave up (see b200norm_device_status) */
};

/* Library version (B200NORM_VERSION of the build). */
B200NORM_API int b200norm_version(void);

/* SM count of the current device and the largest number of dweight/dbias partial rows a
 * backward call can write there.  Cached per device; replaces the per-call
 * torch.cuda.get_device_properties() of layernorm.py:182. */
B200NORM_API int b200norm_query(int* sm_count, int* max_partials);

/* Text for the last non-OK status returned on this thread ("" if none). */
B200NORM_API const char* b200norm_last_error(void);

/* Sticky per-device status word written by kernels whose bounded waits (mbarrier waits on
 * bulk copies) ran out: 0 = never happened.  Reading it does not synchronise; call it after
 * the stream has been synchronised.  `clear` != 0 resets it. */
B200NORM_API int b200norm_device_status(int clear);

/* Bytes of scratch a backward call needs for its fp32 dweight/dbias partial rows
 * (replaces the `_dw`/`_db` (sm_count, N) buffers of layernorm.py:183-184).
 * `row_shards` is the number of equal row groups whose sums are kept apart (1 unless the
 * caller wants results that do not depend on how many GPUs the rows are spread over). */
B200NORM_API size_t b200norm_bwd_workspace_bytes(int64_t M, int64_t N, int io_dtype, int row_shards);

/*
 * LayerNorm forward (layernorm.py:14-87): per row
 *   mean = sum(x)/N; var = sum((x-mean)^2)/N; rstd = 1/sqrt(var+eps);
 *   y = (x-mean)*rstd [*w] [+b]
 * w, b may each be NULL (HAS_WEIGHT / HAS_BIAS false).  mean and rstd are (M,) fp32 outputs
 * saved for backward.
 */
B200NORM_API int b200norm_ln_fwd(const void* x, int64_t x_row_stride, const void* w, const void* b, void* y,
                    int64_t y_row_stride, float* mean, float* rstd, int64_t M, int64_t N, float eps,
                    int io_dtype, int w_dtype, void* stream);

/*
 * RMSNorm forward (rmsnorm.py:14-70): rstd = 1/sqrt(sum(x^2)/N + eps); y = x*rstd [*w].
 */
B200NORM_API int b200norm_rms_fwd(const void* x, int64_t x_row_stride, const void* w, void* y, int64_t y_row_stride,
                     float* rstd, int64_t M, int64_t N, float eps, int io_dtype, int w_dtype,
                     void* stream);

/*
 * LayerNorm backward (layernorm.py:94-209): per row, with xhat = (x-mean)*rstd, wdy = w*dy
 * (w = 1 when NULL):
 *   c1 = sum(xhat*wdy)/N; c2 = sum(wdy)/N; dx = (wdy - (xhat*c1 + c2))*rstd
 *   dw = sum_rows(dy*xhat); db = sum_rows(dy)
 * dw / db: (N,) outputs in w_dtype, or NULL to skip that gradient.
 * group_sums: optional fp32 output (row_shards, 2, N): the dweight (slot 0) and dbias (slot 1)
 *   sums of each row shard before the final add and cast -- what a multi-GPU caller
 *   exchanges.  NULL if not wanted.  When given, dw/db are still written if non-NULL.
 * row_shards >= 1 splits the M rows into that many equal groups (M % row_shards == 0) whose
 *   partial sums are formed separately and then added left to right, so that a run over one
 *   shard per GPU followed by b200norm_finalize_dwdb gives bit-identical dw/db.
 * workspace: at least b200norm_bwd_workspace_bytes(M, N, io_dtype, row_shards) bytes,
 *   256-byte aligned; contents undefined on entry and on exit.
 */
B200NORM_API int b200norm_ln_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                    const void* w, const float* mean, const float* rstd, void* dx,
                    int64_t dx_row_stride, void* dw, void* db, float* group_sums, int row_shards,
                    void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int io_dtype,
                    int w_dtype, void* stream);

/*
 * RMSNorm backward (rmsnorm.py:77-167): xhat = x*rstd; c1 = sum(xhat*wdy)/N;
 *   dx = (wdy - xhat*c1)*rstd; dw = sum_rows(dy*xhat).
 * group_sums, when given, is (row_shards, 1, N) fp32.
 */
B200NORM_API int b200norm_rms_bwd(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                     const void* w, const float* rstd, void* dx, int64_t dx_row_stride, void* dw,
                     float* group_sums, int row_shards, void* workspace, size_t workspace_bytes,
                     int64_t M, int64_t N, int io_dtype, int w_dtype, void* stream);

/*
 * Finish dweight/dbias from gathered shard sums: out[k][n] = sum_{g=0..groups-1} in[g][k][n]
 * added left to right in fp32, then cast to w_dtype.  `slots` is 2 for LayerNorm (dw, db) and
 * 1 for RMSNorm.  This is the step after an all-gather of every rank's group_sums; it has no
 * counterpart in the single-GPU reference beyond the `.sum(0).to(dtype)` of layernorm.py:207-208.
 * dw / db may be NULL.
 */
B200NORM_API int b200norm_finalize_dwdb(const float* group_sums, int groups, int slots, void* dw, void* db, int64_t N,
                           int w_dtype, void* stream);

/*
 * The activation that follows the norm in the reference's Quick Start (README.md:44-48):
 * GeLU, erf or tanh form (TritonHub/Activations/gelu.py).
 *
 * b200norm_gelu_fwd / _bwd replace _gelu_fwd (gelu.py:31-49, kernel :12-29) and _gelu_bwd
 *   (gelu.py:83-105, kernel :56-81): y = gelu(x); dx = dout * gelu'(x).  approximate: 0 = 'none'
 *   (erf), 1 = 'tanh'.  Any alignment is accepted.
 * b200norm_*_act_fwd / _bwd fuse it into the norm (the reference runs two kernels and writes the
 *   normalised tensor to memory in between; these do not): forward writes z = act(norm(x)) and
 *   the same mean / rstd; backward takes dz, rebuilds y = xhat*w + b from the row (hence `b`),
 *   forms dy = dz * act'(y) rounded to the storage type, and continues as b200norm_*_bwd.  Rows
 *   must be 16-byte aligned in base, stride and length (B200NORM_ERR_UNSUPPORTED otherwise: run
 *   the two steps separately).  act = B200NORM_ACT_NONE makes them identical to the plain entry
 *   points.
 */
enum b200norm_act { B200NORM_ACT_NONE = 0, B200NORM_ACT_GELU_ERF = 1, B200NORM_ACT_GELU_TANH = 2 };

B200NORM_API int b200norm_gelu_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int64_t M,
                                   int64_t N, int approximate, int io_dtype, void* stream);
B200NORM_API int b200norm_gelu_bwd(const void* x, int64_t x_row_stride, const void* dout, int64_t dout_row_stride,
                                   void* dx, int64_t dx_row_stride, int64_t M, int64_t N, int approximate,
                                   int io_dtype, void* stream);
B200NORM_API int b200norm_ln_act_fwd(const void* x, int64_t x_row_stride, const void* w, const void* b, void* z,
                                     int64_t z_row_stride, float* mean, float* rstd, int64_t M, int64_t N,
                                     float eps, int act, int io_dtype, int w_dtype, void* stream);
B200NORM_API int b200norm_rms_act_fwd(const void* x, int64_t x_row_stride, const void* w, void* z,
                                      int64_t z_row_stride, float* rstd, int64_t M, int64_t N, float eps, int act,
                                      int io_dtype, int w_dtype, void* stream);
B200NORM_API int b200norm_ln_act_bwd(const void* x, int64_t x_row_stride, const void* dz, int64_t dz_row_stride,
                                     const void* w, const void* b, const float* mean, const float* rstd, void* dx,
                                     int64_t dx_row_stride, void* dw, void* db, float* group_sums, int row_shards,
                                     void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int act,
                                     int io_dtype, int w_dtype, void* stream);
B200NORM_API int b200norm_rms_act_bwd(const void* x, int64_t x_row_stride, const void* dz, int64_t dz_row_stride,
                                      const void* w, const float* rstd, void* dx, int64_t dx_row_stride, void* dw,
                                      float* group_sums, int row_shards, void* workspace, size_t workspace_bytes,
                                      int64_t M, int64_t N, int act, int io_dtype, int w_dtype, void* stream);

/*
 * Row-wise Softmax / LogSoftmax over the last dimension, the reference's other "row in registers
 * + row reduction" kernels (TritonHub/Activations/softmax.py, logsoftmax.py; Softmin is Softmax of
 * -x, softmin.py:103).  b200norm_softmax_fwd replaces _softmax_fwd / _logsoftmax_fwd
 * (softmax.py:24-41, logsoftmax.py:26-48): y = exp(x - max) / sum exp(x - max), or its logarithm
 * when log_softmax != 0.  b200norm_softmax_bwd replaces _softmax_bwd / _logsoftmax_bwd
 * (softmax.py:64-84, logsoftmax.py:69-91); like them it takes the saved OUTPUT y, not x:
 *   Softmax dx = y * (dout - sum(dout * y));  LogSoftmax dx = dout - exp(y) * sum(dout).
 * fp32 arithmetic, any alignment, rows up to 64 KB.
 */
B200NORM_API int b200norm_softmax_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, int64_t M,
                                      int64_t N, int log_softmax, int io_dtype, void* stream);
B200NORM_API int b200norm_softmax_bwd(const void* y, int64_t y_row_stride, const void* dout, int64_t dout_row_stride,
                                      void* dx, int64_t dx_row_stride, int64_t M, int64_t N, int log_softmax,
                                      int io_dtype, void* stream);

/*
 * p-norm and normalisation over the last dimension, the reference's TritonHub.Ops.norm / normalize
 * (Ops/norm.py, Ops/normalize.py), on (M, N) rows (the reference's (B, M, K) flattened):
 *   b200norm_pnorm_fwd      replaces _norm_fwd (norm.py:47-60):
 *                           norms[m] = max((sum_k |x[m,k]|^p)^(1/p), eps), stored in the storage type;
 *   b200norm_pnorm_bwd      replaces _norm_bwd (norm.py:103-126); dout and norms are (M,) contiguous:
 *                           p = 1: dout*sign(x); p = 2: dout*x/norms; else dout*sign(x)*|x|^(p-1)/norms^(p-1);
 *   b200norm_normalize_fwd  replaces _normalize_fwd (normalize.py:35-59), both of its kernels in one:
 *                           norms as above, y = x / norms with norms as stored (rounded);
 *   b200norm_normalize_bwd  replaces _normalize_bwd (normalize.py:119-144); x is read for p = 1 and for p
 *                           other than 2, y for every p but 1; either may be NULL where it is not read.
 * 1 <= p <= 6 and eps >= 0 as in the reference's wrappers (norm.py:143-144); fp32 arithmetic, any
 * alignment, rows up to 64 KB.
 */
B200NORM_API int b200norm_pnorm_fwd(const void* x, int64_t x_row_stride, void* norms, int64_t M, int64_t N, float p,
                                    float eps, int io_dtype, void* stream);
B200NORM_API int b200norm_pnorm_bwd(const void* x, int64_t x_row_stride, const void* norms, const void* dout, void* dx,
                                    int64_t dx_row_stride, int64_t M, int64_t N, float p, int io_dtype, void* stream);
B200NORM_API int b200norm_normalize_fwd(const void* x, int64_t x_row_stride, void* y, int64_t y_row_stride, void* norms,
                                        int64_t M, int64_t N, float p, float eps, int io_dtype, void* stream);
B200NORM_API int b200norm_normalize_bwd(const void* x, int64_t x_row_stride, const void* y, int64_t y_row_stride,
                                        const void* norms, const void* dout, int64_t dout_row_stride, void* dx,
                                        int64_t dx_row_stride, int64_t M, int64_t N, float p, int io_dtype,
                                        void* stream);

/*
 * Multi-GPU exchange fused into the backward's column reduce.  (No counterpart in the reference,
 * which is single-GPU.)  One process per GPU; every rank owns an inbox of `depth` equal slots of
 * inbox_bytes / depth each, in memory that is peer-mapped into all ranks (CUDA IPC / VMM --
 * torch.distributed._symmetric_memory provides it).  A slot holds one exchange's
 * (total_shards, slots, N) shard sums as 8-byte entries {fp32 value, 32-bit tag of the exchange
 * number}; an entry is written with one store, so a matching tag vouches for its value and the
 * exchange needs neither flags nor fences.
 *
 * b200norm_*_bwd_push: like b200norm_*_bwd, but instead of writing dw / db the column-reduce
 *   kernel stores this rank's fp32 shard sums directly into slot `seq % depth` of EVERY rank's
 *   inbox (plain stores over NVLink, no loads from remote memory).  This rank fills shards
 *   [rank*row_shards, (rank+1)*row_shards); world * row_shards must equal peers->total_shards.
 *   With `finish` non-NULL the same kernel then finishes an exchange (see below) -- an earlier one
 *   (the usual pipeline: exchange s finishes s - 1, whose entries arrived a step ago, and a step
 *   costs no launch more than on one GPU), or `seq` itself (the kernel then ends once every peer's
 *   push of `seq` has arrived).
 * b200norm_finalize_pushed: the finish as a kernel of its own.
 * Finishing exchange f = waiting (bounded, 2 s; then B200NORM_ERR_TIMEOUT in the status word and the
 *   kernel carries on) until the entries of slot f % depth carry f's tag, adding the total_shards
 *   sums of every column left to right in fp32 and casting to w_dtype.  Same bits on every rank and
 *   as a single GPU summing the same shards.
 *
 * `seq` starts at 1 and grows by 1 per exchange on all ranks alike.  Slot reuse: exchange s + depth
 * overwrites exchange s in every inbox, so it may start only once every rank has finished s.  A
 * rank's finish of exchange k proves that every peer has PUSHED k, hence -- by the peer's stream
 * order -- that the peer has finished whatever it had to finish before pushing k.  Two patterns
 * keep the slots safe (3 <= depth <= 8; use depth >= 4):
 *   - finishes fused into later pushes (exchange s finishes s - 1 or s): safe from depth 4 on;
 *   - finishes launched on their own: every rank finishes exchange s before it starts exchange
 *     s + depth / 2 (integer division), i.e. at most depth / 2 exchanges are pushed-but-unfinished.
 * A rank that breaks the rule makes a slower peer's wait run out (the tag it waits for has been
 * overwritten); it does not make the peer add up another exchange's numbers.
 * Passing seq = 0 (in `seq` and in finish->seq) makes the kernels number the exchanges themselves
 * from counters kept in `counter` (pushes and finishes each count up from 1): nothing in the launch
 * then changes from step to step, so a captured CUDA graph of the step can be replayed; the
 * caller keeps the slot rule.  inbox and counter (128 bytes) must be zero before the first exchange.
 */
#define B200NORM_MAX_PEERS 8
typedef struct b200norm_peers {
  int world, rank, depth, total_shards;
  size_t inbox_bytes;                   /* size of each rank's inbox: a multiple of 16 * depth, at least
                                           depth * total_shards * slots * N * 8 */
  void* inbox[B200NORM_MAX_PEERS];      /* inbox[r]: rank r's inbox as mapped in THIS process (16-byte aligned) */
  void* counter;                        /* this rank's own 128 bytes of bookkeeping, zeroed once */
} b200norm_peers;

/* An exchange to finish: its number (0 = the one after the last finished, by the device-side count),
 * its shape and where dweight [and dbias] go (either may be NULL). */
typedef struct b200norm_finish {
  uint64_t seq;
  int slots;      /* 1: dweight; 2: dweight and dbias */
  int w_dtype;
  int64_t N;
  void* dw;
  void* db;
} b200norm_finish;

B200NORM_API int b200norm_ln_bwd_push(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                                      const void* w, const float* mean, const float* rstd, void* dx,
                                      int64_t dx_row_stride, int row_shards, void* workspace,
                                      size_t workspace_bytes, int64_t M, int64_t N, int io_dtype, int w_dtype,
                                      const b200norm_peers* peers, uint64_t seq, const b200norm_finish* finish,
                                      void* stream);
B200NORM_API int b200norm_rms_bwd_push(const void* x, int64_t x_row_stride, const void* dy, int64_t dy_row_stride,
                                       const void* w, const float* rstd, void* dx, int64_t dx_row_stride,
                                       int row_shards, void* workspace, size_t workspace_bytes, int64_t M,
                                       int64_t N, int io_dtype, int w_dtype, const b200norm_peers* peers,
                                       uint64_t seq, const b200norm_finish* finish, void* stream);
B200NORM_API int b200norm_finalize_pushed(const b200norm_peers* peers, uint64_t seq, int slots, void* dw, void* db,
                                          int64_t N, int w_dtype, void* stream);

/*
 * RMSNorm backward for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose wrapper allocates its partial-sum buffers with torch on every call.)
 *
 * b200norm_rms_bwd needs a caller-provided workspace for its fp32 dweight partial rows.  A host
 * runtime that plans all of its device memory once at start-up -- an inference or training
 * engine with a static memory planner, or a real-time loop that may not call cudaMalloc because
 * it synchronises the device and can fail mid-run -- has no such buffer to hand over.  This
 * variant computes the same dx and dweight with the partial rows kept in a fixed array of
 * B200NORM_STATIC_SCRATCH_BYTES that is part of the library image: every GPU that loads
 * libb200norm.so holds that much memory until the process exits.  The caller still passes x, dy,
 * w, rstd, dx and dw.
 *
 *   - It calls no cudaMalloc / cudaFree / cudaHostAlloc and no allocating library routine.
 *   - The first call on each device looks up the array's device address, the SM count and kernel
 *     occupancies; make that first call before any stream capture.
 *   - Shapes whose partial rows exceed B200NORM_STATIC_SCRATCH_BYTES (roughly: resident CTAs x N x
 *     4 bytes, e.g. N = 16384 on a 148-SM GPU) are refused with B200NORM_ERR_UNSUPPORTED; use
 *     b200norm_rms_bwd with a caller workspace for those.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     Nothing in it has to start at zero (each call overwrites every partial row it later reads),
 *     but two calls that overlap on the GPU -- different streams, or different threads -- race
 *     on it.  Serialise them.
 *   - A bounded device-side wait that expires poisons only that launch; this variant has no
 *     host-readable status word (b200norm_device_status covers the other entry points).
 */
#define B200NORM_STATIC_SCRATCH_BYTES (8u << 20)
B200NORM_API int b200norm_rms_bwd_static(const void* x, int64_t x_row_stride, const void* dy,
                                         int64_t dy_row_stride, const void* w, const float* rstd, void* dx,
                                         int64_t dx_row_stride, void* dw, int64_t M, int64_t N, int io_dtype,
                                         int w_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NORM_H_ */
