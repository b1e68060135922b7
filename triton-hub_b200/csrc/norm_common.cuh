// Shared device helpers for the LayerNorm / RMSNorm kernels: 16-byte packets of each storage
// type, streaming loads and stores, warp and row-group reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200norm {

// Storage type codes; the numbering is the C ABI's enum b200norm_dtype.
enum : int { kF32 = 0, kF16 = 1, kBF16 = 2, kF64 = 3 };

// ---------------------------------------------------------------------------------------
// Packed fp32 arithmetic: sm_100 executes fma / mul / add on two fp32 values held in a register pair
// as ONE instruction, each lane rounded exactly like the scalar instruction.  The row kernels keep
// their per-element values as such pairs, which nearly halves the arithmetic instructions of
// kernels that are bound by instruction issue rather than by memory.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// ---------------------------------------------------------------------------------------
// Pack16<T>: one 128-bit packet of T and its fp32 view (kElems floats, or kElems / 2 pairs).
// ---------------------------------------------------------------------------------------
template <typename T>
struct Pack16;

template <>
struct Pack16<float> {
  static constexpr int kElems = 4;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
    f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
    f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
  }
  __device__ __forceinline__ static uint4 pack2(const float2* f) {
    return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x),
                      __float_as_uint(f[1].y));
  }
};

template <>
struct Pack16<__half> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 p = __half22float2(h);
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
  }
  __device__ __forceinline__ static uint4 pack2(const float2* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __float22half2_rn(f[i]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Pack16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // bf16 -> fp32 is a 16-bit shift: exact and cheaper than the library call.
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
  __device__ __forceinline__ static uint4 pack2(const float2* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[i].x, f[i].y);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Pack16<double> {
  static constexpr int kElems = 2;
  __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
    f[0] = static_cast<float>(__hiloint2double(static_cast<int>(v.y), static_cast<int>(v.x)));
    f[1] = static_cast<float>(__hiloint2double(static_cast<int>(v.w), static_cast<int>(v.z)));
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    const double a = static_cast<double>(f[0]), b = static_cast<double>(f[1]);
    return make_uint4(static_cast<uint32_t>(__double2loint(a)), static_cast<uint32_t>(__double2hiint(a)),
                      static_cast<uint32_t>(__double2loint(b)), static_cast<uint32_t>(__double2hiint(b)));
  }
  __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
    float t[2];
    unpack(v, t);
    f[0] = make_float2(t[0], t[1]);
  }
  __device__ __forceinline__ static uint4 pack2(const float2* f) {
    const float t[2] = {f[0].x, f[0].y};
    return pack(t);
  }
};

// 2^x and 1/x on the special-function unit, one instruction each (denormal results and inputs
// flush to zero; the callers' arguments keep far from both).
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Makes the compiler forget what it knows about a packet, so that a later unpack is redone from
// the packed registers instead of keeping every fp32 copy alive across the row reduction.
__device__ __forceinline__ void forget(uint4& v) { asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)); }

// Scalar conversions for the any-alignment kernels.
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(double v) { return static_cast<float>(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ double from_f32<double>(float v) { return static_cast<double>(v); }

// One element of a parameter vector (weight, bias) whose storage type is only known at run
// time.  Parameters are read once per CTA, so the switch costs nothing.
__device__ __forceinline__ float load_param(const void* p, int dtype, int64_t i) {
  switch (dtype) {
    case kF32: return static_cast<const float*>(p)[i];
    case kF16: return __half2float(static_cast<const __half*>(p)[i]);
    case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    default: return static_cast<float>(static_cast<const double*>(p)[i]);
  }
}
__device__ __forceinline__ void store_param(void* p, int dtype, int64_t i, float v) {
  switch (dtype) {
    case kF32: static_cast<float*>(p)[i] = v; break;
    case kF16: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case kBF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    default: static_cast<double*>(p)[i] = static_cast<double>(v); break;
  }
}

// Storage type code of a compile-time element type.
template <typename T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr int value = kF32; };
template <> struct DTypeOf<__half> { static constexpr int value = kF16; };
template <> struct DTypeOf<__nv_bfloat16> { static constexpr int value = kBF16; };
template <> struct DTypeOf<double> { static constexpr int value = kF64; };

// The Pack16<T>::kElems parameter values that line up with packet `v` of a row of T: one
// cached 16-byte load when the parameters are stored as T too, element loads otherwise.
template <typename T>
__device__ __forceinline__ void load_param_packet(const void* p, int dtype, int v, float* out) {
  constexpr int VEC = Pack16<T>::kElems;
  if (dtype == DTypeOf<T>::value) {
    const uint4 pk = __ldg(static_cast<const uint4*>(p) + v);
    Pack16<T>::unpack(pk, out);
  } else {
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = load_param(p, dtype, (int64_t)v * VEC + e);
  }
}

// The parameter values that line up with a thread's packets, for up to two parameter vectors of one
// storage type (weight and bias; a null pointer is skipped): packets v0 + j * stride + t (j < LDGS)
// of a row of T whose part handled here is `limit` packets long; `take(j)` says which of them this
// thread fetches.  ALL loads are issued before any value is used, so the whole set costs one trip to
// memory -- a loop that loads and converts packet by packet pays one trip per packet, which for a
// CTA with a few dozen rows is a visible share of its life.  `issued()` runs between the loads and
// their first use: the kernels start their bulk row copies there, BEHIND the small parameter
// requests, which would otherwise queue up after hundreds of kilobytes of row data.  Vector loads
// when the storage type and alignment allow (same type as the rows; fp32 parameters with 16-bit
// rows; 16-bit parameters with fp32 rows), element loads otherwise.  `sink(which, j, values)`
// receives each packet of vector `which`.
template <typename T, int LDGS, typename Take, typename Issued, typename Sink>
__device__ __forceinline__ void load_param_packets(const void* p0, const void* p1, int dtype, int v0, int t,
                                                   int stride, int limit, Take take, Issued issued, Sink sink) {
  constexpr int VEC = Pack16<T>::kElems;
  const void* const ptr[2] = {p0, p1};
  const uintptr_t addr = reinterpret_cast<uintptr_t>(p0) | reinterpret_cast<uintptr_t>(p1);
  if (dtype == DTypeOf<T>::value && (addr & 15u) == 0) {
    uint4 raw[2][LDGS];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) raw[w][j] = __ldg(static_cast<const uint4*>(ptr[w]) + v0 + v);
      }
    issued();
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) {
          float f[VEC];
          Pack16<T>::unpack(raw[w][j], f);
          sink(w, j, f);
        }
      }
  } else if (dtype == kF32 && VEC == 8 && (addr & 15u) == 0) {  // fp32 parameters, 16-bit rows
    float4 raw[2][LDGS][2];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) {
          raw[w][j][0] = __ldg(static_cast<const float4*>(ptr[w]) + (size_t)(v0 + v) * 2);
          raw[w][j][1] = __ldg(static_cast<const float4*>(ptr[w]) + (size_t)(v0 + v) * 2 + 1);
        }
      }
    issued();
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) {
          const float f[8] = {raw[w][j][0].x, raw[w][j][0].y, raw[w][j][0].z, raw[w][j][0].w,
                              raw[w][j][1].x, raw[w][j][1].y, raw[w][j][1].z, raw[w][j][1].w};
          sink(w, j, f);
        }
      }
  } else if ((dtype == kF16 || dtype == kBF16) && VEC == 4 && (addr & 7u) == 0) {  // 16-bit parameters, fp32 rows
    uint2 raw[2][LDGS];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) raw[w][j] = __ldg(static_cast<const uint2*>(ptr[w]) + v0 + v);
      }
    issued();
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) {
          float f[VEC > 4 ? VEC : 4];
          const uint32_t w2[2] = {raw[w][j].x, raw[w][j].y};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            if (dtype == kBF16) {
              f[2 * i] = __uint_as_float(w2[i] << 16);
              f[2 * i + 1] = __uint_as_float(w2[i] & 0xffff0000u);
            } else {
              const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&w2[i]));
              f[2 * i] = h.x;
              f[2 * i + 1] = h.y;
            }
          }
          sink(w, j, f);
        }
      }
  } else {
    issued();
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int j = 0; j < LDGS; ++j) {
        const int v = j * stride + t;
        if (ptr[w] != nullptr && v < limit && take(j)) {
          float f[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) f[e] = load_param(ptr[w], dtype, (int64_t)(v0 + v) * VEC + e);
          sink(w, j, f);
        }
      }
  }
}

// ---------------------------------------------------------------------------------------
// Streaming 128-bit global accesses.  x, dy, y and dx are touched exactly once per kernel, so
// they bypass L1 on the way in and are marked evict-first on the way out; that keeps L1 for
// the parameter vectors, which every row re-reads.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// VEC consecutive fp32 values (a thread's share of a dweight / dbias partial row) in one store:
// a whole 32-byte sector per thread for 8 values, so the memory system sees each sector once
// instead of once per element.  `p` is aligned to VEC * 4 bytes.
template <int VEC>
__device__ __forceinline__ void st_f32_vec(float* p, const float* v) {
  if constexpr (VEC == 8) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]),
                 "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
  } else if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int e = 0; e < VEC; ++e) p[e] = v[e];
  }
}

// The same for H pairs (2 * H consecutive values).
template <int H>
__device__ __forceinline__ void st_f32_pairs(float* p, const float2* v) {
  if constexpr (H == 4) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0].x), "f"(v[0].y), "f"(v[1].x),
                 "f"(v[1].y), "f"(v[2].x), "f"(v[2].y), "f"(v[3].x), "f"(v[3].y)
                 : "memory");
  } else if constexpr (H == 2) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
  } else {
#pragma unroll
    for (int h = 0; h < H; ++h) *reinterpret_cast<float2*>(p + 2 * h) = v[h];
  }
}

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  The kernels are launched with the "programmatic stream
// serialization" attribute: a kernel may be scheduled while its predecessor in the stream is
// still draining, and must call grid_dependency_sync() before it touches global memory; that
// returns once the predecessor has completed and its writes are visible.  Calling
// trigger_dependents() early lets the successor's CTAs take SM slots as this grid's CTAs retire,
// which hides launch latency and the ramp-up of the next kernel behind this kernel's tail.
// After a predecessor that never triggers (any ordinary kernel) the launch behaves as usual.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_sync() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void trigger_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// Reductions.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Barrier over the WARPS_N warps that share a row.  Barrier 0 is __syncthreads; row group m
// uses hardware barrier m + FIRST (at most 15 row groups per CTA).  A kernel that never calls
// __syncthreads once its row groups run apart may pass FIRST = 0: the SM has 16 barriers, so one
// barrier less per CTA is up to twice as many small CTAs per SM.
template <int WARPS_N, int FIRST = 1>
__device__ __forceinline__ void group_sync(int warp_m) {
  if (WARPS_N > 1) {
    asm volatile("bar.sync %0, %1;" ::"r"(warp_m + FIRST), "r"(WARPS_N * 32) : "memory");
  }
}

// Sum of NV values over the WARPS_N*32 threads of a row group; every thread gets the result.
// `scratch` points at this row group's 2*NV*WARPS_N floats of shared memory.  The two halves
// are used alternately (`phase` flips on every call), so one barrier per call is enough: a
// warp cannot overwrite a half before every warp has read it, because a full barrier lies
// between.  The cross-warp add runs in warp order in every thread: deterministic and
// identical across the group.
template <int WARPS_N, int NV, int FIRST = 1>
__device__ __forceinline__ void group_sum(float (&v)[NV], float* scratch, int& phase, int warp_m, int warp_n,
                                          int lane) {
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
  if (WARPS_N > 1) {
    float* buf = scratch + phase * (NV * WARPS_N);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) buf[i * WARPS_N + warp_n] = v[i];
    }
    group_sync<WARPS_N, FIRST>(warp_m);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < WARPS_N; ++k) s += buf[i * WARPS_N + k];
      v[i] = s;
    }
    phase ^= 1;
  }
}

// Mean and centred sum of squares of a row from per-thread (mean, M2) pairs over equal element
// counts, merged pairwise with Chan's update
//   n = na + nb;  d = mb - ma;  mean = ma + d * nb / n;  M2 = M2a + M2b + d * d * na * nb / n
// -- one reduction (one barrier) per row where the two-pass form needs two, with the same
// numerical quality: no E[x^2] - E[x]^2 cancellation.  With equal counts the weights are
// constants (nb/n = 1/2 in the butterfly, 1/(k+1) across warps), so nothing is divided and both
// butterfly partners compute the same bits.  The warp pairs go through shared memory and every
// thread folds them in warp order: the whole row group ends with identical statistics.
// `n` is the element count per thread on entry and per row group on return.
template <int WARPS_N, int FIRST = 1>
__device__ __forceinline__ void group_moments(float& n, float& mean, float& m2, float* scratch, int& phase,
                                              int warp_m, int warp_n, int lane) {
  float half = 0.5f * n;  // na * nb / (na + nb) for equal counts
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float mb = __shfl_xor_sync(0xffffffffu, mean, o);
    const float qb = __shfl_xor_sync(0xffffffffu, m2, o);
    const float d = mb - mean;
    mean = 0.5f * (mean + mb);
    m2 = (m2 + qb) + d * d * half;
    half += half;
  }
  n *= 32.f;
  if (WARPS_N > 1) {
    float* buf = scratch + phase * (2 * WARPS_N);
    if (lane == 0) {
      buf[warp_n] = mean;
      buf[WARPS_N + warp_n] = m2;
    }
    group_sync<WARPS_N, FIRST>(warp_m);
    const float nw = n;  // elements per warp
    mean = buf[0];
    m2 = buf[WARPS_N];
#pragma unroll
    for (int k = 1; k < WARPS_N; ++k) {
      const float f = 1.f / static_cast<float>(k + 1);  // folded at compile time
      const float d = buf[k] - mean;
      mean = mean + d * f;
      m2 = (m2 + buf[WARPS_N + k]) + d * d * (static_cast<float>(k) * f * nw);
    }
    n = nw * static_cast<float>(WARPS_N);
    phase ^= 1;
  }
}

}  // namespace b200norm
