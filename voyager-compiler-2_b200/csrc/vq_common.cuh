// Shared device/host helpers for the sm_100a quantized-ops kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/vq_b200.h"

namespace vq {

// ---------------------------------------------------------------------------
// error reporting across the C ABI
// ---------------------------------------------------------------------------
char* error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define VQ_REQUIRE(cond, ...)                     \
  do {                                            \
    if (!(cond)) return vq::fail(VQ_EINVAL, __VA_ARGS__); \
  } while (0)

constexpr int kSmCount = 148;

// Per-device one-time set-up (function attributes such as the dynamic shared-memory limit
// belong to a device, not to the process).  `done` holds one bit per device ordinal; returns
// true, and marks the bit, the first time it is called with the current device.  Racing callers
// may both see "first": the set-up they repeat is idempotent.
inline bool first_call_on_device(unsigned long long* done) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return true;
  const unsigned long long bit = 1ull << device;
  if (*done & bit) return false;
  *done |= bit;
  return true;
}

// ---------------------------------------------------------------------------
// storage dtypes.  All arithmetic is exact float32 followed by one RNE
// rounding into the storage dtype, which is what the reference's CPU ops do.
// ---------------------------------------------------------------------------
template <int DT> struct Elem;

template <> struct Elem<VQ_BF16> {
  using T = __nv_bfloat16;
  static constexpr int kVec = 8;  // elements per 16-byte access
  static __device__ __forceinline__ float to_float(T v) { return __bfloat162float(v); }
  static __device__ __forceinline__ T from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Elem<VQ_F16> {
  using T = __half;
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_float(T v) { return __half2float(v); }
  static __device__ __forceinline__ T from_float(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Elem<VQ_F32> {
  using T = float;
  static constexpr int kVec = 4;
  static __device__ __forceinline__ float to_float(T v) { return v; }
  static __device__ __forceinline__ T from_float(float v) { return v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float bf16_from_bits(uint32_t b) {
  return __uint_as_float(b << 16);
}

// ---------------------------------------------------------------------------
// rounding onto a format's grid
// ---------------------------------------------------------------------------
// Device-side copy of VqRound (passed by value as a kernel parameter).
struct Round {
  int32_t mode;
  const uint16_t* table;
  float lo, hi;
  int32_t emin, mbits;
  float max_norm;
  int32_t is_signed;
  const float* edges;
  const float* levels;
  int32_t n_edges, n_levels;
  const int64_t* seed;
  const uint16_t* steps;  // n_steps keys then n_steps values (global or shared)
  int32_t n_steps;
  uint32_t nan_value;
};

inline Round make_round(const VqRound* r) {
  Round d{};
  if (r == nullptr) {
    d.mode = VQ_ROUND_NONE;
    return d;
  }
  d.mode = r->mode;
  d.table = static_cast<const uint16_t*>(r->table);
  d.lo = r->lo;
  d.hi = r->hi;
  d.emin = r->emin;
  d.mbits = r->mbits;
  d.max_norm = r->max_norm;
  d.is_signed = r->is_signed;
  d.edges = r->edges;
  d.levels = r->levels;
  d.n_edges = r->n_edges;
  d.n_levels = r->n_levels;
  d.seed = r->seed;
  d.steps = static_cast<const uint16_t*>(r->steps);
  d.n_steps = r->n_steps;
  d.nan_value = r->nan_value;
  return d;
}

int validate_round(const VqRound* r, const char* what);

// Sign-magnitude bf16 bits -> a key that is monotone in value:
// negatives map below positives, larger magnitude negative = smaller key.
__device__ __forceinline__ uint32_t ordered_key(uint32_t bits) {
  return (bits & 0x8000u) ? (0x7FFFu - (bits & 0x7FFFu)) : (0x8000u + bits);
}

__device__ __forceinline__ float round_int(float v, float lo, float hi) {
  // torch.round = half to even; clamp keeps NaN; a zero result keeps its sign.
  float r = rintf(v);
  if (r == 0.0f || r != r) return r;
  return fminf(fmaxf(r, lo), hi);
}

__device__ __forceinline__ float round_minifloat(float v, int emin, int mbits, float max_norm,
                                                 int is_signed) {
  if (v != v) return v;
  float a = fabsf(v);
  a = fminf(a, max_norm);
  // exponent of a, floored at emin; a == 0 behaves as exponent emin.
  int e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
  e = e < emin ? emin : e;
  // a / 2^(e - mbits), exact; |e - mbits| stays inside the normal range here.
  float up = __uint_as_float((uint32_t)(127 - (e - mbits)) << 23);
  float down = __uint_as_float((uint32_t)(127 + (e - mbits)) << 23);
  float q = rintf(a * up) * down;
  q = fminf(q, max_norm);
  if (!is_signed) return q;
  // sign(-0) is +0 but a negative value that rounds to nothing stays -0.
  if (v == 0.0f) return 0.0f;
  return copysignf(q, v);
}

__device__ __forceinline__ uint32_t philox_byte(uint64_t index, uint64_t seed) {
  // Philox4x32-10 on counter = index / 16 (high words zero); element takes
  // byte index % 4 of word (index % 16) / 4.
  uint64_t counter = index >> 4;
  uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)c0 * 0xD2511F53ull;
    uint64_t p1 = (uint64_t)c2 * 0xCD9E8D57ull;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  uint32_t word_index = (uint32_t)(index & 15) >> 2;
  uint32_t w = word_index == 0 ? c0 : word_index == 1 ? c1 : word_index == 2 ? c2 : c3;
  return (w >> (8 * (uint32_t)(index & 3))) & 0xFFu;
}

// v: the scaled value, already rounded to the storage dtype.  `flat` is the
// element's index in the input's logical row-major order (stochastic only).
// Returns the grid value (or codebook index) as a float, exact in bf16.
// MODE >= 0 fixes the rounding mode at compile time; -1 switches at run time.
template <int MODE = -1>
__device__ __forceinline__ float apply_round(const Round& r, float v, int64_t flat) {
  const int mode = MODE >= 0 ? MODE : r.mode;
  switch (mode) {
    case VQ_ROUND_NONE:
      return v;
    case VQ_ROUND_TABLE:
      return bf16_from_bits(__ldg(r.table + bf16_bits(v)));
    case VQ_ROUND_INT:
      return round_int(bf16_from_bits(bf16_bits(v)), r.lo, r.hi);
    case VQ_ROUND_MINIFLOAT:
      return round_minifloat(bf16_from_bits(bf16_bits(v)), r.emin, r.mbits, r.max_norm, r.is_signed);
    case VQ_ROUND_STEPS: {
      uint32_t bits = bf16_bits(v);
      if ((bits & 0x7FFFu) > 0x7F80u) return bf16_from_bits(r.nan_value);
      uint32_t key = ordered_key(bits);
      int lo = 0, hi = r.n_steps - 1;  // first k with key < steps[k]
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (key < r.steps[mid]) hi = mid; else lo = mid + 1;
      }
      return bf16_from_bits(r.steps[r.n_steps + lo]);
    }
    case VQ_ROUND_SEARCH: {
      float x = bf16_from_bits(bf16_bits(v));
      int lo = 0, hi = r.n_edges;  // count of edges < x (NaN compares false everywhere)
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (__ldg(r.edges + mid) >= x) hi = mid; else lo = mid + 1;
      }
      return r.levels ? __ldg(r.levels + lo) : (float)lo;
    }
    case VQ_ROUND_STOCHASTIC: {
      const int n = r.n_levels;
      float first = __ldg(r.levels), last = __ldg(r.levels + n - 1);
      float x = fminf(fmaxf(v, first), last);
      if (v != v) x = v;
      int lo = 0, hi = n;  // first index with level >= x
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (__ldg(r.levels + mid) >= x) hi = mid; else lo = mid + 1;
      }
      int up = lo < n - 1 ? lo : n - 1;
      float high = __ldg(r.levels + up);
      float low = (high == x) ? high : __ldg(r.levels + (up > 0 ? up - 1 : 0));
      float noise = (float)philox_byte((uint64_t)flat, (uint64_t)__ldg(r.seed)) * (1.0f / 256.0f);
      float near = x < 0.0f ? high : low;
      float far = x < 0.0f ? low : high;
      bool away = __fadd_rn(fabsf(x), __fmul_rn(noise, __fsub_rn(high, low))) >= fabsf(far);
      return away ? far : near;
    }
  }
  return v;
}

// Step tables are searched from shared memory: copy them once per CTA.  Every
// thread of the CTA must call this (it synchronises when the mode is STEPS).
__device__ __forceinline__ void stage_steps(Round& r, uint16_t* smem /* 2*VQ_MAX_STEPS */) {
  if (r.mode == VQ_ROUND_STEPS) {
    for (int i = threadIdx.x; i < 2 * r.n_steps; i += blockDim.x) smem[i] = r.steps[i];
    __syncthreads();
    r.steps = smem;
  }
}

}  // namespace vq
