// bfloat16 fast paths of the quantizers.
//
// The generic kernels in quantize_kernels.cu are exact for every dtype and
// rounding mode but spend ~40 instructions per element, which caps them near
// 2 TB/s.  These kernels cover the hot cases -- bfloat16 data, blocks along the
// contiguous axis, integer or hardware-convertible minifloat grids -- in about
// ten instructions per element so that HBM is the limit:
//   * block amax on packed 16-bit lanes (NaN bit patterns order above inf, so
//     an unsigned max propagates NaN exactly like torch.amax);
//   * power-of-two scales straight from the exponent field;
//   * division by a general scale as a product with the correctly rounded
//     reciprocal, re-done with a true division only when the product lies
//     within 2 ulp of a bfloat16 rounding boundary (so the result always
//     equals round_bf16(x / s));
//   * integer grids by rint + clamp, e4m3 / e5m2 / e2m1 / e2m3 / e3m2 grids by
//     the hardware's saturating converts.
// Any block that is not "ordinary" (zero, subnormal, infinite or NaN amax, or a
// scale outside the normal range) is handed to the exact generic code.

#include <cuda_fp4.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>

#include "quantize_shared.cuh"

namespace vq {

enum {
  FAST_NONE = 0,   // keep the scaled value
  FAST_INT,        // signed integer grid (lo < 0)
  FAST_E4M3,
  FAST_E5M2,
  FAST_E2M1,
  FAST_E2M3,
  FAST_E3M2,
  FAST_GENERIC,    // apply_round at run time (tables, steps, ...)
};

int fast_mode_of(const VqRound* r) {
  if (r == nullptr || r->mode == VQ_ROUND_NONE) return FAST_NONE;
  if (r->mode == VQ_ROUND_INT && r->lo < 0.0f && r->hi > 0.0f) return FAST_INT;
  if (r->mode == VQ_ROUND_MINIFLOAT && r->is_signed) {
    if (r->mbits == 3 && r->emin == -6 && r->max_norm == 448.0f) return FAST_E4M3;
    if (r->mbits == 2 && r->emin == -14 && r->max_norm == 57344.0f) return FAST_E5M2;
    if (r->mbits == 1 && r->emin == 0 && r->max_norm == 6.0f) return FAST_E2M1;
    if (r->mbits == 3 && r->emin == 0 && r->max_norm == 7.5f) return FAST_E2M3;
    if (r->mbits == 2 && r->emin == -2 && r->max_norm == 28.0f) return FAST_E3M2;
  }
  return FAST_GENERIC;
}

namespace {

#ifndef VQ_FAST_UNROLL
#define VQ_FAST_UNROLL 4
#endif
#ifndef VQ_FAST_CTAS_PER_SM
#define VQ_FAST_CTAS_PER_SM 4
#endif
constexpr int kT = 256;
constexpr int kU = VQ_FAST_UNROLL;            // 16-byte loads in flight per thread
constexpr int kCtasPerSm = VQ_FAST_CTAS_PER_SM;
// The per-tensor / per-row quantizer has no block reduction and little state: more resident CTAs
// win there (measured: 4.8 TB/s at six per SM against 4.4 at four), fewer for the MX kernels.
constexpr int kCtasPerSmPlain = 6;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float lo_of(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_of(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Two scaled values (exact bfloat16 values held as floats) -> two grid values
// packed as bfloat16.  The tables map -0 to +0 but keep the sign of a negative
// value that rounds to nothing; adding +0 reproduces that (-0 + 0 = +0).
template <int FM>
__device__ __forceinline__ uint32_t round_pair(float a, float b, const Round& r, int64_t flat) {
  if constexpr (FM == FAST_NONE) {
    return pack_bf16(a, b);
  } else if constexpr (FM == FAST_INT) {
    a = fminf(fmaxf(rintf(a), r.lo), r.hi);
    b = fminf(fmaxf(rintf(b), r.lo), r.hi);
    return pack_bf16(a, b);
  } else if constexpr (FM == FAST_E4M3 || FM == FAST_E5M2) {
    float2 v = make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
    __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(v, __NV_SATFINITE, FM == FAST_E4M3 ? __NV_E4M3 : __NV_E5M2);
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(q, FM == FAST_E4M3 ? __NV_E4M3 : __NV_E5M2);
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
    return pack_bf16(f.x, f.y);
  } else if constexpr (FM == FAST_E2M1) {
    float2 v = make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
    __nv_fp4x2_storage_t q = __nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest);
    __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(q, __NV_E2M1);
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
    return pack_bf16(f.x, f.y);
  } else if constexpr (FM == FAST_E2M3 || FM == FAST_E3M2) {
    float2 v = make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
    __nv_fp6x2_storage_t q = __nv_cvt_float2_to_fp6x2(v, FM == FAST_E2M3 ? __NV_E2M3 : __NV_E3M2, cudaRoundNearest);
    __half2_raw h = __nv_cvt_fp6x2_to_halfraw2(q, FM == FAST_E2M3 ? __NV_E2M3 : __NV_E3M2);
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
    return pack_bf16(f.x, f.y);
  } else {
    return pack_bf16(apply_round(r, a, flat), apply_round(r, b, flat + 1));
  }
}

// Exact generic treatment of one 16-byte vector (8 elements) given its block's amax.
__device__ __noinline__ uint4 slow_vector(uint4 raw, uint32_t amax_bits, const ScaleRule& rule, const Round& r,
                                          int64_t flat, float* scale_out) {
  float es;
  float scale = block_scale<VQ_BF16>(amax_bits, rule, &es);
  *scale_out = scale;
  Vec<VQ_BF16> x, y;
  x.raw = raw;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    y.set(j, apply_round(r, Elem<VQ_BF16>::round(__fdiv_rn(x.get(j), es)), flat + j));
  return y.raw;
}

// Blocks along the contiguous axis, K a whole number of blocks: the tensor is a
// flat run of blocks; vector v belongs to block v >> gshift (G = 1 << gshift
// lanes per block).
// U vectors per thread and step: kU for streaming tensors; 1 for small ones (a decode step's few rows), which
// then spread over four times as many CTAs and have a quarter of the dependent latency per thread.
template <int FM, bool POT, bool WRITE_CODES, int U = kU>
__global__ void __launch_bounds__(kT, kCtasPerSm)
mx_flat_bf16_kernel(const uint4* __restrict__ in, __nv_bfloat16* __restrict__ scale_out, uint4* __restrict__ codes_out,
                    int64_t nvec, int G, int gshift, ScaleRule rule, Round r) {
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(rule.scale_round, s_steps[1]);
  float gs = 0.0f;
  const bool has_gs = rule.global_scale != nullptr;
  if (has_gs) gs = loadp(rule.global_scale, 0, rule.global_scale_dtype);
  const int64_t chunk = (int64_t)kT * U;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int64_t v = base + u * kT + threadIdx.x;
      x[u] = make_uint4(0, 0, 0, 0);
      if (v < nvec) x[u] = __ldg(in + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * kT + threadIdx.x;
      const bool active = v < nvec;
      // block amax of the bf16 magnitudes, two lanes at a time
      uint32_t m2 = __vmaxu2(__vmaxu2(x[u].x & 0x7FFF7FFFu, x[u].y & 0x7FFF7FFFu),
                             __vmaxu2(x[u].z & 0x7FFF7FFFu, x[u].w & 0x7FFF7FFFu));
      uint32_t m = max(m2 & 0xFFFFu, m2 >> 16);
      for (int off = 1; off < G; off <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
      const uint32_t ex = m >> 7;  // exponent field of the amax (sign is clear)

      float scale, es, rcp = 0.0f;
      bool ordinary;
      if (POT) {
        // scale = 2^(floor(log2 amax) - qexp): exponent field ex - qexp
        const int se = (int)ex - rule.qmax_exp;
        ordinary = ex >= 1u && ex <= 254u && se >= 1 && se <= 253 && !has_gs;
        scale = __uint_as_float((uint32_t)se << 23);
        es = scale;
        rcp = __uint_as_float((uint32_t)(254 - se) << 23);  // exact reciprocal
        if (m == 0u && !has_gs) {
          // all-zero block: every quotient is a zero of the element's sign
          ordinary = true;
          scale = rule.zero_scale_bf16;
          es = scale;
          rcp = 0.0f;
        }
      } else {
        // an all-zero block takes the ordinary route: its scale comes out as 1
        ordinary = (ex >= 1u && ex <= 254u) || m == 0u;
        const float amax = __uint_as_float(m << 16);
        scale = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(amax, rule.quant_max)));
        if (has_gs) scale = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(scale, gs)));
        if (rule.scale_round.mode != VQ_ROUND_NONE)
          scale = __bfloat162float(__float2bfloat16_rn(apply_round(rule.scale_round, scale, 0)));
        scale = scale > 0.0f ? scale : 1.0f;
        es = has_gs ? __bfloat162float(__float2bfloat16_rn(__fmul_rn(scale, gs))) : scale;
        const uint32_t eex = (__float_as_uint(es) >> 23) & 0xFFu;
        ordinary = ordinary && eex >= 1u && eex <= 253u && es > 0.0f;
        rcp = __frcp_rn(es);
      }

      uint4 y;
      if (ordinary) {
        if (WRITE_CODES) {
          const int64_t flat = v * 8;
          uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float a, b;
            if (POT) {
              // exact products; a subnormal product still rounds like the quotient
              a = __fmul_rn(lo_of(w[j]), rcp);
              b = __fmul_rn(hi_of(w[j]), rcp);
              if (FM != FAST_INT) {
                a = __bfloat162float(__float2bfloat16_rn(a));
                b = __bfloat162float(__float2bfloat16_rn(b));
              }
            } else {
              a = div_to_bf16(lo_of(w[j]), es, rcp);
              b = div_to_bf16(hi_of(w[j]), es, rcp);
            }
            o[j] = round_pair<FM>(a, b, r, flat + 2 * j);
          }
          y = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
        y = slow_vector(x[u], m << 16, rule, r, v * 8, &scale);
      }
      if (active) {
        if ((threadIdx.x & (G - 1)) == 0) scale_out[v >> gshift] = __float2bfloat16_rn(scale);
        if (WRITE_CODES) codes_out[v] = y;
      }
    }
  }
}

// out = round(in / scale) with one scale per `d` consecutive elements
// (d a multiple of 8; d = 0: a single scale), no zero point.
template <int FM>
__global__ void __launch_bounds__(kT, kCtasPerSmPlain)
quantize_bf16_kernel(const uint4* __restrict__ in, const void* __restrict__ scale, int pdt, uint4* __restrict__ out,
                     int64_t nvec, uint32_t vecs_per_scale, int vshift, Round r) {
  __shared__ uint16_t s_steps[2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps);
  float s0 = 1.0f, rcp0 = 1.0f;
  bool ord0 = false;
  if (vecs_per_scale == 0) {
    s0 = loadp(scale, 0, pdt);
    const uint32_t ex = (__float_as_uint(s0) >> 23) & 0xFFu;
    ord0 = ex >= 1u && ex <= 253u && s0 > 0.0f;
    rcp0 = __frcp_rn(s0);
  }
  const int64_t chunk = (int64_t)kT * kU;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    uint4 x[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      int64_t v = base + u * kT + threadIdx.x;
      if (v < nvec) x[u] = __ldg(in + v);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = base + u * kT + threadIdx.x;
      if (v >= nvec) continue;
      float s = s0, rcp = rcp0;
      bool ordinary = ord0;
      if (vecs_per_scale != 0) {
        const int64_t pi = vshift >= 0 ? (v >> vshift) : (int64_t)((uint64_t)v / vecs_per_scale);
        s = loadp(scale, pi, pdt);
        const uint32_t ex = (__float_as_uint(s) >> 23) & 0xFFu;
        ordinary = ex >= 1u && ex <= 253u && s > 0.0f;
        rcp = __frcp_rn(s);
      }
      const int64_t flat = v * 8;
      uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
      uint32_t o[4];
      if (ordinary) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[j] = round_pair<FM>(div_to_bf16(lo_of(w[j]), s, rcp), div_to_bf16(hi_of(w[j]), s, rcp), r, flat + 2 * j);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(lo_of(w[j]), s)));
          float b = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(hi_of(w[j]), s)));
          o[j] = pack_bf16(apply_round(r, a, flat + 2 * j), apply_round(r, b, flat + 2 * j + 1));
        }
      }
      out[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// out = bf16(in * scale), one scale per `d` consecutive elements (operand read-back).
__global__ void __launch_bounds__(kT, kCtasPerSm)
scale_bf16_kernel(const uint4* __restrict__ in, const __nv_bfloat16* __restrict__ scale, uint4* __restrict__ out,
                  int64_t nvec, uint32_t vecs_per_scale, int vshift) {
  const int64_t chunk = (int64_t)kT * kU;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    uint4 x[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      int64_t v = base + u * kT + threadIdx.x;
      if (v < nvec) x[u] = __ldg(in + v);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = base + u * kT + threadIdx.x;
      if (v >= nvec) continue;
      const int64_t pi = vshift >= 0 ? (v >> vshift) : (int64_t)((uint64_t)v / vecs_per_scale);
      const float s = __bfloat162float(scale[pi]);
      uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = pack_bf16(__fmul_rn(lo_of(w[j]), s), __fmul_rn(hi_of(w[j]), s));
      out[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Real FP8 bytes for the tensor-core GEMM: out[i] = e4m3|e5m2(round_bf16(in[i] / scale)),
// the byte encoding of exactly the grid value the table rounding yields.  Each
// thread turns 16 bfloat16 elements into one 16-byte store.
template <bool E4M3>
__global__ void __launch_bounds__(kT, kCtasPerSm)
quantize_fp8_kernel(const uint4* __restrict__ in, const void* __restrict__ scale, int pdt, uint4* __restrict__ out,
                    int64_t n16, uint32_t v16_per_scale, int vshift) {
  float s0 = 1.0f, rcp0 = 1.0f;
  bool ord0 = false;
  if (v16_per_scale == 0) {
    s0 = loadp(scale, 0, pdt);
    const uint32_t ex = (__float_as_uint(s0) >> 23) & 0xFFu;
    ord0 = ex >= 1u && ex <= 253u && s0 > 0.0f;
    rcp0 = __frcp_rn(s0);
  }
  constexpr int U = 2;
  const int64_t chunk = (int64_t)kT * U;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < n16; base += (int64_t)gridDim.x * chunk) {
    uint4 x[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int64_t v = base + u * kT + threadIdx.x;
      if (v < n16) {
        x[u][0] = __ldg(in + 2 * v);
        x[u][1] = __ldg(in + 2 * v + 1);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * kT + threadIdx.x;
      if (v >= n16) continue;
      float s = s0, rcp = rcp0;
      bool ordinary = ord0;
      if (v16_per_scale != 0) {
        const int64_t pi = vshift >= 0 ? (v >> vshift) : (int64_t)((uint64_t)v / v16_per_scale);
        s = loadp(scale, pi, pdt);
        const uint32_t ex = (__float_as_uint(s) >> 23) & 0xFFu;
        ordinary = ex >= 1u && ex <= 253u && s > 0.0f;
        rcp = __frcp_rn(s);
      }
      const uint32_t w[8] = {x[u][0].x, x[u][0].y, x[u][0].z, x[u][0].w, x[u][1].x, x[u][1].y, x[u][1].z, x[u][1].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a, b;
        if (ordinary) {
          a = div_to_bf16(lo_of(w[j]), s, rcp);
          b = div_to_bf16(hi_of(w[j]), s, rcp);
        } else {
          a = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(lo_of(w[j]), s)));
          b = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(hi_of(w[j]), s)));
        }
        float2 f = make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
        uint32_t q = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, E4M3 ? __NV_E4M3 : __NV_E5M2);
        if (j & 1) o[j >> 1] |= q << 16; else o[j >> 1] = q;
      }
      out[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

inline int grid_of(int64_t nvec, int ctas_per_sm = kCtasPerSm) {
  int64_t blocks = (nvec + kT * kU - 1) / (kT * kU);
  int64_t cap = (int64_t)kSmCount * ctas_per_sm;  // all CTAs resident at once
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <int FM>
void launch_mx_fm(bool pot, bool write, const void* in, void* scale_out, void* codes_out, int64_t nvec, int G,
                  int gshift, const ScaleRule& rule, const Round& r, cudaStream_t st) {
  const uint4* i = static_cast<const uint4*>(in);
  __nv_bfloat16* s = static_cast<__nv_bfloat16*>(scale_out);
  uint4* c = static_cast<uint4*>(codes_out);
  if (FM == FAST_GENERIC && write && nvec <= (int64_t)kSmCount * kT) {
    // a small tensor through a gathered table: latency, not bandwidth
    const int small_grid = (int)((nvec + kT - 1) / kT);
    if (pot) mx_flat_bf16_kernel<FM, true, true, 1><<<small_grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
    else mx_flat_bf16_kernel<FM, false, true, 1><<<small_grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
    return;
  }
  const int grid = grid_of(nvec);
  if (pot) {
    if (write) mx_flat_bf16_kernel<FM, true, true><<<grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
    else mx_flat_bf16_kernel<FAST_NONE, true, false><<<grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
  } else {
    if (write) mx_flat_bf16_kernel<FM, false, true><<<grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
    else mx_flat_bf16_kernel<FAST_NONE, false, false><<<grid, kT, 0, st>>>(i, s, c, nvec, G, gshift, rule, r);
  }
}

}  // namespace

#define VQ_DISPATCH_FM(fm, ...)                                            \
  switch (fm) {                                                            \
    case FAST_NONE:  { constexpr int FM = FAST_NONE;  __VA_ARGS__; break; } \
    case FAST_INT:   { constexpr int FM = FAST_INT;   __VA_ARGS__; break; } \
    case FAST_E4M3:  { constexpr int FM = FAST_E4M3;  __VA_ARGS__; break; } \
    case FAST_E5M2:  { constexpr int FM = FAST_E5M2;  __VA_ARGS__; break; } \
    case FAST_E2M1:  { constexpr int FM = FAST_E2M1;  __VA_ARGS__; break; } \
    case FAST_E2M3:  { constexpr int FM = FAST_E2M3;  __VA_ARGS__; break; } \
    case FAST_E3M2:  { constexpr int FM = FAST_E3M2;  __VA_ARGS__; break; } \
    default:         { constexpr int FM = FAST_GENERIC; __VA_ARGS__; break; } \
  }

int fast_mx_flat_bf16(const void* in, void* scale_out, void* codes_out, int64_t nvec, int G, int gshift,
                      const ScaleRule& rule, const Round& r, int fast_mode, bool write_codes, cudaStream_t st) {
  VQ_DISPATCH_FM(fast_mode, (launch_mx_fm<FM>(rule.power_of_two != 0, write_codes, in, scale_out, codes_out, nvec, G,
                                              gshift, rule, r, st)));
  return check_launch("mx_flat_bf16_kernel");
}

int fast_quantize_bf16(const void* in, const void* scale, int pdt, void* out, int64_t nvec, uint32_t vecs_per_scale,
                       const Round& r, int fast_mode, cudaStream_t st) {
  int vshift = -1;
  if (vecs_per_scale && (vecs_per_scale & (vecs_per_scale - 1)) == 0) {
    vshift = 0;
    while ((1u << vshift) < vecs_per_scale) ++vshift;
  }
  const int grid = grid_of(nvec, kCtasPerSmPlain);
  VQ_DISPATCH_FM(fast_mode, (quantize_bf16_kernel<FM><<<grid, kT, 0, st>>>(
      static_cast<const uint4*>(in), scale, pdt, static_cast<uint4*>(out), nvec, vecs_per_scale, vshift, r)));
  return check_launch("quantize_bf16_kernel");
}

int fast_scale_bf16(const void* in, const void* scale, void* out, int64_t nvec, uint32_t vecs_per_scale,
                    cudaStream_t st) {
  int vshift = -1;
  if ((vecs_per_scale & (vecs_per_scale - 1)) == 0) {
    vshift = 0;
    while ((1u << vshift) < vecs_per_scale) ++vshift;
  }
  scale_bf16_kernel<<<grid_of(nvec), kT, 0, st>>>(static_cast<const uint4*>(in),
                                                  static_cast<const __nv_bfloat16*>(scale),
                                                  static_cast<uint4*>(out), nvec, vecs_per_scale, vshift);
  return check_launch("scale_bf16_kernel");
}

int fast_quantize_fp8(const void* in, const void* scale, int pdt, void* out, int64_t n16, uint32_t v16_per_scale,
                      bool e4m3, cudaStream_t st) {
  int vshift = -1;
  if (v16_per_scale && (v16_per_scale & (v16_per_scale - 1)) == 0) {
    vshift = 0;
    while ((1u << vshift) < v16_per_scale) ++vshift;
  }
  int64_t blocks = (n16 + kT * 2 - 1) / (kT * 2);
  const int64_t cap = (int64_t)kSmCount * 4;
  const int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  if (e4m3)
    quantize_fp8_kernel<true><<<grid, kT, 0, st>>>(static_cast<const uint4*>(in), scale, pdt, static_cast<uint4*>(out),
                                                   n16, v16_per_scale, vshift);
  else
    quantize_fp8_kernel<false><<<grid, kT, 0, st>>>(static_cast<const uint4*>(in), scale, pdt, static_cast<uint4*>(out),
                                                    n16, v16_per_scale, vshift);
  return check_launch("quantize_fp8_kernel");
}

}  // namespace vq

using namespace vq;

extern "C" int vq_quantize_fp8(const void* in, const void* scale, int scale_dtype, void* out, int format, int64_t n,
                               int64_t elems_per_scale, void* stream) {
  VQ_REQUIRE(n >= 0, "vq_quantize_fp8: negative size");
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(in && scale && out, "vq_quantize_fp8: null argument");
  VQ_REQUIRE(format == VQ_IN_E4M3 || format == VQ_IN_E5M2, "vq_quantize_fp8: format must be e4m3 or e5m2");
  VQ_REQUIRE(scale_dtype >= VQ_BF16 && scale_dtype <= VQ_F32, "vq_quantize_fp8: bad scale dtype");
  VQ_REQUIRE(n % 16 == 0, "vq_quantize_fp8: the element count must be a multiple of 16");
  VQ_REQUIRE(elems_per_scale >= 0 && elems_per_scale % 16 == 0 && elems_per_scale < (1ll << 35),
             "vq_quantize_fp8: elements per scale must be 0 (one scale) or a multiple of 16");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
             "vq_quantize_fp8: buffers must be 16-byte aligned");
  return fast_quantize_fp8(in, scale, scale_dtype, out, n / 16, (uint32_t)(elems_per_scale / 16),
                           format == VQ_IN_E4M3, static_cast<cudaStream_t>(stream));
}
