// Pieces shared by the generic and the bfloat16 fast-path quantizer kernels.
#pragma once

#include "vq_common.cuh"

namespace vq {

// ---------------------------------------------------------------------------
// 16-byte vector access
// ---------------------------------------------------------------------------
template <int DT> struct Vec {
  using E = Elem<DT>;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    if constexpr (DT == VQ_F32) {
      return reinterpret_cast<const float*>(&raw)[i];
    } else {
      return E::to_float(reinterpret_cast<const typename E::T*>(&raw)[i]);
    }
  }
  __device__ __forceinline__ void set(int i, float v) {
    if constexpr (DT == VQ_F32) {
      reinterpret_cast<float*>(&raw)[i] = v;
    } else {
      reinterpret_cast<typename E::T*>(&raw)[i] = E::from_float(v);
    }
  }
};

template <int DT>
__device__ __forceinline__ float load1(const void* p, int64_t i) {
  return Elem<DT>::to_float(static_cast<const typename Elem<DT>::T*>(p)[i]);
}
template <int DT>
__device__ __forceinline__ void store1(void* p, int64_t i, float v) {
  static_cast<typename Elem<DT>::T*>(p)[i] = Elem<DT>::from_float(v);
}

// A parameter (scale, zero point, global scale) whose dtype is only known at
// run time: a 0-d float32 scale next to bfloat16 data is used at full
// precision, as torch does for scalar operands.
__device__ __forceinline__ float loadp(const void* p, int64_t i, int pdt) {
  if (pdt == VQ_F32) return static_cast<const float*>(p)[i];
  if (pdt == VQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

// ---------------------------------------------------------------------------
// microscaling: scale rule
// ---------------------------------------------------------------------------
struct ScaleRule {
  float quant_max;
  int power_of_two;
  int qmax_exp;  // floor(log2(quant_max))
  const void* global_scale;
  int global_scale_dtype;
  Round scale_round;
  float zero_scale_bf16;  // power-of-two rule: the bfloat16 scale of an all-zero block
};

// amax_bits: |amax| as float bits (NaN patterns compare above inf, so an
// integer max over |x| bits propagates NaN like torch.amax).
// Returns the block scale (value of dtype DT, as float); *elem_scale gets the
// divisor of the elements (scale * global_scale when present).
template <int DT>
__device__ __forceinline__ float block_scale(uint32_t amax_bits, const ScaleRule& rule, float* elem_scale) {
  using E = Elem<DT>;
  float amax = __uint_as_float(amax_bits);
  float scale;
  float gs = 0.f;
  const bool has_gs = rule.global_scale != nullptr;
  if (has_gs) gs = loadp(rule.global_scale, 0, rule.global_scale_dtype);
  if (rule.power_of_two) {
    if (amax != amax) {
      scale = amax;
    } else if (amax_bits == 0x7F800000u) {
      scale = amax;  // infinite block -> infinite scale
    } else {
      int e = (amax == 0.0f) ? -126 : ilogbf(amax);
      scale = E::round(ldexpf(1.0f, e - rule.qmax_exp));
    }
  } else {
    scale = E::round(__fdiv_rn(amax, rule.quant_max));
    if (has_gs) scale = E::round(__fdiv_rn(scale, gs));
    if (rule.scale_round.mode != VQ_ROUND_NONE) scale = E::round(apply_round(rule.scale_round, scale, 0));
  }
  scale = (scale > 0.0f) ? scale : 1.0f;
  *elem_scale = has_gs ? E::round(__fmul_rn(scale, gs)) : scale;
  return scale;
}

__device__ __forceinline__ uint32_t abs_bits(float v) { return __float_as_uint(v) & 0x7FFFFFFFu; }


// round_bf16(x / s) for a normal, finite, positive s with rcp = 1/s correctly
// rounded.  x * rcp is within 2 ulp of the correctly rounded quotient; when it
// is that close to the midpoint between two bfloat16 values, or not a normal
// number, the exact division decides.
__device__ __forceinline__ float div_to_bf16(float x, float s, float rcp) {
  float q = __fmul_rn(x, rcp);
  uint32_t b = __float_as_uint(q);
  uint32_t ex = (b >> 23) & 0xFFu;
  uint32_t low = b & 0xFFFFu;
  if (ex == 0u || ex == 0xFFu || (low - 0x7FFDu) <= 6u) q = __fdiv_rn(x, s);
  return __bfloat162float(__float2bfloat16_rn(q));
}

// True when s is a normal, finite, positive float whose reciprocal is normal too.
__device__ __forceinline__ bool ordinary_divisor(float s) {
  const uint32_t ex = (__float_as_uint(s) >> 23) & 0xFFu;
  return ex >= 1u && ex <= 253u && s > 0.0f;
}

// bfloat16 fast paths (quantize_fast.cu)
int fast_mode_of(const VqRound* r);
int fast_mx_flat_bf16(const void* in, void* scale_out, void* codes_out, int64_t nvec, int G, int gshift,
                      const ScaleRule& rule, const Round& r, int fast_mode, bool write_codes, cudaStream_t st);
int fast_quantize_bf16(const void* in, const void* scale, int pdt, void* out, int64_t nvec, uint32_t vecs_per_scale,
                       const Round& r, int fast_mode, cudaStream_t st);
int fast_scale_bf16(const void* in, const void* scale, void* out, int64_t nvec, uint32_t vecs_per_scale,
                    cudaStream_t st);

}  // namespace vq
