// Device helpers shared by the kernels that cast bfloat16 values to FP8 with a per-tensor
// scale: bfloat16 rounding, the bfloat16 quotient x / scale, and the packed FP8 conversion.
#pragma once

#include <cuda_fp8.h>

#include "quantize_shared.cuh"

namespace vq {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float lo_of(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_of(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

struct Divisor {
  float s, rcp;
  bool ordinary;
};
__device__ __forceinline__ Divisor make_divisor(const void* scale, int dt) {
  Divisor d;
  d.s = loadp(scale, 0, dt);
  d.ordinary = ordinary_divisor(d.s);
  d.rcp = __frcp_rn(d.s);
  return d;
}
__device__ __forceinline__ float quot(float x, const Divisor& d) {
  return d.ordinary ? div_to_bf16(x, d.s, d.rcp) : bf16r(__fdiv_rn(x, d.s));
}
template <bool E4M3>
__device__ __forceinline__ uint32_t fp8_pair(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f)), __NV_SATFINITE,
                                            E4M3 ? __NV_E4M3 : __NV_E5M2);
}

}  // namespace vq
