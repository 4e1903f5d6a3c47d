// Delayed-scaling state of a per-tensor / per-channel fake-quantizer, kept on the device:
// a ring of the last `length` absolute maxima per channel, a ring position per channel, and
// the scale derived from the ring.  One call = one observed tensor:
//
//   amax  = max over the ring as it stood BEFORE this tensor (a NaN entry makes it NaN)
//   ring[position] = this tensor's amax; position advances
//   scale = amax / quant_max in the tensor dtype, kept unchanged while amax is 0, negative,
//           infinite or NaN; optionally rounded up to a power of two, 2^ceil(log2 scale),
//           with the logarithm itself rounded to the tensor dtype first
//
// which is the update rule of FusedAmaxObsFakeQuantize (reference
// quantization/fake_quantize.py:406-437): a tensor is quantized with the scale of its
// predecessors, before its own amax counts.  One thread owns one channel, so nothing is
// shared between threads and the call can be captured in a CUDA graph (no host counter).

#include <cmath>

#include "vq_common.cuh"

namespace vq {
namespace {

__device__ __forceinline__ float load_any(const void* p, int64_t i, int dt) {
  if (dt == VQ_F32) return static_cast<const float*>(p)[i];
  if (dt == VQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

template <int DT>
__global__ void amax_history_kernel(typename Elem<DT>::T* ring, int length, int64_t channels, int32_t* position,
                                    const void* amax_now, int amax_dt, int64_t amax_count, float quant_max,
                                    int power_of_two, typename Elem<DT>::T* scale) {
  using E = Elem<DT>;
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float amax = E::to_float(ring[c]);
  for (int l = 1; l < length; ++l) {
    const float v = E::to_float(ring[(int64_t)l * channels + c]);
    amax = (isnan(v) || isnan(amax)) ? NAN : fmaxf(amax, v);
  }
  int at = position[c];
  if (at < 0 || at >= length) at = 0;
  ring[(int64_t)at * channels + c] = E::from_float(load_any(amax_now, amax_count == 1 ? 0 : c, amax_dt));
  position[c] = at + 1 == length ? 0 : at + 1;
  if (!(amax > 0.0f) || isinf(amax)) return;      // zero, negative, infinite or NaN: the scale stays
  float s = E::round(__fdiv_rn(amax, quant_max));
  if (power_of_two) {
    const float e = ceilf(E::round(log2f(s)));     // the reference takes the logarithm in the tensor dtype
    s = isnan(e) ? NAN : (isinf(e) ? (e < 0.0f ? 0.0f : INFINITY) : ldexpf(1.0f, (int)fmaxf(fminf(e, 400.0f), -400.0f)));
  }
  scale[c] = E::from_float(s);
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_amax_history_update(void* ring, int dtype, int64_t length, int64_t channels, int32_t* position,
                                      const void* amax, int amax_dtype, int64_t amax_count, float quant_max,
                                      int power_of_two, void* scale, void* stream) {
  VQ_REQUIRE(length > 0 && length < (1ll << 30) && channels >= 0, "vq_amax_history_update: bad extents");
  if (channels == 0) return VQ_OK;
  VQ_REQUIRE(ring && position && amax && scale, "vq_amax_history_update: null argument");
  VQ_REQUIRE(amax_count == 1 || amax_count == channels, "vq_amax_history_update: one amax, or one per channel");
  VQ_REQUIRE(amax_dtype >= VQ_BF16 && amax_dtype <= VQ_F32, "vq_amax_history_update: bad amax dtype");
  VQ_REQUIRE(quant_max > 0.0f, "vq_amax_history_update: quant_max must be positive");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = 128;
  const unsigned grid = (unsigned)((channels + threads - 1) / threads);
  switch (dtype) {
    case VQ_BF16:
      amax_history_kernel<VQ_BF16><<<grid, threads, 0, st>>>(static_cast<__nv_bfloat16*>(ring), (int)length, channels,
                                                             position, amax, amax_dtype, amax_count, quant_max,
                                                             power_of_two, static_cast<__nv_bfloat16*>(scale));
      break;
    case VQ_F16:
      amax_history_kernel<VQ_F16><<<grid, threads, 0, st>>>(static_cast<__half*>(ring), (int)length, channels, position,
                                                            amax, amax_dtype, amax_count, quant_max, power_of_two,
                                                            static_cast<__half*>(scale));
      break;
    case VQ_F32:
      amax_history_kernel<VQ_F32><<<grid, threads, 0, st>>>(static_cast<float*>(ring), (int)length, channels, position,
                                                            amax, amax_dtype, amax_count, quant_max, power_of_two,
                                                            static_cast<float*>(scale));
      break;
    default:
      return fail(VQ_EINVAL, "vq_amax_history_update: unknown dtype %d", dtype);
  }
  return check_launch("amax_history_kernel");
}
