// Fused attention-probability kernel: scale, mask, softmax and FP8 cast in one pass.
//
// An eager-attention graph runs, per score row,
//     s = bf16(score * scale); s = bf16(s + mask); p = bf16(softmax_fp32(s)); code = fp8(bf16(p / s_p))
// as five separate elementwise / reduction passes over a [heads*T, T] matrix.
// Here one warp owns one row, keeps it in registers, and writes only the FP8
// codes: the bfloat16 scores are read once and one byte per element is written.
// Under a causal mask the columns past the diagonal are never read (their
// probability is exactly zero).  Every rounding step of the unfused sequence is
// kept; the exponential and the two quotients are within an ulp of the unfused ones
// before they are rounded to bfloat16, so a code differs by one FP8 step only when such
// a value sits on a rounding boundary (about one entry in a few thousand).

#include <cuda_fp8.h>

#include "quantize_shared.cuh"

namespace vq {
namespace {

constexpr int kWarpsPerCta = 4;

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// VPL = 16-byte vectors (8 columns) per lane; a row has up to 32 * 8 * VPL columns.
template <int VPL, bool E4M3>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
softmax_quantize_kernel(const uint4* __restrict__ scores, uint2* __restrict__ out, int64_t rows, int cols,
                        float score_scale, const __nv_bfloat16* __restrict__ mask, int64_t mask_rows,
                        int causal_period, const void* __restrict__ out_scale, int out_scale_dt) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int vecs = cols >> 3;
  const float sp = loadp(out_scale, 0, out_scale_dt);
  // columns [0, limit) can be non-zero
  int limit = cols;
  if (causal_period > 0) limit = min(cols, (int)(row % causal_period) + 1);
  const uint4* src = scores + row * vecs;
  const __nv_bfloat16* mrow = mask ? mask + (row % mask_rows) * (int64_t)cols : nullptr;

  float x[VPL][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    const int c0 = v << 3;
    const bool live = v < vecs && c0 < limit;  // a vector past the diagonal is neither read nor computed
    if (live) {
      const uint4 raw = __ldg(src + v);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s = __uint_as_float((j & 1) ? (w[j >> 1] & 0xFFFF0000u) : (w[j >> 1] << 16));
        s = bf16r(__fmul_rn(s, score_scale));
        if (mrow) s = bf16r(__fadd_rn(s, __bfloat162float(mrow[c0 + j])));
        if (c0 + j >= limit) s = -INFINITY;
        x[i][j] = s;
        mx = fmaxf(mx, s);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[i][j] = -INFINITY;
    }
  }
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c0 = (lane + 32 * i) << 3;
    if (c0 < limit && (lane + 32 * i) < vecs) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // exp(-inf) = 0 for masked entries; a fully masked row (max = -inf) yields NaN, as torch.softmax does
        const float e = __expf(x[i][j] - mx);
        x[i][j] = e;
        sum += e;
      }
    }
  }
  for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);

  // p = bf16(e / sum), code = fp8(bf16(p / s_p)): both quotients are taken as products
  // with the correctly rounded reciprocal (within an ulp of the division before the
  // bfloat16 rounding, like the exponential itself).
  const float rsum = __frcp_rn(sum), rsp = __frcp_rn(sp);
  uint2* dst = out + row * vecs;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + 32 * i;
    if (v >= vecs) continue;
    uint32_t o[2] = {0u, 0u};
    if ((v << 3) < limit) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float p0 = bf16r(__fmul_rn(bf16r(__fmul_rn(x[i][j], rsum)), rsp));
        const float p1 = bf16r(__fmul_rn(bf16r(__fmul_rn(x[i][j + 1], rsum)), rsp));
        const float2 f = make_float2(__fadd_rn(p0, 0.0f), __fadd_rn(p1, 0.0f));
        const uint32_t q = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, E4M3 ? __NV_E4M3 : __NV_E5M2);
        o[j >> 2] |= q << (16 * ((j >> 1) & 1));
      }
    } else if (sum != sum) {
      o[0] = o[1] = E4M3 ? 0x7F7F7F7Fu : 0x7E7E7E7Eu;  // NaN row
    }
    dst[v] = make_uint2(o[0], o[1]);
  }
}

template <bool E4M3>
int launch(int vpl, const void* scores, void* out, int64_t rows, int cols, float score_scale, const void* mask,
           int64_t mask_rows, int causal_period, const void* out_scale, int out_scale_dt, cudaStream_t st) {
  const int64_t grid = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  const uint4* s = static_cast<const uint4*>(scores);
  uint2* o = static_cast<uint2*>(out);
  const __nv_bfloat16* m = static_cast<const __nv_bfloat16*>(mask);
#define VQ_SM_CASE(V)                                                                                          \
  case V:                                                                                                      \
    softmax_quantize_kernel<V, E4M3><<<(unsigned)grid, kWarpsPerCta * 32, 0, st>>>(                          \
        s, o, rows, cols, score_scale, m, mask_rows, causal_period, out_scale, out_scale_dt);                  \
    break;
  switch (vpl) {
    VQ_SM_CASE(1) VQ_SM_CASE(2) VQ_SM_CASE(4) VQ_SM_CASE(8) VQ_SM_CASE(16)
    default:
      return fail(VQ_EUNSUPPORTED, "softmax row too long");
  }
#undef VQ_SM_CASE
  return check_launch("softmax_quantize_kernel");
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_softmax_quantize_fp8(const void* scores, void* out, int64_t rows, int64_t cols, float score_scale,
                                       const void* mask, int64_t mask_rows, int64_t causal_period,
                                       const void* out_scale, int out_scale_dtype, int format, void* stream) {
  VQ_REQUIRE(rows >= 0 && cols >= 0, "vq_softmax_quantize_fp8: negative extent");
  if (rows == 0 || cols == 0) return VQ_OK;
  VQ_REQUIRE(scores && out && out_scale, "vq_softmax_quantize_fp8: null argument");
  VQ_REQUIRE(format == VQ_IN_E4M3 || format == VQ_IN_E5M2, "vq_softmax_quantize_fp8: format must be e4m3 or e5m2");
  VQ_REQUIRE(cols % 8 == 0, "vq_softmax_quantize_fp8: the row length must be a multiple of 8");
  VQ_REQUIRE(cols <= 32 * 8 * 16, "vq_softmax_quantize_fp8: rows longer than 4096 are not supported");
  VQ_REQUIRE(!mask || mask_rows > 0, "vq_softmax_quantize_fp8: mask without rows");
  VQ_REQUIRE(causal_period >= 0 && causal_period < (1ll << 31), "vq_softmax_quantize_fp8: bad causal period");
  VQ_REQUIRE(rows < (1ll << 33), "vq_softmax_quantize_fp8: too many rows");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(scores) & 15) | (reinterpret_cast<uintptr_t>(out) & 7)) == 0,
             "vq_softmax_quantize_fp8: misaligned buffers");
  const int vecs = (int)(cols / 8);
  int vpl = 1;
  while (vpl * 32 < vecs) vpl <<= 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (format == VQ_IN_E4M3)
    return launch<true>(vpl, scores, out, rows, (int)cols, score_scale, mask, mask_rows, (int)causal_period,
                        out_scale, out_scale_dtype, st);
  return launch<false>(vpl, scores, out, rows, (int)cols, score_scale, mask, mask_rows, (int)causal_period,
                       out_scale, out_scale_dtype, st);
}
