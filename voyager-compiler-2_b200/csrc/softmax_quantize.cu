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
// two floats rounded to bfloat16 by one instruction: `lo` in bits [0,16), `hi` in bits [16,32)
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// the two bfloat16 values of a word as floats
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
// both floats rounded to bfloat16 (one packed conversion) and widened again
__device__ __forceinline__ float2 round_pair_bf16(float2 v) { return unpack_bf16x2(pack_bf16x2(v.x, v.y)); }
// max of three floats in one instruction; like fmaxf, a NaN operand is ignored
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ex2_approx(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// barrier over the THREADS threads that share a row (at most two rows per CTA); id 0 is left to __syncthreads
template <int THREADS>
__device__ __forceinline__ void group_barrier(int group) {
  // the id is an immediate so that the CTA reserves only the barriers it uses
  if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
  else asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");
}

// VPL = 16-byte vectors (8 columns) per lane; a row has up to 32 * 8 * VPL * WPR columns.
// WPR warps share a row (its vectors interleaved between them, so a causal row's live part is
// split evenly) and combine their maximum and sum through shared memory.  The kernel is bound
// by instruction issue, not by DRAM: a row costs each of its warps about 130 instructions of
// indexing, shuffles and reciprocals beside the 84 per live vector, so long rows want few
// warps, while one warp per 2048-column row needs 90 registers and leaves too few warps
// resident.  Two warps with four vectors per lane measured fastest for such rows.
template <int VPL, int WPR, bool E4M3>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
softmax_quantize_kernel(const uint4* __restrict__ scores, uint2* __restrict__ out, int64_t rows, int cols,
                        float score_scale, const __nv_bfloat16* __restrict__ mask, int64_t mask_rows,
                        int causal_period, const void* __restrict__ out_scale, int out_scale_dt) {
  __shared__ float part_max[kWarpsPerCta], part_sum[kWarpsPerCta];
  constexpr int kStride = 32 * WPR;                    // vectors between a thread's consecutive vectors
  const int lane = threadIdx.x % kStride;              // position among the row's threads
  const int warp = threadIdx.x >> 5;
  const int w0 = warp - warp % WPR;                    // first warp of this row's group
  const int group = threadIdx.x / kStride;             // which of the CTA's rows
  const int64_t row = (int64_t)blockIdx.x * (kWarpsPerCta / WPR) + group;
  if (row >= rows) return;                             // the barriers below are per row group
  const int vecs = cols >> 3;
  // columns [0, lim) can be non-zero: t + 1 under a causal mask, t the row's place in its period
  int lim = cols;
  if (causal_period > 0) {
    // a 64-bit remainder costs dozens of instructions: take the 32-bit one whenever the row fits
    const int t = row < (1ll << 31) ? (int)((uint32_t)row % (uint32_t)causal_period) : (int)(row % causal_period);
    lim = min(cols, t + 1);
  }
  const uint4* src = scores + row * vecs;
  const __nv_bfloat16* mrow = mask ? mask + (row % mask_rows) * (int64_t)cols : nullptr;

  // A lane's vectors are live up to a lane-dependent count; dead vectors (past the row's end or
  // wholly past the diagonal) are never touched.  Only a row's last live vector can straddle
  // the diagonal and needs per-element masking.
  // All of a lane's loads are issued before the first is used.
  uint4 raw[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + kStride * i;
    if (v < vecs && (v << 3) < lim) raw[i] = __ldg(src + v);
  }
  float2 x[VPL][4];                                    // packed pairs: the fp32 pipe takes two per instruction
  float mx = -INFINITY;
  const float2 scale2 = make_float2(score_scale, score_scale);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + kStride * i;
    const int c0 = v << 3;
    if (v < vecs && c0 < lim) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j)  // s = bf16(score * scale)
        x[i][j] = round_pair_bf16(__fmul2_rn(unpack_bf16x2(w[j]), scale2));
      if (mrow) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          x[i][j] = round_pair_bf16(__fadd2_rn(x[i][j], make_float2(__bfloat162float(mrow[c0 + 2 * j]),
                                                                    __bfloat162float(mrow[c0 + 2 * j + 1]))));
      }
      if (c0 + 8 > lim) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (c0 + 2 * j >= lim) x[i][j].x = -INFINITY;
          if (c0 + 2 * j + 1 >= lim) x[i][j].y = -INFINITY;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) mx = fmax3(mx, x[i][j].x, x[i][j].y);
    }
  }
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
  if (WPR > 1) {
    if ((threadIdx.x & 31) == 0) part_max[warp] = mx;
    group_barrier<kStride>(group);
#pragma unroll
    for (int q = 0; q < WPR; ++q) mx = fmaxf(mx, part_max[w0 + q]);
  }
  // exp(s - max) = 2^(s * log2(e) - max * log2(e)): one fused multiply-add and one ex2 per element.
  // exp(-inf) = 0 for masked entries; a fully masked row (max = -inf) yields NaN, as torch.softmax does.
  constexpr float kLog2e = 1.4426950408889634f;
  const float2 log2e2 = make_float2(kLog2e, kLog2e);
  const float2 shift2 = make_float2(-mx * kLog2e, -mx * kLog2e);
  float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + kStride * i;
    if (v < vecs && (v << 3) < lim) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __ffma2_rn(x[i][j], log2e2, shift2);
        x[i][j] = make_float2(ex2_approx(a.x), ex2_approx(a.y));
        sum2 = __fadd2_rn(sum2, x[i][j]);
      }
    }
  }
  float sum = sum2.x + sum2.y;
  for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  if (WPR > 1) {
    if ((threadIdx.x & 31) == 0) part_sum[warp] = sum;
    group_barrier<kStride>(group);
    sum = 0.0f;
#pragma unroll
    for (int q = 0; q < WPR; ++q) sum += part_sum[w0 + q];   // same order in every warp
  }

  // p = bf16(e / sum), code = fp8(bf16(p / s_p)): both quotients are taken as products
  // with the correctly rounded reciprocal (within an ulp of the division before the
  // bfloat16 rounding, like the exponential itself).  p >= 0, so no -0 can arise.
  const float rsum = __frcp_rn(sum), rsp = __frcp_rn(loadp(out_scale, 0, out_scale_dt));
  const float2 rsum2 = make_float2(rsum, rsum), rsp2 = make_float2(rsp, rsp);
  uint2* dst = out + row * vecs;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + kStride * i;
    if (v >= vecs) continue;
    uint32_t o[2] = {0u, 0u};
    if ((v << 3) < lim) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 prob = round_pair_bf16(__fmul2_rn(x[i][j], rsum2));
        const float2 f = round_pair_bf16(__fmul2_rn(prob, rsp2));
        const uint32_t code = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, E4M3 ? __NV_E4M3 : __NV_E5M2);
        o[j >> 1] |= code << (16 * (j & 1));
      }
    } else if (sum != sum) {
      o[0] = o[1] = E4M3 ? 0x7F7F7F7Fu : 0x7E7E7E7Eu;  // NaN row
    }
    dst[v] = make_uint2(o[0], o[1]);
  }
}

template <bool E4M3>
int launch(int vecs, const void* scores, void* out, int64_t rows, int cols, float score_scale, const void* mask,
           int64_t mask_rows, int causal_period, const void* out_scale, int out_scale_dt, cudaStream_t st) {
  const uint4* s = static_cast<const uint4*>(scores);
  uint2* o = static_cast<uint2*>(out);
  const __nv_bfloat16* m = static_cast<const __nv_bfloat16*>(mask);
  // up to 1024 columns one warp per row, up to 2048 two, beyond that the CTA's four
  const int wpr = vecs > 256 ? 4 : vecs > 128 ? 2 : 1;
  int vpl = 1;
  while (vpl * 32 * wpr < vecs) vpl <<= 1;
  const int64_t rows_per_cta = kWarpsPerCta / wpr;
  const int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
#define VQ_SM_CASE(V, W)                                                                                       \
  softmax_quantize_kernel<V, W, E4M3><<<(unsigned)grid, kWarpsPerCta * 32, 0, st>>>(                         \
      s, o, rows, cols, score_scale, m, mask_rows, causal_period, out_scale, out_scale_dt)
  if (wpr == 1) {
    switch (vpl) {
      case 1: VQ_SM_CASE(1, 1); break;
      case 2: VQ_SM_CASE(2, 1); break;
      default: VQ_SM_CASE(4, 1); break;
    }
  } else if (wpr == 2) {
    VQ_SM_CASE(4, 2);
  } else {
    if (vpl != 4) return fail(VQ_EUNSUPPORTED, "softmax row too long");
    VQ_SM_CASE(4, 4);
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (format == VQ_IN_E4M3)
    return launch<true>(vecs, scores, out, rows, (int)cols, score_scale, mask, mask_rows, (int)causal_period,
                        out_scale, out_scale_dtype, st);
  return launch<false>(vecs, scores, out, rows, (int)cols, score_scale, mask, mask_rows, (int)causal_period,
                       out_scale, out_scale_dtype, st);
}
