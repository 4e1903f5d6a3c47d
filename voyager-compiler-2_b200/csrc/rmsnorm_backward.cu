// RMSNorm's backward for a training step: input and weight gradients from one read of the rows.
//
// Forward: r = rsqrt(mean(x^2) + eps) in float32, y = w * bf16(x * r).  Backward, with every
// elementwise value rounded to bfloat16 where the decomposed aten program rounds it:
//   dy   = the sum of up to three gradients, rounded after each addition
//   dw  += bf16(dy * bf16(x * r))                          summed over the rows in float32
//   g    = bf16(dy * w)
//   s    = sum_k(g * x) * -0.5 * r^3 / cols                the row's dot product, float32
//   dx   = bf16(g * r + s * (2 x)) (+ residual, rounded again)
// Only the two sums (a row's dot product, the weight gradient over the rows) add in an order of
// their own.  A CTA walks ROWS consecutive rows keeping its columns' weight-gradient sums in
// registers and writes one partial row; a second kernel adds the partial rows.

#include "quantize_shared.cuh"

namespace vq {
namespace {

constexpr int RB_THREADS = 256;

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float lo16(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi16(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// VPT 16-byte vectors (8 columns) per thread; cols <= 8 * VPT * RB_THREADS.
template <int VPT, int GRADIENTS, bool RESIDUAL>
__global__ void __launch_bounds__(RB_THREADS, VPT <= 2 ? 4 : 2)
rmsnorm_backward_kernel(const uint4* __restrict__ dy0, const uint4* __restrict__ dy1, const uint4* __restrict__ dy2,
                        const uint4* __restrict__ x, const float* __restrict__ rsqrt_rows,
                        const uint4* __restrict__ weight, const uint4* __restrict__ residual, uint4* __restrict__ dx,
                        float* __restrict__ partial_dw, int64_t rows, int cols, int rows_per_cta) {
  __shared__ float warp_sums[2][RB_THREADS / 32];
  const int vecs = cols >> 3;
  const float inv_cols = __fdiv_rn(1.0f, (float)cols);
  // Weights, the summed gradient and x stay packed (two bfloat16 per register) between the row's two
  // phases; only the weight-gradient sums are float32.  Fewer registers, more CTAs per SM.
  uint4 w[VPT];
  float dw[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + RB_THREADS * i;
    w[i] = make_uint4(0, 0, 0, 0);
    if (v < vecs) w[i] = __ldg(weight + v);
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.0f;
  }
  const int64_t first = (int64_t)blockIdx.x * rows_per_cta;
  const int64_t last = min(first + rows_per_cta, rows);
  for (int64_t m = first; m < last; ++m) {
    const float r = rsqrt_rows[m];
    uint4 dyp[VPT], xp[VPT];   // dy (the gradients summed) and x of this thread's vectors
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + RB_THREADS * i;
      dyp[i] = xp[i] = make_uint4(0, 0, 0, 0);
      if (v < vecs) {
        const int64_t at = m * vecs + v;
        const uint4 a = __ldg(dy0 + at);
        xp[i] = __ldg(x + at);
        uint4 b = make_uint4(0, 0, 0, 0), c = make_uint4(0, 0, 0, 0);
        if (GRADIENTS > 1) b = __ldg(dy1 + at);
        if (GRADIENTS > 2) c = __ldg(dy2 + at);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, cw[4] = {c.x, c.y, c.z, c.w};
        const uint32_t xw[4] = {xp[i].x, xp[i].y, xp[i].z, xp[i].w};
        const uint32_t ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
        uint32_t sum[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float dy[2] = {lo16(aw[q]), hi16(aw[q])};
          if (GRADIENTS > 1) {
            dy[0] = bf16_round(__fadd_rn(dy[0], lo16(bw[q])));
            dy[1] = bf16_round(__fadd_rn(dy[1], hi16(bw[q])));
          }
          if (GRADIENTS > 2) {
            dy[0] = bf16_round(__fadd_rn(dy[0], lo16(cw[q])));
            dy[1] = bf16_round(__fadd_rn(dy[1], hi16(cw[q])));
          }
          sum[q] = pack_bf16(dy[0], dy[1]);   // exact: both are bfloat16 values
          const float xe[2] = {lo16(xw[q]), hi16(xw[q])}, we[2] = {lo16(ww[q]), hi16(ww[q])};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            dw[i][2 * q + h] = __fadd_rn(dw[i][2 * q + h], bf16_round(__fmul_rn(dy[h], bf16_round(__fmul_rn(xe[h], r)))));
            dot = __fadd_rn(dot, __fmul_rn(bf16_round(__fmul_rn(dy[h], we[h])), xe[h]));
          }
        }
        dyp[i] = make_uint4(sum[0], sum[1], sum[2], sum[3]);
      }
    }
    // the row's dot product: warps, then the CTA (the two buffers alternate so one barrier per row is enough)
    for (int off = 16; off; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
    float* sums = warp_sums[m & 1];
    if ((threadIdx.x & 31) == 0) sums[threadIdx.x >> 5] = dot;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int q = 0; q < RB_THREADS / 32; ++q) total += sums[q];   // same order in every thread
    // d(rsqrt)/dx: -0.5 r^3 * 2 x / cols, times the row's g . x
    const float scale = __fmul_rn(__fmul_rn(__fmul_rn(total, -0.5f), __fmul_rn(__fmul_rn(r, r), r)), inv_cols);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + RB_THREADS * i;
      if (v < vecs) {
        const int64_t at = m * vecs + v;
        uint4 rv = make_uint4(0, 0, 0, 0);
        if (RESIDUAL) rv = __ldg(residual + at);
        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
        const uint32_t dw4[4] = {dyp[i].x, dyp[i].y, dyp[i].z, dyp[i].w};
        const uint32_t xw[4] = {xp[i].x, xp[i].y, xp[i].z, xp[i].w};
        const uint32_t ww[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float dy[2] = {lo16(dw4[q]), hi16(dw4[q])}, xe[2] = {lo16(xw[q]), hi16(xw[q])};
          const float we[2] = {lo16(ww[q]), hi16(ww[q])}, re[2] = {lo16(rw[q]), hi16(rw[q])};
          float e[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float g = bf16_round(__fmul_rn(dy[h], we[h]));
            float grad = bf16_round(__fadd_rn(__fmul_rn(g, r), __fmul_rn(scale, __fmul_rn(xe[h], 2.0f))));
            if (RESIDUAL) grad = __fadd_rn(grad, re[h]);
            e[h] = grad;
          }
          o[q] = pack_bf16(e[0], e[1]);
        }
        dx[at] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + RB_THREADS * i;
    if (v < vecs) {
      float4* dst = reinterpret_cast<float4*>(partial_dw + (int64_t)blockIdx.x * cols + (int64_t)v * 8);
      dst[0] = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      dst[1] = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

// dw[c] = bf16(sum over the partial rows): 32 columns x 8 row lanes per CTA
__global__ void __launch_bounds__(256)
rmsnorm_dw_sum_kernel(const float* __restrict__ partial_dw, __nv_bfloat16* __restrict__ dw, int programs, int cols) {
  __shared__ float part[8][32];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int lane_row = threadIdx.x >> 5;
  float total = 0.0f;
  if (c < cols)
    for (int p = lane_row; p < programs; p += 8) total += partial_dw[(int64_t)p * cols + c];
  part[lane_row][threadIdx.x & 31] = total;
  __syncthreads();
  if (lane_row == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += part[q][threadIdx.x];
    dw[c] = __float2bfloat16_rn(t);
  }
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int64_t vq_rmsnorm_backward_programs(int64_t rows, int64_t cols) {
  // as many CTAs as are resident at once (the kernels are compiled for 4 per SM, 2 for rows of more than
  // 4096 columns), at least one row each
  const int vpt = (int)((cols / 8 + RB_THREADS - 1) / RB_THREADS);
  const int64_t target = (int64_t)kSmCount * (vpt <= 2 ? 4 : 2);
  const int64_t per = rows <= target ? 1 : (rows + target - 1) / target;
  return rows <= 0 ? 0 : (rows + per - 1) / per;
}

extern "C" int vq_rmsnorm_backward(const void* dy0, const void* dy1, const void* dy2, int gradients, const void* x,
                                   const float* rsqrt_rows, const void* weight, const void* residual, void* dx,
                                   float* partial_dw, void* dw, int64_t rows, int64_t cols, void* stream) {
  VQ_REQUIRE(rows >= 0 && cols > 0, "vq_rmsnorm_backward: bad extent");
  VQ_REQUIRE(gradients >= 1 && gradients <= 3, "vq_rmsnorm_backward: one to three gradients");
  VQ_REQUIRE(cols % 8 == 0 && cols <= 8 * 4 * RB_THREADS, "vq_rmsnorm_backward: the row length must be a multiple of 8, at most 8192");
  VQ_REQUIRE(weight && dw, "vq_rmsnorm_backward: null argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    cudaMemsetAsync(dw, 0, (size_t)cols * 2, st);
    return check_launch("vq_rmsnorm_backward (memset)");
  }
  VQ_REQUIRE(dy0 && x && rsqrt_rows && dx && partial_dw && (gradients < 2 || dy1) && (gradients < 3 || dy2),
             "vq_rmsnorm_backward: null argument");
  const uintptr_t all = reinterpret_cast<uintptr_t>(dy0) | reinterpret_cast<uintptr_t>(dy1) |
                        reinterpret_cast<uintptr_t>(dy2) | reinterpret_cast<uintptr_t>(x) |
                        reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(residual) |
                        reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(partial_dw);
  VQ_REQUIRE((all & 15) == 0, "vq_rmsnorm_backward: misaligned buffers");
  const int64_t programs = vq_rmsnorm_backward_programs(rows, cols);
  const int rows_per_cta = (int)((rows + programs - 1) / programs);
  VQ_REQUIRE(programs < (1ll << 31), "vq_rmsnorm_backward: too many rows");
  const int vecs = (int)(cols / 8);
  const int vpt = (vecs + RB_THREADS - 1) / RB_THREADS;
  const uint4 *a = static_cast<const uint4*>(dy0), *b = static_cast<const uint4*>(dy1), *c = static_cast<const uint4*>(dy2);
  const uint4 *xi = static_cast<const uint4*>(x), *wi = static_cast<const uint4*>(weight), *ri = static_cast<const uint4*>(residual);
  uint4* out = static_cast<uint4*>(dx);
#define VQ_RB_LAUNCH(V, G, R)                                                                                      \
  rmsnorm_backward_kernel<V, G, R><<<(unsigned)programs, RB_THREADS, 0, st>>>(a, b, c, xi, rsqrt_rows, wi, ri, out, \
                                                                             partial_dw, rows, (int)cols, rows_per_cta)
#define VQ_RB_RES(V, G) do { if (residual) VQ_RB_LAUNCH(V, G, true); else VQ_RB_LAUNCH(V, G, false); } while (0)
#define VQ_RB_GRAD(V) do { if (gradients == 1) VQ_RB_RES(V, 1); else if (gradients == 2) VQ_RB_RES(V, 2); else VQ_RB_RES(V, 3); } while (0)
  if (vpt <= 1) VQ_RB_GRAD(1);
  else if (vpt == 2) VQ_RB_GRAD(2);
  else VQ_RB_GRAD(4);
#undef VQ_RB_GRAD
#undef VQ_RB_RES
#undef VQ_RB_LAUNCH
  int rc = check_launch("rmsnorm_backward_kernel");
  if (rc != VQ_OK) return rc;
  rmsnorm_dw_sum_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, st>>>(partial_dw, static_cast<__nv_bfloat16*>(dw),
                                                                     (int)programs, (int)cols);
  return check_launch("rmsnorm_dw_sum_kernel");
}
