// FP8 casts fused with the bfloat16 operation that produces their input.
//
// In a per-tensor FP8 decoder layer every quantized tensor is produced by a cheap
// bfloat16 operation (RMSNorm, rotary embedding, SiLU * up, a head transpose) and
// immediately cast.  Running them as separate passes writes and re-reads every
// activation several times; here each pair is one kernel that reads the
// bfloat16 input once and writes one byte per element, in the layout the next
// GEMM wants.  Each kernel keeps the bfloat16 rounding steps of the unfused
// sequence (products, sums and the normalised value are rounded to bfloat16
// before the division by the scale), so the codes are those of the unfused
// graph up to the last-bit behaviour of expf / rsqrtf.

#include "fp8_cast.cuh"

namespace vq {
namespace {

// ---- RMSNorm + cast: one CTA per row ------------------------------------------
// y = bf16(x * rsqrt(mean(x^2) + eps) * w) in fp32 as torch's rms_norm computes it.
// A thread keeps its VPT vectors of the row in registers between the two phases.
template <int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_quantize_kernel(const uint4* __restrict__ x, const uint4* __restrict__ weight, uint2* __restrict__ out,
                        int cols, float eps, const void* __restrict__ scale, int scale_dt) {
  __shared__ float warp_sums[8];
  const int64_t row = blockIdx.x;
  const int vecs = cols >> 3;
  const Divisor d = make_divisor(scale, scale_dt);
  // the row's vectors and the weights they meet are all requested before the first is used
  uint4 raw[VPT], wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + blockDim.x * i;
    raw[i] = make_uint4(0, 0, 0, 0);
    wv[i] = make_uint4(0, 0, 0, 0);
    if (v < vecs) {
      raw[i] = __ldg(x + row * vecs + v);
      wv[i] = __ldg(weight + v);
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = lo_of(w[j]), b = hi_of(w[j]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_sums[w];   // same order in every thread
  const float inv = rsqrtf(total / (float)cols + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + blockDim.x * i;
    if (v >= vecs) continue;
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    const uint32_t g[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = bf16r(lo_of(w[j]) * inv * lo_of(g[j]));
      const float b = bf16r(hi_of(w[j]) * inv * hi_of(g[j]));
      o[j >> 1] |= fp8_pair<true>(quot(a, d), quot(b, d)) << (16 * (j & 1));
    }
    out[row * vecs + v] = make_uint2(o[0], o[1]);
  }
}

// ---- SiLU(gate) * up + cast ---------------------------------------------------
// gate / up: [rows, cols] with row strides ld_gate / ld_up (in 8-element vectors here).
__global__ void __launch_bounds__(256, 4)
silu_mul_quantize_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint2* __restrict__ out,
                         int64_t nvec, int vecs_per_row, int64_t ld_gate, int64_t ld_up,
                         const void* __restrict__ scale, int scale_dt) {
  const Divisor d = make_divisor(scale, scale_dt);
  // (row, column) of this thread's vector, advanced by the grid stride without further divisions
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t r = first / vecs_per_row;
  int c = (int)(first - r * vecs_per_row);
  const int64_t dr = stride / vecs_per_row;
  const int dc = (int)(stride - dr * vecs_per_row);
  for (int64_t v = first; v < nvec; v += stride) {
    const int64_t gi = r * ld_gate + c, ui = r * ld_up + c;
    r += dr;
    c += dc;
    if (c >= vecs_per_row) { c -= vecs_per_row; ++r; }
    const uint4 gv = __ldg(gate + gi), uv = __ldg(up + ui);
    const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t u[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g0 = lo_of(g[j]), g1 = hi_of(g[j]);
      const float s0 = bf16r(__fdividef(g0, 1.0f + __expf(-g0)));
      const float s1 = bf16r(__fdividef(g1, 1.0f + __expf(-g1)));
      const float a = bf16r(__fmul_rn(s0, lo_of(u[j])));
      const float b = bf16r(__fmul_rn(s1, hi_of(u[j])));
      o[j >> 1] |= fp8_pair<true>(quot(a, d), quot(b, d)) << (16 * (j & 1));
    }
    out[v] = make_uint2(o[0], o[1]);
  }
}

// ---- rotary embedding + cast + head/token layout change ----------------------
// Element (t, h, j) is read at x[t * in_t + h * in_h + j] and its byte written at
// out[t * out_t + h * out_h + j]; cos/sin: [T, d] bf16 or absent (no rotation).
// y = bf16(bf16(x * cos) + bf16(rot(x) * sin)), rot(x) = (-x[d/2:], x[:d/2]).
// `block` of `blocks`: the caller's share of the grid (a kernel that does several jobs gives each a range of its blocks).
__device__ __forceinline__ void rope_quantize_body(const uint4* __restrict__ x, const uint4* __restrict__ cosv,
                                                   const uint4* __restrict__ sinv, uint2* __restrict__ out, int T,
                                                   int heads, int d, int64_t in_t, int64_t in_h, int64_t out_t,
                                                   int64_t out_h, int apply_rope, const void* __restrict__ scale,
                                                   int scale_dt, int block, int blocks) {
  const Divisor dv = make_divisor(scale, scale_dt);
  const int vpd = d >> 3;          // 8-element vectors per head row; strides are in vectors here
  const int half = vpd >> 1;
  const int64_t total = (int64_t)T * heads * vpd;
  // vpd a power of two (head_dim 64, 128, ...): the vector within the head row is a mask of the
  // thread index and one 32-bit division splits the head row's index into (t, h)
  const bool pow2 = (vpd & (vpd - 1)) == 0 && (int64_t)T * heads < (1ll << 31);
  const int vshift = 31 - __clz(vpd);
  for (int64_t idx = (int64_t)block * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)blocks * blockDim.x) {
    int v, h, t;
    if (pow2) {
      v = (int)(idx & (vpd - 1));
      const uint32_t r = (uint32_t)(idx >> vshift);
      t = (int)(r / (uint32_t)heads);
      h = (int)(r - (uint32_t)t * (uint32_t)heads);
    } else {
      v = (int)(idx % vpd);
      h = (int)((idx / vpd) % heads);
      t = (int)(idx / ((int64_t)vpd * heads));
    }
    const uint4* row = x + t * in_t + h * in_h;
    const uint4 xv = __ldg(row + v);
    uint32_t o[2] = {0, 0};
    const uint32_t a[4] = {xv.x, xv.y, xv.z, xv.w};
    if (apply_rope) {
      const uint4 pvv = __ldg(row + (v < half ? v + half : v - half));   // partner in the other half
      const uint4 cv = __ldg(cosv + (int64_t)t * vpd + v), sv = __ldg(sinv + (int64_t)t * vpd + v);
      const uint32_t p[4] = {pvv.x, pvv.y, pvv.z, pvv.w};
      const uint32_t c[4] = {cv.x, cv.y, cv.z, cv.w};
      const uint32_t s[4] = {sv.x, sv.y, sv.z, sv.w};
      const float sign = v < half ? -1.0f : 1.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y0 = bf16r(__fadd_rn(bf16r(__fmul_rn(lo_of(a[j]), lo_of(c[j]))),
                                         bf16r(__fmul_rn(sign * lo_of(p[j]), lo_of(s[j])))));
        const float y1 = bf16r(__fadd_rn(bf16r(__fmul_rn(hi_of(a[j]), hi_of(c[j]))),
                                         bf16r(__fmul_rn(sign * hi_of(p[j]), hi_of(s[j])))));
        o[j >> 1] |= fp8_pair<true>(quot(y0, dv), quot(y1, dv)) << (16 * (j & 1));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j >> 1] |= fp8_pair<true>(quot(lo_of(a[j]), dv), quot(hi_of(a[j]), dv)) << (16 * (j & 1));
    }
    out[t * out_t + h * out_h + v] = make_uint2(o[0], o[1]);
  }
}
__global__ void __launch_bounds__(256)
rope_quantize_kernel(const uint4* __restrict__ x, const uint4* __restrict__ cosv, const uint4* __restrict__ sinv,
                     uint2* __restrict__ out, int T, int heads, int d, int64_t in_t, int64_t in_h, int64_t out_t,
                     int64_t out_h, int apply_rope, const void* __restrict__ scale, int scale_dt) {
  rope_quantize_body(x, cosv, sinv, out, T, heads, d, in_t, in_h, out_t, out_h, apply_rope, scale, scale_dt,
                     (int)blockIdx.x, (int)gridDim.x);
}

// ---- cast + transpose: x [T, heads, d] bf16 -> transposed fp8 [heads, d, T] ----
// Optionally also the codes in x's own layout and the bit pattern of max |x|
// (bfloat16 magnitudes order as their bit patterns do, NaN above all).
// (bx, by, bz): the 64-token tile, the 64-column tile and the head this block takes.
template <bool E4M3>
__device__ __forceinline__ void transpose_quantize_body(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out,
                                                        uint8_t* __restrict__ codes, int* __restrict__ amax_bits, int T,
                                                        int heads, int d, int64_t ldx, const void* __restrict__ scale,
                                                        int scale_dt, int bx, int by, int bz) {
  __shared__ __align__(16) uint8_t tile[64][64 + 4];
  __shared__ int block_max;
  const Divisor dv = make_divisor(scale, scale_dt);
  const int h = bz;
  const int t0 = bx * 64, j0 = by * 64;
  if (threadIdx.x == 0) block_max = 0;
  int local_max = 0;
  const uint16_t* xs = reinterpret_cast<const uint16_t*>(x);
  if ((d & 7) == 0 && (ldx & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // eight elements of a token per thread: one 16-byte load, eight codes
    for (int i = threadIdx.x; i < 64 * 8; i += blockDim.x) {
      const int tt = i >> 3, jv = (i & 7) << 3;
      if (t0 + tt >= T || j0 + jv >= d) continue;   // d % 8 == 0: a vector is inside or outside as a whole
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xs + (int64_t)(t0 + tt) * ldx + (int64_t)h * d + j0 + jv));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t packed[2] = {0, 0};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        local_max = max(local_max, max((int)(w[e] & 0x7FFFu), (int)((w[e] >> 16) & 0x7FFFu)));
        const uint32_t pair = fp8_pair<E4M3>(quot(lo_of(w[e]), dv), quot(hi_of(w[e]), dv));
        tile[jv + 2 * e][tt] = (uint8_t)(pair & 0xFFu);
        tile[jv + 2 * e + 1][tt] = (uint8_t)(pair >> 8);
        packed[e >> 1] |= pair << (16 * (e & 1));
      }
      if (codes != nullptr)
        *reinterpret_cast<uint2*>(codes + ((int64_t)(t0 + tt) * heads + h) * d + j0 + jv) = make_uint2(packed[0], packed[1]);
    }
  } else {
    for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
      const int tt = i >> 6, jj = i & 63;
      uint32_t q = 0;
      if (t0 + tt < T && j0 + jj < d) {
        const int64_t at = ((int64_t)(t0 + tt) * heads + h) * d + j0 + jj;          // dense position
        const uint16_t raw = xs[(int64_t)(t0 + tt) * ldx + (int64_t)h * d + j0 + jj];
        local_max = max(local_max, (int)(raw & 0x7FFFu));
        q = fp8_pair<E4M3>(quot(__uint_as_float((uint32_t)raw << 16), dv), 0.0f) & 0xFFu;
        if (codes != nullptr) codes[at] = (uint8_t)q;
      }
      tile[jj][tt] = (uint8_t)q;
    }
  }
  __syncthreads();
  if (amax_bits != nullptr) {
    for (int off = 16; off; off >>= 1) local_max = max(local_max, __shfl_xor_sync(0xFFFFFFFFu, local_max, off));
    if ((threadIdx.x & 31) == 0) atomicMax(&block_max, local_max);
  }
  const bool wide = (T & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0;
  if (wide) {
    for (int i = threadIdx.x; i < 64 * 16; i += blockDim.x) {
      const int jj = i >> 4, tq = (i & 15) << 2;
      if (t0 + tq < T && j0 + jj < d)   // T % 4 == 0: a group of four is inside or outside as a whole
        *reinterpret_cast<uint32_t*>(out + ((int64_t)h * d + j0 + jj) * T + t0 + tq) =
            *reinterpret_cast<const uint32_t*>(&tile[jj][tq]);
    }
  } else {
    for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
      const int jj = i >> 6, tt = i & 63;
      if (t0 + tt < T && j0 + jj < d) out[((int64_t)h * d + j0 + jj) * T + t0 + tt] = tile[jj][tt];
    }
  }
  if (amax_bits != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(amax_bits, block_max);
  }
}
template <bool E4M3>
__global__ void __launch_bounds__(256)
transpose_quantize_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, uint8_t* __restrict__ codes,
                          int* __restrict__ amax_bits, int T, int heads, int d, int64_t ldx,
                          const void* __restrict__ scale, int scale_dt) {
  transpose_quantize_body<E4M3>(x, out, codes, amax_bits, T, heads, d, ldx, scale, scale_dt, (int)blockIdx.x,
                                (int)blockIdx.y, (int)blockIdx.z);
}

// The three casts between the merged q/k/v projection and the attention kernel as one launch: RoPE + cast of the
// query heads and of the key heads (head-major outputs), cast + transpose of the value heads.  Blocks
// [0, q_blocks) take the queries, the next k_blocks the keys, the rest one value tile each.
struct QkvPostParams {
  const uint4 *q, *k, *cosv, *sinv;
  const __nv_bfloat16* v;
  uint2 *q_out, *k_out;
  uint8_t* vt_out;
  int T, q_heads, kv_heads, d;
  int64_t ld;               // elements between consecutive tokens of q, k and v (slices of one [T, *] matrix)
  const void *q_scale, *k_scale, *v_scale;
  int q_scale_dt, k_scale_dt, v_scale_dt;
  int q_blocks, k_blocks, v_tiles_t, v_tiles_d;
};
__global__ void __launch_bounds__(256)
qkv_post_kernel(const QkvPostParams p) {
  const int b = (int)blockIdx.x;
  const int vpd = p.d >> 3;
  if (b < p.q_blocks) {
    rope_quantize_body(p.q, p.cosv, p.sinv, p.q_out, p.T, p.q_heads, p.d, p.ld / 8, vpd, vpd, (int64_t)p.T * vpd, 1,
                       p.q_scale, p.q_scale_dt, b, p.q_blocks);
  } else if (b < p.q_blocks + p.k_blocks) {
    rope_quantize_body(p.k, p.cosv, p.sinv, p.k_out, p.T, p.kv_heads, p.d, p.ld / 8, vpd, vpd, (int64_t)p.T * vpd, 1,
                       p.k_scale, p.k_scale_dt, b - p.q_blocks, p.k_blocks);
  } else {
    const int i = b - p.q_blocks - p.k_blocks;
    const int per_head = p.v_tiles_t * p.v_tiles_d;
    const int h = i / per_head, rem = i - h * per_head;
    transpose_quantize_body<true>(p.v, p.vt_out, nullptr, nullptr, p.T, p.kv_heads, p.d, p.ld, p.v_scale, p.v_scale_dt,
                                  rem % p.v_tiles_t, rem / p.v_tiles_t, h);
  }
}

// out = bf16(bf16(silu(gate)) * up) in bfloat16, and max |out| over the whole tensor (atomicMax on the float bits of
// a zero-initialised word): the SwiGLU nodes of a graph whose next node needs a tensor-wide amax (an NVFP4 cast).
__global__ void __launch_bounds__(256, 4)
silu_mul_amax_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out,
                     int64_t nvec, int vecs_per_row, int64_t ld_gate, int64_t ld_up, uint32_t* __restrict__ amax_bits) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t r = first / vecs_per_row;
  int c = (int)(first - r * vecs_per_row);
  const int64_t dr = stride / vecs_per_row;
  const int dc = (int)(stride - dr * vecs_per_row);
  uint32_t m = 0;
  for (int64_t v = first; v < nvec; v += stride) {
    const int64_t gi = r * ld_gate + c, ui = r * ld_up + c;
    r += dr;
    c += dc;
    if (c >= vecs_per_row) { c -= vecs_per_row; ++r; }
    const uint4 gv = __ldg(gate + gi), uv = __ldg(up + ui);
    const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t u[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g0 = lo_of(g[j]), g1 = hi_of(g[j]);
      const float s0 = bf16r(__fdividef(g0, 1.0f + __expf(-g0)));
      const float s1 = bf16r(__fdividef(g1, 1.0f + __expf(-g1)));
      const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(s0, lo_of(u[j])), __fmul_rn(s1, hi_of(u[j])));
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
      m = max(m, max((o[j] << 16) & 0x7FFFFFFFu, o[j] & 0x7FFF0000u));
    }
    out[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int off = 16; off; off >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  __shared__ uint32_t warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = max(m, warp_max[w]);
    atomicMax(amax_bits, m);   // non-negative float bits order like unsigned integers
  }
}

// Rotary embedding of x [T, heads, d] (strided: a slice of a merged projection's output) written head-major,
// out[h * out_h + t * out_t + j], in bfloat16: y = bf16(bf16(x * cos) + bf16(rot(x) * sin)), the graph's
// elementwise nodes with their roundings, and the layout the attention kernel reads.  Strides in 8-element vectors.
__global__ void __launch_bounds__(256)
rope_heads_kernel(const uint4* __restrict__ x, const uint4* __restrict__ cosv, const uint4* __restrict__ sinv,
                  uint4* __restrict__ out, int T, int heads, int d, int64_t in_t, int64_t in_h, int64_t out_t,
                  int64_t out_h) {
  const int vpd = d >> 3, half = vpd >> 1;
  const int64_t total = (int64_t)T * heads * vpd;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vpd);
    const int h = (int)((idx / vpd) % heads);
    const int t = (int)(idx / ((int64_t)vpd * heads));
    const uint4* row = x + t * in_t + h * in_h;
    const uint4 xv = __ldg(row + v);
    const uint4 pvv = __ldg(row + (v < half ? v + half : v - half));
    const uint4 cv = __ldg(cosv + (int64_t)t * vpd + v), sv = __ldg(sinv + (int64_t)t * vpd + v);
    const uint32_t a[4] = {xv.x, xv.y, xv.z, xv.w}, p[4] = {pvv.x, pvv.y, pvv.z, pvv.w};
    const uint32_t c[4] = {cv.x, cv.y, cv.z, cv.w}, s[4] = {sv.x, sv.y, sv.z, sv.w};
    const float sign = v < half ? -1.0f : 1.0f;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = __fadd_rn(bf16r(__fmul_rn(lo_of(a[j]), lo_of(c[j]))), bf16r(__fmul_rn(sign * lo_of(p[j]), lo_of(s[j]))));
      const float y1 = __fadd_rn(bf16r(__fmul_rn(hi_of(a[j]), hi_of(c[j]))), bf16r(__fmul_rn(sign * hi_of(p[j]), hi_of(s[j]))));
      const __nv_bfloat162 hh = __floats2bfloat162_rn(y0, y1);
      o[j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    out[h * out_h + t * out_t + v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// One decode step's RoPE and cache append.  qkv: [B, (hq + 2 hkv) * d] bfloat16, the merged projection's
// output.  Query head h goes, rotated, to q_out[b, h, :]; key head h, rotated, to k_dst + (b * hkv + h) *
// kv_stride; value head h, as it is, to v_dst + (b * hkv + h) * kv_stride (the slot of this step's
// position in a [B, hkv, R, d] window: kv_stride = R * d).  cos / sin: [d] (cs_stride = 0) or one row per
// sequence.  y = bf16(bf16(x * cos) + bf16(rot(x) * sin)), rot(x) = (-x[d/2:], x[:d/2]): the graph's
// four elementwise nodes with their roundings.  One thread per 8 elements.
__global__ void __launch_bounds__(256)
rope_decode_append_kernel(const uint4* __restrict__ qkv, const uint4* __restrict__ cosv, const uint4* __restrict__ sinv,
                          uint4* __restrict__ q_out, uint4* __restrict__ k_dst, uint4* __restrict__ v_dst, int B, int hq,
                          int hkv, int d, int64_t kv_stride, int64_t cs_stride) {
  const int vpd = d >> 3, half = vpd >> 1;
  const int heads = hq + 2 * hkv;
  const int64_t total = (int64_t)B * heads * vpd;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vpd);
    const int h = (int)((idx / vpd) % heads);
    const int b = (int)(idx / ((int64_t)vpd * heads));
    const uint4* row = qkv + ((int64_t)b * heads + h) * vpd;
    const uint4 xv = __ldg(row + v);
    if (h >= hq + hkv) {   // a value head: appended unrotated
      v_dst[((int64_t)b * hkv + (h - hq - hkv)) * kv_stride + v] = xv;
      continue;
    }
    const uint4 pvv = __ldg(row + (v < half ? v + half : v - half));
    const uint4 cv = __ldg(cosv + b * cs_stride + v), sv = __ldg(sinv + b * cs_stride + v);
    const uint32_t a[4] = {xv.x, xv.y, xv.z, xv.w}, p[4] = {pvv.x, pvv.y, pvv.z, pvv.w};
    const uint32_t c[4] = {cv.x, cv.y, cv.z, cv.w}, s[4] = {sv.x, sv.y, sv.z, sv.w};
    const float sign = v < half ? -1.0f : 1.0f;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = __fadd_rn(bf16r(__fmul_rn(lo_of(a[j]), lo_of(c[j]))), bf16r(__fmul_rn(sign * lo_of(p[j]), lo_of(s[j]))));
      const float y1 = __fadd_rn(bf16r(__fmul_rn(hi_of(a[j]), hi_of(c[j]))), bf16r(__fmul_rn(sign * hi_of(p[j]), hi_of(s[j]))));
      const __nv_bfloat162 hh = __floats2bfloat162_rn(y0, y1);
      o[j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
    if (h < hq) q_out[((int64_t)b * hq + h) * vpd + v] = ov;
    else k_dst[((int64_t)b * hkv + (h - hq)) * kv_stride + v] = ov;
  }
}

// out = bf16(dequantize(quantize(x)) + y): the value x keeps after a per-tensor e4m3 cast,
//   q = e4m3(bf16(x / s)) (saturating), d = bf16(q * s),
// added to y (or alone when y is null).  Eight elements per thread.
__device__ __forceinline__ float e4m3_byte_to_float(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__global__ void __launch_bounds__(256)
fp8_roundtrip_add_kernel(const uint4* __restrict__ x, const uint4* __restrict__ y, uint4* __restrict__ out, int64_t nvec,
                         const void* __restrict__ scale, int scale_dt) {
  const Divisor dv = make_divisor(scale, scale_dt);
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    const uint4 xv = __ldg(x + v);
    uint4 yv = make_uint4(0, 0, 0, 0);
    if (y != nullptr) yv = __ldg(y + v);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
    uint32_t ow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t codes = fp8_pair<true>(quot(lo_of(xw[j]), dv), quot(hi_of(xw[j]), dv));
      float d0 = bf16r(__fmul_rn(e4m3_byte_to_float(codes & 0xFFu), dv.s));
      float d1 = bf16r(__fmul_rn(e4m3_byte_to_float((codes >> 8) & 0xFFu), dv.s));
      if (y != nullptr) {
        d0 = __fadd_rn(d0, lo_of(yw[j]));
        d1 = __fadd_rn(d1, hi_of(yw[j]));
      }
      const __nv_bfloat162 h = __floats2bfloat162_rn(d0, d1);
      ow[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    out[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

inline int stream_grid(int64_t items, int threads, int per_sm) {
  int64_t blocks = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)kSmCount * per_sm;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_rmsnorm_quantize_fp8(const void* x, const void* weight, void* out, int64_t rows, int64_t cols,
                                       float eps, const void* scale, int scale_dtype, void* stream) {
  VQ_REQUIRE(rows >= 0 && cols > 0, "vq_rmsnorm_quantize_fp8: bad extent");
  if (rows == 0) return VQ_OK;
  VQ_REQUIRE(x && weight && out && scale, "vq_rmsnorm_quantize_fp8: null argument");
  VQ_REQUIRE(cols % 8 == 0 && cols <= 32 * 8 * 32, "vq_rmsnorm_quantize_fp8: the row length must be a multiple of 8, at most 8192");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(out) & 7) == 0, "vq_rmsnorm_quantize_fp8: misaligned buffers");
  const int vecs = (int)(cols / 8);
  // four vectors per thread where the row allows: small CTAs, so that a few thousand rows are
  // resident at once instead of queueing behind one another
  int threads = ((((vecs + 3) / 4) + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  const int vpt = (vecs + threads - 1) / threads;   // <= 4 for cols <= 8192
  const unsigned grid = (unsigned)rows;
  VQ_REQUIRE(rows < (1ll << 31), "vq_rmsnorm_quantize_fp8: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint4* xi = static_cast<const uint4*>(x);
  const uint4* wi = static_cast<const uint4*>(weight);
  uint2* o = static_cast<uint2*>(out);
  switch (vpt) {
    case 1: rmsnorm_quantize_kernel<1><<<grid, threads, 0, st>>>(xi, wi, o, (int)cols, eps, scale, scale_dtype); break;
    case 2: rmsnorm_quantize_kernel<2><<<grid, threads, 0, st>>>(xi, wi, o, (int)cols, eps, scale, scale_dtype); break;
    default: rmsnorm_quantize_kernel<4><<<grid, threads, 0, st>>>(xi, wi, o, (int)cols, eps, scale, scale_dtype); break;
  }
  return check_launch("rmsnorm_quantize_kernel");
}

extern "C" int vq_silu_mul_quantize_fp8(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                                        int64_t ld_gate, int64_t ld_up, const void* scale, int scale_dtype,
                                        void* stream) {
  VQ_REQUIRE(rows >= 0 && cols >= 0, "vq_silu_mul_quantize_fp8: negative size");
  if (rows == 0 || cols == 0) return VQ_OK;
  VQ_REQUIRE(gate && up && out && scale, "vq_silu_mul_quantize_fp8: null argument");
  VQ_REQUIRE(cols % 8 == 0 && ld_gate % 8 == 0 && ld_up % 8 == 0 && ld_gate >= cols && ld_up >= cols,
             "vq_silu_mul_quantize_fp8: the row length and strides must be multiples of 8, strides at least a row");
  VQ_REQUIRE(cols < (1ll << 31), "vq_silu_mul_quantize_fp8: row too long");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(out) & 7) == 0, "vq_silu_mul_quantize_fp8: misaligned buffers");
  const int64_t nvec = rows * (cols / 8);
  silu_mul_quantize_kernel<<<stream_grid(nvec, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint2*>(out), nvec, (int)(cols / 8),
      ld_gate / 8, ld_up / 8, scale, scale_dtype);
  return check_launch("silu_mul_quantize_kernel");
}

extern "C" int vq_silu_mul_amax(const void* gate, const void* up, void* out, void* amax, int64_t rows, int64_t cols,
                                int64_t ld_gate, int64_t ld_up, void* stream) {
  VQ_REQUIRE(rows >= 0 && cols >= 0, "vq_silu_mul_amax: negative size");
  if (rows == 0 || cols == 0) return VQ_OK;
  VQ_REQUIRE(gate && up && out && amax, "vq_silu_mul_amax: null argument");
  VQ_REQUIRE(cols % 8 == 0 && ld_gate % 8 == 0 && ld_up % 8 == 0 && ld_gate >= cols && ld_up >= cols,
             "vq_silu_mul_amax: the row length and strides must be multiples of 8, strides at least a row");
  VQ_REQUIRE(cols < (1ll << 31), "vq_silu_mul_amax: row too long");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(amax) & 3) == 0, "vq_silu_mul_amax: misaligned buffers");
  const int64_t nvec = rows * (cols / 8);
  silu_mul_amax_kernel<<<stream_grid(nvec, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(out), nvec, (int)(cols / 8),
      ld_gate / 8, ld_up / 8, static_cast<uint32_t*>(amax));
  return check_launch("silu_mul_amax_kernel");
}

extern "C" int vq_rope_heads_bf16(const void* x, const void* cosv, const void* sinv, void* out, int64_t T, int64_t heads,
                                  int64_t d, int64_t in_stride_t, int64_t in_stride_h, int64_t out_stride_t,
                                  int64_t out_stride_h, void* stream) {
  VQ_REQUIRE(T >= 0 && heads >= 0 && d > 0, "vq_rope_heads_bf16: bad extent");
  if (T == 0 || heads == 0) return VQ_OK;
  VQ_REQUIRE(x && cosv && sinv && out, "vq_rope_heads_bf16: null argument");
  VQ_REQUIRE(d % 16 == 0, "vq_rope_heads_bf16: head_dim must be a multiple of 16");
  VQ_REQUIRE(((in_stride_t | in_stride_h | out_stride_t | out_stride_h) & 7) == 0 && in_stride_t >= 0 &&
             in_stride_h >= 0 && out_stride_t >= 0 && out_stride_h >= 0,
             "vq_rope_heads_bf16: strides must be non-negative multiples of 8 elements");
  VQ_REQUIRE(T < (1ll << 31) && heads < (1 << 20) && d < (1 << 20), "vq_rope_heads_bf16: extent too large");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(cosv) |
               reinterpret_cast<uintptr_t>(sinv)) & 15) == 0, "vq_rope_heads_bf16: misaligned buffers");
  rope_heads_kernel<<<stream_grid(T * heads * (d / 8), 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(cosv), static_cast<const uint4*>(sinv),
      static_cast<uint4*>(out), (int)T, (int)heads, (int)d, in_stride_t / 8, in_stride_h / 8, out_stride_t / 8,
      out_stride_h / 8);
  return check_launch("rope_heads_kernel");
}

extern "C" int vq_rope_decode_append(const void* qkv, const void* cosv, const void* sinv, void* q_out, void* k_dst,
                                     void* v_dst, int64_t B, int64_t q_heads, int64_t kv_heads, int64_t d,
                                     int64_t kv_stride, int64_t cs_stride, void* stream) {
  VQ_REQUIRE(B >= 0 && q_heads >= 0 && kv_heads >= 0 && d > 0, "vq_rope_decode_append: bad extent");
  if (B == 0 || q_heads + kv_heads == 0) return VQ_OK;
  VQ_REQUIRE(qkv && cosv && sinv && (q_heads == 0 || q_out) && (kv_heads == 0 || (k_dst && v_dst)),
             "vq_rope_decode_append: null argument");
  VQ_REQUIRE(d % 16 == 0 && d < (1 << 20), "vq_rope_decode_append: head_dim must be a multiple of 16");
  VQ_REQUIRE(kv_stride % 8 == 0 && kv_stride >= d && cs_stride % 8 == 0 && cs_stride >= 0,
             "vq_rope_decode_append: strides are multiples of 8 elements, the window's at least one head row");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv) |
               reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_dst) | reinterpret_cast<uintptr_t>(v_dst)) & 15) == 0,
             "vq_rope_decode_append: buffers must be 16-byte aligned");
  VQ_REQUIRE(B < (1ll << 31) && q_heads + 2 * kv_heads < (1 << 20), "vq_rope_decode_append: extent too large");
  const int64_t total = B * (q_heads + 2 * kv_heads) * (d / 8);
  rope_decode_append_kernel<<<stream_grid(total, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(qkv), static_cast<const uint4*>(cosv), static_cast<const uint4*>(sinv),
      static_cast<uint4*>(q_out), static_cast<uint4*>(k_dst), static_cast<uint4*>(v_dst), (int)B, (int)q_heads,
      (int)kv_heads, (int)d, kv_stride / 8, cs_stride / 8);
  return check_launch("rope_decode_append_kernel");
}

extern "C" int vq_fp8_roundtrip_add(const void* x, const void* y, void* out, int64_t n, const void* scale,
                                    int scale_dtype, void* stream) {
  VQ_REQUIRE(n >= 0, "vq_fp8_roundtrip_add: negative size");
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(x && out && scale, "vq_fp8_roundtrip_add: null argument");
  VQ_REQUIRE(scale_dtype >= VQ_BF16 && scale_dtype <= VQ_F32, "vq_fp8_roundtrip_add: bad scale dtype");
  VQ_REQUIRE(n % 8 == 0, "vq_fp8_roundtrip_add: the element count must be a multiple of 8");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
             "vq_fp8_roundtrip_add: buffers must be 16-byte aligned");
  const int64_t nvec = n / 8;
  fp8_roundtrip_add_kernel<<<stream_grid(nvec, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(y), static_cast<uint4*>(out), nvec, scale, scale_dtype);
  return check_launch("fp8_roundtrip_add_kernel");
}

extern "C" int vq_rope_quantize_fp8(const void* x, const void* cosv, const void* sinv, void* out, int64_t T,
                                    int64_t heads, int64_t d, int64_t in_stride_t, int64_t in_stride_h,
                                    int64_t out_stride_t, int64_t out_stride_h, const void* scale, int scale_dtype,
                                    void* stream) {
  VQ_REQUIRE(T >= 0 && heads >= 0 && d > 0, "vq_rope_quantize_fp8: bad extent");
  if (T == 0 || heads == 0) return VQ_OK;
  VQ_REQUIRE(x && out && scale, "vq_rope_quantize_fp8: null argument");
  VQ_REQUIRE((cosv == nullptr) == (sinv == nullptr), "vq_rope_quantize_fp8: cos and sin come together");
  VQ_REQUIRE(d % 16 == 0, "vq_rope_quantize_fp8: head_dim must be a multiple of 16");
  VQ_REQUIRE(((in_stride_t | in_stride_h | out_stride_t | out_stride_h) & 7) == 0 && in_stride_t >= 0 &&
             in_stride_h >= 0 && out_stride_t >= 0 && out_stride_h >= 0,
             "vq_rope_quantize_fp8: strides must be non-negative multiples of 8 elements");
  VQ_REQUIRE(T < (1ll << 31) && heads < 65536 && d < 65536, "vq_rope_quantize_fp8: extent too large");
  VQ_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
             ((reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv)) & 15) == 0,
             "vq_rope_quantize_fp8: misaligned buffers");
  rope_quantize_kernel<<<stream_grid(T * heads * (d / 8), 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(cosv), static_cast<const uint4*>(sinv),
      static_cast<uint2*>(out), (int)T, (int)heads, (int)d, in_stride_t / 8, in_stride_h / 8, out_stride_t / 8,
      out_stride_h / 8, cosv != nullptr, scale, scale_dtype);
  return check_launch("rope_quantize_kernel");
}

extern "C" int vq_qkv_post_fp8(const void* q, const void* k, const void* v, int64_t ld, const void* cosv, const void* sinv,
                               void* q_out, void* k_out, void* vt_out, int64_t T, int64_t q_heads, int64_t kv_heads,
                               int64_t d, const void* q_scale, int q_scale_dtype, const void* k_scale,
                               int k_scale_dtype, const void* v_scale, int v_scale_dtype, void* stream) {
  VQ_REQUIRE(T >= 0 && q_heads >= 0 && kv_heads >= 0 && d >= 0, "vq_qkv_post_fp8: bad extent");
  if (T == 0 || d == 0 || (q_heads == 0 && kv_heads == 0)) return VQ_OK;
  VQ_REQUIRE(q && k && v && cosv && sinv && q_out && k_out && vt_out && q_scale && k_scale && v_scale,
             "vq_qkv_post_fp8: null argument");
  VQ_REQUIRE(d % 16 == 0 && ld % 8 == 0 && ld >= d, "vq_qkv_post_fp8: head_dim must be a multiple of 16, the token stride of 8");
  VQ_REQUIRE(T < (1ll << 31) && q_heads < 65536 && kv_heads < 65536 && d < (1 << 22), "vq_qkv_post_fp8: extent too large");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
               reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv)) & 15) == 0 &&
                 ((reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_out)) & 7) == 0,
             "vq_qkv_post_fp8: misaligned buffers");
  QkvPostParams p{};
  p.q = static_cast<const uint4*>(q); p.k = static_cast<const uint4*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.cosv = static_cast<const uint4*>(cosv); p.sinv = static_cast<const uint4*>(sinv);
  p.q_out = static_cast<uint2*>(q_out); p.k_out = static_cast<uint2*>(k_out); p.vt_out = static_cast<uint8_t*>(vt_out);
  p.T = (int)T; p.q_heads = (int)q_heads; p.kv_heads = (int)kv_heads; p.d = (int)d; p.ld = ld;
  p.q_scale = q_scale; p.k_scale = k_scale; p.v_scale = v_scale;
  p.q_scale_dt = q_scale_dtype; p.k_scale_dt = k_scale_dtype; p.v_scale_dt = v_scale_dtype;
  // the rope jobs get blocks in proportion to their elements, about eight blocks per SM in all
  const int64_t q_items = T * q_heads * (d / 8), k_items = T * kv_heads * (d / 8);
  p.q_blocks = q_items > 0 ? stream_grid(q_items, 256, 6) : 0;
  p.k_blocks = k_items > 0 ? stream_grid(k_items, 256, 2) : 0;
  p.v_tiles_t = (int)((T + 63) / 64); p.v_tiles_d = (int)((d + 63) / 64);
  const int64_t v_blocks = (int64_t)p.v_tiles_t * p.v_tiles_d * kv_heads;
  VQ_REQUIRE(v_blocks < (1ll << 30), "vq_qkv_post_fp8: too many value tiles");
  qkv_post_kernel<<<(unsigned)(p.q_blocks + p.k_blocks + v_blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("qkv_post_kernel");
}

extern "C" int vq_transpose_quantize_fp8(const void* x, void* out, void* codes, void* amax_bits, int format, int64_t T,
                                         int64_t heads, int64_t d, int64_t ldx, const void* scale, int scale_dtype,
                                         void* stream) {
  VQ_REQUIRE(T >= 0 && heads >= 0 && d >= 0, "vq_transpose_quantize_fp8: bad extent");
  if (T == 0 || heads == 0 || d == 0) return VQ_OK;
  VQ_REQUIRE(x && out && scale, "vq_transpose_quantize_fp8: null argument");
  VQ_REQUIRE(format == VQ_IN_E4M3 || format == VQ_IN_E5M2, "vq_transpose_quantize_fp8: format must be e4m3 or e5m2");
  VQ_REQUIRE(T < (1ll << 31) && heads < 65536 && d < (1 << 22), "vq_transpose_quantize_fp8: extent too large");
  VQ_REQUIRE(ldx >= heads * d, "vq_transpose_quantize_fp8: row stride smaller than a row");
  dim3 grid((unsigned)((T + 63) / 64), (unsigned)((d + 63) / 64), (unsigned)heads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (format == VQ_IN_E4M3)
    transpose_quantize_kernel<true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(out),
                                                          static_cast<uint8_t*>(codes), static_cast<int*>(amax_bits),
                                                          (int)T, (int)heads, (int)d, ldx, scale, scale_dtype);
  else
    transpose_quantize_kernel<false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(out),
                                                           static_cast<uint8_t*>(codes), static_cast<int*>(amax_bits),
                                                           (int)T, (int)heads, (int)d, ldx, scale, scale_dtype);
  return check_launch("transpose_quantize_kernel");
}
