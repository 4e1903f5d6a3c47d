// One decode step's attention straight from a packed KIVI cache.
//
// For every (sequence, KV head) the graph of a decode step runs, on bfloat16 tensors,
//
//   k_main = dequantize(k_codes, k_scale, k_zero)        keys   [Tm, 128], groups of `k_block` positions per channel
//   v_main = dequantize(v_codes, v_scale, v_zero)        values [Tm, 128], groups of `v_block` channels per position
//   scores = cat(matmul(q, k_main^T), matmul(q, k_res^T))           q: the KV group's G query heads, [G, 128]
//   p      = softmax_fp32(scores * score_scale) -> bfloat16
//   out    = matmul(p[:, :Tm], v_main) + matmul(p[:, Tm:], v_res)
//
// (quantized_ops::dequantize, ops/quantized.py:527-571, as emitted for the KIVI cache by
// codegen/transform/quant_folding.py:2391-2547, then the eager attention nodes), every node's
// output rounded to bfloat16.  Here one CTA owns one (sequence, KV head): it streams the 2-bit codes
// and their parameters through shared memory with cp.async (two 1024-position chunks in flight),
// decodes them in registers into mma.sync.m16n8k16 operand fragments with two packed bfloat16
// instructions per pair of values -- bf16(bf16(code - zero) * scale), the operator's own two
// roundings -- and keeps the scores and probabilities of its G rows in shared memory, so the
// dequantized cache (8 x the packed bytes) is never written or read.  G <= 8 query rows fill the
// top half of the 16-row MMA tile; the tensor-core work is negligible, the kernel is bound by the
// packed bytes and their latency.
//
// Fragment layouts (lane = 4 g + t): A a0 = rows g, columns 2t, 2t+1; a2 = columns 2t+8, 2t+9 (a1, a3 are
// rows g + 8: zero); B b0 = k 2t, 2t+1 of column g, b1 = k 2t+8, 2t+9; C c0, c1 = row g, columns 2t, 2t+1.
#include <cuda_bf16.h>

#include "vq_common.cuh"

namespace vq {
namespace {

constexpr int KA_D = 128;                  // head_dim
constexpr int KA_ROW = KA_D / 4;           // packed bytes per position
constexpr int KA_THREADS = 512;
constexpr int KA_WARPS = KA_THREADS / 32;
constexpr int KA_WKEYS = 64;               // positions a warp takes from a chunk
constexpr int KA_CHUNK = KA_WARPS * KA_WKEYS;   // 1024 positions per chunk
// A stage buffer: the chunk's packed rows, then its parameters -- keys: one 512-byte row (128 scales, 128 zero
// points) per 64 positions; values: NGRP scales per position, then NGRP zero points per position.
__host__ __device__ constexpr int ka_stage_bytes(int ngrp) {
  return KA_CHUNK * KA_ROW + (KA_CHUNK * ngrp * 4 > KA_CHUNK * 8 ? KA_CHUNK * ngrp * 4 : KA_CHUNK * 8);
}
constexpr int KA_RES_LD = KA_D + 8;        // padded row of the staged recent values (bank spread)
constexpr int KA_MAX_G = 8;

struct KaParams {
  const __nv_bfloat16* q;        // [outer, G, 128]
  const uint8_t* k_packed;       // [outer, Tm, 32]
  const __nv_bfloat16* k_scale;  // [outer, Tm / k_block, 128]
  const __nv_bfloat16* k_zero;
  const uint8_t* v_packed;       // [outer, Tm, 32]
  const __nv_bfloat16* v_scale;  // [outer, Tm, 128 / v_block]
  const __nv_bfloat16* v_zero;
  const __nv_bfloat16* k_res;    // [outer, R, 128]
  const __nv_bfloat16* v_res;
  __nv_bfloat16* out;            // [outer, G, 128]
  int G, Tm, R, k_block;
  float score_scale;
};

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t mul_bf16x2_(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// NGRP = 128 / v_block value groups per position (1, 2 or 4).
template <int NGRP>
__global__ void __launch_bounds__(KA_THREADS, 1)
kivi_decode_attention_kernel(const KaParams p) {
  extern __shared__ __align__(16) uint8_t ka_smem[];
  const int N = p.Tm + p.R;                                   // keys per row
  float* scores = reinterpret_cast<float*>(ka_smem);                                  // [G][N]
  __nv_bfloat16* probs = reinterpret_cast<__nv_bfloat16*>(scores + (size_t)p.G * N);   // [G][N]
  constexpr int KA_STAGE_BYTES = ka_stage_bytes(NGRP);
  uint8_t* stage = reinterpret_cast<uint8_t*>(probs + (size_t)p.G * N);               // [2][KA_STAGE_BYTES]; N is a multiple of 8
  float* red = reinterpret_cast<float*>(stage + 2 * KA_STAGE_BYTES);                  // [KA_WARPS][G][128]
  float* row_stat = red + KA_WARPS * p.G * KA_D;                                      // [KA_WARPS]
  float* main_out = row_stat + KA_WARPS;                                              // [KA_MAX_G][128]
  uint32_t* lut = reinterpret_cast<uint32_t*>(main_out + KA_MAX_G * KA_D);            // [16] bf16x2 of a pair of codes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t outer = blockIdx.x;
  const int n_chunks = (p.Tm + KA_CHUNK - 1) / KA_CHUNK;
  const bool row_live = g < p.G;

  if (threadIdx.x < 16) {
    const float c0 = (float)(threadIdx.x & 3), c1 = (float)(threadIdx.x >> 2);
    lut[threadIdx.x] = pack_bf16x2(c0, c1);
  }

  // ---- the query rows as A fragments, one pair of registers per 16 channels ----
  uint32_t qa[8][2];
  {
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(p.q + (outer * p.G + (row_live ? g : 0)) * KA_D);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      qa[k][0] = row_live ? __ldg(qrow + 8 * k + t) : 0u;
      qa[k][1] = row_live ? __ldg(qrow + 8 * k + t + 4) : 0u;
    }
  }

  // Chunk c of a packed tensor and its parameters into stage buffer b.  Keys: groups of k_block positions
  // (a multiple of 64): 128 scales + 128 zero points per group; values: NGRP of each per position.
  auto issue = [&](bool keys, int c, int b) {
    const int key0 = c * KA_CHUNK;
    const int count = min(KA_CHUNK, p.Tm - key0);
    uint8_t* dst = stage + b * KA_STAGE_BYTES;
    const uint8_t* src = (keys ? p.k_packed : p.v_packed) + (outer * p.Tm + key0) * KA_ROW;
    for (int i = threadIdx.x; i < count * (KA_ROW / 16); i += KA_THREADS) cp_async16(dst + i * 16, src + i * 16);
    uint8_t* pdst = dst + KA_CHUNK * KA_ROW;
    if (keys) {
      // one parameter row per 64 positions of the chunk (repeated when a group spans several)
      const int rows = count / KA_WKEYS;
      for (int i = threadIdx.x; i < rows * 32; i += KA_THREADS) {
        const int r = i >> 5, part = i & 31;                       // 16 bytes each: 16 for scales, 16 for zero points
        const int64_t grp = outer * (p.Tm / p.k_block) + (key0 + r * KA_WKEYS) / p.k_block;
        const __nv_bfloat16* s = (part < 16 ? p.k_scale : p.k_zero) + grp * KA_D + (part & 15) * 8;
        cp_async16(pdst + r * 512 + part * 16, s);
      }
    } else {
      const int bytes = count * NGRP * 2;                          // per tensor; a multiple of 16 (count % 64 == 0)
      const __nv_bfloat16* s = p.v_scale + (outer * p.Tm + key0) * NGRP;
      const __nv_bfloat16* z = p.v_zero + (outer * p.Tm + key0) * NGRP;
      for (int i = threadIdx.x; i < bytes / 16; i += KA_THREADS) {
        cp_async16(pdst + i * 16, reinterpret_cast<const uint8_t*>(s) + i * 16);
        cp_async16(pdst + KA_CHUNK * NGRP * 2 + i * 16, reinterpret_cast<const uint8_t*>(z) + i * 16);
      }
    }
    cp_async_commit();
  };

  // =========================== phase 1: scores ===========================
  if (n_chunks > 0) issue(true, 0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) {
      issue(true, c + 1, (c + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = c * KA_CHUNK;
    const int count = min(KA_CHUNK, p.Tm - key0);
    if (warp * KA_WKEYS < count) {
      const uint8_t* buf = stage + (c & 1) * KA_STAGE_BYTES;
      const uint32_t* ps = reinterpret_cast<const uint32_t*>(buf + KA_CHUNK * KA_ROW + warp * 512);   // scales, then zero points
      uint32_t sc[16], zp[16];   // [2 k + h]: channels 16 k + 8 h + 2 t, +1
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          sc[2 * k + h] = ps[8 * k + 4 * h + t];
          zp[2 * k + h] = ps[64 + 8 * k + 4 * h + t];
        }
#pragma unroll 2
      for (int nb = 0; nb < KA_WKEYS / 8; ++nb) {
        const int kl = warp * KA_WKEYS + nb * 8;                    // first position of the block within the chunk
        const uint4* row = reinterpret_cast<const uint4*>(buf + (kl + g) * KA_ROW);
        const uint4 r0 = row[0], r1 = row[1];
        const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};   // word k: channels 16 k .. 16 k + 15
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t bits = w[k] >> (4 * t);
          const uint32_t b0 = mul_bf16x2_(sub_bf16x2(lut[bits & 15u], zp[2 * k]), sc[2 * k]);
          const uint32_t b1 = mul_bf16x2_(sub_bf16x2(lut[(bits >> 16) & 15u], zp[2 * k + 1]), sc[2 * k + 1]);
          mma_16816(acc, qa[k][0], qa[k][1], b0, b1);
        }
        if (row_live) {
          float2 s;
          s.x = bf16_round(bf16_round(acc[0]) * p.score_scale);
          s.y = bf16_round(bf16_round(acc[1]) * p.score_scale);
          *reinterpret_cast<float2*>(scores + (size_t)g * N + key0 + kl + 2 * t) = s;
        }
      }
    }
    __syncthreads();   // the buffer is refilled by the next iteration's issue
  }
  // the newest positions, kept in bfloat16
  for (int nb = warp; nb < p.R / 8; nb += KA_WARPS) {
    const uint32_t* row = reinterpret_cast<const uint32_t*>(p.k_res + (outer * p.R + nb * 8 + g) * KA_D);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint32_t b[16];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      b[2 * k] = __ldg(row + 8 * k + t);
      b[2 * k + 1] = __ldg(row + 8 * k + t + 4);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) mma_16816(acc, qa[k][0], qa[k][1], b[2 * k], b[2 * k + 1]);
    if (row_live) {
      float2 s;
      s.x = bf16_round(bf16_round(acc[0]) * p.score_scale);
      s.y = bf16_round(bf16_round(acc[1]) * p.score_scale);
      *reinterpret_cast<float2*>(scores + (size_t)g * N + p.Tm + nb * 8 + 2 * t) = s;
    }
  }
  // the first value chunk can start while the softmax runs
  if (n_chunks > 0) issue(false, 0, 0);
  __syncthreads();

  // =========================== softmax: p = bf16(exp(s - max) / sum) ===========================
  for (int r = 0; r < p.G; ++r) {
    const float* srow = scores + (size_t)r * N;
    float m = -INFINITY;
    for (int j = threadIdx.x; j < N; j += KA_THREADS) m = fmaxf(m, srow[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) row_stat[warp] = m;
    __syncthreads();
    m = row_stat[0];
#pragma unroll
    for (int w = 1; w < KA_WARPS; ++w) m = fmaxf(m, row_stat[w]);
    __syncthreads();
    float l = 0.0f;
    for (int j = threadIdx.x; j < N; j += KA_THREADS) l += __expf(srow[j] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o);
    if (lane == 0) row_stat[warp] = l;
    __syncthreads();
    l = 0.0f;
#pragma unroll
    for (int w = 0; w < KA_WARPS; ++w) l += row_stat[w];
    const float rl = __frcp_rn(l);
    __nv_bfloat16* prow = probs + (size_t)r * N;
    for (int j = threadIdx.x; j < N; j += KA_THREADS) prow[j] = __float2bfloat16_rn(__expf(srow[j] - m) * rl);
    __syncthreads();
  }

  // =========================== phase 2: out = P V ===========================
  float acc[16][4];
#pragma unroll
  for (int nb = 0; nb < 16; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nb][e] = 0.0f;

  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) {
      issue(false, c + 1, (c + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = c * KA_CHUNK;
    const int count = min(KA_CHUNK, p.Tm - key0);
    if (warp * KA_WKEYS < count) {
      const uint8_t* buf = stage + (c & 1) * KA_STAGE_BYTES;
      const uint16_t* vs = reinterpret_cast<const uint16_t*>(buf + KA_CHUNK * KA_ROW);
      const uint16_t* vz = reinterpret_cast<const uint16_t*>(buf + KA_CHUNK * KA_ROW + KA_CHUNK * NGRP * 2);
#pragma unroll 1
      for (int ks = 0; ks < KA_WKEYS / 16; ++ks) {
        const int kl = warp * KA_WKEYS + ks * 16;
        // A: probabilities of positions kl + 2t, +1 and kl + 2t + 8, +9
        const uint32_t* prow = reinterpret_cast<const uint32_t*>(probs + (size_t)(row_live ? g : 0) * N + key0 + kl);
        const uint32_t a0 = row_live ? prow[t] : 0u, a2 = row_live ? prow[t + 4] : 0u;
        // the packed rows of the four positions
        uint32_t w[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int pos = kl + 2 * t + (i & 1) + 8 * (i >> 1);
          const uint4* row = reinterpret_cast<const uint4*>(buf + pos * KA_ROW);
          const uint4 r0 = row[0], r1 = row[1];
          w[i][0] = r0.x; w[i][1] = r0.y; w[i][2] = r0.z; w[i][3] = r0.w;
          w[i][4] = r1.x; w[i][5] = r1.y; w[i][6] = r1.z; w[i][7] = r1.w;
        }
        // scales and zero points of position pairs (2t, 2t+1) and (2t+8, 2t+9), per channel group
        uint32_t s2[2][NGRP], z2[2][NGRP];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int q = 0; q < NGRP; ++q) {
            const int pos = kl + 2 * t + 8 * h;
            s2[h][q] = (uint32_t)vs[pos * NGRP + q] | ((uint32_t)vs[(pos + 1) * NGRP + q] << 16);
            z2[h][q] = (uint32_t)vz[pos * NGRP + q] | ((uint32_t)vz[(pos + 1) * NGRP + q] << 16);
          }
#pragma unroll
        for (int nb = 0; nb < 16; ++nb) {
          // channel 8 nb + g: word nb / 2 of the row, bit 16 (nb % 2) + 2 g
          const int sh = 16 * (nb & 1) + 2 * g;
          const int q = nb / (16 / NGRP);
          const uint32_t i0 = ((w[0][nb >> 1] >> sh) & 3u) | (((w[1][nb >> 1] >> sh) & 3u) << 2);
          const uint32_t i1 = ((w[2][nb >> 1] >> sh) & 3u) | (((w[3][nb >> 1] >> sh) & 3u) << 2);
          const uint32_t b0 = mul_bf16x2_(sub_bf16x2(lut[i0], z2[0][q]), s2[0][q]);
          const uint32_t b1 = mul_bf16x2_(sub_bf16x2(lut[i1], z2[1][q]), s2[1][q]);
          mma_16816(acc[nb], a0, a2, b0, b1);
        }
      }
    }
    __syncthreads();
  }

  // Sum of the warps' partial tiles in warp order: red[w][g][channel], then main_out = bf16(sum).
  auto reduce_to = [&](float* dst, bool add_rounded) {
    if (row_live) {
#pragma unroll
      for (int nb = 0; nb < 16; ++nb)
        *reinterpret_cast<float2*>(red + ((size_t)warp * p.G + g) * KA_D + nb * 8 + 2 * t) =
            make_float2(acc[nb][0], acc[nb][1]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.G * KA_D; i += KA_THREADS) {
      const int r = i / KA_D, ch = i - r * KA_D;
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < KA_WARPS; ++w) s += red[((size_t)w * p.G + r) * KA_D + ch];
      s = bf16_round(s);
      if (add_rounded) p.out[(outer * p.G + r) * KA_D + ch] = __float2bfloat16_rn(dst[r * KA_D + ch] + s);
      else dst[r * KA_D + ch] = s;
    }
    __syncthreads();
  };
  reduce_to(main_out, false);

  // ---- the newest positions' values: staged [R][128 + 8] bfloat16, 128 positions at a time ----
#pragma unroll
  for (int nb = 0; nb < 16; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nb][e] = 0.0f;
  __nv_bfloat16* vres = reinterpret_cast<__nv_bfloat16*>(stage);
  for (int base = 0; base < p.R; base += 128) {
    const int rows = min(128, p.R - base);
    for (int i = threadIdx.x; i < rows * 16; i += KA_THREADS) {
      const int r = i >> 4, part = i & 15;
      cp_async16(vres + r * KA_RES_LD + part * 8, p.v_res + (outer * p.R + base + r) * KA_D + part * 8);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    for (int ks = warp; ks < rows / 16; ks += KA_WARPS) {
      const uint32_t* prow = reinterpret_cast<const uint32_t*>(probs + (size_t)(row_live ? g : 0) * N + p.Tm + base + ks * 16);
      const uint32_t a0 = row_live ? prow[t] : 0u, a2 = row_live ? prow[t + 4] : 0u;
      const uint16_t* v16 = reinterpret_cast<const uint16_t*>(vres);
#pragma unroll
      for (int nb = 0; nb < 16; ++nb) {
        const int ch = nb * 8 + g;
        const int pos = ks * 16 + 2 * t;
        const uint32_t b0 = (uint32_t)v16[pos * KA_RES_LD + ch] | ((uint32_t)v16[(pos + 1) * KA_RES_LD + ch] << 16);
        const uint32_t b1 = (uint32_t)v16[(pos + 8) * KA_RES_LD + ch] | ((uint32_t)v16[(pos + 9) * KA_RES_LD + ch] << 16);
        mma_16816(acc[nb], a0, a2, b0, b1);
      }
    }
    __syncthreads();
  }
  reduce_to(main_out, true);
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_kivi_decode_attention(const void* q, const void* k_packed, const void* k_scale, const void* k_zero,
                                        const void* v_packed, const void* v_scale, const void* v_zero,
                                        const void* k_res, const void* v_res, void* out, int64_t outer, int64_t G,
                                        int64_t Tm, int64_t R, int64_t D, int64_t k_block, int64_t v_block,
                                        float score_scale, void* stream) {
  VQ_REQUIRE(outer >= 0 && G > 0 && Tm >= 0 && R >= 0, "vq_kivi_decode_attention: bad extents");
  if (outer == 0) return VQ_OK;
  VQ_REQUIRE(Tm + R > 0, "vq_kivi_decode_attention: no keys");
  VQ_REQUIRE(q && out && (Tm == 0 || (k_packed && k_scale && k_zero && v_packed && v_scale && v_zero)) &&
                 (R == 0 || (k_res && v_res)), "vq_kivi_decode_attention: null argument");
  const int ngrp = v_block > 0 && v_block <= KA_D ? (int)(KA_D / v_block) : 1;
  const size_t smem = (size_t)G * (Tm + R) * 6 + 2 * (size_t)ka_stage_bytes(ngrp) +
                      (size_t)(KA_WARPS * G * KA_D + KA_WARPS + KA_MAX_G * KA_D) * 4 + 64;
  if (D != KA_D || G > KA_MAX_G || k_block <= 0 || k_block % KA_WKEYS != 0 || Tm % k_block != 0 || R % 16 != 0 ||
      (v_block != 32 && v_block != 64 && v_block != 128) || smem > 227 * 1024 || outer >= (1ll << 31) ||
      Tm >= (1ll << 24) || R >= (1ll << 24))
    return fail(VQ_EUNSUPPORTED,
                "vq_kivi_decode_attention: needs head_dim 128, at most 8 query heads per KV head, key groups of a "
                "multiple of 64 positions, value groups of 32, 64 or 128 channels, a multiple of 16 recent positions "
                "and G * (Tm + R) * 6 bytes of scores beside two staged chunks within 227 KB of shared memory");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_packed) | reinterpret_cast<uintptr_t>(k_scale) |
               reinterpret_cast<uintptr_t>(k_zero) | reinterpret_cast<uintptr_t>(v_packed) | reinterpret_cast<uintptr_t>(v_scale) |
               reinterpret_cast<uintptr_t>(v_zero) | reinterpret_cast<uintptr_t>(k_res) | reinterpret_cast<uintptr_t>(v_res)) & 15) == 0,
             "vq_kivi_decode_attention: buffers must be 16-byte aligned");
  KaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_packed = static_cast<const uint8_t*>(k_packed);
  p.k_scale = static_cast<const __nv_bfloat16*>(k_scale);
  p.k_zero = static_cast<const __nv_bfloat16*>(k_zero);
  p.v_packed = static_cast<const uint8_t*>(v_packed);
  p.v_scale = static_cast<const __nv_bfloat16*>(v_scale);
  p.v_zero = static_cast<const __nv_bfloat16*>(v_zero);
  p.k_res = static_cast<const __nv_bfloat16*>(k_res);
  p.v_res = static_cast<const __nv_bfloat16*>(v_res);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.G = (int)G; p.Tm = (int)Tm; p.R = (int)R; p.k_block = (int)k_block;
  p.score_scale = score_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    const int limit = 227 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kivi_decode_attention_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kivi_decode_attention_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kivi_decode_attention_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit);
    if (e != cudaSuccess) return fail(VQ_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  if (ngrp == 1) kivi_decode_attention_kernel<1><<<(unsigned)outer, KA_THREADS, smem, st>>>(p);
  else if (ngrp == 2) kivi_decode_attention_kernel<2><<<(unsigned)outer, KA_THREADS, smem, st>>>(p);
  else kivi_decode_attention_kernel<4><<<(unsigned)outer, KA_THREADS, smem, st>>>(p);
  return check_launch("kivi_decode_attention_kernel");
}
