// Weight-streaming linear for a decode step: a few activation rows (M <= 32) against a weight
// stored PACKED -- two 4-bit codebook indices per byte plus one scale per block of K -- which is
// what a `lut4_to_int6, bs=64, scale=fp8_e5m3` weight costs in memory (0.53 bytes per parameter
// here, against 2 for the bfloat16-valued index tensor the operator contract passes around).
//
//   Y[m][n] = alpha * sum_k a[m][k] * w[n][k] + bias[n]
//   a[m][k] = bf16(levels_a[A[m][k]] * scale_a[m][k / bs])     (or A itself when it has no scale / codebook)
//   w[n][k] = bf16(levels_w[code(n, k)] * scale_w[n][k / bs])
//
// Both operands are rounded to bfloat16 exactly as quantized_ops::linear_mx's read-back does
// (reference ops/quantized.py:574-591), the products are exact in float32 and the sum is float32:
// the result differs from the operator's dequantize-then-matmul in summation order only.
//
// The kernel is bound by HBM (the weight bytes) and, next, by instruction issue (decoding a weight
// is a table lookup and a multiply).  A CTA owns 256 weight rows x one K slice (1024, or 512 for small weights):
//   * prologue: the activation slice is decoded into shared memory once (M x 1024 bfloat16, the
//     four elements a lane needs per MMA step stored so that a warp's loads touch every bank once)
//     and a 256-entry table maps a packed byte to its two codebook values as a bfloat16 pair --
//     one copy per lane (32 random indices into a single table would collide on banks about
//     3.5-fold), rows 256 bytes apart at a 64 KB-aligned shared address, because the lookups are
//     what the loop does most and this makes a lookup three instructions: byte-permute (address),
//     load, packed multiply (scale);
//   * sixteen warps of 16 rows each stream the weight slice with 16-byte loads (32 weights per
//     lane and load, two rows per lane in flight), look both nibbles of a byte up with one
//     shared-memory load, scale them with one packed multiply and feed mma.sync m16n8k16 --
//     M = 16 activation rows is exactly the instruction's height, the tensor-core form that fits a
//     16-row problem (a 128-row tcgen05 tile would be 7/8 padding);
//   * K slices are combined deterministically: every CTA writes its float32 partial tile to a
//     workspace, and the last CTA of a row tile to arrive (a counter per tile) adds the partials in
//     slice order, applies alpha and bias, rounds once and resets the counter.

#include <cuda_bf16.h>
#include <mma.h>

#include "vq_common.cuh"

namespace vq {
namespace {

constexpr int L4_ROWS_PER_WARP = 16;
constexpr int L4_WARPS = 16;
constexpr int L4_ROWS = L4_ROWS_PER_WARP * L4_WARPS;   // 256 weight rows per CTA
constexpr int L4_KC = 1024;                            // longest K slice per CTA
constexpr int L4_THREADS = 32 * L4_WARPS;
// The byte table: one 256-byte row per byte value, lane l reading word l of the row.  It sits at
// shared-memory address 0x10000, so that a lookup address is the lane's base address with its second
// byte replaced by the packed byte -- one byte-permute instruction, no shift, mask or add.
constexpr uint32_t L4_TABLE_ADDR = 0x10000u;
constexpr int L4_TABLE_BYTES = 256 * 256;
constexpr int L4_APAD = 16;                            // bfloat16 elements of padding per activation row (bank spread)

struct Lut4Params {
  const void* a;            // [M, K] bfloat16: values, or codebook indices when a_levels != null
  const void* a_scale;      // [M, K / bs] bfloat16 or null
  const void* a_levels;     // [n_a_levels] bfloat16 or null
  int n_a_levels;
  const uint8_t* w;         // [N, K / 2]
  const void* w_scale;      // [N, K / bs] bfloat16
  const void* w_levels;     // [16] bfloat16
  void* out;
  int out_dt;
  int M, N, K, bs;
  int64_t lda;              // elements between activation rows
  const void* alpha;
  int alpha_dt;
  const void* bias;
  int bias_dt;
  float* workspace;         // [k_slices][row_tiles][M_pad][128]
  int* counters;            // [row_tiles], zero between launches
  int k_slices, row_tiles;
  int kc;                   // K slice length (a multiple of 128, at most L4_KC)
  int a_after_table;        // the activation slice lies behind the table (two row tiles of activations)
};

__device__ __forceinline__ float lparam(const void* p, int64_t i, int dt) {
  if (dt == VQ_F32) return static_cast<const float*>(p)[i];
  if (dt == VQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t v, uint32_t s) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(s));
  return r;
}

// MT: 16-row activation tiles (1 or 2).
template <int MT>
__global__ void __launch_bounds__(L4_THREADS, 1)
gemm_lut4_kernel(Lut4Params p) {
  extern __shared__ __align__(16) uint8_t l4_smem[];
  // dynamic shared memory starts a little above the window's first kilobyte; the table is placed so that
  // its shared address is exactly L4_TABLE_ADDR, the activation slice before it (or behind it when large)
  const uint32_t dyn_base = (uint32_t)__cvta_generic_to_shared(l4_smem);
  const uint32_t table_offset = L4_TABLE_ADDR - dyn_base;
  uint32_t* table = reinterpret_cast<uint32_t*>(l4_smem + table_offset);           // [256][64 words], 32 used
  __nv_bfloat16* sa = reinterpret_cast<__nv_bfloat16*>(
      l4_smem + (p.a_after_table ? table_offset + L4_TABLE_BYTES : ((16u - (dyn_base & 15u)) & 15u)));   // [MT * 16][L4_KC + pad]
  constexpr int SA_LD = L4_KC + L4_APAD;
  __shared__ int s_last;
  __shared__ float a_levels[256];                                                  // the activation's codebook

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.y;
  const int k0 = slice * p.kc;
  const int kc = min(p.kc, p.K - k0);                                              // a multiple of 128

  // ---- prologue: byte table and the decoded activation slice ----
  __shared__ uint16_t w_levels[16];
  if (threadIdx.x < 16) w_levels[threadIdx.x] = static_cast<const uint16_t*>(p.w_levels)[threadIdx.x];
  if (p.a_levels != nullptr && (int)threadIdx.x < p.n_a_levels)
    a_levels[threadIdx.x] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.a_levels)[threadIdx.x]);
  __syncthreads();
  for (int i = threadIdx.x; i < 256 * 32; i += L4_THREADS) {
    const int byte = i >> 5;
    table[byte * 64 + (i & 31)] = (uint32_t)w_levels[byte & 15] | ((uint32_t)w_levels[byte >> 4] << 16);   // even element low
  }
  {
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.a);
    const __nv_bfloat16* S = static_cast<const __nv_bfloat16*>(p.a_scale);
    const bool coded = p.a_levels != nullptr;
    const int groups = kc >> 3;                                                    // 8 elements per thread and step
    constexpr int BATCH = 8;                                                       // loads in flight per thread
    for (int base = 0; base < MT * 16 * groups; base += BATCH * L4_THREADS) {
      uint4 raw[BATCH];
      float scl[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int idx = base + u * L4_THREADS + threadIdx.x;
        const int m = idx / groups, kk = (idx - m * groups) << 3;
        raw[u] = make_uint4(0, 0, 0, 0);
        scl[u] = 1.0f;
        if (idx < MT * 16 * groups && m < p.M) {
          raw[u] = *reinterpret_cast<const uint4*>(A + (int64_t)m * p.lda + k0 + kk);
          if (S) scl[u] = __bfloat162float(S[(int64_t)m * (p.K / p.bs) + (k0 + kk) / p.bs]);
        }
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int idx = base + u * L4_THREADS + threadIdx.x;
        if (idx >= MT * 16 * groups) continue;
        const int m = idx / groups, kk = (idx - m * groups) << 3;
        uint4 packed = raw[u];
        if (m < p.M && (S != nullptr || coded)) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
          uint32_t o4[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v0 = __uint_as_float(w4[q] << 16), v1 = __uint_as_float(w4[q] & 0xFFFF0000u);
            if (coded) {   // indices are exact small integers in bfloat16
              v0 = a_levels[min(max((int)v0, 0), p.n_a_levels - 1)];
              v1 = a_levels[min(max((int)v1, 0), p.n_a_levels - 1)];
            }
            const __nv_bfloat162 h = __floats2bfloat162_rn(v0 * scl[u], v1 * scl[u]);   // one rounding of the exact product
            o4[q] = *reinterpret_cast<const uint32_t*>(&h);
          }
          packed = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
        // element 128 i + 32 t + 4 s + e of the slice lives at column 128 i + 16 s + 4 t + e: lane t of a warp
        // reads its four elements of step s eight bytes after lane t - 1's
        const int seg = kk & 127, tt = seg >> 5, ss = (seg & 31) >> 2;              // ss is even: steps ss and ss + 1
        __nv_bfloat16* dst = sa + m * SA_LD + (kk & ~127) + 16 * ss + 4 * tt;
        *reinterpret_cast<uint2*>(dst) = make_uint2(packed.x, packed.y);
        *reinterpret_cast<uint2*>(dst + 16) = make_uint2(packed.z, packed.w);
      }
    }
  }
  __syncthreads();

  // ---- main loop: this warp's 16 weight rows over the K slice, one row tile of the CTA after the other ----
  for (int row_tile = blockIdx.x; row_tile < p.row_tiles; row_tile += gridDim.x) {
  const int n_base = row_tile * L4_ROWS + warp * L4_ROWS_PER_WARP;
  float acc[MT][2][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][j][e] = 0.0f;

  // This lane's column of the table as a 32-bit shared address; its second byte is zero.
  const uint32_t tb_lane = L4_TABLE_ADDR + 4u * lane;
  const int row_bytes = p.K >> 1;
  const int blocks_per_row = p.K / p.bs;
  const int bs_shift = 31 - __clz(p.bs);                  // the block size is a power of two (32, 64, 128, ...)
  // rows past the end of the weight read row N - 1 again (valid memory); their results are never stored
  const uint8_t* wrow[2];
  const uint16_t* srow[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int n = min(n_base + 8 * j + g, p.N - 1);
    wrow[j] = p.w + (int64_t)n * row_bytes + (k0 >> 1) + t * 16;
    srow[j] = static_cast<const uint16_t*>(p.w_scale) + (int64_t)n * blocks_per_row + ((k0 + t * 32) >> bs_shift);
  }
  const int iters = kc >> 7;                              // 128 weights per row and iteration
  const int scale_step_shift = 7 - bs_shift;              // blocks per iteration = 128 / bs (>= 0 for bs <= 128)

  struct Vec { uint4 w[2]; uint32_t s[2]; };
  auto fetch = [&](int it, Vec& v) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      v.w[j] = __ldcs(reinterpret_cast<const uint4*>(wrow[j] + it * 64));          // streamed once: evict first
      const int blk = scale_step_shift >= 0 ? (it << scale_step_shift) : (it >> -scale_step_shift);
      const uint32_t h = __ldg(srow[j] + blk);
      v.s[j] = h | (h << 16);
    }
  };
  // the table entry of byte `which` (0..3) of `word`: address = tb_lane with byte 1 replaced by that byte
  auto lookup = [&](uint32_t word, int which) {
    uint32_t r;
    // not volatile: the table is constant once the CTA has passed its barrier, and the scheduler may then
    // hoist an iteration's lookups ahead of the MMAs that consume them
    asm("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(__byte_perm(word, tb_lane, 0x7604u | ((uint32_t)which << 4))));
    return r;
  };
  // the eight MMA steps of one iteration: step s takes bytes 2 s and 2 s + 1 of each row's 16-byte vector
  auto compute = [&](int it, const Vec& v) {
    const __nv_bfloat16* a_it = sa + it * 128 + t * 4;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      uint32_t af[MT][4];   // rows g and g + 8 of every 16-row tile, elements k = 32 t + 4 s + {0..3}
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint2 top = *reinterpret_cast<const uint2*>(a_it + (mt * 16 + g) * SA_LD + 16 * s);
        const uint2 bot = *reinterpret_cast<const uint2*>(a_it + (mt * 16 + g + 8) * SA_LD + 16 * s);
        af[mt][0] = top.x; af[mt][1] = bot.x; af[mt][2] = top.y; af[mt][3] = bot.y;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t word = s < 2 ? v.w[j].x : s < 4 ? v.w[j].y : s < 6 ? v.w[j].z : v.w[j].w;
        const uint32_t b0 = mul_bf16x2(lookup(word, 2 * (s & 1)), v.s[j]);         // weights k, k + 1
        const uint32_t b1 = mul_bf16x2(lookup(word, 2 * (s & 1) + 1), v.s[j]);     // weights k + 2, k + 3
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(acc[mt][j], af[mt][0], af[mt][1], af[mt][2], af[mt][3], b0, b1);
      }
    }
  };
  // three vector sets rotate by name, not by copy: two iterations' loads are always in flight
  Vec va, vb, vc;
  if (iters > 0) fetch(0, va);
  if (iters > 1) fetch(1, vb);
  int it = 0;
  for (; it + 3 <= iters; it += 3) {
    if (it + 2 < iters) fetch(it + 2, vc);
    compute(it, va);
    if (it + 3 < iters) fetch(it + 3, va);
    compute(it + 1, vb);
    if (it + 4 < iters) fetch(it + 4, vb);
    compute(it + 2, vc);
  }
  if (it < iters) {
    if (it + 2 < iters) fetch(it + 2, vc);
    compute(it, va);
    if (it + 1 < iters) compute(it + 1, vb);
    if (it + 2 < iters) compute(it + 2, vc);
  }

  // ---- partial tile to the workspace: [slice][row_tile][m][128 columns] ----
  // accumulator element e of group j: row m = g (+8 for e >= 2), column n = 8 j + 2 t + (e & 1)
  const int m_pad = MT * 16;
  float* part = p.workspace + ((int64_t)slice * p.row_tiles + row_tile) * m_pad * L4_ROWS;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int col = warp * L4_ROWS_PER_WARP + 8 * j + 2 * t;
      *reinterpret_cast<float2*>(part + (mt * 16 + g) * L4_ROWS + col) = make_float2(acc[mt][j][0], acc[mt][j][1]);
      *reinterpret_cast<float2*>(part + (mt * 16 + g + 8) * L4_ROWS + col) = make_float2(acc[mt][j][2], acc[mt][j][3]);
    }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&p.counters[row_tile], 1) == p.k_slices - 1;
  __syncthreads();
  const bool last = s_last != 0;
  __syncthreads();   // s_last is rewritten for the CTA's next row tile
  if (!last) continue;
  __threadfence();

  // ---- the last CTA of the row tile adds the slices in order and writes the output ----
  const float alpha = p.alpha ? lparam(p.alpha, 0, p.alpha_dt) : 1.0f;
  for (int idx = threadIdx.x; idx < p.M * L4_ROWS; idx += L4_THREADS) {
    const int m = idx / L4_ROWS, c = idx - m * L4_ROWS;
    const int n = row_tile * L4_ROWS + c;
    if (n >= p.N) continue;
    float sum = 0.0f;
    for (int sl = 0; sl < p.k_slices; ++sl)
      sum += __ldcg(p.workspace + (((int64_t)sl * p.row_tiles + row_tile) * m_pad + m) * L4_ROWS + c);
    if (p.alpha) sum = __fmul_rn(sum, alpha);
    if (p.bias) sum = __fadd_rn(sum, lparam(p.bias, n, p.bias_dt));
    const int64_t o = (int64_t)m * p.N + n;
    if (p.out_dt == VQ_F32) static_cast<float*>(p.out)[o] = sum;
    else if (p.out_dt == VQ_BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(sum);
    else static_cast<__half*>(p.out)[o] = __float2half_rn(sum);
  }
  if (threadIdx.x == 0) p.counters[row_tile] = 0;   // ready for the next launch
  }
}

// Pack bfloat16-valued codebook indices (0..15) two per byte, even element in the low nibble.
__global__ void pack_lut4_kernel(const __nv_bfloat16* __restrict__ codes, uint8_t* __restrict__ out, int64_t bytes,
                                 int* bad) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= bytes) return;
  const float lo = __bfloat162float(codes[2 * i]), hi = __bfloat162float(codes[2 * i + 1]);
  const int a = (int)lo, b = (int)hi;
  if (!(lo == (float)a && hi == (float)b && a >= 0 && a < 16 && b >= 0 && b < 16)) atomicExch(bad, 1);
  out[i] = (uint8_t)((a & 15) | ((b & 15) << 4));
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" {

// K slice length: 1024, or 512 when the weight has too few 256-row tiles to give every SM a CTA
static int lut4_slice_length(int64_t N, int64_t K) {
  const int64_t tiles = (N + L4_ROWS - 1) / L4_ROWS;
  return tiles * ((K + L4_KC - 1) / L4_KC) < kSmCount && K > 512 ? 512 : L4_KC;
}

int64_t vq_gemm_lut4_workspace_floats(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int64_t m_pad = M <= 16 ? 16 : 32;
  const int64_t kc = lut4_slice_length(N, K);
  const int64_t slices = (K + kc - 1) / kc, tiles = (N + L4_ROWS - 1) / L4_ROWS;
  return slices * tiles * m_pad * L4_ROWS;
}

int64_t vq_gemm_lut4_counters(int64_t N) { return N <= 0 ? 0 : (N + L4_ROWS - 1) / L4_ROWS; }

int vq_pack_lut4(const void* codes, void* packed, int64_t rows, int64_t K, int* bad, void* stream) {
  VQ_REQUIRE(rows >= 0 && K >= 0 && K % 2 == 0, "vq_pack_lut4: K must be even");
  const int64_t bytes = rows * (K / 2);
  if (bytes == 0) return VQ_OK;
  VQ_REQUIRE(codes && packed && bad, "vq_pack_lut4: null argument");
  pack_lut4_kernel<<<(unsigned)((bytes + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(codes), static_cast<uint8_t*>(packed), bytes, bad);
  return check_launch("pack_lut4_kernel");
}

int vq_gemm_lut4(const void* a, int64_t lda, const void* a_scale, const void* a_levels, int n_a_levels, int64_t M,
                 const void* w_packed, const void* w_scale, const void* w_levels, int block_size, void* out,
                 int out_dtype, int64_t N, int64_t K, const void* alpha, int alpha_dtype, const void* bias,
                 int bias_dtype, float* workspace, int* counters, void* stream) {
  VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, "vq_gemm_lut4: negative extent");
  if (M == 0 || N == 0) return VQ_OK;
  VQ_REQUIRE(M <= 32, "vq_gemm_lut4: at most 32 activation rows (a decode step); larger products take linear_mx's GEMM");
  VQ_REQUIRE(K > 0 && K % 128 == 0, "vq_gemm_lut4: K must be a positive multiple of 128");
  VQ_REQUIRE(block_size >= 32 && (block_size & (block_size - 1)) == 0 && K % block_size == 0,
             "vq_gemm_lut4: the block size must be a power of two, at least 32, that divides K");
  VQ_REQUIRE(a && w_packed && w_scale && w_levels && out && workspace && counters, "vq_gemm_lut4: null argument");
  VQ_REQUIRE(lda >= K && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(w_packed) & 15) == 0,
             "vq_gemm_lut4: operands must be 16-byte aligned with rows a multiple of 8 elements apart");
  VQ_REQUIRE(out_dtype >= VQ_BF16 && out_dtype <= VQ_F32, "vq_gemm_lut4: bad output dtype");
  VQ_REQUIRE(a_levels == nullptr || (n_a_levels > 0 && n_a_levels <= 256),
             "vq_gemm_lut4: an activation codebook has 1 to 256 entries");
  VQ_REQUIRE(N < (1ll << 31) && K < (1ll << 31), "vq_gemm_lut4: extent too large");
  Lut4Params p{};
  p.a = a; p.a_scale = a_scale; p.a_levels = a_levels; p.n_a_levels = n_a_levels;
  p.w = static_cast<const uint8_t*>(w_packed); p.w_scale = w_scale; p.w_levels = w_levels;
  p.out = out; p.out_dt = out_dtype;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.bs = block_size; p.lda = lda;
  p.alpha = alpha; p.alpha_dt = alpha_dtype; p.bias = bias; p.bias_dt = bias_dtype;
  p.workspace = workspace; p.counters = counters;
  p.kc = lut4_slice_length(N, K);
  p.k_slices = (int)((K + p.kc - 1) / p.kc);
  p.row_tiles = (int)((N + L4_ROWS - 1) / L4_ROWS);
  VQ_REQUIRE(p.k_slices <= 65535, "vq_gemm_lut4: K too large");
  const int mt = M <= 16 ? 1 : 2;
  // Shared memory: the table must sit at shared address L4_TABLE_ADDR.  Dynamic memory starts somewhere in
  // [1 KB, 4 KB) of the window (system + static variables), so reserving up to the table's end measured from
  // 1 KB always suffices; one row tile of activations (33 KB) fits before the table, two go behind it.
  const int a_bytes = mt * 16 * (L4_KC + L4_APAD) * (int)sizeof(__nv_bfloat16);
  p.a_after_table = mt == 2;
  const size_t smem = (size_t)L4_TABLE_ADDR + L4_TABLE_BYTES - 1024 + (p.a_after_table ? a_bytes : 0);
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    cudaFuncSetAttribute(gemm_lut4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)L4_TABLE_ADDR + L4_TABLE_BYTES - 1024);
    cudaFuncSetAttribute(gemm_lut4_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)L4_TABLE_ADDR + L4_TABLE_BYTES - 1024 + 32 * (L4_KC + L4_APAD) * 2);
  }
  // about two CTAs' worth of row tiles per SM in all; with many row tiles a CTA takes several of them, one
  // after the other, and decodes its activation slice once
  const int per_slice = (2 * kSmCount + p.k_slices - 1) / p.k_slices;
  dim3 grid((unsigned)(p.row_tiles < per_slice ? p.row_tiles : per_slice), (unsigned)p.k_slices);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mt == 1) gemm_lut4_kernel<1><<<grid, L4_THREADS, smem, st>>>(p);
  else gemm_lut4_kernel<2><<<grid, L4_THREADS, smem, st>>>(p);
  return check_launch("gemm_lut4_kernel");
}

}  // extern "C"
