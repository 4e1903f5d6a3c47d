// Causal self-attention on per-tensor FP8 operands in one kernel:
//     scores = bf16(q8 k8^T * alpha_qk)                  (the FP8 GEMM's rounding)
//     s      = bf16(scores * score_scale), causal mask
//     p      = bf16(softmax_fp32(s)),  p8 = fp8(bf16(p / s_p))
//     ctx    = bf16(p8 v8 * alpha_pv), ctx8 = fp8(bf16(ctx / s_ctx))
// which an eager graph runs as GEMM, softmax + cast, GEMM, cast, writing and re-reading
// the [heads * T, T] score and probability matrices.  Here neither leaves the SM.
//
// One CTA owns 128 query rows of one head.  Because p8 is the FP8 code of the
// normalised probability, the row maximum and sum must be final before the first
// code can be formed, so the CTA walks its key blocks twice:
//   pass A: S_j = Q K_j^T in tensor memory; running row maximum and sum
//   pass B: S_j again (bit-identical), probabilities and their FP8 codes written to
//           shared memory in the MMA operand layout, O += P_j V_j
// Every rounding step of the unfused sequence is kept.  The exponential and the
// reciprocal products are within an ulp of the unfused ones before they are rounded
// to bfloat16 and the row sum is accumulated in another order, so a probability code
// differs by one FP8 step only when a value sits on a rounding boundary.
//
// Warps: 0 TMA producer, 1 MMA issuer, then four softmax groups of four warps.  A
// softmax thread owns one query row (one tensor-memory lane) of 64 columns, so row
// statistics need no shuffles: a group takes the key blocks of one parity and one half
// of their columns, and the groups merge their statistics once, between the passes.
// Every wait is bounded.

#include <cuda.h>

#include <cstring>

#include "fp8_cast.cuh"
#include "sm100_ptx.cuh"

namespace vq {
namespace {

using namespace sm100;

constexpr int AT_BLK = 128;                 // query rows per CTA, keys per block, head_dim
constexpr int AT_STAGES = 3;                // K / V tiles in flight

// FP8 operands: 16 KB tiles, one score tile in tensor memory, two softmax groups, two CTAs per SM (one
// computes while the other waits or starts up).  bfloat16 operands: 32 KB tiles (two 128-byte-swizzled
// halves of 64 contraction elements each), so one CTA per SM, which overlaps the tensor core with the
// softmax inside itself instead: two score / probability tiles and four softmax groups.
template <bool BF16>
struct AtCfg {
  static constexpr int TILE = AT_BLK * AT_BLK * (BF16 ? 2 : 1);   // bytes of one operand tile
  static constexpr int HALF = TILE / 2;                          // bfloat16: bytes of one 64-element half
  static constexpr int KSTEPS = 4 * (BF16 ? 2 : 1);              // MMA instructions per tile (32 bytes of K each)
  static constexpr int SBUFS = BF16 ? 2 : 1;                     // score tiles in tensor memory (and probability tiles in shared memory)
  static constexpr int GROUPS = BF16 ? 4 : 2;                    // softmax groups of four warps: (score buffer) x (column part)
  static constexpr int PARTS = GROUPS / SBUFS;                   // column parts of a score tile
  static constexpr int CPT = 4 / PARTS;                          // 32-column chunks per thread and tile
  static constexpr int THREADS = 64 + GROUPS * 128;
  static constexpr int CTAS_PER_SM = BF16 ? 1 : 2;
  static constexpr int TMEM_COLS = SBUFS == 1 ? 256 : 512;       // score tiles, then the context accumulator
  static constexpr uint32_t O_COL = SBUFS * AT_BLK;
  static constexpr int STATS_BYTES = GROUPS * 2 * AT_BLK * 4;    // (max, sum) x groups x 128 rows
  static constexpr size_t SMEM_BYTES = 1024 + (1 + AT_STAGES + SBUFS) * TILE + STATS_BYTES + 256;
};

__device__ int g_attention_error = 0;

struct AttnParams {
  int T, groups, kv_heads;
  const void* alpha_qk;
  int alpha_qk_dt;
  float score_scale;
  const void* p_scale;
  int p_scale_dt;
  const void* alpha_pv;
  int alpha_pv_dt;
  const void* ctx_scale;   // scale of the FP8 output
  int ctx_scale_dt;
  uint8_t* out8;           // [T, ld8] e4m3, head h at columns [h * 128, +128), or null
  int64_t ld8;
  __nv_bfloat16* out16;    // [kv_heads, groups * T, 128] (ld16 = 0) or [T, ld16] with head h at columns [h * 128, +128); or null
  int64_t ld16;
  int round_acc;           // both products are rounded to bfloat16 before their scale is applied
};

__device__ __forceinline__ float2 unpack2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack2(float2 v) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 round2(float2 v) { return unpack2(pack2(v)); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ex2(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
template <int THREADS>
__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }

constexpr float kLog2e = 1.4426950408889634f;

// s = bf16(bf16(acc * alpha_qk) * score_scale) for 32 accumulator columns, as 16 pairs.
// In the diagonal block, column c of the block is masked for row r when c > r.
// ALPHA = false (bfloat16 operands: the product has no dequantization factor) skips that step, so that
// without round_acc the scores meet their first rounding only after the scale.
template <bool DIAG, bool ALPHA = true>
__device__ __forceinline__ void scores_of_chunk(const uint32_t (&v)[32], float2 (&s)[16], float alpha, float scale,
                                                int col0, int r, bool round_acc) {
  const float2 a2 = make_float2(alpha, alpha), s2 = make_float2(scale, scale);
#pragma unroll
  for (int i = 0; i < 16; ++i) s[i] = make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
  if (round_acc) {   // bf16(q8 k8^T) first: the matmul's own rounding (warp-uniform)
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = round2(s[i]);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float2 x = s[i];
    if (ALPHA) x = round2(__fmul2_rn(x, a2));
    x = round2(__fmul2_rn(x, s2));
    if (DIAG) {
      if (col0 + 2 * i > r) x.x = -INFINITY;
      if (col0 + 2 * i + 1 > r) x.y = -INFINITY;
    }
    s[i] = x;
  }
}

// Pass A on one chunk: the running maximum m and the sum l of exp(s - m) take in 32 more columns.
template <bool DIAG, bool ALPHA = true>
__device__ __forceinline__ void accumulate_chunk(const uint32_t (&v)[32], float alpha, float scale, int col0, int r,
                                                 float& m, float& l, bool round_acc) {
  float2 s[16];
  scores_of_chunk<DIAG, ALPHA>(v, s, alpha, scale, col0, r, round_acc);
  float cmax = m;
#pragma unroll
  for (int i = 0; i < 16; ++i) cmax = max3(cmax, s[i].x, s[i].y);
  // a live chunk's first column is at or before the warp's first row, so cmax is finite
  const float shift = -cmax * kLog2e;
  const float2 shift2 = make_float2(shift, shift), log2e2 = make_float2(kLog2e, kLog2e);
  float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 a = __ffma2_rn(s[i], log2e2, shift2);
    sum2 = __fadd2_rn(sum2, make_float2(ex2(a.x), ex2(a.y)));
  }
  l = fmaf(l, ex2(fmaf(m, kLog2e, shift)), sum2.x + sum2.y);   // m = -inf only while l = 0
  m = cmax;
}

// Pass B on one chunk: the 32 probabilities' FP8 codes.  p = bf16(e / sum), code = fp8(bf16(p / s_p)),
// both quotients as products with the correctly rounded reciprocal; p >= 0, so no -0 can arise.
template <bool DIAG>
__device__ __forceinline__ void codes_of_chunk(const uint32_t (&v)[32], uint32_t (&codes)[8], float alpha, float scale,
                                               int col0, int r, float shift, float rl, float rsp, bool round_acc) {
  float2 s[16];
  scores_of_chunk<DIAG>(v, s, alpha, scale, col0, r, round_acc);
  const float2 log2e2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(shift, shift);
  const float2 rl2 = make_float2(rl, rl), rsp2 = make_float2(rsp, rsp);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 a = __ffma2_rn(s[i], log2e2, shift2);
    const float2 prob = round2(__fmul2_rn(make_float2(ex2(a.x), ex2(a.y)), rl2));
    const float2 f = round2(__fmul2_rn(prob, rsp2));
    const uint32_t code = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
    if ((i & 1) == 0) codes[i >> 1] = code;
    else codes[i >> 1] |= code << 16;
  }
}

// Pass B on one chunk of bfloat16 attention: the 32 probabilities p = bf16(e / sum) as 16 packed pairs.
template <bool DIAG>
__device__ __forceinline__ void probs_of_chunk(const uint32_t (&v)[32], uint32_t (&words)[16], float alpha, float scale,
                                               int col0, int r, float shift, float rl, bool round_acc) {
  float2 s[16];
  scores_of_chunk<DIAG, false>(v, s, alpha, scale, col0, r, round_acc);
  const float2 log2e2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(shift, shift);
  const float2 rl2 = make_float2(rl, rl);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 a = __ffma2_rn(s[i], log2e2, shift2);
    words[i] = pack2(__fmul2_rn(make_float2(ex2(a.x), ex2(a.y)), rl2));
  }
}

template <bool BF16>
__global__ void __launch_bounds__(AtCfg<BF16>::THREADS, AtCfg<BF16>::CTAS_PER_SM)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttnParams p) {
  using C = AtCfg<BF16>;
  constexpr int AT_TILE = C::TILE, AT_SBUFS = C::SBUFS, AT_GROUPS = C::GROUPS, AT_PARTS = C::PARTS, AT_CPT = C::CPT;
  constexpr int AT_STATS_BYTES = C::STATS_BYTES, AT_TMEM_COLS = C::TMEM_COLS;
  constexpr uint32_t AT_O_COL = C::O_COL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;
  uint8_t* ring = smem + AT_TILE;                              // [AT_STAGES] K or V tiles
  uint8_t* smem_p = ring + AT_STAGES * AT_TILE;                // [AT_SBUFS] probability tiles
  float* stats = reinterpret_cast<float*>(smem_p + AT_SBUFS * AT_TILE);   // [groups][max, sum][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_p + AT_SBUFS * AT_TILE + AT_STATS_BYTES);
  uint64_t* q_full = bars;                        // [1]
  uint64_t* kv_full = bars + 1;                   // [AT_STAGES]
  uint64_t* kv_empty = kv_full + AT_STAGES;       // [AT_STAGES]
  uint64_t* s_full = kv_empty + AT_STAGES;        // [AT_SBUFS] score tile complete in tensor memory
  uint64_t* s_empty = s_full + AT_SBUFS;          // [AT_SBUFS] score tile read by its groups
  uint64_t* p_full = s_empty + AT_SBUFS;          // [AT_SBUFS] probability tile written
  uint64_t* p_empty = p_full + AT_SBUFS;          // [AT_SBUFS] probability tile read by the MMA
  uint64_t* o_full = p_empty + AT_SBUFS;          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work item: CTAs with the most key blocks come first in launch order.
  const int nb = p.T / AT_BLK;
  const int per_level = p.kv_heads * p.groups;
  const int jd = nb - 1 - (int)(blockIdx.x / per_level);      // the diagonal block; blocks 0..jd are live
  const int rest = (int)(blockIdx.x % per_level);
  const int kvh = rest / p.groups, g = rest % p.groups;
  const int qrow0 = g * p.T + jd * AT_BLK;                    // first query row within the KV head's [groups * T]

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < AT_SBUFS; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 4 * AT_PARTS);   // the warps of the groups that share the tile
      mbar_init(&p_full[b], 4 * AT_PARTS);
      mbar_init(&p_empty[b], 1);
    }
    mbar_init(o_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      // a bfloat16 tile arrives as two boxes of 64 contraction elements (x is the contraction coordinate)
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
        tma_load_3d(dst, map, bar, x, y, kvh);
        if (BF16) tma_load_3d(dst + C::HALF, map, bar, x + 64, y, kvh);
      };
      mbar_arrive_expect_tx(q_full, AT_TILE);
      load_tile(smem_q, &map_q, q_full, 0, qrow0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto load = [&](const CUtensorMap* map, int x, int y) {
        if (!ok) return;
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, abort_flag)) { ok = false; return; }
        mbar_arrive_expect_tx(&kv_full[stage], AT_TILE);
        load_tile(ring + stage * AT_TILE, map, &kv_full[stage], x, y);
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      };
      for (int j = 0; j <= jd; ++j) load(&map_k, 0, j * AT_BLK);          // pass A
      // pass B, in the order the MMA warp consumes: the first K blocks, then V_j and K_{j + AT_SBUFS} alternating
      for (int j = 0; j < AT_SBUFS && j <= jd; ++j) load(&map_k, 0, j * AT_BLK);
      for (int j = 0; j <= jd; ++j) {
        load(&map_v, j * AT_BLK, 0);
        if (j + AT_SBUFS <= jd) load(&map_k, 0, (j + AT_SBUFS) * AT_BLK);
      }
      if (!ok) {
        // Drain: let copies already issued land before the CTA's shared memory goes away.
        for (int s = 0; s < AT_STAGES; ++s)
          for (int spin = 0; spin < (1 << 14); ++spin)
            if (mbar_try_wait(&kv_full[s], 0) || mbar_try_wait(&kv_full[s], 1)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      // e4m3 x e4m3 or bfloat16 x bfloat16, M = N = 128; step k of a tile covers 32 bytes of K
      constexpr uint32_t idesc = BF16 ? make_idesc(AT_BLK, AT_BLK, 1, 1, 0, 0) : make_idesc(AT_BLK, AT_BLK, 0, 0, 0, 0);
      auto operand = [](uint32_t tile_addr, int k) {
        return smem_desc_k_major_sw128(tile_addr + (BF16 ? (uint32_t)((k >> 2) * C::HALF) : 0u) + (uint32_t)((k & 3) * 32));
      };
      auto mma = [&](uint32_t d, uint32_t a_addr, uint32_t b_addr, int k, uint32_t accumulate) {
        if (BF16) mma_f16_ss(d, operand(a_addr, k), operand(b_addr, k), idesc, accumulate);
        else mma_f8f6f4_ss(d, operand(a_addr, k), operand(b_addr, k), idesc, accumulate);
      };
      int stage = 0;
      uint32_t phase = 0;
      uint32_t s_uses[AT_SBUFS] = {}, p_uses[AT_SBUFS] = {};
      bool ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(smem_q);
      // S[j % AT_SBUFS] = Q K_j^T
      auto issue_scores = [&](int j) {
        if (!ok) return;
        const int b = j % AT_SBUFS;
        if (!mbar_wait(&kv_full[stage], phase, abort_flag) ||
            !mbar_wait(&s_empty[b], (s_uses[b] & 1) ^ 1, abort_flag)) { ok = false; return; }
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(ring + stage * AT_TILE);
#pragma unroll
        for (int k = 0; k < C::KSTEPS; ++k) mma(tmem_base + (uint32_t)(b * AT_BLK), q_addr, k_addr, k, k > 0 ? 1u : 0u);
        mma_commit(&kv_empty[stage]);
        mma_commit(&s_full[b]);
        ++s_uses[b];
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      };
      // O += P_j V_j
      auto issue_context = [&](int j) {
        if (!ok) return;
        const int b = j % AT_SBUFS;
        if (!mbar_wait(&kv_full[stage], phase, abort_flag) ||
            !mbar_wait(&p_full[b], p_uses[b] & 1, abort_flag)) { ok = false; return; }
        tc_fence_after_sync();
        const uint32_t p_addr = smem_u32(smem_p + b * AT_TILE);
        const uint32_t v_addr = smem_u32(ring + stage * AT_TILE);
#pragma unroll
        for (int k = 0; k < C::KSTEPS; ++k) mma(tmem_base + AT_O_COL, p_addr, v_addr, k, (j > 0 || k > 0) ? 1u : 0u);
        mma_commit(&kv_empty[stage]);
        mma_commit(&p_empty[b]);
        ++p_uses[b];
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      };
      for (int j = 0; j <= jd; ++j) issue_scores(j);                       // pass A
      for (int j = 0; j < AT_SBUFS && j <= jd; ++j) issue_scores(j);       // pass B
      for (int j = 0; j <= jd; ++j) {
        issue_context(j);
        if (j + AT_SBUFS <= jd) issue_scores(j + AT_SBUFS);
      }
      if (ok) mma_commit(o_full);
    }
  } else {
    // ------------------------------ softmax groups ----------------------------
    const int group = (warp - 2) >> 2;
    const int w = group % AT_SBUFS;                // key blocks j = w, w + AT_SBUFS, ...
    const int part = group / AT_SBUFS;             // columns [32 AT_CPT part, +32 AT_CPT) of each block
    const int quarter = warp & 3;                  // tensor-memory lanes [32 * quarter, +32) are this warp's
    const int r = quarter * 32 + lane;             // this thread's query row within the block
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float alpha = p.alpha_qk != nullptr ? loadp(p.alpha_qk, 0, p.alpha_qk_dt) : 1.0f;
    const bool round_acc = p.round_acc != 0;
    uint32_t s_uses = 0, p_uses = 0;               // tiles taken from S[w], tiles written to P[w]
    bool ok = true;
    uint32_t v[32];

    // ---- pass A: running maximum m and sum l of exp(s - m) over this group's part of the scores ----
    float m = -INFINITY, l = 0.0f;
    for (int j = w; j <= jd && ok; j += AT_SBUFS) {
      // The warp must stay convergent for the .sync.aligned tensor-memory loads below.
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s_full[w], s_uses & 1, abort_flag))) { ok = false; break; }
      ++s_uses;
      tc_fence_after_sync();
      const bool diag = j == jd;
      // in the diagonal block a chunk whose first column exceeds the warp's last row is masked for the whole warp
      const int live = diag ? min(max(quarter + 1 - AT_CPT * part, 0), AT_CPT) : AT_CPT;
      const uint32_t taddr = lane_addr + (uint32_t)(w * AT_BLK + part * 32 * AT_CPT);
      for (int c = 0; c < live; ++c) {
        const int col0 = (part * AT_CPT + c) * 32;
        tmem_ld_32x32(taddr + 32 * c, v);
        tmem_ld_wait();
        if (c == live - 1) {   // the tile is in registers: hand it back before working on the last chunk
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[w]);
        }
        if (diag) accumulate_chunk<true, !BF16>(v, alpha, p.score_scale, col0, r, m, l, round_acc);
        else accumulate_chunk<false, !BF16>(v, alpha, p.score_scale, col0, r, m, l, round_acc);
      }
      if (live == 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[w]);
      }
    }

    // ---- merge the two groups' statistics (every softmax thread reaches this barrier) ----
    stats[(group * 2 + 0) * AT_BLK + r] = m;
    stats[(group * 2 + 1) * AT_BLK + r] = l;
    softmax_barrier<AT_GROUPS * 128>();
    if (*abort_flag) ok = false;
    float mf = -INFINITY;
#pragma unroll
    for (int q = 0; q < AT_GROUPS; ++q) mf = fmaxf(mf, stats[(q * 2) * AT_BLK + r]);
    float lf = 0.0f;   // a group that saw nothing holds (-inf, 0); group 0 always sees column 0
#pragma unroll
    for (int q = 0; q < AT_GROUPS; ++q)
      lf = fmaf(stats[(q * 2 + 1) * AT_BLK + r], ex2((stats[(q * 2) * AT_BLK + r] - mf) * kLog2e), lf);
    const float rl = __frcp_rn(lf), rsp = BF16 ? 1.0f : __frcp_rn(loadp(p.p_scale, 0, p.p_scale_dt));
    const float shift = -mf * kLog2e;

    // ---- pass B: probabilities of this group's blocks as FP8 codes in the MMA operand layout ----
    // Row r of a K-major tile with the 128-byte swizzle: 16-byte chunk a sits at chunk a ^ (r % 8).
    uint8_t* p_row = smem_p + w * AT_TILE + (r >> 3) * 1024 + (r & 7) * 128;
    for (int j = w; j <= jd && ok; j += AT_SBUFS) {
      // the score tile is complete and the MMA that read this buffer's previous probabilities has finished
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s_full[w], s_uses & 1, abort_flag) &&
                                       mbar_wait(&p_empty[w], (p_uses & 1) ^ 1, abort_flag))) { ok = false; break; }
      ++s_uses;
      ++p_uses;
      tc_fence_after_sync();
      const bool diag = j == jd;
      const int live = diag ? min(max(quarter + 1 - AT_CPT * part, 0), AT_CPT) : AT_CPT;
      const uint32_t taddr = lane_addr + (uint32_t)(w * AT_BLK + part * 32 * AT_CPT);
      for (int c = 0; c < AT_CPT; ++c) {
        const int cidx = AT_CPT * part + c;        // 32-column chunk of the tile
        const int col0 = cidx * 32;
        const bool have = c < live;
        if (have) {
          tmem_ld_32x32(taddr + 32 * c, v);
          tmem_ld_wait();
          if (c == live - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[w]);
          }
        }
        if (BF16) {
          // 32 probabilities = 64 bytes = four 16-byte chunks of the half tile holding keys [64 (cidx / 2), +64)
          uint32_t words[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
          if (have) {
            if (diag) probs_of_chunk<true>(v, words, alpha, p.score_scale, col0, r, shift, rl, round_acc);
            else probs_of_chunk<false>(v, words, alpha, p.score_scale, col0, r, shift, rl, round_acc);
          }
          uint8_t* half_row = p_row + (cidx >> 1) * C::HALF;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(half_row + ((((cidx & 1) * 4 + q) ^ (r & 7)) << 4)) =
                make_uint4(words[4 * q], words[4 * q + 1], words[4 * q + 2], words[4 * q + 3]);
        } else {
          uint32_t codes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          if (have) {
            if (diag) codes_of_chunk<true>(v, codes, alpha, p.score_scale, col0, r, shift, rl, rsp, round_acc);
            else codes_of_chunk<false>(v, codes, alpha, p.score_scale, col0, r, shift, rl, rsp, round_acc);
          }
          const int chunk16 = 2 * cidx;
          *reinterpret_cast<uint4*>(p_row + ((chunk16 ^ (r & 7)) << 4)) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
          *reinterpret_cast<uint4*>(p_row + (((chunk16 + 1) ^ (r & 7)) << 4)) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
        }
      }
      if (live == 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[w]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[w]);
    }

    // ---- output: each group converts its share of the accumulator columns of its rows ----
    if (ok && !__all_sync(0xFFFFFFFFu, mbar_wait(o_full, 0, abort_flag))) ok = false;
    if (ok) {
      tc_fence_after_sync();
      const float alpha_pv = p.alpha_pv != nullptr ? loadp(p.alpha_pv, 0, p.alpha_pv_dt) : 1.0f;
      const int t = jd * AT_BLK + r;                         // position in the sequence
      const int head = kvh * p.groups + g;
      Divisor dv;
      if (p.out8 != nullptr) dv = make_divisor(p.ctx_scale, p.ctx_scale_dt);
      for (int c = 0; c < 4 / AT_GROUPS; ++c) {
        const int col0 = (group * (4 / AT_GROUPS) + c) * 32;
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + AT_O_COL + (uint32_t)col0, v);
        tmem_ld_wait();
        uint32_t words[16];   // ctx = bf16(acc * alpha_pv), or bf16(bf16(acc) * alpha_pv), two per word
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 acc = make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
          if (p.round_acc) acc = round2(acc);
          words[i] = pack2(__fmul2_rn(acc, make_float2(alpha_pv, alpha_pv)));
        }
        if (p.out16 != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(
              p.ld16 > 0 ? p.out16 + (int64_t)t * p.ld16 + head * AT_BLK + col0
                         : p.out16 + ((int64_t)kvh * p.groups * p.T + qrow0 + r) * AT_BLK + col0);
#pragma unroll
          for (int q = 0; q < 4; ++q) dst[q] = make_uint4(words[4 * q], words[4 * q + 1], words[4 * q + 2], words[4 * q + 3]);
        }
        if (p.out8 != nullptr) {
          uint32_t codes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int i = 0; i < 16; ++i)
            codes[i >> 1] |= fp8_pair<true>(quot(lo_of(words[i]), dv), quot(hi_of(words[i]), dv)) << (16 * (i & 1));
          uint4* dst = reinterpret_cast<uint4*>(p.out8 + (int64_t)t * p.ld8 + head * AT_BLK + col0);
          dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
          dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
        }
      }
      tc_fence_before_sync();
    }
  }

  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attention_error, VQ_ETIMEOUT);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Tensor map over a [batch, rows, cols] matrix of 1- or 2-byte elements, cols contiguous; boxes of
// 128 rows x 128 bytes in the 128-byte swizzle (the K-major MMA operand layout).
int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t batch, int elem_bytes = 1) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(cols * elem_bytes), (cuuint64_t)(rows * cols * elem_bytes)};
  cuuint32_t box[3] = {(cuuint32_t)(AT_BLK / elem_bytes), AT_BLK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return VQ_OK;
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_attention_fp8(const void* q8, const void* k8, const void* vt8, void* out8, int64_t ld8, void* out16,
                                int64_t T, int64_t kv_heads, int64_t groups, int64_t head_dim, const void* alpha_qk,
                                int alpha_qk_dtype, float score_scale, const void* p_scale, int p_scale_dtype,
                                const void* alpha_pv, int alpha_pv_dtype, const void* ctx_scale, int ctx_scale_dtype,
                                int round_acc, void* stream) {
  VQ_REQUIRE(T >= 0 && kv_heads >= 0 && groups >= 0, "vq_attention_fp8: negative extent");
  if (T == 0 || kv_heads == 0 || groups == 0) return VQ_OK;
  if (head_dim != AT_BLK || T % AT_BLK != 0)
    return fail(VQ_EUNSUPPORTED, "vq_attention_fp8: head_dim must be 128 and T a multiple of 128");
  VQ_REQUIRE(q8 && k8 && vt8 && alpha_qk && p_scale && alpha_pv, "vq_attention_fp8: null argument");
  VQ_REQUIRE(out8 || out16, "vq_attention_fp8: no output");
  VQ_REQUIRE(!out8 || (ctx_scale && ld8 >= kv_heads * groups * AT_BLK && ld8 % 16 == 0),
             "vq_attention_fp8: the FP8 output needs its scale and a row stride of at least heads * 128, a multiple of 16");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(q8) | reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(vt8) |
               reinterpret_cast<uintptr_t>(out8) | reinterpret_cast<uintptr_t>(out16)) & 15) == 0,
             "vq_attention_fp8: misaligned buffers");
  const int64_t items = kv_heads * groups * (T / AT_BLK);
  VQ_REQUIRE(T < (1ll << 24) && groups * T < (1ll << 31) && kv_heads < 65536 && items < (1ll << 31),
             "vq_attention_fp8: extent too large");
  CUtensorMap map_q, map_k, map_v;
  int rc;
  if ((rc = make_tile_map(&map_q, q8, groups * T, AT_BLK, kv_heads)) != VQ_OK) return rc;
  if ((rc = make_tile_map(&map_k, k8, T, AT_BLK, kv_heads)) != VQ_OK) return rc;
  if ((rc = make_tile_map(&map_v, vt8, AT_BLK, T, kv_heads)) != VQ_OK) return rc;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.T = (int)T;
  p.groups = (int)groups;
  p.kv_heads = (int)kv_heads;
  p.alpha_qk = alpha_qk;
  p.alpha_qk_dt = alpha_qk_dtype;
  p.score_scale = score_scale;
  p.p_scale = p_scale;
  p.p_scale_dt = p_scale_dtype;
  p.alpha_pv = alpha_pv;
  p.alpha_pv_dt = alpha_pv_dtype;
  p.ctx_scale = ctx_scale;
  p.ctx_scale_dt = ctx_scale_dtype;
  p.out8 = static_cast<uint8_t*>(out8);
  p.ld8 = ld8;
  p.out16 = static_cast<__nv_bfloat16*>(out16);
  p.round_acc = round_acc != 0;
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AtCfg<false>::SMEM_BYTES);
    if (e != cudaSuccess) return fail(VQ_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  attention_kernel<false><<<(unsigned)items, AtCfg<false>::THREADS, AtCfg<false>::SMEM_BYTES,
                            static_cast<cudaStream_t>(stream)>>>(map_q, map_k, map_v, p);
  return check_launch("attention_kernel<fp8>");
}

extern "C" int vq_attention_bf16(const void* q, const void* k, const void* vt, void* out, int64_t ldo, int64_t T,
                                 int64_t kv_heads, int64_t groups, int64_t head_dim, float score_scale, int round_acc,
                                 void* stream) {
  VQ_REQUIRE(T >= 0 && kv_heads >= 0 && groups >= 0, "vq_attention_bf16: negative extent");
  if (T == 0 || kv_heads == 0 || groups == 0) return VQ_OK;
  if (head_dim != AT_BLK || T % AT_BLK != 0)
    return fail(VQ_EUNSUPPORTED, "vq_attention_bf16: head_dim must be 128 and T a multiple of 128");
  VQ_REQUIRE(q && k && vt && out, "vq_attention_bf16: null argument");
  VQ_REQUIRE(ldo >= kv_heads * groups * AT_BLK && ldo % 8 == 0,
             "vq_attention_bf16: the output's row stride must be at least heads * 128 and a multiple of 8 elements");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(vt) |
               reinterpret_cast<uintptr_t>(out)) & 15) == 0, "vq_attention_bf16: misaligned buffers");
  const int64_t items = kv_heads * groups * (T / AT_BLK);
  VQ_REQUIRE(T < (1ll << 24) && groups * T < (1ll << 31) && kv_heads < 65536 && items < (1ll << 31),
             "vq_attention_bf16: extent too large");
  CUtensorMap map_q, map_k, map_v;
  int rc;
  if ((rc = make_tile_map(&map_q, q, groups * T, AT_BLK, kv_heads, 2)) != VQ_OK) return rc;
  if ((rc = make_tile_map(&map_k, k, T, AT_BLK, kv_heads, 2)) != VQ_OK) return rc;
  if ((rc = make_tile_map(&map_v, vt, AT_BLK, T, kv_heads, 2)) != VQ_OK) return rc;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.T = (int)T;
  p.groups = (int)groups;
  p.kv_heads = (int)kv_heads;
  p.score_scale = score_scale;
  p.out16 = static_cast<__nv_bfloat16*>(out);
  p.ld16 = ldo;
  p.round_acc = round_acc != 0;
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)AtCfg<true>::SMEM_BYTES);
    if (e != cudaSuccess) return fail(VQ_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  attention_kernel<true><<<(unsigned)items, AtCfg<true>::THREADS, AtCfg<true>::SMEM_BYTES,
                           static_cast<cudaStream_t>(stream)>>>(map_q, map_k, map_v, p);
  return check_launch("attention_kernel<bf16>");
}

// A wait inside the kernel ran out (VQ_ETIMEOUT) since the last reset, else VQ_OK.  Synchronises the device.
extern "C" int vq_attention_status(int reset) {
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(VQ_ECUDA, "vq_attention_status: %s", cudaGetErrorString(e));
  cudaMemcpyFromSymbol(&v, g_attention_error, sizeof(int));
  if (reset) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attention_error, &zero, sizeof(int));
  }
  return v;
}
