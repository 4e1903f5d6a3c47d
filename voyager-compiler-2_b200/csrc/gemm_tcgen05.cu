// Dense GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   C[b][m][n] = alpha * sum_k A[b][m][k] * B[b][n][k]  (+ bias[n])
//
// A and B are K-contiguous ("TN"): 16-bit (bf16 / f16) or 8-bit (e4m3 / e5m2)
// elements; accumulation is fp32 in tensor memory; the result is rounded once.
// This is the contraction behind quantized_ops::linear_mx / matmul_mx
// (operands first read back through their codebooks and block scales, which
// are exact bf16 values) and behind the real-FP8 linear.
//
// Structure: a persistent kernel, one CTA per SM, 128x256 output tiles.
//   warp 0   : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, 4 stages)
//   warp 1   : MMA issuer    (one thread; tcgen05.mma 128x256x{16|32}), owns TMEM
//   warps 2-9: epilogue      (tcgen05.ld -> alpha/bias -> global), overlapped with
//              the next tile's main loop through two TMEM accumulator buffers.
// TMA zero-fills out-of-range rows/columns, so M, N, K tails need no special
// main-loop code; the epilogue predicates its stores.
// Every mbarrier wait is bounded; on timeout the kernel records an error code
// in a device flag, drains, frees TMEM and exits.

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include <cuda_fp8.h>

#include "quantize_shared.cuh"
#include "sm100_ptx.cuh"
#include "vq_common.cuh"

namespace vq {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK_BYTES = 128;          // one swizzle row per operand row per stage
constexpr int STAGES = 4;
constexpr int MMA_K_BYTES = 32;        // K extent of one tcgen05.mma in bytes (16 x 16-bit / 32 x 8-bit)
constexpr int A_STAGE_BYTES = BM * BK_BYTES;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK_BYTES;   // 32 KB
constexpr int TMEM_COLS = 512;         // two 128x256 fp32 accumulators
constexpr int NUM_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;              // two per tensor-memory lane quadrant, one per half of the tile's columns
constexpr int EPI_STAGE_BYTES = EPI_WARPS * 32 * 128;   // per epilogue warp: 32 rows x 128 bytes of output
constexpr size_t SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + EPI_STAGE_BYTES;

__device__ int g_gemm_error = 0;

struct GemmParams {
  void* C;
  int M, N, K;          // K in elements
  int elem_bytes;       // 2 or 1
  int64_t ldc, strideC;
  int batch;
  const void* alpha;
  int alpha_dt;
  const void* bias;
  int bias_dt;
  const void* alpha_cols;   // per-column factor [N], or null
  int alpha_cols_dt;
  const void* residual;     // [batch, M, N] of the output dtype added after the first rounding, or null
  int64_t ldr, strideR;
  int causal_period;        // > 0: row r belongs to position t = r % period of a causal sequence
  int causal_mode;          // 1: tiles whose columns all exceed t are not computed; 2: A is zero beyond column t
  int bn;                   // CTA-pair kernel: tile width, 256 or 128
  int tma_store;            // the output has a tensor map: staged rows leave shared memory as TMA stores
  const void* gate_scale;   // gated mode (SwiGLU): per-tensor scale of the e4m3 output, or null
  int gate_scale_dt;
  int out_dt;
  int round_acc;            // round the accumulator to out_dt before alpha / alpha_cols / bias
  uint32_t idesc;
  int kind_f8;
};

__device__ __forceinline__ float load_param(const void* p, int64_t i, int dt) {
  if (dt == VQ_F32) return static_cast<const float*>(p)[i];
  if (dt == VQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

// alpha, the per-column factor and the bias for 32 consecutive accumulator columns.
// Every lane of a warp works on the same 32 columns (one row each): lane j fetches
// column j's factor and bias with one coalesced load and the warp shares them by
// shuffle.  All 32 lanes must call this together.
// This lane's column factor and bias of the 32-column chunk at col0 (1 and 0 where there is none).
__device__ __forceinline__ void load_col_params(const GemmParams& p, int col0, float* col_factor, float* col_bias) {
  const int lane = threadIdx.x & 31;
  *col_factor = 1.0f;
  *col_bias = 0.0f;
  if (p.alpha_cols != nullptr && col0 + lane < p.N) *col_factor = load_param(p.alpha_cols, col0 + lane, p.alpha_cols_dt);
  if (p.bias != nullptr && col0 + lane < p.N) *col_bias = load_param(p.bias, col0 + lane, p.bias_dt);
}
__device__ __forceinline__ void scale_chunk_with(const GemmParams& p, const uint32_t (&v)[32], float (&f)[32],
                                                 float col_factor, float col_bias, bool has_alpha, float alpha);
__device__ __forceinline__ void scale_chunk(const GemmParams& p, const uint32_t (&v)[32], float (&f)[32], int col0,
                                            bool has_alpha, float alpha) {
  float col_factor, col_bias;
  load_col_params(p, col0, &col_factor, &col_bias);
  scale_chunk_with(p, v, f, col_factor, col_bias, has_alpha, alpha);
}
// The per-column parameters come from the caller, which can fetch them long before the accumulator is ready:
// loaded here they put a trip to global memory in front of every chunk.
__device__ __forceinline__ void scale_chunk_with(const GemmParams& p, const uint32_t (&v)[32], float (&f)[32],
                                                 float col_factor, float col_bias, bool has_alpha, float alpha) {
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
  if (p.round_acc) {   // the matmul's own rounding, before the dequantize's scale
    if (p.out_dt == VQ_BF16) {
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(f[j], f[j + 1]);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
        f[j] = __uint_as_float(w << 16);
        f[j + 1] = __uint_as_float(w & 0xFFFF0000u);
      }
    } else if (p.out_dt == VQ_F16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __half2float(__float2half_rn(f[j]));
    }
  }
  if (has_alpha) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __fmul_rn(f[j], alpha);
  }
  if (p.alpha_cols != nullptr) {
    // one factor for all 32 columns (tensor-wise scales of merged projections): no exchange per element
    const float first = __shfl_sync(0xFFFFFFFFu, col_factor, 0);
    if (__all_sync(0xFFFFFFFFu, col_factor == first)) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __fmul_rn(f[j], first);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __fmul_rn(f[j], __shfl_sync(0xFFFFFFFFu, col_factor, j));
    }
  }
  if (p.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __fadd_rn(f[j], __shfl_sync(0xFFFFFFFFu, col_bias, j));
  }
}

// One rounded output element plus one residual element, rounded again (x + linear(...)).
__device__ __forceinline__ uint16_t add_residual16(uint16_t y, uint16_t r, int out_dt) {
  if (out_dt == VQ_BF16) {
    const float s = __fadd_rn(__uint_as_float((uint32_t)y << 16), __uint_as_float((uint32_t)r << 16));
    return __bfloat16_as_ushort(__float2bfloat16_rn(s));
  }
  const float s = __fadd_rn(__half2float(__ushort_as_half(y)), __half2float(__ushort_as_half(r)));
  return __half_as_ushort(__float2half_rn(s));
}
__device__ __forceinline__ uint32_t add_residual_word(uint32_t y, uint32_t r, int out_dt) {
  if (out_dt == VQ_F32) return __float_as_uint(__fadd_rn(__uint_as_float(y), __uint_as_float(r)));
  return (uint32_t)add_residual16((uint16_t)(y & 0xFFFFu), (uint16_t)(r & 0xFFFFu), out_dt) |
         ((uint32_t)add_residual16((uint16_t)(y >> 16), (uint16_t)(r >> 16), out_dt) << 16);
}

// Epilogue for 32 consecutive accumulator columns of one output row:
// alpha, bias, one rounding, 16-byte stores where the row allows.
__device__ __forceinline__ void store_chunk(const GemmParams& p, const uint32_t (&v)[32], uint8_t* c_row,
                                            const uint8_t* r_row, int row, int col0, bool has_alpha, float alpha) {
  float f[32];
  scale_chunk(p, v, f, col0, has_alpha, alpha);   // warp-wide: before the per-row guard
  if (row < p.M && col0 < p.N) {
    const bool full = (col0 + 32 <= p.N);
    if (p.out_dt == VQ_F32) {
      float* dst = reinterpret_cast<float*>(c_row) + col0;
      if (r_row != nullptr) {
        const float* res = reinterpret_cast<const float*>(r_row) + col0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) f[j] = __fadd_rn(f[j], res[j]);
      }
      if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) dst[j] = f[j];
      }
    } else {
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (p.out_dt == VQ_BF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
          packed[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
          packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      uint16_t* dst = reinterpret_cast<uint16_t*>(c_row) + col0;
      if (r_row != nullptr) {
        const uint16_t* res = reinterpret_cast<const uint16_t*>(r_row) + col0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) {
            const uint16_t y = add_residual16((uint16_t)(packed[j >> 1] >> (16 * (j & 1))), res[j], p.out_dt);
            packed[j >> 1] = (packed[j >> 1] & ~(0xFFFFu << (16 * (j & 1)))) | ((uint32_t)y << (16 * (j & 1)));
          }
      }
      if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) dst[j] = (uint16_t)(packed[j >> 1] >> (16 * (j & 1)));
      }
    }
  }
}

// Ask L2 for the residual values one warp's part of a tile will add (32 rows x
// [c_begin, c_end) columns), while the tile's accumulator is still being computed.
__device__ __forceinline__ void prefetch_residual(const GemmParams& p, int row0, int lane, int n0, int b, int c_begin,
                                                  int c_end) {
  if (p.residual == nullptr) return;
  const int esz = p.out_dt == VQ_F32 ? 4 : 2;
  const int row = row0 + lane;
  if (row >= p.M) return;
  const uint8_t* base = static_cast<const uint8_t*>(p.residual) +
                        ((int64_t)b * p.strideR + (int64_t)row * p.ldr) * esz;
  const int64_t row_bytes = (int64_t)p.N * esz;
  for (int64_t off = (int64_t)(n0 + c_begin) * esz; off < (int64_t)(n0 + c_end) * esz && off < row_bytes; off += 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

template <int OUT_DT>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if (OUT_DT == VQ_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Phase 1 of the staged epilogue: this thread's 32 scaled values of one row go to
// its row of the warp's staging buffer (16-byte units XOR-swizzled by the row).
// `res` (16-bit outputs only): the residual's 32 elements of this row and chunk, added to the rounded values and
// rounded again before they are staged.
template <int OUT_DT>
__device__ __forceinline__ void stage_chunk(const GemmParams& p, const uint32_t (&v)[32], uint8_t* srow, int lane,
                                            int col0, int half, bool has_alpha, float alpha,
                                            const uint4 (&res)[4], bool add_res) {
  float f[32];
  scale_chunk(p, v, f, col0, has_alpha, alpha);
  if (OUT_DT != VQ_F32 && add_res) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t r4[4] = {res[u].x, res[u].y, res[u].z, res[u].w};
      uint32_t o4[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o4[q] = add_residual_word(pack_pair<OUT_DT>(f[8 * u + 2 * q], f[8 * u + 2 * q + 1]), r4[q], OUT_DT);
      *reinterpret_cast<uint4*>(srow + (((half * 4 + u) ^ (lane & 7)) << 4)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
    return;
  }
  if (OUT_DT == VQ_F32) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
      *reinterpret_cast<float4*>(srow + ((u ^ (lane & 7)) << 4)) =
          make_float4(f[4 * u], f[4 * u + 1], f[4 * u + 2], f[4 * u + 3]);
  } else {
#pragma unroll
    for (int u = 0; u < 4; ++u)
      *reinterpret_cast<uint4*>(srow + (((half * 4 + u) ^ (lane & 7)) << 4)) =
          make_uint4(pack_pair<OUT_DT>(f[8 * u], f[8 * u + 1]), pack_pair<OUT_DT>(f[8 * u + 2], f[8 * u + 3]),
                     pack_pair<OUT_DT>(f[8 * u + 4], f[8 * u + 5]), pack_pair<OUT_DT>(f[8 * u + 6], f[8 * u + 7]));
  }
}

// Phase 2: the staged 32 rows x 128 bytes go to C, eight consecutive lanes writing
// 128 contiguous bytes of one row.  `interior` (warp-uniform): every row and column
// of the block lies inside C, so no element needs a bounds check.
template <int OUT_DT>
__device__ __forceinline__ void flush_stage(const GemmParams& p, const uint8_t* stage, uint8_t* c_batch,
                                            const uint8_t* r_batch, int64_t row_stride, int64_t r_row_stride,
                                            bool r_wide, int row0, int lane, int round_col0, bool interior) {
  constexpr int ESZ = OUT_DT == VQ_F32 ? 4 : 2;
  constexpr int UNIT_COLS = 16 / ESZ;
  const int u = lane & 7;
  const int rq = lane >> 3;
  const int col = round_col0 + u * UNIT_COLS;
  if (interior && r_batch == nullptr) {
    uint8_t* dst = c_batch + (int64_t)(row0 + rq) * row_stride + (int64_t)col * ESZ;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = 4 * i + rq;
      *reinterpret_cast<uint4*>(dst + (int64_t)(4 * i) * row_stride) =
          *reinterpret_cast<const uint4*>(stage + r * 128 + ((u ^ (r & 7)) << 4));
    }
    return;
  }
  // general path: bounds-checked, with the residual.  Two groups of four rows per lane; a group's
  // residual loads are all in flight before its first store (coalesced like the stores).
#pragma unroll 1
  for (int i0 = 0; i0 < 8; i0 += 4) {
    uint4 rv[4];
    if (r_batch != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = row0 + 4 * (i0 + i) + rq;
        rv[i] = make_uint4(0, 0, 0, 0);
        if (row < p.M && col < p.N) {
          const uint8_t* rsrc = r_batch + (int64_t)row * r_row_stride + (int64_t)col * ESZ;
          if (r_wide && col + UNIT_COLS <= p.N) {
            rv[i] = *reinterpret_cast<const uint4*>(rsrc);
          } else {
            uint32_t w[4] = {0, 0, 0, 0};
            const int valid = p.N - col < UNIT_COLS ? p.N - col : UNIT_COLS;
            if (ESZ == 4) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (e < valid) w[e] = reinterpret_cast<const uint32_t*>(rsrc)[e];
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (e < valid) w[e >> 1] |= (uint32_t)reinterpret_cast<const uint16_t*>(rsrc)[e] << (16 * (e & 1));
            }
            rv[i] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * (i0 + i) + rq;
      const int row = row0 + r;
      if (row < p.M && col < p.N) {
        uint4 val = *reinterpret_cast<const uint4*>(stage + r * 128 + ((u ^ (r & 7)) << 4));
        uint8_t* dst = c_batch + (int64_t)row * row_stride + (int64_t)col * ESZ;
        if (r_batch != nullptr) {
          val.x = add_residual_word(val.x, rv[i].x, OUT_DT);
          val.y = add_residual_word(val.y, rv[i].y, OUT_DT);
          val.z = add_residual_word(val.z, rv[i].z, OUT_DT);
          val.w = add_residual_word(val.w, rv[i].w, OUT_DT);
        }
        if (col + UNIT_COLS <= p.N) {
          *reinterpret_cast<uint4*>(dst) = val;
        } else {
          const uint32_t w[4] = {val.x, val.y, val.z, val.w};
          const int valid = p.N - col;
          if (ESZ == 4) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (e < valid) reinterpret_cast<uint32_t*>(dst)[e] = w[e];
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (e < valid) reinterpret_cast<uint16_t*>(dst)[e] = (uint16_t)(w[e >> 1] >> (16 * (e & 1)));
          }
        }
      }
    }
  }
}

// The epilogue of one warp for one tile: its 32 accumulator rows x [c_begin, c_end)
// columns.  A thread owns a row in tensor memory, which would make every 16-byte
// store of a warp touch 32 different rows of C.  Rows are therefore staged in shared
// memory (32 rows x 128 bytes, conflict-free in both phases) and written back with
// eight consecutive lanes covering 128 contiguous bytes of one row.  The tensor-memory
// load of the next 32 columns is in flight while the current ones are processed.
// Outputs that are not 16-byte aligned fall back to per-row stores.
// Epilogue for an output that is not 16-byte aligned: every thread stores its own row.
__device__ __noinline__ void epilogue_warp_tile_unstaged(const GemmParams& p, uint32_t taddr, int row0, int lane, int n0,
                                                         int b, bool has_alpha, float alpha, int c_begin, int c_end) {
  const int esz = p.out_dt == VQ_F32 ? 4 : 2;
  const int my_row = row0 + lane;
  uint8_t* c_row = static_cast<uint8_t*>(p.C) + ((int64_t)b * p.strideC + (int64_t)my_row * p.ldc) * esz;
  const uint8_t* r_row = p.residual == nullptr
                             ? nullptr
                             : static_cast<const uint8_t*>(p.residual) + ((int64_t)b * p.strideR + (int64_t)my_row * p.ldr) * esz;
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + (uint32_t)c0, v);
    tmem_ld_wait();
    if (n0 + c0 >= p.N) continue;  // warp-uniform
    store_chunk(p, v, c_row, r_row, my_row, n0 + c0, has_alpha, alpha);
  }
}

// `release_bar` (a shared::cluster barrier address, or 0): arrived on by lane 0 as soon as the LAST tensor-memory
// load of [c_begin, c_end) has completed -- before the values still in registers are converted and stored -- for
// callers that hand the columns back to the MMA warp.
template <int OUT_DT, int EPI_BUFS>
__device__ __forceinline__ void epilogue_warp_tile_t(const GemmParams& p, const CUtensorMap* map_c, uint32_t taddr,
                                                     uint8_t* stage0, uint32_t& buf, int row0, int lane, int n0, int b,
                                                     bool has_alpha, float alpha, int c_begin, int c_end,
                                                     uint32_t release_bar = 0) {
  constexpr int ESZ = OUT_DT == VQ_F32 ? 4 : 2;
  constexpr int ROUND_COLS = 128 / ESZ;   // output columns per 128-byte staged row
  const int64_t row_stride = p.ldc * ESZ;
  uint8_t* c_batch = static_cast<uint8_t*>(p.C) + (int64_t)b * p.strideC * ESZ;
  const int64_t r_row_stride = p.ldr * ESZ;
  const uint8_t* r_batch = p.residual == nullptr ? nullptr
                                                 : static_cast<const uint8_t*>(p.residual) + (int64_t)b * p.strideR * ESZ;
  const bool r_wide = ((reinterpret_cast<uintptr_t>(p.residual) | (uintptr_t)r_row_stride | (uintptr_t)(p.strideR * ESZ)) & 15) == 0;
  const bool rows_inside = row0 + 32 <= p.M;
  // With EPI_BUFS = 2 the warp alternates between two 4 KB staging buffers (`buf`, which lives
  // across tiles), so the TMA store of one block drains while the next block is being staged.
  uint8_t* stage = stage0 + (EPI_BUFS == 2 ? buf * (32 * 128) : 0);
  uint8_t* srow = stage + lane * 128;
  // A 16-bit residual whose rows are 16-byte aligned is fetched by the lane that owns the row, 64 bytes per chunk,
  // when the chunk's tensor-memory load is issued, and added before staging: the block then leaves like any other.
  const bool early_res = r_batch != nullptr && ESZ == 2 && r_wide && p.tma_store != 0 && (p.N & 31) == 0;
  // With a tensor map for C (and no residual left to add) a finished 32 x 128-byte block leaves
  // shared memory as one TMA store issued by lane 0; the hardware clips it at the edges of C.
  const bool by_tma = p.tma_store != 0 && (r_batch == nullptr || early_res);
  const uint8_t* r_row = early_res && row0 + lane < p.M ? r_batch + (int64_t)(row0 + lane) * r_row_stride : nullptr;
  auto load_res = [&](uint4 (&r)[4], int c0) {
    if (!early_res) return;
    const bool in = r_row != nullptr && n0 + c0 < p.N;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      r[u] = in ? __ldg(reinterpret_cast<const uint4*>(r_row + (int64_t)(n0 + c0) * ESZ) + u) : make_uint4(0, 0, 0, 0);
  };

  // one 32-column chunk: scale, stage, and flush when its 128-byte round is complete
  auto process = [&](const uint32_t (&v)[32], int c0, const uint4 (&res)[4]) {
    const int col0 = n0 + c0;
    if (col0 >= p.N) return;  // warp-uniform
    const int half = ESZ == 4 ? 0 : (c0 >> 5) & 1;   // a 128-byte row holds two 32-column chunks of 16-bit values
    if (by_tma && half == 0) {   // the store that last used this staging buffer must have read it
      if (lane == 0) {
        if (EPI_BUFS == 2) tma_store_wait_read_but_one(); else tma_store_wait_read();
      }
      __syncwarp();
    }
    stage_chunk<OUT_DT>(p, v, srow, lane, col0, half, has_alpha, alpha, res, early_res);
    if (ESZ != 4 && half == 0 && col0 + 32 < p.N && c0 + 32 < c_end) return;  // the round's second chunk follows
    const int round_col0 = col0 - half * 32;
    if (by_tma) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (row0 < p.M) tma_store_3d(map_c, stage, round_col0, row0, b);   // a block entirely below C stores nothing
        tma_store_commit();                                                 // (an empty group keeps the count in step)
      }
      if (EPI_BUFS == 2) {
        buf ^= 1u;
        stage = stage0 + buf * (32 * 128);
        srow = stage + lane * 128;
      }
      return;
    }
    __syncwarp();
    flush_stage<OUT_DT>(p, stage, c_batch, r_batch, row_stride, r_row_stride, r_wide, row0, lane, round_col0,
                        rows_inside && round_col0 + ROUND_COLS <= p.N);
    __syncwarp();
  };

  uint32_t va[32], vb[32];
  uint4 ra[4] = {}, rb[4] = {};
  tmem_ld_32x32(taddr + (uint32_t)c_begin, va);
  load_res(ra, c_begin);
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 64) {
    const bool has_b = c0 + 32 < c_end;   // warp-uniform
    tmem_ld_wait();
    if (has_b) {
      tmem_ld_32x32(taddr + (uint32_t)(c0 + 32), vb);
      load_res(rb, c0 + 32);
    }
    const bool release_now = release_bar != 0 && c0 + 64 >= c_end;   // these are the range's last loads
    if (release_now) {
      if (has_b) tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release_bar);
    }
    process(va, c0, ra);
    if (has_b) {
      if (!release_now) tmem_ld_wait();
      if (c0 + 64 < c_end) {
        tmem_ld_32x32(taddr + (uint32_t)(c0 + 64), va);
        load_res(ra, c0 + 64);
      }
      process(vb, c0 + 32, rb);
    }
  }
}

// Gated epilogue (SwiGLU): the tile's columns alternate between 32 gate columns and their 32 up
// columns (the caller interleaved the two weight matrices that way), so a warp's consecutive
// 32-column chunks are a (gate, up) pair.  Per pair and row:
//   g = bf16(gate), u = bf16(up)            the two linears' outputs as a bfloat16 GEMM rounds them
//   a = bf16(bf16(silu(g)) * u)             the activation, every rounding of the unfused graph kept
//   C = e4m3(bf16(a / scale))               32 bytes per row: one full sector per lane, stored directly
// C is [M, N / 2] bytes.
//
// The arithmetic of a 32-column pair is written as three branch-free passes over 16 independent two-element
// chains (activation, quotient, code), so that the compiler interleaves the chains: with a branch inside the
// chain (the quotient's rare exact-division case) every chain ran alone and the epilogue, not the main loop,
// set the time of the merged gate/up GEMM.  The rare cases are collected in a mask and redone after the pass.
__device__ __forceinline__ uint32_t mul_rn_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void store_32_bytes(uint8_t* dst, const uint32_t (&q)[8], bool aligned32) {
  if (aligned32) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(dst), "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7])
                 : "memory");
  } else {
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(q[0], q[1], q[2], q[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(q[4], q[5], q[6], q[7]);
  }
}
// g: 32 gate values as bfloat16 pairs; f: the 32 up values (float32, scaled); q: the 32 output bytes.
template <bool ORDINARY>
__device__ __forceinline__ void gated_pair(const uint32_t (&g)[16], const float (&f)[32], float s_out, float r_out,
                                           uint32_t (&q)[8]) {
  uint32_t a[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t u = pack_pair<VQ_BF16>(f[2 * j], f[2 * j + 1]);
    const float g0 = __uint_as_float(g[j] << 16), g1 = __uint_as_float(g[j] & 0xFFFF0000u);
    const uint32_t sl = pack_pair<VQ_BF16>(__fdividef(g0, 1.0f + __expf(-g0)), __fdividef(g1, 1.0f + __expf(-g1)));
    a[j] = mul_rn_bf16x2(sl, u);   // the float32 product of two bfloat16 values is exact: one rounding either way
  }
  float y[32];
  uint32_t slow = 0;   // bit i: element i needs the exact division
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float a0 = __uint_as_float(a[j] << 16), a1 = __uint_as_float(a[j] & 0xFFFF0000u);
    if (ORDINARY) {
      // div_to_bf16 without its branch; a zero numerator gives the exact (signed) zero through the product too
      const float q0 = __fmul_rn(a0, r_out), q1 = __fmul_rn(a1, r_out);
      const uint32_t b0 = __float_as_uint(q0), b1 = __float_as_uint(q1);
      const uint32_t e0 = (b0 >> 23) & 0xFFu, e1 = (b1 >> 23) & 0xFFu;
      const bool s0 = (e0 == 0u && a0 != 0.0f) || e0 == 0xFFu || ((b0 & 0xFFFFu) - 0x7FFDu) <= 6u;
      const bool s1 = (e1 == 0u && a1 != 0.0f) || e1 == 0xFFu || ((b1 & 0xFFFFu) - 0x7FFDu) <= 6u;
      slow |= (s0 ? 1u : 0u) << (2 * j) | (s1 ? 1u : 0u) << (2 * j + 1);
      const uint32_t w = pack_pair<VQ_BF16>(q0, q1);
      y[2 * j] = __uint_as_float(w << 16);
      y[2 * j + 1] = __uint_as_float(w & 0xFFFF0000u);
    } else {
      y[2 * j] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(a0, s_out)));
      y[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(a1, s_out)));
    }
  }
  if (ORDINARY && slow != 0u) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (slow & (1u << (2 * j)))
        y[2 * j] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(__uint_as_float(a[j] << 16), s_out)));
      if (slow & (1u << (2 * j + 1)))
        y[2 * j + 1] = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(__uint_as_float(a[j] & 0xFFFF0000u), s_out)));
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t code = (uint32_t)__nv_cvt_float2_to_fp8x2(
        make_float2(__fadd_rn(y[2 * j], 0.0f), __fadd_rn(y[2 * j + 1], 0.0f)), __NV_SATFINITE, __NV_E4M3);
    if (j & 1) q[j >> 1] |= code << 16; else q[j >> 1] = code;
  }
}
__device__ __forceinline__ void epilogue_warp_tile_gated(const GemmParams& p, uint32_t taddr, int row0, int lane,
                                                         int n0, int b, bool has_alpha, float alpha, int c_begin,
                                                         int c_end) {
  const int my_row = row0 + lane;
  uint8_t* out_row = static_cast<uint8_t*>(p.C) + (int64_t)b * p.strideC + (int64_t)my_row * p.ldc;
  const float s_out = load_param(p.gate_scale, 0, p.gate_scale_dt);
  const bool ordinary = ordinary_divisor(s_out);
  const float r_out = __frcp_rn(s_out);
  const bool aligned32 = ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)p.ldc | (uintptr_t)p.strideC) & 31) == 0;
  // the column factors of the warp's (at most four) chunks, fetched before the first accumulator values arrive
  float factor[4], unused_bias;
#pragma unroll
  for (int i = 0; i < 4; ++i) load_col_params(p, n0 + c_begin + 32 * i, &factor[i], &unused_bias);
  uint32_t va[32], vb[32];
  tmem_ld_32x32(taddr + (uint32_t)c_begin, va);
#pragma unroll 1
  for (int c0 = c_begin; c0 < c_end; c0 += 64) {
    tmem_ld_wait();
    tmem_ld_32x32(taddr + (uint32_t)(c0 + 32), vb);
    float f[32];
    const int round = (c0 - c_begin) >> 6;   // 0 or 1 with the kernels' 128-column ranges
    float gate_factor = round ? factor[2] : factor[0], up_factor = round ? factor[3] : factor[1];
    if (round > 1) {
      load_col_params(p, n0 + c0, &gate_factor, &unused_bias);
      load_col_params(p, n0 + c0 + 32, &up_factor, &unused_bias);
    }
    scale_chunk_with(p, va, f, gate_factor, 0.0f, has_alpha, alpha);
    uint32_t g[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) g[j] = pack_pair<VQ_BF16>(f[2 * j], f[2 * j + 1]);
    tmem_ld_wait();
    if (c0 + 64 < c_end) tmem_ld_32x32(taddr + (uint32_t)(c0 + 64), va);
    scale_chunk_with(p, vb, f, up_factor, 0.0f, has_alpha, alpha);
    uint32_t q[8];
    if (ordinary) gated_pair<true>(g, f, s_out, r_out, q);
    else gated_pair<false>(g, f, s_out, r_out, q);
    if (my_row < p.M && n0 + c0 < p.N) store_32_bytes(out_row + ((n0 + c0) >> 1), q, aligned32);
  }
}

// Returns true when `release_bar` (see epilogue_warp_tile_t) has been arrived on; otherwise the caller does it.
template <int OUT_DT, int EPI_BUFS = 1>
__device__ __forceinline__ bool epilogue_warp_tile(const GemmParams& p, const CUtensorMap* map_c, uint32_t taddr,
                                                   uint8_t* stage, uint32_t& buf, int row0, int lane, int n0, int b,
                                                   bool has_alpha, float alpha, int c_begin, int c_end,
                                                   uint32_t release_bar = 0) {
  constexpr int ESZ = OUT_DT == VQ_F32 ? 4 : 2;
  if (OUT_DT == VQ_BF16 && p.gate_scale != nullptr) {   // gated launches use the bfloat16 instantiation
    epilogue_warp_tile_gated(p, taddr, row0, lane, n0, b, has_alpha, alpha, c_begin, c_end);
    return false;
  }
  if (((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.ldc * ESZ) | (uintptr_t)(p.strideC * ESZ)) & 15) != 0) {
    epilogue_warp_tile_unstaged(p, taddr, row0, lane, n0, b, has_alpha, alpha, c_begin, c_end);
    return false;
  }
  epilogue_warp_tile_t<OUT_DT, EPI_BUFS>(p, map_c, taddr, stage, buf, row0, lane, n0, b, has_alpha, alpha, c_begin,
                                         c_end, release_bar);
  return release_bar != 0 && c_begin < c_end;
}

// The MMAs of one pipeline stage (128 bytes of K = four instructions) as straight-line code, the operand
// kind a template parameter.  Choosing the kind at run time between consecutive tcgen05.mma instructions
// (`if (f8) mma_f8 else mma_f16` inside the unrolled loop) was measured to cost a third of the tensor
// throughput: 2048x28672x4096 e4m3 207 us with the choice inside the sequence, 141 us with it outside.
template <bool F8, bool PAIR>
__device__ __forceinline__ void issue_stage(uint32_t tmem_acc, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                            bool accumulate_first) {
#pragma unroll
  for (int k = 0; k < BK_BYTES / MMA_K_BYTES; ++k) {
    const uint64_t da = smem_desc_k_major_sw128(a_addr + k * MMA_K_BYTES);
    const uint64_t db = smem_desc_k_major_sw128(b_addr + k * MMA_K_BYTES);
    const uint32_t accumulate = (accumulate_first || k > 0) ? 1u : 0u;
    if constexpr (F8 && PAIR) mma_f8f6f4_ss_pair(tmem_acc, da, db, idesc, accumulate);
    else if constexpr (F8) mma_f8f6f4_ss(tmem_acc, da, db, idesc, accumulate);
    else if constexpr (PAIR) mma_f16_ss_pair(tmem_acc, da, db, idesc, accumulate);
    else mma_f16_ss(tmem_acc, da, db, idesc, accumulate);
  }
}

template <int OUT_DT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint8_t* epi_stage = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);   // 1024-byte aligned: TMA stores read it with the 128-byte swizzle
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;    // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  const int k_elems_per_stage = BK_BYTES / p.elem_bytes;
  const int k_blocks = (p.K + k_elems_per_stage - 1) / k_elems_per_stage;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_WARPS);  // one arrival per epilogue warp
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = (int)(tile % tiles_m);
        const int n_blk = (int)((tile / tiles_m) % tiles_n);
        const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_3d(smem_a + stage * A_STAGE_BYTES, &map_a, &full_bar[stage], kb * k_elems_per_stage, m_blk * BM, b);
          tma_load_3d(smem_b + stage * B_STAGE_BYTES, &map_b, &full_bar[stage], kb * k_elems_per_stage, n_blk * BN, b);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Drain: let copies already issued land before the CTA's shared memory goes away.
        for (int s = 0; s < STAGES; ++s)
          for (int spin = 0; spin < (1 << 14); ++spin) {
            if (mbar_try_wait(&full_bar[s], 0) || mbar_try_wait(&full_bar[s], 1)) break;
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    auto mma_role = [&](auto kind_tag) {   // compiled once per operand kind: no branch between MMA instructions
      constexpr bool F8 = decltype(kind_tag)::value;
      const uint32_t idesc = p.idesc;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_stage<F8, false>(tmem_acc, smem_u32(smem_a + stage * A_STAGE_BYTES), smem_u32(smem_b + stage * B_STAGE_BYTES),
                                 idesc, kb > 0);
          mma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&acc_full[acc]);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    };
    if (lane == 0) {
      if (p.kind_f8) mma_role(std::true_type{});
      else mma_role(std::false_type{});
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) are this warp's
    const int chalf = (warp - 2) >> 2;  // which half of the tile's columns
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;   // which staging buffer this warp fills next
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      prefetch_residual(p, m_blk * BM + quarter * 32, lane, n_blk * BN, b, chalf * (BN / 2), (chalf + 1) * (BN / 2));
      // The warp must stay convergent for the .sync.aligned TMEM loads below.
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
      epilogue_warp_tile<OUT_DT>(p, &map_c, taddr, epi_stage + (warp - 2) * (32 * 128), epi_buf, m_blk * BM + quarter * 32, lane, n_blk * BN, b,
                         has_alpha, alpha, chalf * (BN / 2), (chalf + 1) * (BN / 2));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait_read();   // staging buffers stay valid until their stores have read them
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant: two CTAs (a cluster of 2 on neighbouring SMs) share one
// 256x256 tile.  Each CTA loads its own 128 rows of A and its own 128 of the
// tile's 256 B rows (32 KB per stage, so twice the flops per byte fetched from
// L2), the even CTA's thread issues tcgen05.mma.cta_group::2 (M = 256), and each
// CTA's tensor memory receives its 128 rows of the accumulator.
//   full barrier  : lives in the even CTA; both CTAs' TMA loads complete on it
//   empty barrier : one per CTA, released by a tcgen05.commit sent to both CTAs
//   acc_full      : one per CTA, same commit mechanism
//   acc_empty     : lives in the even CTA; 8 arrivals (4 epilogue warps x 2 CTAs)
// ---------------------------------------------------------------------------
constexpr int P_THREADS = 384;             // one warpgroup of {TMA warp, MMA warp, two idle warps} + two epilogue warpgroups
constexpr int P_EPI_WARP0 = 4;             // first epilogue warp
constexpr int P_STAGES = 6;
constexpr int P_EPI_BUFS = 1;              // staging buffers per epilogue warp (2 was measured: no gain, and it costs a pipeline stage)
constexpr int P_A_BYTES = 128 * BK_BYTES;  // 16 KB
constexpr int P_B_BYTES = 128 * BK_BYTES;  // 16 KB (half of the tile's B rows)
constexpr size_t P_SMEM_BYTES = 1024 + P_STAGES * (P_A_BYTES + P_B_BYTES) + 256 + P_EPI_BUFS * EPI_STAGE_BYTES;

template <int OUT_DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tn_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + P_STAGES * P_A_BYTES;
  uint8_t* epi_stage = smem + P_STAGES * (P_A_BYTES + P_B_BYTES);   // 1024-byte aligned: TMA stores read it with the 128-byte swizzle
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * (P_A_BYTES + P_B_BYTES) + P_EPI_BUFS * EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                        // [P_STAGES] (used in the even CTA)
  uint64_t* empty_bar = bars + P_STAGES;            // [P_STAGES]
  uint64_t* acc_full = bars + 2 * P_STAGES;         // [2]
  uint64_t* acc_empty = bars + 2 * P_STAGES + 2;    // [2] (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = even (leader), 1 = odd
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int bn = p.bn;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + bn - 1) / bn;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  const int k_elems_per_stage = BK_BYTES / p.elem_bytes;
  const int k_blocks = (p.K + k_elems_per_stage - 1) / k_elems_per_stage;
  const uint32_t stage_tx_bytes = 2u * (uint32_t)(P_A_BYTES + (bn / 2) * BK_BYTES);

  // Causal hints: the number of K blocks a tile needs (0 = the tile is not computed at all).
  // The three roles evaluate this identically, so they walk the same tile sequence.
  auto tile_k_blocks = [&](int m_blk, int n_blk) -> int {
    if (p.causal_period <= 0) return k_blocks;
    const int t_lo = (m_blk * 2 * BM) % p.causal_period;
    int t_hi = t_lo + 2 * BM - 1;                       // largest position among the tile's rows
    if (t_hi >= p.causal_period) t_hi = p.causal_period - 1;   // the tile runs into the next sequence
    if (p.causal_mode == 1) return n_blk * bn > t_hi ? 0 : k_blocks;
    const int need = (t_hi + k_elems_per_stage) / k_elems_per_stage;   // ceil((t_hi + 1) / k per stage)
    return need < k_blocks ? need : k_blocks;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // the peer's barriers are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Registers by warpgroup (384 threads x 168 at launch): the producer / MMA group keeps 40 per thread,
  // the two epilogue groups take 232, so that the epilogue's double-buffered tensor-memory loads and its
  // arithmetic fit without spilling to local memory.
  if (warp < P_EPI_WARP0) {
  reg_dealloc<40>();
  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m_blk = (int)(tile % tiles_m);
        const int n_blk = (int)((tile / tiles_m) % tiles_n);
        const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        const int n0 = n_blk * bn + (int)rank * (bn / 2);
        const int kb_end = tile_k_blocks(m_blk, n_blk);
        for (int kb = 0; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          // the even CTA arms its barrier for the bytes of both CTAs
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], stage_tx_bytes);
          const uint32_t leader_full = map_to_cta(&full_bar[stage], 0);
          tma_load_3d_pair(smem_a + stage * P_A_BYTES, &map_a, leader_full, kb * k_elems_per_stage, m0, b);
          tma_load_3d_pair(smem_b + stage * P_B_BYTES, &map_b, leader_full, kb * k_elems_per_stage, n0, b);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ----------------
    // The whole role is compiled once per operand kind, so that nothing but the barrier wait separates the
    // MMA instructions of consecutive stages.
    auto mma_role = [&](auto kind_tag) {
      constexpr bool F8 = decltype(kind_tag)::value;
      const uint32_t idesc = p.idesc;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int kb_end = tile_k_blocks((int)(tile % tiles_m), (int)((tile / tiles_m) % tiles_n));
        if (kb_end == 0) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_stage<F8, true>(tmem_acc, smem_u32(smem_a + stage * P_A_BYTES), smem_u32(smem_b + stage * P_B_BYTES),
                                idesc, kb > 0);
          mma_commit_pair(&empty_bar[stage], 0x3);  // both CTAs may refill this stage
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit_pair(&acc_full[acc], 0x3);  // both CTAs' epilogues may read their rows
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    };
    if (lane == 0 && rank == 0) {
      if (p.kind_f8) mma_role(std::true_type{});
      else mma_role(std::false_type{});
    }
  }
  } else {
    reg_alloc<232>();
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quarter = warp & 3;
    const int chalf = (warp - P_EPI_WARP0) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;   // which staging buffer this warp fills next
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      if (tile_k_blocks(m_blk, n_blk) == 0) continue;
      prefetch_residual(p, m_blk * 2 * BM + (int)rank * BM + quarter * 32, lane, n_blk * bn, b, chalf * (bn / 2),
                        (chalf + 1) * (bn / 2));
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
      epilogue_warp_tile<OUT_DT, P_EPI_BUFS>(p, &map_c, taddr, epi_stage + (warp - P_EPI_WARP0) * (P_EPI_BUFS * 32 * 128), epi_buf,
                                             m_blk * 2 * BM + (int)rank * BM + quarter * 32,
                         lane, n_blk * bn, b, has_alpha, alpha, chalf * (bn / 2), (chalf + 1) * (bn / 2));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (warp >= P_EPI_WARP0 && lane == 0) tma_store_wait_read();   // staging buffers stay valid until their stores have read them
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  cluster_sync();  // neither CTA leaves while the other may still signal its barriers or read its tiles
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Block-scaled (MX) operands dequantized inside the main loop.  The GEMM of
// linear_mx / matmul_mx multiplies bf16(code * scale) values, the scale shared by
// `block` consecutive elements of K.  This kernel is the CTA-pair kernel above with
// one more role: four "transform" warps per CTA take each stage as TMA delivers it
// (the raw codes), multiply it in place by the rows' block scales (mul.rn.bf16x2:
// the one bfloat16 rounding the separate read-back pass applies) and only then hand
// it to the MMA thread.  The dequantized operands never exist in device memory.
//   full_bar[s]  : per CTA; its own producer arms it with the CTA's own bytes
//   ready_bar[s] : lives in the even CTA; 8 arrivals (4 transform warps x 2 CTAs)
//   empty_bar[s], acc_full, acc_empty: as in the pair kernel
// A transform thread owns one row of the CTA's A tile and the same row of its B half; a row
// of a stage is eight 16-byte chunks, chunk c of row r sitting at ((c ^ (r & 7)) << 4) under
// the 128-byte swizzle.  Every stage costs a tile's CTA 64 KB of shared-memory traffic on top of
// the 32 KB the tensor core reads, and is repeated for every tile that shares the operand rows: this
// kernel wins where the read-back pass it replaces is a large part of the time (weight-bound
// shapes, a single wave of tiles) and loses on compute-bound ones; the caller chooses.
// ---------------------------------------------------------------------------
constexpr int MX_XFORM_WARPS = 4;
constexpr int MX_ROWS_PER_THREAD = 128 / (32 * MX_XFORM_WARPS);
// Four warpgroups: {TMA warp, MMA warp, two idle warps}, two epilogue warpgroups (one per half of the
// tile's columns; a warp's position in its group is its tensor-memory lane quarter), the transform warps.
// The kernel starts with 128 registers per thread and redistributes them by role: 40 / 184 / 184 / 104.
constexpr int MX_THREADS = 512;
constexpr int MX_EPI_WARP0 = 4;            // first epilogue warp
constexpr int MX_XFORM_WARP0 = 12;         // first transform warp

struct MxScales {
  const __nv_bfloat16* a;   // [batch, M, lds_a] or null (operand taken as is)
  const __nv_bfloat16* b;   // [batch, N, lds_b] or null
  int64_t lds_a, lds_b, stride_a, stride_b;
  int shift;                // block size = 1 << shift elements of K
};

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Scales of one row for the stage starting at element k0: one per 16-byte chunk, duplicated into
// both halves of a word.  `count` scales exist in the row; indices past the end (the zero-filled
// tail of K) reuse the last one.
__device__ __forceinline__ void load_row_scales(const __nv_bfloat16* row, int64_t count, int k0, int shift,
                                                uint32_t (&s)[8]) {
  const unsigned short* r16 = reinterpret_cast<const unsigned short*>(row);
  if (shift >= 6) {
    int64_t i = k0 >> shift;
    if (i >= count) i = count - 1;
    const uint32_t v = __ldg(r16 + i);
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = v | (v << 16);
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int64_t i = (k0 + 8 * c) >> shift;
      if (i >= count) i = count - 1;
      const uint32_t v = __ldg(r16 + i);
      s[c] = v | (v << 16);
    }
  }
}

// The same from a 16-byte group of eight consecutive scales of the row (`q`, scales 8g .. 8g + 7, loaded
// once per group instead of once per chunk): `sidx` is the index of the stage's first scale.
__device__ __forceinline__ uint32_t dup_half(uint32_t w, int hi) { return __byte_perm(w, 0, hi ? 0x3232 : 0x1010); }
__device__ __forceinline__ uint32_t pick_word(const uint4& q, int i) {
  return i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w;
}
__device__ __forceinline__ void chunk_scales(const uint4& q, int sidx, int shift, uint32_t (&s)[8]) {
  const int base = sidx & 7;
  const uint32_t w0 = pick_word(q, base >> 1);
  if (shift == 3) {          // 8 scales per stage: the whole group
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = dup_half(pick_word(q, c >> 1), c & 1);
  } else if (shift == 4) {   // 4 per stage: two words
    const uint32_t w1 = pick_word(q, (base >> 1) + 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = dup_half(c < 4 ? w0 : w1, (c >> 1) & 1);
  } else if (shift == 5) {   // 2 per stage: one word
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = dup_half(w0, c >> 2);
  } else {                   // one scale for the stage (and for 2^(shift-6) stages in a row)
    const uint32_t v = dup_half(w0, base & 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = v;
  }
}

__device__ __forceinline__ void scale_row_in_place(uint8_t* tile, int r, const uint32_t (&s)[8]) {
  uint8_t* row = tile + r * BK_BYTES;
  uint4 v[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint4*>(row + ((c ^ (r & 7)) << 4));
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    v[c].x = mul_bf16x2(v[c].x, s[c]);
    v[c].y = mul_bf16x2(v[c].y, s[c]);
    v[c].z = mul_bf16x2(v[c].z, s[c]);
    v[c].w = mul_bf16x2(v[c].w, s[c]);
    *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = v[c];
  }
}

template <int OUT_DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MX_THREADS, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ GemmParams p, const __grid_constant__ MxScales sc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + P_STAGES * P_A_BYTES;
  uint8_t* epi_stage = smem + P_STAGES * (P_A_BYTES + P_B_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * (P_A_BYTES + P_B_BYTES) + P_EPI_BUFS * EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                        // [P_STAGES] per CTA
  uint64_t* empty_bar = bars + P_STAGES;            // [P_STAGES]
  uint64_t* ready_bar = bars + 2 * P_STAGES;        // [P_STAGES] (used in the even CTA)
  uint64_t* acc_full = bars + 3 * P_STAGES;         // [2]
  uint64_t* acc_empty = bars + 3 * P_STAGES + 2;    // [2] (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * P_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int bn = p.bn;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + bn - 1) / bn;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  constexpr int k_per_stage = BK_BYTES / 2;
  const int k_blocks = (p.K + k_per_stage - 1) / k_per_stage;
  const uint32_t stage_tx_bytes = (uint32_t)(P_A_BYTES + (bn / 2) * BK_BYTES);   // this CTA's own loads

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&ready_bar[s], 2 * MX_XFORM_WARPS);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < MX_EPI_WARP0) {
  reg_dealloc<40>();
  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m_blk = (int)(tile % tiles_m);
        const int n_blk = (int)((tile / tiles_m) % tiles_n);
        const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        const int n0 = n_blk * bn + (int)rank * (bn / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], stage_tx_bytes);
          tma_load_3d(smem_a + stage * P_A_BYTES, &map_a, &full_bar[stage], kb * k_per_stage, m0, b);
          tma_load_3d(smem_b + stage * P_B_BYTES, &map_b, &full_bar[stage], kb * k_per_stage, n0, b);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&ready_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem_a + stage * P_A_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + stage * P_B_BYTES);
#pragma unroll
          for (int k = 0; k < BK_BYTES / MMA_K_BYTES; ++k) {
            const uint64_t da = smem_desc_k_major_sw128(a_addr + k * MMA_K_BYTES);
            const uint64_t db = smem_desc_k_major_sw128(b_addr + k * MMA_K_BYTES);
            mma_f16_ss_pair(tmem_acc, da, db, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty_bar[stage], 0x3);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit_pair(&acc_full[acc], 0x3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  }
  } else if (warp < MX_XFORM_WARP0) {
    reg_alloc<184>();
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quarter = warp & 3;
    const int chalf = (warp - MX_EPI_WARP0) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
      epilogue_warp_tile<OUT_DT, P_EPI_BUFS>(p, &map_c, taddr, epi_stage + (warp - MX_EPI_WARP0) * (P_EPI_BUFS * 32 * 128), epi_buf,
                                             m_blk * 2 * BM + (int)rank * BM + quarter * 32, lane, n_blk * bn, b,
                                             has_alpha, alpha, chalf * (bn / 2), (chalf + 1) * (bn / 2));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    reg_dealloc<104>();
    // ------------------------------ transform (both CTAs) ---------------------
    const int t = threadIdx.x - MX_XFORM_WARP0 * 32;   // row of the tile (and the next after 32 x warps rows)
    const int64_t count_a = sc.lds_a, count_b = sc.lds_b;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      const int m0 = m_blk * 2 * BM + (int)rank * BM;
      const int n0 = n_blk * bn + (int)rank * (bn / 2);
      const __nv_bfloat16* row_a[MX_ROWS_PER_THREAD];
      const __nv_bfloat16* row_b[MX_ROWS_PER_THREAD];
#pragma unroll
      for (int h = 0; h < MX_ROWS_PER_THREAD; ++h) {
        const int r = t + 32 * MX_XFORM_WARPS * h;
        row_a[h] = (sc.a != nullptr && m0 + r < p.M) ? sc.a + b * sc.stride_a + (int64_t)(m0 + r) * sc.lds_a : nullptr;
        row_b[h] = (sc.b != nullptr && r < bn / 2 && n0 + r < p.N) ? sc.b + b * sc.stride_b + (int64_t)(n0 + r) * sc.lds_b
                                                                  : nullptr;
      }
      // Scale rows whose length is a multiple of eight are read 16 bytes (eight scales) at a time, one
      // group ahead of its use; other lengths take one 2-byte load per chunk.
      const bool grouped = ((count_a | count_b) & 7) == 0 &&
                           ((reinterpret_cast<uintptr_t>(sc.a) | reinterpret_cast<uintptr_t>(sc.b)) & 15) == 0;
      uint4 cur[2 * MX_ROWS_PER_THREAD] = {}, nxt[2 * MX_ROWS_PER_THREAD] = {};
      int cur_grp = -1;
      auto load_group = [&](uint4 (&dst)[2 * MX_ROWS_PER_THREAD], int grp) {
#pragma unroll
        for (int h = 0; h < MX_ROWS_PER_THREAD; ++h) {
          if (row_a[h] && (int64_t)grp * 8 < count_a) dst[h] = __ldg(reinterpret_cast<const uint4*>(row_a[h]) + grp);
          if (row_b[h] && (int64_t)grp * 8 < count_b) dst[MX_ROWS_PER_THREAD + h] = __ldg(reinterpret_cast<const uint4*>(row_b[h]) + grp);
        }
      };
      if (grouped) load_group(nxt, 0);
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int k0 = kb * k_per_stage;
        const int sidx = k0 >> sc.shift;
        if (grouped && (sidx >> 3) != cur_grp) {
          cur_grp = sidx >> 3;
#pragma unroll
          for (int i = 0; i < 2 * MX_ROWS_PER_THREAD; ++i) cur[i] = nxt[i];
          load_group(nxt, cur_grp + 1);
        }
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&full_bar[stage], phase, abort_flag))) { ok = false; break; }
        // one row at a time: the eight chunk scales live only while their row is in registers
#pragma unroll
        for (int h = 0; h < MX_ROWS_PER_THREAD; ++h) {
          const int r = t + 32 * MX_XFORM_WARPS * h;
          if (row_a[h]) {
            uint32_t s8[8];
            if (grouped) chunk_scales(cur[h], sidx, sc.shift, s8);
            else load_row_scales(row_a[h], count_a, k0, sc.shift, s8);
            scale_row_in_place(smem_a + stage * P_A_BYTES, r, s8);
          }
          if (row_b[h]) {
            uint32_t s8[8];
            if (grouped) chunk_scales(cur[MX_ROWS_PER_THREAD + h], sidx, sc.shift, s8);
            else load_row_scales(row_b[h], count_b, k0, sc.shift, s8);
            scale_row_in_place(smem_b + stage * P_B_BYTES, r, s8);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&ready_bar[stage], 0));
        if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  if (warp >= MX_EPI_WARP0 && warp < MX_XFORM_WARP0 && lane == 0) tma_store_wait_read();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// NVFP4 block-scaled GEMM: packed e2m1 operands (two per byte, K-contiguous), one
// ue4m3 scale per 16 elements, multiplied by the tensor cores' native
// kind::mxf4nvf4 MMA (K = 64 per instruction).  128x128 tiles, one CTA per SM.
// A stage holds 256 elements of K: 128-byte operand rows (TMA, 128-byte swizzle)
// plus four 512-byte scale tiles per operand (bulk copies).  The MMA thread
// moves a stage's scale tiles into tensor memory (tcgen05.cp) right before it
// issues the stage's MMAs; tcgen05 operations of one thread execute in order, so
// the next stage's copies cannot overtake MMAs still reading the scales.
// Tensor-memory columns: [0,256) two accumulators, [256,272) A scales,
// [272,288) B scales.
// ---------------------------------------------------------------------------
constexpr int Q_BN = 128;
constexpr int Q_STAGES = 5;
constexpr int Q_A_BYTES = 128 * BK_BYTES;     // 16 KB
constexpr int Q_B_BYTES = Q_BN * BK_BYTES;    // 16 KB
constexpr int Q_SF_BYTES = 4 * 512;           // 128 rows x 16 scales
constexpr int Q_STAGE_BYTES = Q_A_BYTES + Q_B_BYTES + 2 * Q_SF_BYTES;
constexpr size_t Q_SMEM_BYTES = 1024 + Q_STAGES * Q_STAGE_BYTES + 256 + EPI_STAGE_BYTES;
constexpr uint32_t Q_SFA_COL = 256, Q_SFB_COL = 272;

struct ScaledOperands {
  const uint8_t* sfa;   // scale tiles of A: [batch][M/128][K/64][512]
  const uint8_t* sfb;   // scale tiles of B: [batch][N/128][K/64][512]
  int64_t sfa_batch_stride, sfb_batch_stride;  // bytes
};

template <int OUT_DT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ GemmParams p,
                  ScaledOperands sf) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + Q_STAGES * Q_A_BYTES;
  uint8_t* smem_sfa = smem_b + Q_STAGES * Q_B_BYTES;
  uint8_t* smem_sfb = smem_sfa + Q_STAGES * Q_SF_BYTES;
  uint8_t* epi_stage = smem + Q_STAGES * Q_STAGE_BYTES;   // 1024-byte aligned: TMA stores read it with the 128-byte swizzle
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Q_STAGES * Q_STAGE_BYTES + EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Q_STAGES;
  uint64_t* acc_full = bars + 2 * Q_STAGES;
  uint64_t* acc_empty = bars + 2 * Q_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Q_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + Q_BN - 1) / Q_BN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  const int k64_total = p.K / 64;               // K is a multiple of 64
  const int k_blocks = (k64_total + 3) / 4;     // stages of 256 elements

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = (int)(tile % tiles_m);
        const int n_blk = (int)((tile / tiles_m) % tiles_n);
        const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
        const uint8_t* sfa_row = sf.sfa + (int64_t)b * sf.sfa_batch_stride + (int64_t)m_blk * k64_total * 512;
        const uint8_t* sfb_row = sf.sfb + (int64_t)b * sf.sfb_batch_stride + (int64_t)n_blk * k64_total * 512;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          const int steps = min(4, k64_total - kb * 4);
          const uint32_t sf_bytes = (uint32_t)steps * 512u;
          mbar_arrive_expect_tx(&full_bar[stage], Q_A_BYTES + Q_B_BYTES + 2 * sf_bytes);
          // operand rows are K/2 bytes; a stage is 128 bytes of each row
          tma_load_3d(smem_a + stage * Q_A_BYTES, &map_a, &full_bar[stage], kb * BK_BYTES, m_blk * BM, b);
          tma_load_3d(smem_b + stage * Q_B_BYTES, &map_b, &full_bar[stage], kb * BK_BYTES, n_blk * Q_BN, b);
          bulk_load(smem_sfa + stage * Q_SF_BYTES, sfa_row + (int64_t)kb * 4 * 512, sf_bytes, &full_bar[stage]);
          bulk_load(smem_sfb + stage * Q_SF_BYTES, sfb_row + (int64_t)kb * 4 * 512, sf_bytes, &full_bar[stage]);
          if (++stage == Q_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * Q_BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const int steps = min(4, k64_total - kb * 4);
          const uint32_t a_addr = smem_u32(smem_a + stage * Q_A_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + stage * Q_B_BYTES);
          const uint32_t sfa_addr = smem_u32(smem_sfa + stage * Q_SF_BYTES);
          const uint32_t sfb_addr = smem_u32(smem_sfb + stage * Q_SF_BYTES);
          for (int k = 0; k < steps; ++k) {
            tmem_copy_sf(tmem_base + Q_SFA_COL + 4 * k, smem_desc_sf_chunk(sfa_addr + k * 512));
            tmem_copy_sf(tmem_base + Q_SFB_COL + 4 * k, smem_desc_sf_chunk(sfb_addr + k * 512));
          }
          for (int k = 0; k < steps; ++k) {
            const uint64_t da = smem_desc_k_major_sw128(a_addr + k * MMA_K_BYTES);
            const uint64_t db = smem_desc_k_major_sw128(b_addr + k * MMA_K_BYTES);
            mma_nvfp4_ss(tmem_acc, da, db, p.idesc, tmem_base + Q_SFA_COL + 4 * k, tmem_base + Q_SFB_COL + 4 * k,
                         (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);
          if (++stage == Q_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;   // which staging buffer this warp fills next
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)(acc * Q_BN) + ((uint32_t)(quarter * 32) << 16);
      epilogue_warp_tile<OUT_DT>(p, &map_c, taddr, epi_stage + (warp - 2) * (32 * 128), epi_buf, m_blk * BM + quarter * 32, lane, n_blk * Q_BN, b,
                         has_alpha, alpha, chalf * (Q_BN / 2), (chalf + 1) * (Q_BN / 2));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait_read();   // staging buffers stay valid until their stores have read them
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// NVFP4 block-scaled GEMM on CTA pairs: two CTAs (a cluster of 2) share a 256x256 tile.
// Each CTA loads its 128 rows of A, its 128 of the tile's 256 B rows, the block scales of its
// A rows and the block scales of all 256 B rows (every CTA's tensor core multiplies its rows by
// all of B); the even CTA's thread issues tcgen05.cp.cta_group::2 (each CTA's scale tiles go
// from its own shared memory into its own tensor memory) and tcgen05.mma.cta_group::2
// kind::mxf4nvf4 (M = 256, N = 256, K = 64).  Per byte fetched from L2 this does twice the
// arithmetic of the 128x128 single-CTA kernel.
//
// Tensor memory (512 columns per CTA) cannot hold two 256-column accumulators next to the scale
// columns, so the two accumulators overlap: accumulator 0 is columns [0, 256), accumulator 1 is
// [192, 448), scales live in [448, 512).  The epilogue of a tile drains the 64 shared columns
// first and says so on `ovl_free`; the next tile's first MMA waits for that instead of for the
// whole accumulator, so only that short drain is not overlapped with tensor work.
//   full barrier  : in the even CTA; both CTAs' operand loads complete on it
//   sf_full       : in the even CTA; both CTAs' scale loads complete on it.  The scale tiles of a stage are
//                   small and land before its operands, so the MMA thread copies them into tensor memory
//                   (tcgen05.cp, about 40 ns each, twelve per stage, in order with the MMAs) while it would
//                   otherwise sit waiting for the stage's operands: the kernel is bound by the operand feed
//                   from L2, and the copies fill the tensor pipe's idle time instead of adding to it
//   empty barrier : per CTA, released by tcgen05.commit sent to both CTAs
//   acc_full      : per CTA, same mechanism
//   acc_empty     : in the even CTA; 16 arrivals (8 epilogue warps x 2 CTAs)
//   ovl_free      : in the even CTA; 8 arrivals (the 4 warps that drain the shared columns x 2 CTAs)
// ---------------------------------------------------------------------------
constexpr int QP_STAGES = 5;
constexpr int QP_A_BYTES = 128 * BK_BYTES;      // 16 KB: this CTA's A rows, 256 elements of K
constexpr int QP_B_BYTES = 128 * BK_BYTES;      // 16 KB: this CTA's half of the tile's B rows
constexpr int QP_SFA_BYTES = 4 * 512;           // 128 rows x 16 scales
constexpr int QP_SFB_BYTES = 8 * 512;           // 256 rows x 16 scales
constexpr int QP_STAGE_BYTES = QP_A_BYTES + QP_B_BYTES + QP_SFA_BYTES + QP_SFB_BYTES;
constexpr size_t QP_SMEM_BYTES = 1024 + QP_STAGES * QP_STAGE_BYTES + 256 + EPI_STAGE_BYTES;
constexpr uint32_t QP_ACC1_COL = 192, QP_SF_COL = 448;   // scales: four 16-column groups, one per K64 step of a stage
constexpr int QP_OVERLAP = 64;                  // columns shared by the two accumulators

template <int OUT_DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       const __grid_constant__ CUtensorMap map_c, const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + QP_STAGES * QP_A_BYTES;
  uint8_t* smem_sfa = smem_b + QP_STAGES * QP_B_BYTES;
  uint8_t* smem_sfb = smem_sfa + QP_STAGES * QP_SFA_BYTES;
  uint8_t* epi_stage = smem + QP_STAGES * QP_STAGE_BYTES;   // 1024-byte aligned (the stage size is a multiple of 1024)
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [QP_STAGES] (used in the even CTA)
  uint64_t* empty_bar = bars + QP_STAGES;             // [QP_STAGES]
  uint64_t* acc_full = bars + 2 * QP_STAGES;          // [2]
  uint64_t* acc_empty = bars + 2 * QP_STAGES + 2;     // [2] (used in the even CTA)
  uint64_t* ovl_free = bars + 2 * QP_STAGES + 4;      // [2] (used in the even CTA)
  uint64_t* sf_full = bars + 2 * QP_STAGES + 6;       // [QP_STAGES] (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * QP_STAGES + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  const int k64_total = p.K / 64;               // K is a multiple of 64
  const int k_blocks = (k64_total + 3) / 4;     // stages of 256 elements
  const int m_blocks128 = (p.M + 127) / 128;    // 128-row scale blocks per batch entry
  const int n_blocks128 = (p.N + 127) / 128;
  const uint32_t operand_tx_bytes = 2u * (uint32_t)(QP_A_BYTES + QP_B_BYTES);
  const uint32_t scale_tx_bytes = 2u * (uint32_t)(QP_SFA_BYTES + QP_SFB_BYTES);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < QP_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&sf_full[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);
      mbar_init(&ovl_free[a], EPI_WARPS);   // 4 warps per CTA
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      prefetch_tensormap(&map_sfa);
      prefetch_tensormap(&map_sfb);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m_blk = (int)(tile % tiles_m);
        const int n_blk = (int)((tile / tiles_m) % tiles_n);
        const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        const int n0 = n_blk * BN + (int)rank * (BN / 2);
        const int sfa_blk = b * m_blocks128 + m_blk * 2 + (int)rank;   // this CTA's 128 rows of A
        const int sfb_blk = b * n_blocks128 + n_blk * 2;               // both 128-row blocks of the B tile
        // a scale block past the last row block of its batch entry does not exist: reading the next entry's
        // (or nothing) is harmless, its operand rows are zero-filled -- but keep the coordinate in range
        const bool sfa_in = m_blk * 2 + (int)rank < m_blocks128;
        const bool sfb1_in = n_blk * 2 + 1 < n_blocks128;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (rank == 0) {
            mbar_arrive_expect_tx(&sf_full[stage], scale_tx_bytes);
            mbar_arrive_expect_tx(&full_bar[stage], operand_tx_bytes);
          }
          const uint32_t leader_sf = map_to_cta(&sf_full[stage], 0);
          const uint32_t leader_full = map_to_cta(&full_bar[stage], 0);
          // scale tiles first: [row block][K / 64][128 words]; a box is four K64 steps of one row block (2 KB)
          tma_load_3d_pair(smem_sfa + stage * QP_SFA_BYTES, &map_sfa, leader_sf, 0, kb * 4,
                           sfa_in ? sfa_blk : 0x7FFFFFF0);
          tma_load_3d_pair(smem_sfb + stage * QP_SFB_BYTES, &map_sfb, leader_sf, 0, kb * 4, sfb_blk);
          tma_load_3d_pair(smem_sfb + stage * QP_SFB_BYTES + QP_SFA_BYTES, &map_sfb, leader_sf, 0, kb * 4,
                           sfb1_in ? sfb_blk + 1 : 0x7FFFFFF0);
          tma_load_3d_pair(smem_a + stage * QP_A_BYTES, &map_a, leader_full, kb * BK_BYTES, m0, b);
          tma_load_3d_pair(smem_b + stage * QP_B_BYTES, &map_b, leader_full, kb * BK_BYTES, n0, b);
          if (++stage == QP_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int64_t done = 0;   // tiles issued so far
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs, ++done) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        // the other accumulator's shared columns must have been read out of tensor memory: its tile was
        // issued just before this one, as use number (done - 1) / 2 of that buffer
        if (done > 0 && !mbar_wait(&ovl_free[acc ^ 1], (uint32_t)(((done - 1) >> 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + (acc ? QP_ACC1_COL : 0u);
        for (int kb = 0; kb < k_blocks; ++kb) {
          const int steps = min(4, k64_total - kb * 4);
          const uint32_t a_addr = smem_u32(smem_a + stage * QP_A_BYTES);
          const uint32_t b_addr = smem_u32(smem_b + stage * QP_B_BYTES);
          const uint32_t sfa_addr = smem_u32(smem_sfa + stage * QP_SFA_BYTES);
          const uint32_t sfb_addr = smem_u32(smem_sfb + stage * QP_SFB_BYTES);
          // One 16-column group of tensor memory per K64 step: [B scales 8 | A scales 4 | unused 4].  The copies
          // are issued as soon as the scale tiles are there, ahead of the wait for the operands; tcgen05
          // operations of one thread execute in order, so they cannot overtake the previous stage's MMAs.
          if (!mbar_wait(&sf_full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          for (int k = 0; k < steps; ++k) {
            const uint32_t grp = tmem_base + QP_SF_COL + 16 * k;
            tmem_copy_sf_pair(grp, smem_desc_sf_chunk(sfb_addr + k * 512));
            tmem_copy_sf_pair(grp + 4, smem_desc_sf_chunk(sfb_addr + QP_SFA_BYTES + k * 512));
            tmem_copy_sf_pair(grp + 8, smem_desc_sf_chunk(sfa_addr + k * 512));
          }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          for (int k = 0; k < steps; ++k) {
            const uint32_t grp = tmem_base + QP_SF_COL + 16 * k;
            const uint64_t da = smem_desc_k_major_sw128(a_addr + k * MMA_K_BYTES);
            const uint64_t db = smem_desc_k_major_sw128(b_addr + k * MMA_K_BYTES);
            mma_nvfp4_ss_pair(tmem_acc, da, db, p.idesc, grp + 8, grp, (kb > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty_bar[stage], 0x3);
          if (++stage == QP_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit_pair(&acc_full[acc], 0x3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (acc ? QP_ACC1_COL : 0u) + ((uint32_t)(quarter * 32) << 16);
      const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;
      uint8_t* stage = epi_stage + (warp - 2) * (32 * 128);
      // Tile columns shared with the other accumulator: the last 64 of accumulator 0, the first 64 of
      // accumulator 1.  The four warps of column half 0 drain them first, announce it, then take 64 more
      // columns; the warps of half 1 take the 128 columns at the other end.
      const int ovl0 = acc ? 0 : BN - QP_OVERLAP;
      int seg_begin[2], seg_end[2];
      if (chalf == 0) {
        seg_begin[0] = ovl0;
        seg_begin[1] = acc ? QP_OVERLAP : BN - 2 * QP_OVERLAP;
        seg_end[0] = seg_begin[0] + QP_OVERLAP;
        seg_end[1] = seg_begin[1] + QP_OVERLAP;
      } else {
        seg_begin[0] = acc ? BN / 2 : 0;
        seg_end[0] = seg_begin[0] + BN / 2;
        seg_begin[1] = seg_end[1] = 0;
      }
#pragma unroll 1
      for (int seg = 0; seg < 2 - chalf; ++seg) {
        epilogue_warp_tile<OUT_DT, 1>(p, &map_c, taddr, stage, epi_buf, row0, lane, n_blk * BN, b, has_alpha, alpha,
                                      seg_begin[seg], seg_end[seg]);
        if (chalf == 0 && seg == 0) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(&ovl_free[acc], 0));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait_read();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// NVFP4 GEMM on CTA pairs, scale factors written into tensor memory by warps.
// The kernel above moves a stage's twelve scale tiles with tcgen05.cp from the MMA thread; those
// copies execute in the tensor pipe in order with the MMAs and cost as much time as the MMAs do.
// Here four "scale" warps per CTA read the tiles from shared memory (one 16-byte row per lane)
// and store them into tensor memory with tcgen05.st -- the same lane / column placement as the
// 32x128b.warpx4 copy, each warp writing its own lane quadrant -- into one of two 64-column
// buffers, ahead of the MMAs that read them; the MMA thread only issues MMAs.
//   Tensor memory: accumulator 0 at [0,256), accumulator 1 at [128,384) (they share 128 columns:
//   the half the epilogue warps drain first), scale buffers at [384,448) and [448,512),
//   each four 16-column groups [B scales 8 | A scales 4 | unused 4], one per K64 step.
//   sf_full[s]   : per CTA, its own scale tiles of stage s have landed
//   full_bar[s]  : even CTA; besides the operand bytes it counts 8 arrivals (4 scale warps x 2 CTAs): the
//                  stage's scales are in tensor memory.  A scale buffer is free again when the stage that used
//                  it two stages ago completes its empty barrier, so the MMA thread's loop is wait, four MMAs,
//                  one commit, exactly as in the FP8 kernel: with a barrier pair of their own for the scales
//                  (one more wait and one more commit per stage in that thread) the kernel was a fifth slower.
//   the other barriers as in the kernel above
// Four warpgroups as in gemm_mx_pair_kernel: registers 40 / 184 / 184 / 104.
// ---------------------------------------------------------------------------
constexpr int QS_THREADS = 512;
constexpr int QS_EPI_WARP0 = 4, QS_SF_WARP0 = 12, QS_SF_WARPS = 4;
constexpr uint32_t QS_ACC1_COL = 128, QS_SF_COL = 384, QS_SF_BUF_COLS = 64;
constexpr int QS_OVERLAP = 128;

__device__ __forceinline__ void tmem_st_32x32_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int OUT_DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(QS_THREADS, 1)
gemm_nvfp4_sfw_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                      const __grid_constant__ CUtensorMap map_c, const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + QP_STAGES * QP_A_BYTES;
  uint8_t* smem_sfa = smem_b + QP_STAGES * QP_B_BYTES;
  uint8_t* smem_sfb = smem_sfa + QP_STAGES * QP_SFA_BYTES;
  uint8_t* epi_stage = smem + QP_STAGES * QP_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [QP_STAGES] (used in the even CTA)
  uint64_t* empty_bar = bars + QP_STAGES;             // [QP_STAGES]
  uint64_t* sf_full = bars + 2 * QP_STAGES;           // [QP_STAGES] per CTA
  uint64_t* acc_full = bars + 3 * QP_STAGES;          // [2]
  uint64_t* acc_empty = bars + 3 * QP_STAGES + 2;     // [2] (used in the even CTA)
  uint64_t* ovl_free = bars + 3 * QP_STAGES + 4;      // [2] (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * QP_STAGES + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = (int64_t)tiles_m * tiles_n * p.batch;
  const int k64_total = p.K / 64;
  const int k_blocks = (k64_total + 3) / 4;
  const int m_blocks128 = (p.M + 127) / 128;
  const int n_blocks128 = (p.N + 127) / 128;
  const uint32_t operand_tx_bytes = 2u * (uint32_t)(QP_A_BYTES + QP_B_BYTES);
  const uint32_t scale_tx_bytes = (uint32_t)(QP_SFA_BYTES + QP_SFB_BYTES);   // this CTA's own tiles

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < QP_STAGES; ++s) {
      mbar_init(&full_bar[s], 1 + 2 * QS_SF_WARPS);   // the producer's expect_tx + the scale warps of both CTAs
      mbar_init(&sf_full[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);
      mbar_init(&ovl_free[a], 2 * EPI_WARPS);  // every epilogue warp of both CTAs
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < QS_EPI_WARP0) {
    reg_dealloc<40>();
    if (warp == 0) {
      // ------------------------------ TMA producer (both CTAs) ------------------
      if (lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        prefetch_tensormap(&map_sfa);
        prefetch_tensormap(&map_sfb);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
          const int m_blk = (int)(tile % tiles_m);
          const int n_blk = (int)((tile / tiles_m) % tiles_n);
          const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
          const int m0 = m_blk * 2 * BM + (int)rank * BM;
          const int n0 = n_blk * BN + (int)rank * (BN / 2);
          const int sfa_blk = b * m_blocks128 + m_blk * 2 + (int)rank;
          const int sfb_blk = b * n_blocks128 + n_blk * 2;
          const bool sfa_in = m_blk * 2 + (int)rank < m_blocks128;
          const bool sfb1_in = n_blk * 2 + 1 < n_blocks128;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(&sf_full[stage], scale_tx_bytes);
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], operand_tx_bytes);
            const uint32_t leader_full = map_to_cta(&full_bar[stage], 0);
            tma_load_3d(smem_sfa + stage * QP_SFA_BYTES, &map_sfa, &sf_full[stage], 0, kb * 4,
                        sfa_in ? sfa_blk : 0x7FFFFFF0);
            tma_load_3d(smem_sfb + stage * QP_SFB_BYTES, &map_sfb, &sf_full[stage], 0, kb * 4, sfb_blk);
            tma_load_3d(smem_sfb + stage * QP_SFB_BYTES + QP_SFA_BYTES, &map_sfb, &sf_full[stage], 0, kb * 4,
                        sfb1_in ? sfb_blk + 1 : 0x7FFFFFF0);
            tma_load_3d_pair(smem_a + stage * QP_A_BYTES, &map_a, leader_full, kb * BK_BYTES, m0, b);
            tma_load_3d_pair(smem_b + stage * QP_B_BYTES, &map_b, leader_full, kb * BK_BYTES, n0, b);
            if (++stage == QP_STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer (even CTA only) ----------------
      if (lane == 0 && rank == 0) {
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        int64_t done = 0;   // tiles issued so far
        uint32_t it = 0;    // stages issued so far: scale buffer it & 1, its use number it >> 1
        const uint32_t idesc = p.idesc;
        for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs, ++done) {
          if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          if (done > 0 && !mbar_wait(&ovl_free[acc ^ 1], (uint32_t)(((done - 1) >> 1) & 1), abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t tmem_acc = tmem_base + (acc ? QS_ACC1_COL : 0u);
          for (int kb = 0; kb < k_blocks; ++kb, ++it) {
            const int steps = min(4, k64_total - kb * 4);
            const uint32_t buf = it & 1u;
            const uint32_t a_addr = smem_u32(smem_a + stage * QP_A_BYTES);
            const uint32_t b_addr = smem_u32(smem_b + stage * QP_B_BYTES);
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }   // operands landed, scales stored
            tc_fence_after_sync();
            auto issue = [&](int k) {
              const uint32_t grp = tmem_base + QS_SF_COL + buf * QS_SF_BUF_COLS + 16 * k;
              const uint64_t da = smem_desc_k_major_sw128(a_addr + k * MMA_K_BYTES);
              const uint64_t db = smem_desc_k_major_sw128(b_addr + k * MMA_K_BYTES);
              mma_nvfp4_ss_pair(tmem_acc, da, db, idesc, grp + 8, grp, (kb > 0 || k > 0) ? 1u : 0u);
            };
            if (steps == 4) {   // a full stage: four instructions as straight-line code
#pragma unroll
              for (int k = 0; k < 4; ++k) issue(k);
            } else {
              for (int k = 0; k < steps; ++k) issue(k);
            }
            mma_commit_pair(&empty_bar[stage], 0x3);   // frees the stage and, for the scale warps, scale buffer `buf`
            if (++stage == QP_STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          mma_commit_pair(&acc_full[acc], 0x3);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  } else if (warp < QS_SF_WARP0) {
    reg_alloc<184>();
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quarter = warp & 3;
    const int chalf = (warp - QS_EPI_WARP0) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t epi_buf = 0;
    const bool has_alpha = p.alpha != nullptr;
    const float alpha = has_alpha ? load_param(p.alpha, 0, p.alpha_dt) : 1.0f;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = (int)(tile % tiles_m);
      const int n_blk = (int)((tile / tiles_m) % tiles_n);
      const int b = (int)(tile / ((int64_t)tiles_m * tiles_n));
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[acc], acc_phase, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (acc ? QS_ACC1_COL : 0u) + ((uint32_t)(quarter * 32) << 16);
      const int row0 = m_blk * 2 * BM + (int)rank * BM + quarter * 32;
      uint8_t* stage = epi_stage + (warp - QS_EPI_WARP0) * (32 * 128);
      // The tile's columns shared with the other accumulator (the last 128 of accumulator 0, the first 128 of
      // accumulator 1) are drained first, 64 by each column half, and announced; the next tile's MMAs may
      // then start while the warps take the other 128 columns.
      const int shared0 = acc ? 0 : BN - QS_OVERLAP;
      const int other0 = (BN - QS_OVERLAP) - shared0;
#pragma unroll 1
      for (int seg = 0; seg < 2; ++seg) {
        const int begin = (seg == 0 ? shared0 : other0) + chalf * (QS_OVERLAP / 2);
        // the shared columns are handed back as soon as they are in registers
        const bool released = epilogue_warp_tile<OUT_DT, 1>(p, &map_c, taddr, stage, epi_buf, row0, lane, n_blk * BN, b,
                                                            has_alpha, alpha, begin, begin + QS_OVERLAP / 2,
                                                            seg == 0 ? map_to_cta(&ovl_free[acc], 0) : 0u);
        if (seg == 0 && !released) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(&ovl_free[acc], 0));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    reg_dealloc<104>();
    // ------------------------------ scale warps (both CTAs) -------------------
    const int quadrant = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1u;
        // The tiles have landed, and the MMAs that read this buffer two stages ago have completed: that is the
        // completion of that stage's empty barrier (the same use of the ring when the stage index did not wrap).
        const int prev = stage >= 2 ? stage - 2 : stage - 2 + QP_STAGES;
        const uint32_t prev_phase = stage >= 2 ? phase : phase ^ 1u;
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&sf_full[stage], phase, abort_flag) &&
                                         (it < 2 || mbar_wait(&empty_bar[prev], prev_phase, abort_flag)))) { ok = false; break; }
        tc_fence_after_sync();
        const uint8_t* sfa = smem_sfa + stage * QP_SFA_BYTES + lane * 16;
        const uint8_t* sfb = smem_sfb + stage * QP_SFB_BYTES + lane * 16;
        const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + QS_SF_COL + buf * QS_SF_BUF_COLS;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint4 b0 = *reinterpret_cast<const uint4*>(sfb + k * 512);
          const uint4 b1 = *reinterpret_cast<const uint4*>(sfb + QP_SFA_BYTES + k * 512);
          const uint4 a0 = *reinterpret_cast<const uint4*>(sfa + k * 512);
          const uint32_t r[16] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w, a0.x, a0.y, a0.z, a0.w, 0u, 0u, 0u, 0u};
          tmem_st_32x32_x16(taddr + 16 * k, r);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&full_bar[stage], 0));
        if (++stage == QP_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  if (warp >= QS_EPI_WARP0 && warp < QS_SF_WARP0 && lane == 0) tma_store_wait_read();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_error, VQ_ETIMEOUT);
  cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

// Tensor map over a [batch, rows, k] K-contiguous operand; box = 128 bytes of K x box_rows rows.
int make_operand_map(CUtensorMap* map, const void* base, int elem_kind, int elem_bytes, int64_t rows, int64_t k,
                     int64_t ld, int64_t batch, int64_t batch_stride, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                           : (elem_kind == VQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                  : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(ld * elem_bytes), (cuuint64_t)((batch > 1 ? batch_stride : ld * rows) * elem_bytes)};
  cuuint32_t box[3] = {(cuuint32_t)(BK_BYTES / elem_bytes), (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return VQ_OK;
}

// Tensor map over the output [batch, M, N] for the epilogue's TMA stores: boxes of 32 rows x 128
// bytes in the 128-byte swizzle.  `*usable` is 0 (and the map zeroed) when C is not 16-byte
// aligned in base and strides; the epilogue then stores with ordinary instructions.
int make_output_map(CUtensorMap* map, int* usable, void* C, int out_dtype, int64_t M, int64_t N, int64_t ldc,
                    int64_t batch, int64_t strideC) {
  memset(map, 0, sizeof(*map));
  *usable = 0;
  const int esz = out_dtype == VQ_F32 ? 4 : 2;
  const int64_t batch_stride = batch > 1 ? strideC : ldc * M;
  if (((reinterpret_cast<uintptr_t>(C) | (uintptr_t)(ldc * esz) | (uintptr_t)(batch_stride * esz)) & 15) != 0) return VQ_OK;
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType dt = out_dtype == VQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                               : (out_dtype == VQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                      : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(ldc * esz), (cuuint64_t)(batch_stride * esz)};
  cuuint32_t box[3] = {(cuuint32_t)(128 / esz), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, dt, 3, C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled (output) failed with code %d", (int)r);
  *usable = 1;
  return VQ_OK;
}

// Tensor map over packed NVFP4 block scales, [row blocks][K / 64][512 bytes] seen as 32-bit words:
// a box is four K64 steps of one 128-row block (2 KB, no swizzle).  Boxes that reach past the
// last K step or the last row block read as zero.
int make_scale_map(CUtensorMap* map, const void* base, int64_t k64_total, int64_t row_blocks) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {128, (cuuint64_t)k64_total, (cuuint64_t)row_blocks};
  cuuint64_t strides[2] = {512, (cuuint64_t)k64_total * 512};
  cuuint32_t box[3] = {128, 4, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VQ_ECUDA, "cuTensorMapEncodeTiled (scales) failed with code %d", (int)r);
  return VQ_OK;
}

// Kernel instantiation for an output dtype (the epilogue is compiled per dtype).
#define VQ_FOR_OUT_DTYPE(dt, KERNEL) ((dt) == VQ_BF16 ? KERNEL<VQ_BF16> : (dt) == VQ_F16 ? KERNEL<VQ_F16> : KERNEL<VQ_F32>)

template <typename Kernel>
int allow_big_smem(Kernel k_bf16, Kernel k_f16, Kernel k_f32, size_t bytes) {
  for (Kernel k : {k_bf16, k_f16, k_f32}) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(VQ_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  return VQ_OK;
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" {

int vq_gemm_tn(const void* A, const void* B, void* C, int in_kind, int out_dtype, int64_t M, int64_t N, int64_t K,
               int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t strideA, int64_t strideB,
               int64_t strideC, const void* alpha, int alpha_dtype, const void* bias, int bias_dtype,
               void* stream) {
  return vq_gemm_tn_ex(A, B, C, in_kind, out_dtype, M, N, K, lda, ldb, ldc, batch, strideA, strideB, strideC, alpha,
                       alpha_dtype, bias, bias_dtype, nullptr, stream);
}

int vq_gemm_tn_ex(const void* A, const void* B, void* C, int in_kind, int out_dtype, int64_t M, int64_t N, int64_t K,
                  int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t strideA, int64_t strideB,
                  int64_t strideC, const void* alpha, int alpha_dtype, const void* bias, int bias_dtype,
                  const VqGemmEpilogue* epi, void* stream) {
  VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, "vq_gemm_tn: negative extent");
  if (M == 0 || N == 0 || batch == 0) return VQ_OK;
  VQ_REQUIRE(A && B && C, "vq_gemm_tn: null operand");
  VQ_REQUIRE(K > 0, "vq_gemm_tn: empty contraction");
  VQ_REQUIRE(in_kind == VQ_IN_BF16 || in_kind == VQ_IN_F16 || in_kind == VQ_IN_E4M3 || in_kind == VQ_IN_E5M2,
             "vq_gemm_tn: unknown operand kind %d", in_kind);
  VQ_REQUIRE(out_dtype == VQ_BF16 || out_dtype == VQ_F16 || out_dtype == VQ_F32, "vq_gemm_tn: bad output dtype");
  const int eb = (in_kind == VQ_IN_E4M3 || in_kind == VQ_IN_E5M2) ? 1 : 2;
  VQ_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0,
             "vq_gemm_tn: operands must be 16-byte aligned");
  VQ_REQUIRE((lda * eb) % 16 == 0 && (ldb * eb) % 16 == 0 && (strideA * eb) % 16 == 0 && (strideB * eb) % 16 == 0,
             "vq_gemm_tn: leading dimensions and batch strides must be multiples of 16 bytes");
  VQ_REQUIRE(lda >= K && ldb >= K && (ldc >= N || (epi != nullptr && epi->gate_scale != nullptr)),
             "vq_gemm_tn: leading dimension smaller than the row");
  VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && batch < (1ll << 31), "vq_gemm_tn: extent too large");

  const int kind = in_kind == VQ_IN_F16 ? VQ_F16 : VQ_BF16;
  GemmParams p{};
  p.C = C;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.elem_bytes = eb;
  p.ldc = ldc; p.strideC = strideC;
  p.batch = (int)batch;
  p.alpha = alpha; p.alpha_dt = alpha_dtype;
  p.bias = bias; p.bias_dt = bias_dtype;
  p.out_dt = out_dtype;
  p.kind_f8 = eb == 1;
  if (epi != nullptr) {
    if (epi->alpha_cols != nullptr) {
      VQ_REQUIRE(epi->alpha_cols_dtype >= VQ_BF16 && epi->alpha_cols_dtype <= VQ_F32, "vq_gemm_tn_ex: bad alpha_cols dtype");
      p.alpha_cols = epi->alpha_cols; p.alpha_cols_dt = epi->alpha_cols_dtype;
    }
    if (epi->residual != nullptr) {
      VQ_REQUIRE(epi->ldr >= N, "vq_gemm_tn_ex: residual leading dimension smaller than the row");
      VQ_REQUIRE(epi->residual != C, "vq_gemm_tn_ex: the residual must not alias the output");
      p.residual = epi->residual; p.ldr = epi->ldr; p.strideR = epi->strideR;
    }
    if (epi->gate_scale != nullptr) {
      VQ_REQUIRE(out_dtype == VQ_BF16 && bias == nullptr && epi->residual == nullptr,
                 "vq_gemm_tn_ex: the gated epilogue takes out_dtype VQ_BF16 (of the two linears), no bias, no residual");
      VQ_REQUIRE(N % 64 == 0, "vq_gemm_tn_ex: the gated epilogue needs N (gate and up columns together) to be a multiple of 64");
      VQ_REQUIRE(ldc >= N / 2 && ldc % 16 == 0 && strideC % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0,
                 "vq_gemm_tn_ex: the gated output is [M, N/2] bytes, 16-byte aligned rows");
      VQ_REQUIRE(epi->gate_scale_dtype >= VQ_BF16 && epi->gate_scale_dtype <= VQ_F32, "vq_gemm_tn_ex: bad gate scale dtype");
      p.gate_scale = epi->gate_scale; p.gate_scale_dt = epi->gate_scale_dtype;
    }
    p.round_acc = epi->round_acc != 0;
    if (epi->causal_mode != 0) {
      VQ_REQUIRE((epi->causal_mode == 1 || epi->causal_mode == 2) && epi->causal_period > 0 &&
                 epi->causal_period < (1ll << 31), "vq_gemm_tn_ex: causal_mode is 0, 1 or 2 and needs a positive period");
      p.causal_mode = epi->causal_mode; p.causal_period = (int)epi->causal_period;
    }
  }
  const int fmt = in_kind == VQ_IN_BF16 ? 1 : in_kind == VQ_IN_F16 ? 0 : in_kind == VQ_IN_E4M3 ? 0 : 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // CTA pairs (256x256 tiles) when there is more than one 128-row block of output;
  // VQ_GEMM_PAIR=0 forces the single-CTA kernel.  Function attributes and the cluster occupancy
  // belong to a device, so they are set up once per device ordinal.
  static int pair_mode = -1;        // -1 unknown, 0 off, 1 on (process-wide: the environment)
  static int max_clusters_of[64] = {};
  static unsigned long long pair_configured = 0;
  if (pair_mode < 0) {
    const char* env = getenv("VQ_GEMM_PAIR");
    pair_mode = (env && env[0] == '0') ? 0 : 1;
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  if (pair_mode == 1 && first_call_on_device(&pair_configured)) {
    if (int rc = allow_big_smem(gemm_tn_pair_kernel<VQ_BF16>, gemm_tn_pair_kernel<VQ_F16>,
                                gemm_tn_pair_kernel<VQ_F32>, P_SMEM_BYTES))
      return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSmCount, 1, 1);
    cfg.blockDim = dim3(P_THREADS, 1, 1);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_tn_pair_kernel<VQ_BF16>, &cfg);
    if (e != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      max_clusters_of[device] = 0;   // this device runs the single-CTA kernel
    } else {
      max_clusters_of[device] = n < kSmCount / 2 ? n : kSmCount / 2;
    }
  }
  const int max_clusters = pair_mode == 1 ? max_clusters_of[device] : 0;
  CUtensorMap map_c;
  if (p.gate_scale != nullptr) {
    memset(&map_c, 0, sizeof(map_c));   // the gated epilogue stores from registers
  } else if (int e = make_output_map(&map_c, &p.tma_store, C, out_dtype, M, N, ldc, batch, strideC)) {
    return e;
  }
  if (max_clusters > 0 && M > BM) {
    CUtensorMap map_a, map_b;
    if (int e = make_operand_map(&map_a, A, kind, eb, M, K, lda, batch, strideA, BM)) return e;
    p.bn = N <= BN / 2 ? BN / 2 : BN;   // a narrow output takes half-width tiles instead of multiplying zero padding
    if (int e = make_operand_map(&map_b, B, kind, eb, N, K, ldb, batch, strideB, p.bn / 2)) return e;
    p.idesc = sm100::make_idesc(2 * BM, p.bn, fmt, fmt, 0, 0);
    const int64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + p.bn - 1) / p.bn) * batch;
    const int clusters = (int)(tiles < max_clusters ? tiles : max_clusters);
    VQ_FOR_OUT_DTYPE(out_dtype, gemm_tn_pair_kernel)<<<2 * clusters, P_THREADS, P_SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
    return check_launch("gemm_tn_pair_kernel");
  }

  CUtensorMap map_a, map_b;
  if (int e = make_operand_map(&map_a, A, kind, eb, M, K, lda, batch, strideA, BM)) return e;
  if (int e = make_operand_map(&map_b, B, kind, eb, N, K, ldb, batch, strideB, BN)) return e;
  p.idesc = sm100::make_idesc(BM, BN, fmt, fmt, 0, 0);
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    if (int rc = allow_big_smem(gemm_tn_kernel<VQ_BF16>, gemm_tn_kernel<VQ_F16>, gemm_tn_kernel<VQ_F32>, SMEM_BYTES))
      return rc;
  }
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch;
  const int grid = (int)(tiles < kSmCount ? tiles : kSmCount);
  VQ_FOR_OUT_DTYPE(out_dtype, gemm_tn_kernel)<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(map_a, map_b, map_c, p);
  return check_launch("gemm_tn_kernel");
}

int vq_gemm_mx(const void* A, const void* a_scale, const void* B, const void* b_scale, int64_t block_size, void* C,
               int out_dtype, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch,
               int64_t strideA, int64_t strideB, int64_t strideC, const void* alpha, int alpha_dtype, const void* bias,
               int bias_dtype, void* stream) {
  VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, "vq_gemm_mx: negative extent");
  if (M == 0 || N == 0 || batch == 0) return VQ_OK;
  VQ_REQUIRE(A && B && C, "vq_gemm_mx: null operand");
  VQ_REQUIRE(a_scale || b_scale, "vq_gemm_mx: neither operand has scales (use vq_gemm_tn)");
  VQ_REQUIRE(K > 0, "vq_gemm_mx: empty contraction");
  VQ_REQUIRE(block_size >= 8 && (block_size & (block_size - 1)) == 0,
             "vq_gemm_mx: the block size must be a power of two, 8 or more");
  VQ_REQUIRE(out_dtype == VQ_BF16 || out_dtype == VQ_F16 || out_dtype == VQ_F32, "vq_gemm_mx: bad output dtype");
  VQ_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0,
             "vq_gemm_mx: operands must be 16-byte aligned");
  VQ_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && strideA % 8 == 0 && strideB % 8 == 0,
             "vq_gemm_mx: leading dimensions and batch strides must be multiples of 16 bytes");
  VQ_REQUIRE(lda >= K && ldb >= K && ldc >= N, "vq_gemm_mx: leading dimension smaller than the row");
  VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && batch < (1ll << 31), "vq_gemm_mx: extent too large");

  static int max_clusters_of[64] = {};
  static unsigned long long configured = 0;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  if (first_call_on_device(&configured)) {
    if (int rc = allow_big_smem(gemm_mx_pair_kernel<VQ_BF16>, gemm_mx_pair_kernel<VQ_F16>, gemm_mx_pair_kernel<VQ_F32>,
                                P_SMEM_BYTES))
      return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSmCount, 1, 1);
    cfg.blockDim = dim3(MX_THREADS, 1, 1);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_mx_pair_kernel<VQ_BF16>, &cfg);
    if (e != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      max_clusters_of[device] = 0;
    } else {
      max_clusters_of[device] = n < kSmCount / 2 ? n : kSmCount / 2;
    }
  }
  const int max_clusters = max_clusters_of[device];
  if (max_clusters < 1) return vq::fail(VQ_EUNSUPPORTED, "vq_gemm_mx: this device cannot co-schedule CTA pairs");

  GemmParams p{};
  p.C = C;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.elem_bytes = 2;
  p.ldc = ldc; p.strideC = strideC;
  p.batch = (int)batch;
  p.alpha = alpha; p.alpha_dt = alpha_dtype;
  p.bias = bias; p.bias_dt = bias_dtype;
  p.out_dt = out_dtype;
  p.kind_f8 = false;
  MxScales sc{};
  sc.a = static_cast<const __nv_bfloat16*>(a_scale);
  sc.b = static_cast<const __nv_bfloat16*>(b_scale);
  sc.lds_a = sc.lds_b = (K + block_size - 1) / block_size;
  sc.stride_a = M * sc.lds_a;
  sc.stride_b = strideB == 0 ? 0 : N * sc.lds_b;
  sc.shift = 0;
  while ((1ll << sc.shift) < block_size) ++sc.shift;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap map_a, map_b, map_c;
  if (int e = make_output_map(&map_c, &p.tma_store, C, out_dtype, M, N, ldc, batch, strideC)) return e;
  if (int e = make_operand_map(&map_a, A, VQ_BF16, 2, M, K, lda, batch, strideA, BM)) return e;
  p.bn = N <= BN / 2 ? BN / 2 : BN;
  if (int e = make_operand_map(&map_b, B, VQ_BF16, 2, N, K, ldb, batch, strideB, p.bn / 2)) return e;
  p.idesc = sm100::make_idesc(2 * BM, p.bn, 1, 1, 0, 0);
  const int64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + p.bn - 1) / p.bn) * batch;
  const int clusters = (int)(tiles < max_clusters ? tiles : max_clusters);
  VQ_FOR_OUT_DTYPE(out_dtype, gemm_mx_pair_kernel)<<<2 * clusters, MX_THREADS, P_SMEM_BYTES, st>>>(map_a, map_b, map_c, p, sc);
  return check_launch("gemm_mx_pair_kernel");
}

int vq_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int out_dtype, int64_t M,
                  int64_t N, int64_t K, int64_t ldc, int64_t batch, int64_t strideC, const void* alpha,
                  int alpha_dtype, const void* bias, int bias_dtype, void* stream) {
  return vq_gemm_nvfp4_ex(A, sfa, B, sfb, C, out_dtype, M, N, K, ldc, batch, strideC, alpha, alpha_dtype, bias,
                          bias_dtype, nullptr, 0, stream);
}

int vq_gemm_nvfp4_ex(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int out_dtype, int64_t M,
                     int64_t N, int64_t K, int64_t ldc, int64_t batch, int64_t strideC, const void* alpha,
                     int alpha_dtype, const void* bias, int bias_dtype, const void* alpha_cols, int alpha_cols_dtype,
                     void* stream) {
  VQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, "vq_gemm_nvfp4: negative extent");
  if (M == 0 || N == 0 || batch == 0) return VQ_OK;
  VQ_REQUIRE(A && B && C && sfa && sfb, "vq_gemm_nvfp4: null operand");
  VQ_REQUIRE(K > 0 && K % 64 == 0, "vq_gemm_nvfp4: K must be a positive multiple of 64");
  VQ_REQUIRE(out_dtype == VQ_BF16 || out_dtype == VQ_F16 || out_dtype == VQ_F32, "vq_gemm_nvfp4: bad output dtype");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(sfa) |
               reinterpret_cast<uintptr_t>(sfb)) & 15) == 0, "vq_gemm_nvfp4: operands must be 16-byte aligned");
  VQ_REQUIRE(ldc >= N, "vq_gemm_nvfp4: leading dimension smaller than the row");
  VQ_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && batch < (1ll << 31), "vq_gemm_nvfp4: extent too large");
  const int64_t row_bytes = K / 2;
  CUtensorMap map_a, map_b;
  if (int e = make_operand_map(&map_a, A, VQ_BF16, 1, M, row_bytes, row_bytes, batch, M * row_bytes, BM)) return e;
  // More than one 128-row block of output: CTA pairs on 256x256 tiles, scale factors stored into tensor
  // memory by warps (VQ_NVFP4_PAIR=1: the tcgen05.cp form of the pair kernel; 0: the single-CTA kernel).
  static int pair_mode = -1;
  if (pair_mode < 0) {
    const char* env = getenv("VQ_NVFP4_PAIR");
    pair_mode = (env && env[0] == '0') ? 0 : (env && env[0] == '1') ? 1 : 2;
  }
  const bool pair = pair_mode >= 1 && M > BM;
  if (int e = make_operand_map(&map_b, B, VQ_BF16, 1, N, row_bytes, row_bytes, batch, N * row_bytes, pair ? BN / 2 : Q_BN))
    return e;
  GemmParams p{};
  p.C = C;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.elem_bytes = 1;
  p.ldc = ldc; p.strideC = strideC;
  p.batch = (int)batch;
  p.alpha = alpha; p.alpha_dt = alpha_dtype;
  p.bias = bias; p.bias_dt = bias_dtype;
  p.out_dt = out_dtype;
  if (alpha_cols != nullptr) {
    VQ_REQUIRE(alpha_cols_dtype >= VQ_BF16 && alpha_cols_dtype <= VQ_F32, "vq_gemm_nvfp4_ex: bad alpha_cols dtype");
    p.alpha_cols = alpha_cols; p.alpha_cols_dt = alpha_cols_dtype;
  }
  p.idesc = sm100::make_idesc_nvfp4(BM, Q_BN);
  CUtensorMap map_c;
  if (int e = make_output_map(&map_c, &p.tma_store, C, out_dtype, M, N, ldc, batch, strideC)) return e;
  ScaledOperands sf{};
  sf.sfa = static_cast<const uint8_t*>(sfa);
  sf.sfb = static_cast<const uint8_t*>(sfb);
  sf.sfa_batch_stride = ((M + 127) / 128) * (K / 64) * 512;
  sf.sfb_batch_stride = ((N + 127) / 128) * (K / 64) * 512;
  if (pair) {
    CUtensorMap map_sfa, map_sfb;
    if (int e = make_scale_map(&map_sfa, sfa, K / 64, ((M + 127) / 128) * batch)) return e;
    if (int e = make_scale_map(&map_sfb, sfb, K / 64, ((N + 127) / 128) * batch)) return e;
    p.idesc = sm100::make_idesc_nvfp4(2 * BM, BN);
    static unsigned long long pair_configured = 0;
    if (first_call_on_device(&pair_configured)) {
      if (int rc = allow_big_smem(gemm_nvfp4_pair_kernel<VQ_BF16>, gemm_nvfp4_pair_kernel<VQ_F16>,
                                  gemm_nvfp4_pair_kernel<VQ_F32>, QP_SMEM_BYTES))
        return rc;
    }
    const int64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN) * batch;
    const int clusters = (int)(tiles < kSmCount / 2 ? tiles : kSmCount / 2);
    if (pair_mode == 2) {
      static unsigned long long sfw_configured = 0;
      if (first_call_on_device(&sfw_configured)) {
        if (int rc = allow_big_smem(gemm_nvfp4_sfw_kernel<VQ_BF16>, gemm_nvfp4_sfw_kernel<VQ_F16>,
                                    gemm_nvfp4_sfw_kernel<VQ_F32>, QP_SMEM_BYTES))
          return rc;
      }
      VQ_FOR_OUT_DTYPE(out_dtype, gemm_nvfp4_sfw_kernel)<<<2 * clusters, QS_THREADS, QP_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
          map_a, map_b, map_sfa, map_sfb, map_c, p);
      return check_launch("gemm_nvfp4_sfw_kernel");
    }
    VQ_FOR_OUT_DTYPE(out_dtype, gemm_nvfp4_pair_kernel)<<<2 * clusters, NUM_THREADS, QP_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
        map_a, map_b, map_sfa, map_sfb, map_c, p);
    return check_launch("gemm_nvfp4_pair_kernel");
  }
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured)) {
    if (int rc = allow_big_smem(gemm_nvfp4_kernel<VQ_BF16>, gemm_nvfp4_kernel<VQ_F16>, gemm_nvfp4_kernel<VQ_F32>,
                                Q_SMEM_BYTES))
      return rc;
  }
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + Q_BN - 1) / Q_BN) * batch;
  const int grid = (int)(tiles < kSmCount ? tiles : kSmCount);
  VQ_FOR_OUT_DTYPE(out_dtype, gemm_nvfp4_kernel)<<<grid, NUM_THREADS, Q_SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(map_a, map_b, map_c, p, sf);
  return check_launch("gemm_nvfp4_kernel");
}


int vq_gemm_status(int reset) {
  int value = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&value, g_gemm_error, sizeof(int));
  if (e != cudaSuccess) return fail(VQ_ECUDA, "vq_gemm_status: %s", cudaGetErrorString(e));
  if (reset && value != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  }
  if (value != 0) return fail(value, "a tensor-core GEMM gave up waiting on a barrier");
  return VQ_OK;
}

}  // extern "C"
