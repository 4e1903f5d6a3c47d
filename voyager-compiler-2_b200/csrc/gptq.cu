// GPTQ column sweep against a block-scaled grid, on the device.
//
// For one block of `bs` input channels (columns) of a weight [rows, K]:
//   1. each row takes its scale from the current, already compensated values
//      (microscaling: amax / quant_max through the scale table; or group-wise
//      affine: (max - min) / (qmax - qmin) with a zero point);
//   2. the block's columns are rounded one after the other; each column's
//      error over its pivot U[c][c] is propagated into the block's later
//      columns with U's row c (U = upper Cholesky factor of the inverse Hessian);
//   3. the trailing columns receive  work[:, end:] -= deltas @ U[start:end, end:].
// Rows never interact, so one thread owns one row: its slice of the block lives
// in registers, U's diagonal tile is broadcast from shared memory, and every
// arithmetic step is a separately rounded fp32 operation in the order the
// reference's column loop performs them.

#include "quantize_shared.cuh"

namespace vq {
namespace {

constexpr float kEps = 1e-12f;  // the reference's EPS clamp on scales and pivots
constexpr int kMaxBlock = 128;
constexpr int kRowsPerCta = 32;   // one warp per CTA: twice the CTAs of a 64-row split, and up to 3 CTAs share an SM at 64 KB of shared memory each
constexpr int kShrinkCandidates = 5;

struct GptqBlockParams {
  float* work;          // [rows, K] fp32, updated in place inside the block
  float* out;           // [rows, K] fp32, receives the block's grid values
  float* deltas;        // [rows, bs] fp32
  const float* U;       // [K, K] fp32 upper triangular
  const float* salience;  // [K] fp32 (shrink search weights) or null
  int64_t rows, K;
  int start, n;         // block = columns [start, start + n)
  int affine;           // 0: microscaling scale; 1: group-wise affine (scale + zero point)
  float quant_min, quant_max;
  int shrink;
  Round scale_round;    // rounding of the scale (microscaling)
  Round round;          // element grid
};

__device__ __forceinline__ float grid_value(const Round& r, float w, float scale, float zero, bool affine) {
  // quantize(w / scale [+ zero]) then back to the weight's units
  float y = __fdiv_rn(w, scale);
  if (affine) y = __fadd_rn(y, zero);
  float code = apply_round(r, y, 0);
  if (affine) code = __fsub_rn(code, zero);
  return __fmul_rn(code, scale);
}

template <int MAXN>
__global__ void __launch_bounds__(kRowsPerCta)
gptq_block_kernel(GptqBlockParams p) {
  extern __shared__ float tile[];  // U[start:start+n, start:start+n], row-major n x n
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(p.round, s_steps[0]);
  stage_steps(p.scale_round, s_steps[1]);
  const int n = p.n;
  for (int t = threadIdx.x; t < n * n; t += blockDim.x) {
    const int r = t / n, c = t - r * n;
    tile[t] = p.U[(int64_t)(p.start + r) * p.K + p.start + c];
  }
  __syncthreads();
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= p.rows) return;

  float w[MAXN];
  float* wrow = p.work + row * p.K + p.start;
#pragma unroll
  for (int c = 0; c < MAXN; ++c) w[c] = c < n ? wrow[c] : 0.0f;

  // ---- per-row scale (and zero point) from the block as compensated so far ----
  float scale, zero = 0.0f;
  if (p.affine) {
    float lo = w[0], hi = w[0];
#pragma unroll
    for (int c = 1; c < MAXN; ++c)
      if (c < n) { lo = fminf(lo, w[c]); hi = fmaxf(hi, w[c]); }
    scale = __fdiv_rn(__fsub_rn(hi, lo), __fsub_rn(p.quant_max, p.quant_min));
    scale = scale > 0.0f ? scale : 1.0f;
    zero = __fadd_rn(__fdiv_rn(-lo, scale), p.quant_min);
  } else {
    uint32_t m = 0;
#pragma unroll
    for (int c = 0; c < MAXN; ++c)
      if (c < n) m = max(m, abs_bits(w[c]));
    float base = __fdiv_rn(__uint_as_float(m), p.quant_max);
    if (p.scale_round.mode != VQ_ROUND_NONE) base = apply_round(p.scale_round, base, 0);
    base = base > 0.0f ? base : 1.0f;
    base = fmaxf(base, kEps);
    scale = base;
    if (p.shrink) {
      // try scales below amax / quant_max; keep the one with the least salience-weighted error
      const float factors[kShrinkCandidates] = {1.0f, 0.93f, 0.86f, 0.79f, 0.72f};
      float best_err = 0.0f;
      for (int f = 0; f < kShrinkCandidates; ++f) {
        float s = base;
        if (f > 0) {
          s = __bfloat162float(__float2bfloat16_rn(__fmul_rn(base, factors[f])));
          s = apply_round(p.scale_round, s, 0);
          s = fmaxf(s, kEps);
        }
        float err = 0.0f;
#pragma unroll
        for (int c = 0; c < MAXN; ++c)
          if (c < n) {
            const float d = __fsub_rn(w[c], grid_value(p.round, w[c], s, 0.0f, false));
            err = __fadd_rn(err, __fmul_rn(__fmul_rn(d, d), p.salience[p.start + c]));
          }
        if (f == 0 || err < best_err) { best_err = err; scale = s; }
      }
    }
  }

  // ---- column sweep ----
  float* orow = p.out + row * p.K + p.start;
  float* drow = p.deltas + row * n;
#pragma unroll
  for (int c = 0; c < MAXN; ++c) {
    if (c < n) {
      const float level = grid_value(p.round, w[c], scale, zero, p.affine != 0);
      const float pivot = fmaxf(tile[c * n + c], kEps);
      const float delta = __fdiv_rn(__fsub_rn(w[c], level), pivot);
      orow[c] = level;
      drow[c] = delta;
#pragma unroll
      for (int j = c + 1; j < MAXN; ++j)
        if (j < n) w[j] = __fsub_rn(w[j], __fmul_rn(delta, tile[c * n + j]));
    }
  }
}

// work[r][end + j] -= sum_c deltas[r][c] * U[start + c][end + j], c ascending, fp32.
// A CTA computes a 64-row x 64-column patch; deltas and U's rows are staged in
// shared memory in chunks of 32 c.
constexpr int kUpdTile = 64;
__global__ void __launch_bounds__(256)
gptq_update_kernel(float* __restrict__ work, const float* __restrict__ deltas, const float* __restrict__ U,
                   int64_t rows, int64_t K, int start, int n, int end) {
  __shared__ float sd[kUpdTile][33];
  __shared__ float su[32][kUpdTile + 1];
  const int64_t r0 = (int64_t)blockIdx.y * kUpdTile;
  const int64_t j0 = (int64_t)end + (int64_t)blockIdx.x * kUpdTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
  for (int c0 = 0; c0 < n; c0 += 32) {
    for (int t = threadIdx.x; t < kUpdTile * 32; t += 256) {
      const int r = t >> 5, c = t & 31;
      sd[r][c] = (r0 + r < rows && c0 + c < n) ? deltas[(r0 + r) * n + c0 + c] : 0.0f;
    }
    for (int t = threadIdx.x; t < 32 * kUpdTile; t += 256) {
      const int c = t / kUpdTile, j = t - c * kUpdTile;
      su[c][j] = (c0 + c < n && j0 + j < K) ? U[(int64_t)(start + c0 + c) * K + j0 + j] : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < 32; ++c) {
      float d[4], u[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) d[a] = sd[ty * 4 + a][c];
#pragma unroll
      for (int b = 0; b < 4; ++b) u[b] = su[c][tx * 4 + b];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(d[a], u[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int64_t r = r0 + ty * 4 + a;
    if (r >= rows) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int64_t j = j0 + tx * 4 + b;
      if (j < K) work[r * K + j] = __fsub_rn(work[r * K + j], acc[a][b]);
    }
  }
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_gptq_block(float* work, float* out, float* deltas, const float* U, const float* salience,
                             int64_t rows, int64_t K, int64_t start, int64_t n, int affine, float quant_min,
                             float quant_max, int shrink, const VqRound* scale_round, const VqRound* round,
                             void* stream) {
  VQ_REQUIRE(rows >= 0 && K > 0 && start >= 0 && n > 0 && start + n <= K, "vq_gptq_block: bad block");
  if (rows == 0) return VQ_OK;
  VQ_REQUIRE(work && out && deltas && U && round, "vq_gptq_block: null argument");
  VQ_REQUIRE(n <= kMaxBlock, "vq_gptq_block: blocks of more than %d columns are not supported", kMaxBlock);
  VQ_REQUIRE(!shrink || (salience && !affine && scale_round && scale_round->mode != VQ_ROUND_NONE),
             "vq_gptq_block: the shrink search needs salience weights and a scale table");
  VQ_REQUIRE(affine ? quant_max > quant_min : quant_max > 0.0f, "vq_gptq_block: bad code range");
  if (int e = validate_round(scale_round, "scale rounding")) return e;
  if (int e = validate_round(round, "element rounding")) return e;
  GptqBlockParams p{};
  p.work = work; p.out = out; p.deltas = deltas; p.U = U; p.salience = salience;
  p.rows = rows; p.K = K; p.start = (int)start; p.n = (int)n;
  p.affine = affine; p.quant_min = quant_min; p.quant_max = quant_max; p.shrink = shrink;
  p.scale_round = make_round(scale_round);
  p.round = make_round(round);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = (int)((rows + kRowsPerCta - 1) / kRowsPerCta);
  const size_t smem = (size_t)n * n * sizeof(float);
  static unsigned long long configured = 0;
  if (first_call_on_device(&configured))
    cudaFuncSetAttribute(gptq_block_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 128 * 4);
  if (n <= 32) gptq_block_kernel<32><<<grid, kRowsPerCta, smem, st>>>(p);
  else if (n <= 64) gptq_block_kernel<64><<<grid, kRowsPerCta, smem, st>>>(p);
  else gptq_block_kernel<128><<<grid, kRowsPerCta, smem, st>>>(p);
  return check_launch("gptq_block_kernel");
}

extern "C" int vq_gptq_update(float* work, const float* deltas, const float* U, int64_t rows, int64_t K,
                              int64_t start, int64_t n, void* stream) {
  VQ_REQUIRE(rows >= 0 && K > 0 && start >= 0 && n > 0 && start + n <= K, "vq_gptq_update: bad block");
  const int64_t end = start + n;
  if (rows == 0 || end == K) return VQ_OK;
  VQ_REQUIRE(work && deltas && U, "vq_gptq_update: null argument");
  dim3 grid((unsigned)((K - end + kUpdTile - 1) / kUpdTile), (unsigned)((rows + kUpdTile - 1) / kUpdTile));
  gptq_update_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(work, deltas, U, rows, K, (int)start,
                                                                          (int)n, (int)end);
  return check_launch("gptq_update_kernel");
}

// ---------------------------------------------------------------------------
// One GPTQ block step for callers that cannot allocate device memory
// ---------------------------------------------------------------------------
// vq_gptq_block + vq_gptq_update hand the per-column errors from the sweep to the
// trailing update through a caller-provided [rows, n] fp32 buffer.  Some hosts of
// this library have no allocator to get that buffer from: a runtime that drives
// the solve from inside a fixed, pre-planned memory arena (every byte of the pool
// already assigned to tensors), or a plugin loaded into a process whose policy
// forbids cudaMalloc after start-up.  For them the errors live in the array below,
// which is part of the library image: every GPU that loads the library holds these
// 8 MiB until the process exits.
constexpr int64_t kStaticDeltaFloats = 2 * 1024 * 1024;  // 8 MiB: e.g. 16384 rows x 128 columns
static __device__ __align__(256) float g_static_deltas[kStaticDeltaFloats];

// In host code `g_static_deltas` is only a handle for the symbol, not a device
// address; the address is looked up once per device, with that device current.
static float* static_deltas_for_current_device(int* status) {
  constexpr int kMaxDevices = 64;
  static float* address[kMaxDevices] = {};
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    *status = fail(VQ_ECUDA, "vq_gptq_block_step_static: cannot identify the current device");
    return nullptr;
  }
  if (address[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_deltas);
    if (e != cudaSuccess || p == nullptr) {
      *status = fail(VQ_ECUDA, "vq_gptq_block_step_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return nullptr;
    }
    address[device] = p;
  }
  *status = VQ_OK;
  return address[device];
}

extern "C" int vq_gptq_block_step_static(float* work, float* out, const float* U, const float* salience,
                                         int64_t rows, int64_t K, int64_t start, int64_t n, int affine,
                                         float quant_min, float quant_max, int shrink, const VqRound* scale_round,
                                         const VqRound* round, void* stream) {
  VQ_REQUIRE(rows >= 0 && n > 0, "vq_gptq_block_step_static: bad block");
  VQ_REQUIRE(rows <= kStaticDeltaFloats / n,   // not rows * n: an absurd row count must not wrap around
             "vq_gptq_block_step_static: %lld rows x %lld block columns exceeds the built-in buffer of %lld values "
             "(8 MiB); split the rows or use vq_gptq_block / vq_gptq_update with your own buffer",
             (long long)rows, (long long)n, (long long)kStaticDeltaFloats);
  int status = VQ_OK;
  float* deltas = static_deltas_for_current_device(&status);
  if (deltas == nullptr) return status;
  // Every value of the [rows, n] region is rewritten by the sweep before the update
  // reads it, so nothing left over from an earlier call is ever consumed.
  if (int e = vq_gptq_block(work, out, deltas, U, salience, rows, K, start, n, affine, quant_min, quant_max, shrink,
                            scale_round, round, stream))
    return e;
  return vq_gptq_update(work, deltas, U, rows, K, start, n, stream);
}
