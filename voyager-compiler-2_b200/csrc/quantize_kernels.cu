// Quantizer kernels for sm_100a: table rounding (vmap), scale/zero-point
// quantize and dequantize with block-broadcast parameters, the one-pass
// microscaling quantizer (block amax -> scale -> codes), the group-wise affine
// quantizer used for 2-bit KV caches, codebook read-back, and a tensor amax.
//
// All of these are HBM-bound: every kernel reads its input once with 16-byte
// accesses where the layout allows and writes each output once.

#include "quantize_shared.cuh"

#include <cmath>

namespace vq {

// ---------------------------------------------------------------------------
// error plumbing
// ---------------------------------------------------------------------------
static thread_local char g_error[512];
char* error_buffer() { return g_error; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(VQ_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return VQ_OK;
}

int validate_round(const VqRound* r, const char* what) {
  if (r == nullptr) return VQ_OK;
  switch (r->mode) {
    case VQ_ROUND_NONE:
    case VQ_ROUND_INT:
      return VQ_OK;
    case VQ_ROUND_TABLE:
      if (!r->table) return fail(VQ_EINVAL, "%s: table rounding without a table", what);
      return VQ_OK;
    case VQ_ROUND_MINIFLOAT:
      // The kernel scales by 2^(mbits - e) built directly from exponent bits,
      // which must stay a normal float for every exponent e the format has.
      if (r->mbits < 0 || r->mbits > 10 || !(r->max_norm > 0.0f) || r->emin - r->mbits < -126 ||
          ilogbf(r->max_norm) - r->mbits > 126 || ilogbf(r->max_norm) < r->emin)
        return fail(VQ_EINVAL, "%s: minifloat parameters out of range", what);
      return VQ_OK;
    case VQ_ROUND_STEPS:
      if (r->n_steps < 1 || r->n_steps > VQ_MAX_STEPS || !r->steps)
        return fail(VQ_EINVAL, "%s: %d steps (max %d) or no step table", what, r->n_steps, VQ_MAX_STEPS);
      return VQ_OK;
    case VQ_ROUND_SEARCH:
      if (r->n_edges < 0 || (r->n_edges > 0 && !r->edges))
        return fail(VQ_EINVAL, "%s: search rounding without edges", what);
      return VQ_OK;
    case VQ_ROUND_STOCHASTIC:
      if (!r->levels || r->n_levels < 1 || !r->seed)
        return fail(VQ_EINVAL, "%s: stochastic rounding needs levels and a seed", what);
      return VQ_OK;
  }
  return fail(VQ_EINVAL, "%s: unknown rounding mode %d", what, r->mode);
}

static inline int grid_for(int64_t work_items, int threads, int per_sm = 8) {
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)kSmCount * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// ---------------------------------------------------------------------------
// streaming elementwise kernels: vmap, quantize, dequantize
// ---------------------------------------------------------------------------
struct Geom {
  int ndim;
  int64_t size[VQ_MAX_DIMS];
  int64_t div[VQ_MAX_DIMS];
  int64_t stride[VQ_MAX_DIMS];
};

__device__ __forceinline__ int64_t param_index(const Geom& g, int64_t flat) {
  int64_t idx = 0;
#pragma unroll
  for (int d = VQ_MAX_DIMS - 1; d >= 0; --d) {
    if (d < g.ndim) {
      int64_t c = flat % g.size[d];
      flat /= g.size[d];
      idx += (c / g.div[d]) * g.stride[d];
    }
  }
  return idx;
}

// How the parameter (scale / zero point) index follows from the flat element
// index on the fast path.
enum { PI_SCALAR = 0, PI_DIV = 1, PI_MOD = 2, PI_GENERIC = 3 };
struct ParamIndex {
  int kind;
  uint32_t d;      // PI_DIV: index = flat / d (d a multiple of the vector width)
  int shift;       // PI_DIV: log2(d) when d is a power of two, else -1
  uint32_t c;      // PI_MOD: index = flat % c (c a multiple of the vector width)
};

constexpr int kUnroll = 4;
constexpr int kThreads = 256;

// KIND 0: out = round(in / scale [+ zp])
// KIND 1: out = round_out((round_in(in) - zp) * scale)
// KIND 2: out = round_out(in)                       (vmap)
template <int DT, int KIND>
__device__ __forceinline__ float map_one(float x, float s, float z, bool has_z, const Round& r_in,
                                         const Round& r_out, int64_t flat) {
  using E = Elem<DT>;
  if (KIND == 0) {
    float y = E::round(__fdiv_rn(x, s));
    if (has_z) y = E::round(__fadd_rn(y, z));
    return apply_round(r_out, y, flat);
  } else if (KIND == 1) {
    float y = apply_round(r_in, x, flat);
    if (has_z) y = E::round(__fsub_rn(y, z));
    y = E::round(__fmul_rn(y, s));
    return apply_round(r_out, y, flat);
  } else {
    return apply_round(r_out, x, flat);
  }
}

template <int DT, int KIND>
__global__ void __launch_bounds__(kThreads, 4)
stream_map_kernel(const void* __restrict__ in, const void* __restrict__ scale, const void* __restrict__ zp,
                  void* __restrict__ out, Round r_in, Round r_out, int64_t n, ParamIndex pidx, int pdt,
                  int n_is_32bit) {
  using E = Elem<DT>;
  constexpr int V = E::kVec;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r_in, s_steps[0]);
  stage_steps(r_out, s_steps[1]);
  const bool has_z = zp != nullptr;
  float s0 = 1.0f, z0 = 0.0f;
  if (KIND != 2 && pidx.kind == PI_SCALAR) {
    s0 = loadp(scale, 0, pdt);
    if (has_z) z0 = loadp(zp, 0, pdt);
  }
  const int64_t nvec = n / V;
  const int64_t chunk = (int64_t)kThreads * kUnroll;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    Vec<DT> x[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t v = base + u * kThreads + threadIdx.x;
      if (v < nvec) x[u].raw = __ldg(reinterpret_cast<const uint4*>(in) + v);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t v = base + u * kThreads + threadIdx.x;
      if (v >= nvec) continue;
      const int64_t flat = v * V;
      Vec<DT> y;
      if (KIND == 2 || pidx.kind == PI_SCALAR) {
#pragma unroll
        for (int j = 0; j < V; ++j) y.set(j, map_one<DT, KIND>(x[u].get(j), s0, z0, has_z, r_in, r_out, flat + j));
      } else if (pidx.kind == PI_DIV) {
        int64_t pi;
        if (pidx.shift >= 0) pi = flat >> pidx.shift;
        else pi = n_is_32bit ? (int64_t)((uint32_t)flat / pidx.d) : flat / pidx.d;
        float s = loadp(scale, pi, pdt);
        float z = has_z ? loadp(zp, pi, pdt) : 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) y.set(j, map_one<DT, KIND>(x[u].get(j), s, z, has_z, r_in, r_out, flat + j));
      } else {  // PI_MOD: V consecutive parameters
        int64_t pi = n_is_32bit ? (int64_t)((uint32_t)flat % pidx.c) : flat % pidx.c;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float s = loadp(scale, pi + j, pdt);
          float z = has_z ? loadp(zp, pi + j, pdt) : 0.0f;
          y.set(j, map_one<DT, KIND>(x[u].get(j), s, z, has_z, r_in, r_out, flat + j));
        }
      }
      reinterpret_cast<uint4*>(out)[v] = y.raw;
    }
  }
  // tail elements (n not a multiple of V): scalar parameters only reach here
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * V + threadIdx.x; i < n; i += kThreads)
      store1<DT>(out, i, map_one<DT, KIND>(load1<DT>(in, i), s0, z0, has_z, r_in, r_out, i));
  }
}

// Any broadcast, one element per thread step.
template <int DT, int KIND>
__global__ void __launch_bounds__(kThreads, 4)
generic_map_kernel(const void* __restrict__ in, const void* __restrict__ scale, const void* __restrict__ zp,
                   void* __restrict__ out, Geom g, Round r_in, Round r_out, int64_t n, int pdt) {
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r_in, s_steps[0]);
  stage_steps(r_out, s_steps[1]);
  const bool has_z = zp != nullptr;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float s = 1.0f, z = 0.0f;
    if (KIND != 2) {
      int64_t pi = param_index(g, i);
      s = loadp(scale, pi, pdt);
      if (has_z) z = loadp(zp, pi, pdt);
    }
    store1<DT>(out, i, map_one<DT, KIND>(load1<DT>(in, i), s, z, has_z, r_in, r_out, i));
  }
}

// ---------------------------------------------------------------------------
// packed integer codes (a KIVI-style 2- or 4-bit cache)
// ---------------------------------------------------------------------------
// Element i (row-major flat index) lives in byte i / (8 / BITS), at bit BITS * (i % (8 / BITS)).
// A thread handles 8 consecutive elements: BITS bytes of packed codes.
template <int DT, int BITS>
__global__ void __launch_bounds__(kThreads)
pack_codes_kernel(const void* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n) {
  const int64_t groups = (n + 7) / 8;
  for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (int64_t)gridDim.x * blockDim.x) {
    uint64_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t i = gi * 8 + j;
      if (i < n) {
        const int c = __float2int_rn(load1<DT>(codes, i));
        word |= (uint64_t)((uint32_t)c & ((1u << BITS) - 1u)) << (BITS * j);
      }
    }
    const int64_t nbytes = (n * BITS + 7) / 8;
#pragma unroll
    for (int b = 0; b < BITS; ++b)
      if (gi * BITS + b < nbytes) packed[gi * BITS + b] = (uint8_t)(word >> (8 * b));
  }
}

// out = round_out((code - zero_point) * scale), the dequantize of the codes' bf16-valued form.
template <int DT, int BITS>
__global__ void __launch_bounds__(kThreads, 4)
unpack_dequantize_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ scale,
                         const void* __restrict__ zp, void* __restrict__ out, Geom g, Round r_out, int64_t n,
                         int pdt) {
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  Round none{};
  none.mode = VQ_ROUND_NONE;
  stage_steps(r_out, s_steps[1]);
  const bool has_z = zp != nullptr;
  const int64_t groups = (n + 7) / 8;
  const int64_t nbytes = (n * BITS + 7) / 8;
  for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (int64_t)gridDim.x * blockDim.x) {
    uint64_t word = 0;
#pragma unroll
    for (int b = 0; b < BITS; ++b)
      if (gi * BITS + b < nbytes) word |= (uint64_t)packed[gi * BITS + b] << (8 * b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t i = gi * 8 + j;
      if (i >= n) break;
      const float code = (float)((word >> (BITS * j)) & ((1u << BITS) - 1u));
      const int64_t pi = param_index(g, i);
      const float s = loadp(scale, pi, pdt);
      const float z = has_z ? loadp(zp, pi, pdt) : 0.0f;
      store1<DT>(out, i, map_one<DT, 1>(code, s, z, has_z, none, r_out, i));
    }
  }
}

// Fastest path: blocks along the contiguous last axis and K a whole number of
// blocks, so the tensor is a flat run of blocks: vector v belongs to block
// v / G (G = block / V lanes, a power of two) and no row arithmetic is needed.
// Each thread keeps kUnroll 16-byte loads in flight.
template <int DT, bool WRITE_CODES>
__global__ void __launch_bounds__(kThreads, 4)
mx_flat_kernel(const void* __restrict__ in, void* __restrict__ scale_out, void* __restrict__ codes_out,
               int64_t nvec, int G, int gshift, ScaleRule rule, Round r) {
  using E = Elem<DT>;
  constexpr int V = E::kVec;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(rule.scale_round, s_steps[1]);
  const int64_t chunk = (int64_t)kThreads * kUnroll;
  // nvec is a multiple of G and chunk boundaries are multiples of 32, so a
  // block's G lanes are always either all inside or all outside the tensor.
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    Vec<DT> x[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t v = base + u * kThreads + threadIdx.x;
      x[u].raw = make_uint4(0, 0, 0, 0);
      if (v < nvec) x[u].raw = __ldg(reinterpret_cast<const uint4*>(in) + v);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t v = base + u * kThreads + threadIdx.x;
      uint32_t m = 0;
#pragma unroll
      for (int j = 0; j < V; ++j) m = max(m, abs_bits(x[u].get(j)));
      for (int off = 1; off < G; off <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
      float es;
      float scale = block_scale<DT>(m, rule, &es);
      const bool active = v < nvec;
      if (active && (threadIdx.x & (G - 1)) == 0) store1<DT>(scale_out, v >> gshift, scale);
      if (WRITE_CODES && active) {
        Vec<DT> y;
        const int64_t flat = v * V;
        uint32_t sb = __float_as_uint(es);
        const bool pow2 = (sb & 0x007FFFFFu) == 0 && (sb >> 23) >= 1 && (sb >> 23) <= 253;
        if (pow2) {
          float inv = __uint_as_float((254u - (sb >> 23)) << 23);
#pragma unroll
          for (int j = 0; j < V; ++j) y.set(j, apply_round(r, E::round(__fmul_rn(x[u].get(j), inv)), flat + j));
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) y.set(j, apply_round(r, E::round(__fdiv_rn(x[u].get(j), es)), flat + j));
        }
        reinterpret_cast<uint4*>(codes_out)[v] = y.raw;
      }
    }
  }
}

// Ragged path: blocks along the contiguous last axis; row length K a multiple of
// the vector width; a block is covered by G = block/V consecutive lanes.
// Each row owns `slots_per_row` = ceil(K/block) * G thread slots so groups are
// lane-aligned; slots past the row's end only take part in the shuffles.
template <int DT, bool WRITE_CODES>
__global__ void __launch_bounds__(256)
mx_rows_kernel(const void* __restrict__ in, void* __restrict__ scale_out, void* __restrict__ codes_out,
               int64_t rows, int64_t K, int block, int G, int64_t slots_per_row, int64_t total_slots,
               ScaleRule rule, Round r) {
  using E = Elem<DT>;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(rule.scale_round, s_steps[1]);

  constexpr int V = E::kVec;
  const int64_t nblk = slots_per_row / G;
  const int64_t row_vecs = K / V;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // total_slots is rounded up to a multiple of 32 by the launcher, so whole
  // warps enter and leave the loop together.
  for (int64_t slot = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; slot < total_slots; slot += stride) {
    int64_t row = slot / slots_per_row;
    int64_t s_in_row = slot - row * slots_per_row;
    const bool active = row < rows && s_in_row < row_vecs;
    Vec<DT> x;
    x.raw = make_uint4(0, 0, 0, 0);
    if (active) x.raw = __ldg(reinterpret_cast<const uint4*>(in) + row * row_vecs + s_in_row);
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < V; ++j) m = max(m, abs_bits(x.get(j)));
    for (int off = 1; off < G; off <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    float es;
    float scale = block_scale<DT>(m, rule, &es);
    if (active && (s_in_row % G) == 0)
      store1<DT>(scale_out, row * nblk + s_in_row / G, scale);
    if (WRITE_CODES && active) {
      Vec<DT> y;
      const int64_t flat = (row * row_vecs + s_in_row) * V;
      // Dividing by a power of two with a representable reciprocal is the
      // same correctly rounded result as the product with that reciprocal.
      uint32_t sb = __float_as_uint(es);
      const bool pow2 = (sb & 0x007FFFFFu) == 0 && (sb >> 23) >= 1 && (sb >> 23) <= 253;
      if (pow2) {
        float inv = __uint_as_float((254u - (sb >> 23)) << 23);
#pragma unroll
        for (int j = 0; j < V; ++j) y.set(j, apply_round(r, E::round(__fmul_rn(x.get(j), inv)), flat + j));
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) y.set(j, apply_round(r, E::round(__fdiv_rn(x.get(j), es)), flat + j));
      }
      reinterpret_cast<uint4*>(codes_out)[row * row_vecs + s_in_row] = y.raw;
    }
  }
}

// Generic path: one thread per (o, a-block, m, b-block, i); threads are
// consecutive along i, then b-block.  Two passes over the block (the second
// is served from cache).
struct Blocks {
  int64_t O, A, M, B, I;
  int bA, bB;
  int64_t nA, nB;
};

template <int DT, bool WRITE_CODES>
__global__ void __launch_bounds__(256)
mx_generic_kernel(const void* __restrict__ in, void* __restrict__ scale_out, void* __restrict__ codes_out,
                  Blocks g, ScaleRule rule, Round r) {
  using E = Elem<DT>;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(rule.scale_round, s_steps[1]);

  const int64_t total = g.O * g.nA * g.M * g.nB * g.I;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    int64_t i = t % g.I;
    int64_t q = t / g.I;
    int64_t nb = q % g.nB; q /= g.nB;
    int64_t m = q % g.M;   q /= g.M;
    int64_t na = q % g.nA;
    int64_t o = q / g.nA;
    const int64_t a0 = na * g.bA, b0 = nb * g.bB;
    const int64_t a1 = min(a0 + (int64_t)g.bA, g.A), b1 = min(b0 + (int64_t)g.bB, g.B);
    uint32_t mx = 0;
    for (int64_t a = a0; a < a1; ++a) {
      int64_t base = (((o * g.A + a) * g.M + m) * g.B) * g.I + i;
      for (int64_t b = b0; b < b1; ++b) mx = max(mx, abs_bits(load1<DT>(in, base + b * g.I)));
    }
    float es;
    float scale = block_scale<DT>(mx, rule, &es);
    store1<DT>(scale_out, t, scale);
    if (WRITE_CODES) {
      for (int64_t a = a0; a < a1; ++a) {
        int64_t base = (((o * g.A + a) * g.M + m) * g.B) * g.I + i;
        for (int64_t b = b0; b < b1; ++b) {
          int64_t flat = base + b * g.I;
          float y = E::round(__fdiv_rn(load1<DT>(in, flat), es));
          store1<DT>(codes_out, flat, apply_round(r, y, flat));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// group-wise affine (KIVI)
// ---------------------------------------------------------------------------
// torch.amin/amax propagate NaN.
__device__ __forceinline__ float nan_min(float a, float b) { return (a != a || b != b) ? (a + b) : fminf(a, b); }
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a || b != b) ? (a + b) : fmaxf(a, b); }

template <int DT>
__device__ __forceinline__ void affine_params(float low, float high, float qmin, float qmax,
                                              const Round& sr, float* scale, float* zero) {
  using E = Elem<DT>;
  float range = E::round(__fsub_rn(high, low));
  float s = E::round(__fdiv_rn(range, __fsub_rn(qmax, qmin)));
  s = (s > 0.0f) ? s : 1.0f;
  if (sr.mode != VQ_ROUND_NONE) {
    s = E::round(apply_round(sr, s, 0));
    s = (s > 0.0f) ? s : 1.0f;
  }
  float z = E::round(__fdiv_rn(-low, s));
  z = E::round(__fadd_rn(z, qmin));
  if (sr.mode != VQ_ROUND_NONE) z = E::round(apply_round(sr, z, 0));
  *scale = s;
  *zero = z;
}

// Blocks of `block` along B in a dense [O, B, I] view; thread per (o, b-block, i).
template <int DT>
__global__ void __launch_bounds__(256)
affine_generic_kernel(const void* __restrict__ in, void* __restrict__ scale_out, void* __restrict__ zero_out,
                      void* __restrict__ codes_out, int64_t O, int64_t B, int64_t I, int block, int64_t nB,
                      float qmin, float qmax, Round sr, Round r) {
  using E = Elem<DT>;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(sr, s_steps[1]);

  const int64_t total = O * nB * I;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    int64_t i = t % I;
    int64_t q = t / I;
    int64_t nb = q % nB;
    int64_t o = q / nB;
    int64_t b0 = nb * block, b1 = min(b0 + (int64_t)block, B);
    // A short last block is zero padded before the reduction.
    float low = (b1 - b0 < block) ? 0.0f : INFINITY;
    float high = (b1 - b0 < block) ? 0.0f : -INFINITY;
    for (int64_t b = b0; b < b1; ++b) {
      float v = load1<DT>(in, (o * B + b) * I + i);
      low = nan_min(low, v);
      high = nan_max(high, v);
    }
    float s, z;
    affine_params<DT>(low, high, qmin, qmax, sr, &s, &z);
    store1<DT>(scale_out, t, s);
    store1<DT>(zero_out, t, z);
    for (int64_t b = b0; b < b1; ++b) {
      int64_t flat = (o * B + b) * I + i;
      float y = E::round(__fdiv_rn(load1<DT>(in, flat), s));
      y = E::round(__fadd_rn(y, z));
      store1<DT>(codes_out, flat, apply_round(r, y, flat));
    }
  }
}

// Fast path, I == 1: blocks along the contiguous axis, G lanes per block.
template <int DT>
__global__ void __launch_bounds__(256)
affine_rows_kernel(const void* __restrict__ in, void* __restrict__ scale_out, void* __restrict__ zero_out,
                   void* __restrict__ codes_out, int64_t rows, int64_t K, int block, int G,
                   int64_t slots_per_row, int64_t total_slots, float qmin, float qmax, Round sr, Round r) {
  using E = Elem<DT>;
  __shared__ uint16_t s_steps[2][2 * VQ_MAX_STEPS];
  stage_steps(r, s_steps[0]);
  stage_steps(sr, s_steps[1]);

  constexpr int V = E::kVec;
  const int64_t nblk = slots_per_row / G;
  const int64_t row_vecs = K / V;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t slot = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; slot < total_slots; slot += stride) {
    int64_t row = slot / slots_per_row;
    int64_t s_in_row = slot - row * slots_per_row;
    const bool active = row < rows && s_in_row < row_vecs;
    Vec<DT> x;
    x.raw = make_uint4(0, 0, 0, 0);  // padding of a short last block is zero
    if (active) x.raw = __ldg(reinterpret_cast<const uint4*>(in) + row * row_vecs + s_in_row);
    float low = x.get(0), high = x.get(0);
#pragma unroll
    for (int j = 1; j < V; ++j) {
      low = nan_min(low, x.get(j));
      high = nan_max(high, x.get(j));
    }
    for (int off = 1; off < G; off <<= 1) {
      low = nan_min(low, __shfl_xor_sync(0xFFFFFFFFu, low, off));
      high = nan_max(high, __shfl_xor_sync(0xFFFFFFFFu, high, off));
    }
    float s, z;
    affine_params<DT>(low, high, qmin, qmax, sr, &s, &z);
    if (active && (s_in_row % G) == 0) {
      store1<DT>(scale_out, row * nblk + s_in_row / G, s);
      store1<DT>(zero_out, row * nblk + s_in_row / G, z);
    }
    if (active) {
      Vec<DT> y;
      const int64_t flat = (row * row_vecs + s_in_row) * V;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float q = E::round(__fdiv_rn(x.get(j), s));
        q = E::round(__fadd_rn(q, z));
        y.set(j, apply_round(r, q, flat + j));
      }
      reinterpret_cast<uint4*>(codes_out)[row * row_vecs + s_in_row] = y.raw;
    }
  }
}

// ---------------------------------------------------------------------------
// codebook read-back
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256)
dequantize_mx_kernel(const void* __restrict__ in, const void* __restrict__ scale, const void* __restrict__ code,
                     int n_code, const void* __restrict__ gscale, int gdt, void* __restrict__ out, Geom g,
                     int64_t n) {
  using E = Elem<DT>;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool has_g = gscale != nullptr;
  const float gs = has_g ? loadp(gscale, 0, gdt) : 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = load1<DT>(in, i);
    if (code) {
      long long idx = (long long)v;  // Tensor.to(long) truncates
      idx = idx < 0 ? idx + n_code : idx;
      idx = idx < 0 ? 0 : (idx >= n_code ? n_code - 1 : idx);
      v = load1<DT>(code, idx);
    }
    if (scale) v = E::round(__fmul_rn(v, load1<DT>(scale, param_index(g, i))));
    if (has_g) v = E::round(__fmul_rn(v, gs));
    store1<DT>(out, i, v);
  }
}

// ---------------------------------------------------------------------------
// tensor amax
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) amax_kernel(const void* __restrict__ in, int64_t n, int vec_ok,
                                                   uint32_t* __restrict__ out) {
  using E = Elem<DT>;
  constexpr int V = E::kVec;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  uint32_t m = 0;
  int64_t done = 0;
  if (vec_ok) {
    int64_t nvec = n / V;
    for (int64_t v = tid; v < nvec; v += stride) {
      Vec<DT> x;
      x.raw = __ldg(reinterpret_cast<const uint4*>(in) + v);
#pragma unroll
      for (int j = 0; j < V; ++j) m = max(m, abs_bits(x.get(j)));
    }
    done = nvec * V;
  }
  for (int64_t i = done + tid; i < n; i += stride) m = max(m, abs_bits(load1<DT>(in, i)));
  for (int off = 16; off; off >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  __shared__ uint32_t warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = max(m, warp_max[w]);
    atomicMax(out, m);  // non-negative float bits order like unsigned ints
  }
}


// ---------------------------------------------------------------------------
// 16-point random-Hadamard rotation along one axis
// ---------------------------------------------------------------------------
// Dense [O, A, I] input, runs of 16 along A (zero padded to Ap = ceil16(A)):
// out[o][16 r + j][i] = sum_k in[o][16 r + k][i] * m[k][j], accumulated in fp32
// in ascending k, rounded once to the storage dtype.
template <int DT>
__global__ void __launch_bounds__(256)
hadamard_kernel(const void* __restrict__ in, void* __restrict__ out, const float* __restrict__ matrix, int64_t O,
                int64_t A, int64_t Ap, int64_t I) {
  __shared__ float m[16][16];
  for (int t = threadIdx.x; t < 256; t += blockDim.x) m[t >> 4][t & 15] = matrix[t];
  __syncthreads();
  const int64_t runs = Ap / 16;
  const int64_t total = O * runs * I;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t i = t % I;
    const int64_t r = (t / I) % runs;
    const int64_t o = t / (I * runs);
    float x[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int64_t a = r * 16 + k;
      x[k] = a < A ? load1<DT>(in, (o * A + a) * I + i) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float acc = 0.0f;
#pragma unroll
      for (int k = 0; k < 16; ++k) acc = fmaf(x[k], m[k][j], acc);
      store1<DT>(out, (o * Ap + r * 16 + j) * I + i, acc);
    }
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
static int to_geom(const VqBroadcast* b, Geom* g, int64_t* n) {
  if (!b || b->ndim < 1 || b->ndim > VQ_MAX_DIMS) return fail(VQ_EINVAL, "broadcast geometry: ndim out of range");
  g->ndim = b->ndim;
  int64_t total = 1;
  for (int d = 0; d < VQ_MAX_DIMS; ++d) {
    if (d < b->ndim) {
      if (b->size[d] < 0 || b->div[d] < 1) return fail(VQ_EINVAL, "broadcast geometry: bad size/div at dim %d", d);
      g->size[d] = b->size[d];
      g->div[d] = b->div[d];
      g->stride[d] = b->stride[d];
      total *= b->size[d];
    } else {
      g->size[d] = 1;
      g->div[d] = 1;
      g->stride[d] = 0;
    }
  }
  *n = total;
  return VQ_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define VQ_DISPATCH_DTYPE(dtype, ...)                                    \
  switch (dtype) {                                                       \
    case VQ_BF16: { constexpr int DT = VQ_BF16; __VA_ARGS__; break; }    \
    case VQ_F16:  { constexpr int DT = VQ_F16;  __VA_ARGS__; break; }    \
    case VQ_F32:  { constexpr int DT = VQ_F32;  __VA_ARGS__; break; }    \
    default: return vq::fail(VQ_EINVAL, "unknown dtype %d", dtype);      \
  }

static inline int vec_width(int dtype) { return dtype == VQ_F32 ? 4 : 8; }

static int to_rule(const VqScaleRule* rule, ScaleRule* out) {
  if (!rule) return fail(VQ_EINVAL, "scale rule missing");
  if (!(rule->quant_max > 0.0f)) return fail(VQ_EINVAL, "quant_max must be positive");
  if (int e = validate_round(&rule->scale_round, "scale rounding")) return e;
  out->quant_max = rule->quant_max;
  out->power_of_two = rule->power_of_two;
  int ex;
  // floor(log2(quant_max)) as the reference computes it in double precision
  frexp((double)rule->quant_max, &ex);
  out->qmax_exp = ex - 1;
  out->global_scale = rule->global_scale;
  out->global_scale_dtype = rule->global_scale_dtype;
  out->scale_round = make_round(&rule->scale_round);
  // An all-zero block under the power-of-two rule: amax is read as 2^-126, so the
  // scale is 2^(-126 - qexp) rounded to bfloat16 (whose smallest value is 2^-133;
  // 2^-134 ties to zero), and a scale of zero is replaced by one.
  const int ze = -126 - out->qmax_exp;
  out->zero_scale_bf16 = ze >= -133 ? ldexpf(1.0f, ze) : 1.0f;
  return VQ_OK;
}

static int launch_mx(const void* in, void* scale_out, void* codes_out, int dtype, const VqBlocks* b,
                     const VqScaleRule* rule, const VqRound* round, bool write_codes, cudaStream_t st) {
  if (!b) return fail(VQ_EINVAL, "block geometry missing");
  VQ_REQUIRE(b->O >= 0 && b->A >= 0 && b->M >= 0 && b->B >= 0 && b->I >= 0, "negative extent");
  VQ_REQUIRE(b->block_a >= 1 && b->block_b >= 1, "block sizes must be >= 1");
  ScaleRule sr;
  if (int e = to_rule(rule, &sr)) return e;
  if (int e = validate_round(round, "element rounding")) return e;
  Round r = make_round(round);
  const int64_t n = b->O * b->A * b->M * b->B * b->I;
  if (n == 0) return VQ_OK;
  const int V = vec_width(dtype);
  const bool rows_ok = b->I == 1 && b->block_a == 1 && (b->B % V) == 0 && (b->block_b % V) == 0 &&
                       aligned16(in) && (!write_codes || aligned16(codes_out));
  int G = rows_ok ? b->block_b / V : 0;
  const bool g_ok = rows_ok && G >= 1 && G <= 32 && (G & (G - 1)) == 0;
  if (g_ok && (b->B % b->block_b) == 0) {
    const int64_t nvec = n / V;
    int gshift = 0;
    while ((1 << gshift) < G) ++gshift;
    if (dtype == VQ_BF16) {
      const int fm = fast_mode_of(round);
      if (r.mode != VQ_ROUND_STOCHASTIC && r.mode != VQ_ROUND_SEARCH)
        return fast_mx_flat_bf16(in, scale_out, codes_out, nvec, G, gshift, sr, r, fm, write_codes, st);
    }
    int grid = grid_for(nvec, kThreads * kUnroll, 8);
    VQ_DISPATCH_DTYPE(dtype, {
      if (write_codes)
        mx_flat_kernel<DT, true><<<grid, kThreads, 0, st>>>(in, scale_out, codes_out, nvec, G, gshift, sr, r);
      else
        mx_flat_kernel<DT, false><<<grid, kThreads, 0, st>>>(in, scale_out, codes_out, nvec, G, gshift, sr, r);
    });
    return check_launch("mx_flat_kernel");
  }
  if (g_ok) {
    const int64_t rows = b->O * b->A * b->M;
    const int64_t nblk = (b->B + b->block_b - 1) / b->block_b;
    const int64_t slots_per_row = nblk * G;
    int64_t total = rows * slots_per_row;
    total = (total + 31) / 32 * 32;
    int grid = grid_for(total, 256, 8);
    VQ_DISPATCH_DTYPE(dtype, {
      if (write_codes)
        mx_rows_kernel<DT, true><<<grid, 256, 0, st>>>(in, scale_out, codes_out, rows, b->B, b->block_b, G,
                                                       slots_per_row, total, sr, r);
      else
        mx_rows_kernel<DT, false><<<grid, 256, 0, st>>>(in, scale_out, codes_out, rows, b->B, b->block_b, G,
                                                        slots_per_row, total, sr, r);
    });
    return check_launch("mx_rows_kernel");
  }
  Blocks g{b->O, b->A, b->M, b->B, b->I, b->block_a, b->block_b,
           (b->A + b->block_a - 1) / b->block_a, (b->B + b->block_b - 1) / b->block_b};
  const int64_t total = g.O * g.nA * g.M * g.nB * g.I;
  int grid = grid_for(total, 256, 8);
  VQ_DISPATCH_DTYPE(dtype, {
    if (write_codes)
      mx_generic_kernel<DT, true><<<grid, 256, 0, st>>>(in, scale_out, codes_out, g, sr, r);
    else
      mx_generic_kernel<DT, false><<<grid, 256, 0, st>>>(in, scale_out, codes_out, g, sr, r);
  });
  return check_launch("mx_generic_kernel");
}

}  // namespace vq

using namespace vq;

extern "C" {

const char* vq_last_error(void) { return error_buffer(); }
int vq_version(void) { return 1; }

static int launch_stream(int kind, const void* in, const void* scale, const void* zp, void* out, int dtype,
                         int pdt, const Geom* g, const Round& ri, const Round& ro, int64_t n, cudaStream_t st,
                         int fast_mode = 7 /* FAST_GENERIC */) {
  const int V = vec_width(dtype);
  ParamIndex pi{PI_SCALAR, 1, 0, 1};
  bool fast = aligned16(in) && aligned16(out);
  if (kind != 2) {
    // reduce the collapsed broadcast to scalar / flat-div / flat-mod when possible
    bool scalar = true;
    for (int d = 0; d < g->ndim; ++d)
      if (g->stride[d] != 0 && (g->size[d] + g->div[d] - 1) / g->div[d] > 1) scalar = false;
    if (scalar) {
      pi.kind = PI_SCALAR;
    } else if (g->ndim == 1 && g->stride[0] == 1) {
      pi.kind = PI_DIV;
      pi.d = (uint32_t)g->div[0];
    } else if (g->ndim == 2 && g->div[0] == 1 && g->stride[1] == 1 && g->size[1] % g->div[1] == 0 &&
               g->stride[0] == g->size[1] / g->div[1]) {
      pi.kind = PI_DIV;  // dense per-block parameters of a [rows, K] tensor
      pi.d = (uint32_t)g->div[1];
    } else if (g->ndim == 2 && g->div[0] == 1 && g->stride[0] == 1 && g->stride[1] == 0) {
      pi.kind = PI_DIV;  // one parameter per row
      pi.d = (uint32_t)g->size[1];
    } else if (g->ndim == 2 && g->stride[0] == 0 && g->div[1] == 1 && g->stride[1] == 1) {
      pi.kind = PI_MOD;  // one parameter per column
      pi.c = (uint32_t)g->size[1];
    } else if (g->ndim == 1 && g->div[0] == 1 && g->stride[0] == 1) {
      pi.kind = PI_MOD;
      pi.c = (uint32_t)g->size[0];
    } else {
      pi.kind = PI_GENERIC;
    }
    if (pi.kind == PI_DIV) {
      if (pi.d == 0 || pi.d % V != 0 || g->div[g->ndim - 1] > 0x7FFFFFFF) pi.kind = PI_GENERIC;
      pi.shift = -1;
      if ((pi.d & (pi.d - 1)) == 0) { pi.shift = 0; while ((1u << pi.shift) < pi.d) ++pi.shift; }
    }
    if (pi.kind == PI_MOD && (pi.c % V != 0)) pi.kind = PI_GENERIC;
    if (pi.kind != PI_SCALAR && (n % V) != 0) pi.kind = PI_GENERIC;
  }
  if (!fast || pi.kind == PI_GENERIC) {
    if (kind == 2) {
      Geom gg{};
      gg.ndim = 1; gg.size[0] = n; gg.div[0] = 1; gg.stride[0] = 0;
      int grid = grid_for(n, kThreads, 8);
      VQ_DISPATCH_DTYPE(dtype, (generic_map_kernel<DT, 2><<<grid, kThreads, 0, st>>>(in, scale, zp, out, gg, ri, ro, n, pdt)));
      return check_launch("generic_map_kernel");
    }
    int grid = grid_for(n, kThreads, 8);
    VQ_DISPATCH_DTYPE(dtype, {
      if (kind == 0) generic_map_kernel<DT, 0><<<grid, kThreads, 0, st>>>(in, scale, zp, out, *g, ri, ro, n, pdt);
      else generic_map_kernel<DT, 1><<<grid, kThreads, 0, st>>>(in, scale, zp, out, *g, ri, ro, n, pdt);
    });
    return check_launch("generic_map_kernel");
  }
  if (kind == 0 && dtype == VQ_BF16 && zp == nullptr && (n % V) == 0 && ro.mode != VQ_ROUND_STOCHASTIC &&
      ro.mode != VQ_ROUND_SEARCH && (pi.kind == PI_SCALAR || pi.kind == PI_DIV)) {
    const uint32_t vps = pi.kind == PI_SCALAR ? 0u : pi.d / (uint32_t)V;
    return fast_quantize_bf16(in, scale, pdt, out, n / V, vps, ro, fast_mode, st);
  }
  const int n32 = n < 0xFFFFFFFFll;
  int grid = grid_for((n + V - 1) / V, kThreads * kUnroll, 8);
  VQ_DISPATCH_DTYPE(dtype, {
    if (kind == 0) stream_map_kernel<DT, 0><<<grid, kThreads, 0, st>>>(in, scale, zp, out, ri, ro, n, pi, pdt, n32);
    else if (kind == 1) stream_map_kernel<DT, 1><<<grid, kThreads, 0, st>>>(in, scale, zp, out, ri, ro, n, pi, pdt, n32);
    else stream_map_kernel<DT, 2><<<grid, kThreads, 0, st>>>(in, scale, zp, out, ri, ro, n, pi, pdt, n32);
  });
  return check_launch("stream_map_kernel");
}

int vq_vmap(const void* in, void* out, int dtype, const VqRound* round, int64_t n, void* stream) {
  VQ_REQUIRE(n >= 0, "vq_vmap: negative size");
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(in && out && round, "vq_vmap: null argument");
  if (int e = validate_round(round, "vq_vmap")) return e;
  Round none = make_round(nullptr);
  return launch_stream(2, in, nullptr, nullptr, out, dtype, dtype, nullptr, none, make_round(round), n,
                       static_cast<cudaStream_t>(stream));
}

static int scale_map(int kind, const void* in, const void* scale, const void* zp, void* out, int dtype,
                     int param_dtype, const VqBroadcast* geom, const VqRound* r_in, const VqRound* r_out, void* stream) {
  Geom g;
  int64_t n;
  if (int e = to_geom(geom, &g, &n)) return e;
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(in && scale && out, "quantize/dequantize: null argument");
  VQ_REQUIRE(param_dtype >= VQ_BF16 && param_dtype <= VQ_F32, "quantize/dequantize: bad parameter dtype");
  if (int e = validate_round(r_in, "input rounding")) return e;
  if (int e = validate_round(r_out, "output rounding")) return e;
  Round ri = make_round(r_in), ro = make_round(r_out);
  return launch_stream(kind, in, scale, zp, out, dtype, param_dtype, &g, ri, ro, n, static_cast<cudaStream_t>(stream),
                       fast_mode_of(r_out));
}

int vq_quantize(const void* in, const void* scale, const void* zero_point, void* out, int dtype,
                int param_dtype, const VqBroadcast* geom, const VqRound* round, void* stream) {
  return scale_map(0, in, scale, zero_point, out, dtype, param_dtype, geom, nullptr, round, stream);
}

int vq_dequantize(const void* in, const void* scale, const void* zero_point, void* out, int dtype,
                  int param_dtype, const VqBroadcast* geom, const VqRound* round_in, const VqRound* round_out,
                  void* stream) {
  return scale_map(1, in, scale, zero_point, out, dtype, param_dtype, geom, round_in, round_out, stream);
}

int vq_pack_codes(const void* codes, int dtype, void* packed, int bits, int64_t n, void* stream) {
  VQ_REQUIRE(n >= 0, "vq_pack_codes: negative size");
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(codes && packed, "vq_pack_codes: null argument");
  VQ_REQUIRE(bits == 2 || bits == 4 || bits == 8, "vq_pack_codes: bits must be 2, 4 or 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 7) / 8, kThreads, 8);
#define VQ_PACK(B) VQ_DISPATCH_DTYPE(dtype, (pack_codes_kernel<DT, B><<<grid, kThreads, 0, st>>>(codes, static_cast<uint8_t*>(packed), n)))
  if (bits == 2) { VQ_PACK(2); } else if (bits == 4) { VQ_PACK(4); } else { VQ_PACK(8); }
#undef VQ_PACK
  return check_launch("pack_codes_kernel");
}

int vq_unpack_dequantize(const void* packed, int bits, const void* scale, const void* zero_point, void* out,
                         int dtype, int param_dtype, const VqBroadcast* geom, const VqRound* round_out,
                         void* stream) {
  Geom g;
  int64_t n;
  if (int e = to_geom(geom, &g, &n)) return e;
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(packed && scale && out, "vq_unpack_dequantize: null argument");
  VQ_REQUIRE(bits == 2 || bits == 4 || bits == 8, "vq_unpack_dequantize: bits must be 2, 4 or 8");
  VQ_REQUIRE(param_dtype >= VQ_BF16 && param_dtype <= VQ_F32, "vq_unpack_dequantize: bad parameter dtype");
  if (int e = validate_round(round_out, "output rounding")) return e;
  Round ro = make_round(round_out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 7) / 8, kThreads, 8);
  const uint8_t* src = static_cast<const uint8_t*>(packed);
#define VQ_UNPACK(B) VQ_DISPATCH_DTYPE(dtype, (unpack_dequantize_kernel<DT, B><<<grid, kThreads, 0, st>>>(src, scale, zero_point, out, g, ro, n, param_dtype)))
  if (bits == 2) { VQ_UNPACK(2); } else if (bits == 4) { VQ_UNPACK(4); } else { VQ_UNPACK(8); }
#undef VQ_UNPACK
  return check_launch("unpack_dequantize_kernel");
}

static inline bool empty_blocks(const VqBlocks* b) {
  return b && (b->O == 0 || b->A == 0 || b->M == 0 || b->B == 0 || b->I == 0);
}

int vq_mx_qparam(const void* in, void* scale_out, int dtype, const VqBlocks* blocks, const VqScaleRule* rule,
                 void* stream) {
  if (empty_blocks(blocks)) return VQ_OK;
  VQ_REQUIRE(in && scale_out, "vq_mx_qparam: null argument");
  return launch_mx(in, scale_out, nullptr, dtype, blocks, rule, nullptr, false, static_cast<cudaStream_t>(stream));
}

int vq_quantize_mx(const void* in, void* scale_out, void* codes_out, int dtype, const VqBlocks* blocks,
                   const VqScaleRule* rule, const VqRound* round, void* stream) {
  if (empty_blocks(blocks)) return VQ_OK;
  VQ_REQUIRE(in && scale_out && codes_out, "vq_quantize_mx: null argument");
  return launch_mx(in, scale_out, codes_out, dtype, blocks, rule, round, true, static_cast<cudaStream_t>(stream));
}

int vq_quantize_affine(const void* in, void* scale_out, void* zero_out, void* codes_out, int dtype,
                       const VqBlocks* b, float quant_min, float quant_max, const VqRound* scale_round,
                       const VqRound* round, void* stream) {
  if (empty_blocks(b)) return VQ_OK;
  VQ_REQUIRE(in && scale_out && zero_out && codes_out && b, "vq_quantize_affine: null argument");
  VQ_REQUIRE(b->block_a == 1 && b->A == 1 && b->M == 1, "vq_quantize_affine: blocks lie along one axis (B)");
  VQ_REQUIRE(b->block_b >= 1, "vq_quantize_affine: block size must be >= 1");
  VQ_REQUIRE(quant_max > quant_min, "vq_quantize_affine: empty code range");
  if (int e = validate_round(scale_round, "scale rounding")) return e;
  if (int e = validate_round(round, "element rounding")) return e;
  Round sr = make_round(scale_round), r = make_round(round);
  const int64_t n = b->O * b->B * b->I;
  if (n == 0) return VQ_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int V = vec_width(dtype);
  const int64_t nB = (b->B + b->block_b - 1) / b->block_b;
  int G = b->block_b / V;
  const bool rows_ok = b->I == 1 && (b->B % V) == 0 && (b->block_b % V) == 0 && G >= 1 && G <= 32 &&
                       (G & (G - 1)) == 0 && aligned16(in) && aligned16(codes_out);
  if (rows_ok) {
    const int64_t slots_per_row = nB * G;
    int64_t total = b->O * slots_per_row;
    total = (total + 31) / 32 * 32;
    int grid = grid_for(total, 256, 8);
    VQ_DISPATCH_DTYPE(dtype, (affine_rows_kernel<DT><<<grid, 256, 0, st>>>(
        in, scale_out, zero_out, codes_out, b->O, b->B, b->block_b, G, slots_per_row, total, quant_min,
        quant_max, sr, r)));
    return check_launch("affine_rows_kernel");
  }
  int grid = grid_for(b->O * nB * b->I, 256, 8);
  VQ_DISPATCH_DTYPE(dtype, (affine_generic_kernel<DT><<<grid, 256, 0, st>>>(
      in, scale_out, zero_out, codes_out, b->O, b->B, b->I, b->block_b, nB, quant_min, quant_max, sr, r)));
  return check_launch("affine_generic_kernel");
}

int vq_dequantize_mx(const void* in, const void* scale, const void* code, int32_t n_code,
                     const void* global_scale, int global_scale_dtype, void* out, int dtype,
                     const VqBroadcast* geom, void* stream) {
  Geom g;
  int64_t n;
  if (int e = to_geom(geom, &g, &n)) return e;
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(in && out, "vq_dequantize_mx: null argument");
  VQ_REQUIRE(!code || n_code > 0, "vq_dequantize_mx: empty codebook");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == VQ_BF16 && !code && scale && !global_scale && (n % 8) == 0 && aligned16(in) && aligned16(out)) {
    // dense per-block scales along the last axis: parameter index = flat / block
    int64_t d = 0;
    if (g.ndim == 1 && g.stride[0] == 1) d = g.div[0];
    else if (g.ndim == 2 && g.div[0] == 1 && g.stride[1] == 1 && g.size[1] % g.div[1] == 0 &&
             g.stride[0] == g.size[1] / g.div[1]) d = g.div[1];
    if (d >= 8 && d % 8 == 0 && d < (1ll << 31))
      return fast_scale_bf16(in, scale, out, n / 8, (uint32_t)(d / 8), st);
  }
  int grid = grid_for(n, 256, 8);
  VQ_DISPATCH_DTYPE(dtype, (dequantize_mx_kernel<DT><<<grid, 256, 0, st>>>(in, scale, code, n_code, global_scale,
                                                                         global_scale_dtype, out, g, n)));
  return check_launch("dequantize_mx_kernel");
}

int vq_amax(const void* in, int dtype, int64_t n, float* out, void* stream) {
  VQ_REQUIRE(n >= 0 && out, "vq_amax: bad argument");
  if (n == 0) return VQ_OK;
  VQ_REQUIRE(in != nullptr, "vq_amax: null input");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int vec_ok = aligned16(in);
  int grid = grid_for((n + vec_width(dtype) - 1) / vec_width(dtype), 256, 4);
  VQ_DISPATCH_DTYPE(dtype, (amax_kernel<DT><<<grid, 256, 0, st>>>(in, n, vec_ok, reinterpret_cast<uint32_t*>(out))));
  return check_launch("amax_kernel");
}

int vq_hadamard_rotate(const void* in, void* out, int dtype, const float* matrix, int64_t O, int64_t A, int64_t I,
                       void* stream) {
  VQ_REQUIRE(O >= 0 && A >= 0 && I >= 0, "vq_hadamard_rotate: negative extent");
  if (O == 0 || A == 0 || I == 0) return VQ_OK;
  VQ_REQUIRE(in && out && matrix, "vq_hadamard_rotate: null argument");
  const int64_t Ap = (A + 15) / 16 * 16;
  int grid = grid_for(O * (Ap / 16) * I, 256, 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VQ_DISPATCH_DTYPE(dtype, (hadamard_kernel<DT><<<grid, 256, 0, st>>>(in, out, matrix, O, A, Ap, I)));
  return check_launch("hadamard_kernel");
}

}  // extern "C"
