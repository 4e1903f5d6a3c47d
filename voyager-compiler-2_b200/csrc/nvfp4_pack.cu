// NVFP4 operands in the form the block-scaled tensor-core MMA consumes.
//
//   codes : e2m1, two per byte (even element in the low nibble), rows of K/2 bytes
//   scales: e4m3 bytes, one per 16 elements, in 512-byte tiles of 128 rows x 4
//           scales: byte (r % 32) * 16 + (r / 32) * 4 + s of tile
//           (row_block * K/64 + k64_block)
// which is the layout the reference's NVFP4 cast writes for cuBLAS
// (backend/gpu/nvfp4.py:351-372) and what tcgen05.cp moves into tensor memory
// with one 32x128b.warpx4 copy per tile.
//
// Two producers: a fused cast from bfloat16 activations/weights (the arithmetic of
// quantized_ops::quantize_mx with an e2m1 table, e4m3 scale table and a global
// scale, every step rounded to bfloat16 as the op does), and a packer of the
// op's own outputs (bfloat16-valued codes and scales), which also verifies that
// every value is representable.

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "quantize_shared.cuh"

namespace vq {
namespace {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ int64_t scale_tile_offset(int64_t row, int64_t k64, int64_t k64_blocks) {
  return ((row >> 7) * k64_blocks + k64) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4;
}

// One thread = one 16-byte vector (8 elements); two neighbouring lanes share a
// 16-element block (amax by one shuffle) and eight lanes a 64-element group, whose
// four scale bytes its first lane collects and writes as one word.  Loads and
// stores of a warp are contiguous: 512 bytes in, 128 bytes of codes out.
__global__ void __launch_bounds__(256, 4)
quantize_nvfp4_kernel(const uint4* __restrict__ in, const void* __restrict__ global_scale, int gs_dt,
                      uint32_t* __restrict__ codes, uint8_t* __restrict__ scales, int64_t rows, int64_t K) {
  constexpr int U = 4;
  const int64_t k64_blocks = K >> 6;
  const int64_t nvec = rows * (K >> 3);
  const float t = loadp(global_scale, 0, gs_dt);
  const bool t_ordinary = ordinary_divisor(t);
  const bool small = (nvec >> 3) < 0x7FFFFFFFll && k64_blocks < 0x7FFFFFFFll;
  const float rcp_t = __frcp_rn(t), rcp6 = __frcp_rn(6.0f);
  const int64_t chunk = (int64_t)blockDim.x * U;
  for (int64_t base = (int64_t)blockIdx.x * chunk; base < nvec; base += (int64_t)gridDim.x * chunk) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * blockDim.x + threadIdx.x;
      x[u] = make_uint4(0, 0, 0, 0);
      if (v < nvec) x[u] = __ldg(in + v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * blockDim.x + threadIdx.x;
      const uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
      uint32_t m2 = __vmaxu2(__vmaxu2(w[0] & 0x7FFF7FFFu, w[1] & 0x7FFF7FFFu),
                             __vmaxu2(w[2] & 0x7FFF7FFFu, w[3] & 0x7FFF7FFFu));
      uint32_t m = max(m2 & 0xFFFFu, m2 >> 16);
      m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
      // scale = e4m3(bf16(bf16(amax / 6) / t)), replaced by 1 when it is not positive
      const float amax = __uint_as_float(m << 16);
      float s;
      if (t_ordinary && (m >> 7) >= 1u && (m >> 7) <= 254u) {
        s = div_to_bf16(div_to_bf16(amax, 6.0f, rcp6), t, rcp_t);  // exact quotients, no true division
      } else {
        s = bf16r(__fdiv_rn(bf16r(__fdiv_rn(amax, 6.0f)), t));
      }
      uint32_t sb = (uint32_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
      s = e4m3_to_float(sb);
      if (!(s > 0.0f)) { s = 1.0f; sb = 0x38u; }
      const float es = bf16r(__fmul_rn(s, t));
      const bool ordinary = ordinary_divisor(es);
      const float rcp = __frcp_rn(es);
      uint32_t nib = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
        float a, b;
        if (ordinary) {
          a = div_to_bf16(lo, es, rcp);
          b = div_to_bf16(hi, es, rcp);
        } else {
          a = bf16r(__fdiv_rn(lo, es));
          b = bf16r(__fdiv_rn(hi, es));
        }
        const float2 f = make_float2(__fadd_rn(a, 0.0f), __fadd_rn(b, 0.0f));
        nib |= (uint32_t)__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest) << (8 * j);
      }
      // the group's four scale bytes sit in lanes 0, 2, 4, 6 of each aligned group of 8 lanes
      const int lane8 = threadIdx.x & 7;
      const int first = (threadIdx.x & 31) & ~7;
      uint32_t sbytes = __shfl_sync(0xFFFFFFFFu, sb, first) | (__shfl_sync(0xFFFFFFFFu, sb, first + 2) << 8) |
                        (__shfl_sync(0xFFFFFFFFu, sb, first + 4) << 16) | (__shfl_sync(0xFFFFFFFFu, sb, first + 6) << 24);
      if (v < nvec) {
        codes[v] = nib;
        if (lane8 == 0) {
          const int64_t g = v >> 3;  // 64-element group index
          // 64-bit division is ~100 instructions; almost every tensor fits 32 bits
          const int64_t row = small ? (int64_t)((uint32_t)g / (uint32_t)k64_blocks) : g / k64_blocks;
          const int64_t k64 = g - row * k64_blocks;
          *reinterpret_cast<uint32_t*>(scales + scale_tile_offset(row, k64, k64_blocks)) = sbytes;
        }
      }
    }
  }
}

// Pack the operator's outputs: bfloat16-valued e2m1 codes [rows, K] and bfloat16 scales
// [rows, K/16] whose values are e4m3 numbers.  A value that is not representable sets *bad.
__global__ void __launch_bounds__(128)
pack_nvfp4_kernel(const uint4* __restrict__ codes_in, const uint2* __restrict__ scales_in, uint4* __restrict__ codes,
                  uint8_t* __restrict__ scales, int64_t rows, int64_t K, int* __restrict__ bad) {
  const int64_t k64_blocks = K >> 6;
  const int64_t total = rows * k64_blocks;
  bool wrong = false;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / k64_blocks;
    const int64_t k64 = idx - row * k64_blocks;
    const uint4* src = codes_in + idx * 8;
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 x = __ldg(src + i);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      uint32_t nib = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
        const uint32_t q = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
        __half2_raw back = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)q, __NV_E2M1);
        const float2 fb = __half22float2(*reinterpret_cast<__half2*>(&back));
        wrong |= (fb.x != lo) | (fb.y != hi);
        nib |= q << (8 * j);
      }
      packed[i] = nib;
    }
    const uint2 sraw = __ldg(scales_in + idx);  // four bfloat16 scales
    const uint32_t sw[2] = {sraw.x, sraw.y};
    uint32_t sbytes = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float s = __uint_as_float((j & 1) ? (sw[j >> 1] & 0xFFFF0000u) : (sw[j >> 1] << 16));
      const uint32_t sb = (uint32_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
      wrong |= e4m3_to_float(sb) != s;
      sbytes |= sb << (8 * j);
    }
    uint4* dst = codes + idx * 2;
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    *reinterpret_cast<uint32_t*>(scales + scale_tile_offset(row, k64, k64_blocks)) = sbytes;
  }
  if (wrong) atomicExch(bad, 1);
}

inline int grid_for_items(int64_t items) {
  int64_t blocks = (items + 127) / 128;
  const int64_t cap = (int64_t)kSmCount * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int64_t vq_nvfp4_scale_bytes(int64_t rows, int64_t K) {
  if (rows < 0 || K < 0) return -1;
  return ((rows + 127) / 128) * ((K + 63) / 64) * 512;
}

extern "C" int vq_quantize_nvfp4(const void* in, const void* global_scale, int global_scale_dtype, void* codes,
                                 void* scales, int64_t rows, int64_t K, void* stream) {
  VQ_REQUIRE(rows >= 0 && K >= 0, "vq_quantize_nvfp4: negative extent");
  if (rows == 0 || K == 0) return VQ_OK;
  VQ_REQUIRE(in && global_scale && codes && scales, "vq_quantize_nvfp4: null argument");
  VQ_REQUIRE(K % 64 == 0, "vq_quantize_nvfp4: K must be a multiple of 64");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(codes) |
               reinterpret_cast<uintptr_t>(scales)) & 15) == 0, "vq_quantize_nvfp4: misaligned buffers");
  const int64_t nvec = rows * (K / 8);
  int64_t blocks = (nvec + 1023) / 1024;
  const int64_t cap = (int64_t)kSmCount * 4;
  const int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  quantize_nvfp4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(in), global_scale, global_scale_dtype, static_cast<uint32_t*>(codes),
      static_cast<uint8_t*>(scales), rows, K);
  return check_launch("quantize_nvfp4_kernel");
}

extern "C" int vq_pack_nvfp4(const void* codes_in, const void* scales_in, void* codes, void* scales, int64_t rows,
                             int64_t K, int* bad_flag, void* stream) {
  VQ_REQUIRE(rows >= 0 && K >= 0, "vq_pack_nvfp4: negative extent");
  if (rows == 0 || K == 0) return VQ_OK;
  VQ_REQUIRE(codes_in && scales_in && codes && scales && bad_flag, "vq_pack_nvfp4: null argument");
  VQ_REQUIRE(K % 64 == 0, "vq_pack_nvfp4: K must be a multiple of 64");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(codes_in) | reinterpret_cast<uintptr_t>(codes) |
               reinterpret_cast<uintptr_t>(scales)) & 15) == 0 && (reinterpret_cast<uintptr_t>(scales_in) & 7) == 0,
             "vq_pack_nvfp4: misaligned buffers");
  pack_nvfp4_kernel<<<grid_for_items(rows * (K / 64)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(codes_in), static_cast<const uint2*>(scales_in), static_cast<uint4*>(codes),
      static_cast<uint8_t*>(scales), rows, K, bad_flag);
  return check_launch("pack_nvfp4_kernel");
}
