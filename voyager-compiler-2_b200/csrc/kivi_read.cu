// Reading a packed KIVI cache: 2-bit codes (four per byte) of a [outer, T, D] bfloat16 tensor
// back to values,
//
//   out = bf16( bf16(code - zero_point) * scale )
//
// which is quantized_ops::dequantize(codes, scale, zero_point, axes, block) on the unpacked codes
// (reference ops/quantized.py:527-571; the KIVI read of quant_folding.py:2391-2547), every step
// rounded to bfloat16 as that operator does.  Keys are grouped along T (one scale and zero point
// per channel and group of `block` positions: parameters [outer, T / block, D]); values along D
// (one per position and group of `block` channels: [outer, T, D / block]).
//
// The kernel is bound by HBM: 0.25 byte in, 2 bytes out per element.  A thread owns eight
// consecutive channels (two packed bytes in, one 16-byte store out).  For keys it keeps its eight
// scales and zero points in registers and walks the positions of its group; for values it reads
// one pair of parameters per position.
#include "vq_common.cuh"

namespace vq {
namespace {

__device__ __forceinline__ uint32_t dq_pair(uint32_t codes, float z0, float z1, float s0, float s1) {
  // two 2-bit codes in bits [0, 4) of `codes`
  const float c0 = (float)(codes & 3u), c1 = (float)((codes >> 2) & 3u);
  const float d0 = __bfloat162float(__float2bfloat16_rn(c0 - z0));
  const float d1 = __bfloat162float(__float2bfloat16_rn(c1 - z1));
  const __nv_bfloat162 h = __floats2bfloat162_rn(d0 * s0, d1 * s1);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// groups along T: grid.x covers (outer x T / block) groups x (D / 8) channel chunks
__global__ void __launch_bounds__(256)
kivi_read_keys_kernel(const uint8_t* __restrict__ packed, const __nv_bfloat16* __restrict__ scale,
                      const __nv_bfloat16* __restrict__ zero, __nv_bfloat16* __restrict__ out, int64_t groups,
                      int T_block, int D) {
  const int chunks = D >> 3;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 1) + (threadIdx.x >> 1);   // (group, chunk); two threads each
  if (item >= groups * chunks) return;
  const int64_t grp = item / chunks;
  const int c = (int)(item - grp * chunks);
  const int parity = threadIdx.x & 1;                                                   // even / odd positions
  const uint4 sv = *reinterpret_cast<const uint4*>(scale + grp * D + c * 8);
  const uint4 zv = *reinterpret_cast<const uint4*>(zero + grp * D + c * 8);
  float s[8], z[8];
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    s[2 * q] = __uint_as_float(sw[q] << 16); s[2 * q + 1] = __uint_as_float(sw[q] & 0xFFFF0000u);
    z[2 * q] = __uint_as_float(zw[q] << 16); z[2 * q + 1] = __uint_as_float(zw[q] & 0xFFFF0000u);
  }
  const int64_t row0 = grp * T_block;                                                   // first position of the group
  const uint8_t* src = packed + (row0 * D >> 2) + c * 2;
  __nv_bfloat16* dst = out + row0 * D + c * 8;
  const int row_bytes = D >> 2;
#pragma unroll 4
  for (int t = parity; t < T_block; t += 2) {
    const uint32_t w = *reinterpret_cast<const uint16_t*>(src + (int64_t)t * row_bytes);
    uint4 o;
    o.x = dq_pair(w, z[0], z[1], s[0], s[1]);
    o.y = dq_pair(w >> 4, z[2], z[3], s[2], s[3]);
    o.z = dq_pair(w >> 8, z[4], z[5], s[4], s[5]);
    o.w = dq_pair(w >> 12, z[6], z[7], s[6], s[7]);
    *reinterpret_cast<uint4*>(dst + (int64_t)t * D) = o;
  }
}

// groups along D: one thread per eight channels of one position, grid-stride
__global__ void __launch_bounds__(256)
kivi_read_values_kernel(const uint8_t* __restrict__ packed, const __nv_bfloat16* __restrict__ scale,
                        const __nv_bfloat16* __restrict__ zero, __nv_bfloat16* __restrict__ out, int64_t vectors,
                        int D, int block_shift) {
  const int chunks = D >> 3;
  const int groups_per_row = D >> block_shift;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vectors; v += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = v / chunks;
    const int c = (int)(v - row * chunks);
    const int64_t pi = row * groups_per_row + ((c * 8) >> block_shift);
    const float s = __bfloat162float(scale[pi]), z = __bfloat162float(zero[pi]);
    const uint32_t w = *reinterpret_cast<const uint16_t*>(packed + v * 2);
    uint4 o;
    o.x = dq_pair(w, z, z, s, s);
    o.y = dq_pair(w >> 4, z, z, s, s);
    o.z = dq_pair(w >> 8, z, z, s, s);
    o.w = dq_pair(w >> 12, z, z, s, s);
    *reinterpret_cast<uint4*>(out + v * 8) = o;
  }
}

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_kivi_read_2bit(const void* packed, const void* scale, const void* zero_point, void* out,
                                 int64_t outer, int64_t T, int64_t D, int along_channels, int64_t block,
                                 void* stream) {
  VQ_REQUIRE(outer >= 0 && T >= 0 && D >= 0 && block > 0, "vq_kivi_read_2bit: bad extents");
  if (outer == 0 || T == 0 || D == 0) return VQ_OK;
  VQ_REQUIRE(packed && scale && zero_point && out, "vq_kivi_read_2bit: null argument");
  VQ_REQUIRE(D % 8 == 0 && D < (1 << 20), "vq_kivi_read_2bit: the channel count must be a multiple of 8");
  VQ_REQUIRE(((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scale) |
               reinterpret_cast<uintptr_t>(zero_point)) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed) & 1) == 0,
             "vq_kivi_read_2bit: buffers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (along_channels) {
    VQ_REQUIRE(block >= 8 && (block & (block - 1)) == 0 && D % block == 0,
               "vq_kivi_read_2bit: channel groups are a power of two, at least 8, dividing D");
    int shift = 0;
    while ((1ll << shift) < block) ++shift;
    const int64_t vectors = outer * T * (D / 8);
    const int64_t want = (vectors + 255) / 256;
    const int grid = (int)(want < (int64_t)kSmCount * 16 ? want : (int64_t)kSmCount * 16);
    kivi_read_values_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(packed),
                                                  static_cast<const __nv_bfloat16*>(scale),
                                                  static_cast<const __nv_bfloat16*>(zero_point),
                                                  static_cast<__nv_bfloat16*>(out), vectors, (int)D, shift);
    return check_launch("kivi_read_values_kernel");
  }
  VQ_REQUIRE(T % block == 0 && block < (1 << 20), "vq_kivi_read_2bit: position groups must divide T");
  const int64_t groups = outer * (T / block);
  const int64_t items = groups * (D / 8);
  const int64_t blocks = (items + 127) / 128;
  VQ_REQUIRE(blocks < (1ll << 31), "vq_kivi_read_2bit: tensor too large");
  kivi_read_keys_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint8_t*>(packed),
                                                         static_cast<const __nv_bfloat16*>(scale),
                                                         static_cast<const __nv_bfloat16*>(zero_point),
                                                         static_cast<__nv_bfloat16*>(out), groups, (int)block, (int)D);
  return check_launch("kivi_read_keys_kernel");
}
