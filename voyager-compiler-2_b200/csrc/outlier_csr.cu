// Outlier side stream: a fixed-capacity CSR matrix of the elements whose magnitude
// reaches a threshold, built on the device without a host read, and its product
// with a dense matrix in float32.
//
// The capacity (entries per matrix) and every output shape depend only on the
// input's shape, so the whole sequence can be captured in a CUDA graph: a row's
// outliers are counted by one warp, the caller turns the counts into row
// pointers with a prefix sum, and a second pass places values and column
// indices.  Entries beyond the capacity are dropped in row-major order.

#include "quantize_shared.cuh"

namespace vq {
namespace {

template <int DT>
__device__ __forceinline__ bool is_stored_outlier(float v, float threshold) {
  // zero-valued entries never enter a sparse matrix
  return fabsf(v) >= threshold && v != 0.0f;
}

// counts[row] = stored outliers of the row; one warp per row of the [rows_total, cols] view
template <int DT>
__global__ void __launch_bounds__(256)
outlier_count_kernel(const void* __restrict__ in, int32_t* __restrict__ counts, int64_t rows_total, int cols,
                     float threshold) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  int n = 0;
  for (int c = lane; c < cols; c += 32) n += is_stored_outlier<DT>(load1<DT>(in, row * cols + c), threshold) ? 1 : 0;
  for (int off = 16; off; off >>= 1) n += __shfl_xor_sync(0xFFFFFFFFu, n, off);
  if (lane == 0) counts[row] = n;
}

// row_start: [batches, rows + 1] exclusive prefix sums of the counts (not clamped to the capacity)
template <int DT>
__global__ void __launch_bounds__(256)
outlier_fill_kernel(const void* __restrict__ in, void* __restrict__ inlier, void* __restrict__ data,
                    int32_t* __restrict__ indices, const int32_t* __restrict__ row_start, int64_t rows_total,
                    int rows, int cols, float threshold, int capacity) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int64_t b = row / rows;
  const int r = (int)(row - b * rows);
  int pos = row_start[b * (rows + 1) + r];
  for (int c0 = 0; c0 < cols; c0 += 32) {
    const int c = c0 + lane;
    float v = 0.0f;
    if (c < cols) v = load1<DT>(in, row * cols + c);
    const bool outlier = c < cols && fabsf(v) >= threshold;
    const bool stored = outlier && v != 0.0f;
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, stored);
    if (stored) {
      const int at = pos + __popc(ballot & ((1u << lane) - 1u));
      if (at < capacity) {
        store1<DT>(data, b * capacity + at, v);
        indices[b * capacity + at] = c;
      }
    }
    if (c < cols) store1<DT>(inlier, row * cols + c, outlier ? 0.0f : v);
    pos += __popc(ballot);
  }
}

// out[b][r][n] = sum over the row's entries of data * B[col][n], float32 accumulation in entry order.
// B element (k, n) of batch b is at B[b * strideB + k * ld_k + n * ld_n].
template <int DT, int BT, int OT>
__global__ void __launch_bounds__(256)
spmm_csr_kernel(const void* __restrict__ data, const int32_t* __restrict__ indices, const int32_t* __restrict__ indptr,
                const void* __restrict__ B, void* __restrict__ out, int rows, int N, int K, int capacity,
                int64_t strideB, int64_t ld_k, int64_t ld_n) {
  const int r = blockIdx.x;
  const int64_t b = blockIdx.z;
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  const int32_t* ptr = indptr + b * (rows + 1);
  // the pointers may continue a longer array: rebase on the first and keep them inside the stored span
  const int base = ptr[0];
  int s = min(max(ptr[r] - base, 0), capacity);
  int e = min(max(ptr[r + 1] - base, 0), capacity);
  if (e < s) e = s;
  if (n >= N) return;
  float acc = 0.0f;
  for (int i = s; i < e; ++i) {
    const int col = min(max(indices[b * capacity + i], 0), K - 1);
    const float a = load1<DT>(data, b * capacity + i);
    acc = __fadd_rn(acc, __fmul_rn(a, load1<BT>(B, b * strideB + (int64_t)col * ld_k + (int64_t)n * ld_n)));
  }
  store1<OT>(out, (b * rows + r) * (int64_t)N + n, acc);
}

#define VQ_DT_SWITCH(dtype, NAME, ...)                                \
  switch (dtype) {                                                    \
    case VQ_BF16: { constexpr int NAME = VQ_BF16; __VA_ARGS__; break; } \
    case VQ_F16:  { constexpr int NAME = VQ_F16;  __VA_ARGS__; break; } \
    case VQ_F32:  { constexpr int NAME = VQ_F32;  __VA_ARGS__; break; } \
    default: return fail(VQ_EINVAL, "unknown dtype %d", dtype);       \
  }

}  // namespace
}  // namespace vq

using namespace vq;

extern "C" int vq_outlier_count(const void* in, int dtype, int32_t* counts, int64_t rows_total, int64_t cols,
                                float threshold, void* stream) {
  VQ_REQUIRE(rows_total >= 0 && cols >= 0 && cols < (1ll << 31), "vq_outlier_count: bad extent");
  if (rows_total == 0) return VQ_OK;
  VQ_REQUIRE(in && counts, "vq_outlier_count: null argument");
  const unsigned grid = (unsigned)((rows_total + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VQ_DT_SWITCH(dtype, DT, (outlier_count_kernel<DT><<<grid, 256, 0, st>>>(in, counts, rows_total, (int)cols, threshold)));
  return check_launch("outlier_count_kernel");
}

extern "C" int vq_outlier_fill(const void* in, int dtype, void* inlier, void* data, int32_t* indices,
                               const int32_t* row_start, int64_t batches, int64_t rows, int64_t cols, float threshold,
                               int64_t capacity, void* stream) {
  VQ_REQUIRE(batches >= 0 && rows >= 0 && cols >= 0 && cols < (1ll << 31) && rows < (1ll << 31) &&
             capacity >= 0 && capacity < (1ll << 31), "vq_outlier_fill: bad extent");
  if (batches * rows == 0) return VQ_OK;
  VQ_REQUIRE(in && inlier && row_start && (capacity == 0 || (data && indices)), "vq_outlier_fill: null argument");
  const int64_t rows_total = batches * rows;
  const unsigned grid = (unsigned)((rows_total + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VQ_DT_SWITCH(dtype, DT, (outlier_fill_kernel<DT><<<grid, 256, 0, st>>>(in, inlier, data, indices, row_start, rows_total,
                                                                       (int)rows, (int)cols, threshold, (int)capacity)));
  return check_launch("outlier_fill_kernel");
}

extern "C" int vq_spmm_csr(const void* data, int data_dtype, const int32_t* indices, const int32_t* indptr,
                           const void* B, int b_dtype, void* out, int out_dtype, int64_t batches, int64_t rows,
                           int64_t N, int64_t K, int64_t capacity, int64_t strideB, int64_t ld_k, int64_t ld_n,
                           void* stream) {
  VQ_REQUIRE(batches >= 0 && rows >= 0 && N >= 0 && K > 0 && capacity >= 0, "vq_spmm_csr: bad extent");
  if (batches * rows * N == 0) return VQ_OK;
  VQ_REQUIRE(indptr && B && out && (capacity == 0 || (data && indices)), "vq_spmm_csr: null argument");
  VQ_REQUIRE(rows < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && capacity < (1ll << 31) && batches < 65536,
             "vq_spmm_csr: extent too large");
  dim3 grid((unsigned)rows, (unsigned)((N + 255) / 256), (unsigned)batches);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  VQ_DT_SWITCH(data_dtype, DT, VQ_DT_SWITCH(b_dtype, BT, VQ_DT_SWITCH(out_dtype, OT,
      (spmm_csr_kernel<DT, BT, OT><<<grid, 256, 0, st>>>(data, indices, indptr, B, out, (int)rows, (int)N, (int)K,
                                                         (int)capacity, strideB, ld_k, ld_n)))));
  return check_launch("spmm_csr_kernel");
}
