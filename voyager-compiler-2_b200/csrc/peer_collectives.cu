// Token-row exchanges of a tensor-parallel layer over peer memory (NVLink), for ranks whose buffers are mapped
// into one another's address space (symmetric memory: every rank holds the same allocation and the array of all
// ranks' base pointers).  Both kernels PULL with plain loads from the peers' buffers into this GPU's memory;
// nothing here waits on another GPU -- the caller places a cross-rank barrier between the producers of the
// buffers and these kernels (and the next barrier of the sequence keeps a buffer from being rewritten while a
// peer still reads it).
//
//   gather : out[p * chunk + i] = peer[p][i]                      all-gather of every rank's rows
//   reduce : out[i] = sum over p = 0 .. world-1 of peer[p][rank * chunk + i]   reduce-scatter of float32 partial
//            sums over token rows, added in rank order (every rank gets a deterministic sum)
//   max    : out[0] = max over p of peer[p][0]                    all-reduce(max) of one non-negative scalar (an amax)
//
// They replace ncclAllGather / ncclReduceScatter in the row-parallel linears of parallel.py where the layer is
// so short that the library collectives' latency dominates the step.
#include "vq_common.cuh"

namespace vq {
namespace {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  const void* p[kMaxPeers];
};

__global__ void __launch_bounds__(256)
peer_gather_kernel(PeerPtrs peers, int world, int64_t chunk_vecs, uint4* __restrict__ out) {
  const int64_t total = (int64_t)world * chunk_vecs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int src = (int)(i / chunk_vecs);
    const int64_t off = i - (int64_t)src * chunk_vecs;
    out[i] = *(static_cast<const uint4*>(peers.p[src]) + off);   // plain load: remote data is never cached read-only
  }
}

__global__ void __launch_bounds__(256)
peer_reduce_rows_kernel(PeerPtrs peers, int world, int rank, int64_t chunk_vecs, float4* __restrict__ out) {
  const int64_t base = (int64_t)rank * chunk_vecs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunk_vecs; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v[kMaxPeers];
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < world) v[p] = *(static_cast<const float4*>(peers.p[p]) + base + i);   // all loads in flight, then the sum
    float4 s = v[0];
#pragma unroll
    for (int p = 1; p < kMaxPeers; ++p)
      if (p < world) { s.x += v[p].x; s.y += v[p].y; s.z += v[p].z; s.w += v[p].w; }
    out[i] = s;
  }
}

// out[0] = max over ranks of peer[p][0] (non-negative floats: an amax), one warp.
__global__ void peer_max_kernel(PeerPtrs peers, int world, float* __restrict__ out) {
  float m = 0.0f;
#pragma unroll
  for (int p = 0; p < kMaxPeers; ++p)
    if (p < world && (int)threadIdx.x == p) m = *static_cast<const volatile float*>(peers.p[p]);
  for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  if (threadIdx.x == 0) out[0] = m;
}

int check_peers(const void* const* peer_ptrs, int64_t world, PeerPtrs* out, const char* what) {
  if (world < 1 || world > kMaxPeers) return fail(VQ_EINVAL, "%s: 1 to %d ranks", what, kMaxPeers);
  if (!peer_ptrs) return fail(VQ_EINVAL, "%s: no peer pointers", what);
  for (int p = 0; p < (int)world; ++p) {
    if (!peer_ptrs[p] || (reinterpret_cast<uintptr_t>(peer_ptrs[p]) & 15) != 0)
      return fail(VQ_EINVAL, "%s: peer buffer %d is null or not 16-byte aligned", what, p);
    out->p[p] = peer_ptrs[p];
  }
  return VQ_OK;
}

inline int peer_grid(int64_t vecs) {
  int64_t blocks = (vecs + 255) / 256;
  const int64_t cap = (int64_t)kSmCount * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace vq

using namespace vq;

// peer_ptrs: HOST array of `world` device pointers (this rank's own buffer included, at index `rank`).
extern "C" int vq_peer_gather(const void* const* peer_ptrs, int64_t world, int64_t chunk_bytes, void* out, void* stream) {
  VQ_REQUIRE(chunk_bytes >= 0, "vq_peer_gather: negative size");
  if (chunk_bytes == 0) return VQ_OK;
  VQ_REQUIRE(out && chunk_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "vq_peer_gather: the chunk and the output must be multiples of 16 bytes / 16-byte aligned");
  PeerPtrs peers{};
  if (int e = check_peers(peer_ptrs, world, &peers, "vq_peer_gather")) return e;
  peer_gather_kernel<<<peer_grid(world * (chunk_bytes / 16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      peers, (int)world, chunk_bytes / 16, static_cast<uint4*>(out));
  return check_launch("peer_gather_kernel");
}

extern "C" int vq_peer_reduce_rows(const void* const* peer_ptrs, int64_t world, int64_t rank, int64_t chunk_floats,
                                   void* out, void* stream) {
  VQ_REQUIRE(chunk_floats >= 0, "vq_peer_reduce_rows: negative size");
  if (chunk_floats == 0) return VQ_OK;
  VQ_REQUIRE(out && chunk_floats % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "vq_peer_reduce_rows: the chunk must be a multiple of 4 floats and the output 16-byte aligned");
  VQ_REQUIRE(rank >= 0 && rank < world, "vq_peer_reduce_rows: rank out of range");
  PeerPtrs peers{};
  if (int e = check_peers(peer_ptrs, world, &peers, "vq_peer_reduce_rows")) return e;
  peer_reduce_rows_kernel<<<peer_grid(chunk_floats / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      peers, (int)world, (int)rank, chunk_floats / 4, static_cast<float4*>(out));
  return check_launch("peer_reduce_rows_kernel");
}

extern "C" int vq_peer_max(const void* const* peer_ptrs, int64_t world, void* out, void* stream) {
  VQ_REQUIRE(out != nullptr, "vq_peer_max: null output");
  PeerPtrs peers{};
  if (int e = check_peers(peer_ptrs, world, &peers, "vq_peer_max")) return e;
  peer_max_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(peers, (int)world, static_cast<float*>(out));
  return check_launch("peer_max_kernel");
}
