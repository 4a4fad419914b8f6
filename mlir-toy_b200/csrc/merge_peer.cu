// Single-sequence decode sharded along the KV length: the merge of the per-rank partials as ONE kernel over
// peer-mapped memory, without a library collective.
//
// Every rank owns one symmetric buffer (nb200_decode_merge_peer_workspace_bytes), mapped into every other
// rank's address space (CUDA IPC; the host side exchanges the handles).  It holds two gather areas
// [world][rows][D + 2] floats, used alternately by consecutive calls, and per area one arrival flag per rank.
// A call with generation g (the same number on every rank, growing by one per call, never 0) does, in one launch
// of `world` CTAs:
//   CTA p     copies this rank's partial into slot `rank` of rank p's gather area (plain 16-byte stores to the
//             peer's memory over NVLink), fences, and releases flag[rank] = g there;
//   all CTAs  wait until the `world` flags of their OWN area read g (acquire loads of local memory, bounded by
//             wait_ns; on expiry the status words say which rank never arrived and the kernel returns without
//             writing the output), then run the log-sum-exp combine over the gathered slots for their rows.
// Nothing here uses multicast: stores go to one peer at a time and every load is of local memory.  Area g & 1
// is free for call g because rank r can only be in call g once it has finished its own combine of call g - 1,
// and nobody can release a flag of call g + 1 in that area before having passed call g.
//
// The waits are on flags written by OTHER GPUs, whose kernels run at the same time on their own devices; the
// CTAs of one launch never wait for one another, so there is no co-residency requirement.
#include <cstring>

#include "nb200_common.cuh"
#include "peer_merge.cuh"

namespace nb200 {
namespace {

using namespace peer;
constexpr int kPeerThreads = 256;

template <int ODT>
__global__ void __launch_bounds__(kPeerThreads)
decode_merge_peer_kernel(const float *__restrict__ local_partial, Ptrs peers, void *__restrict__ out, int rows,
                         int world, int rank, unsigned generation, long long wait_ns, int *status) {
  __shared__ int timed_out;
  const int p = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) timed_out = 0;
  // ---- push this rank's partial to rank p
  push(local_partial, peers, rows, world, rank, generation, p, p + 1, tid, kPeerThreads);
  __threadfence_system();
  __syncthreads();
  if (tid == 0) release_flag(peers, rows, world, rank, generation, p);
  // ---- wait for every rank's partial to have landed here
  if (tid < world && !wait_arrival(peers, rows, world, rank, generation, tid, wait_ns, status)) timed_out = 1;
  __syncthreads();
  if (timed_out) return;
  // ---- combine: one warp per output row
  const float *gathered = peers.buf[rank] + (generation & 1u) * area_floats(rows, world);
  for (int row = p * (kPeerThreads / 32) + (tid >> 5); row < rows; row += world * (kPeerThreads / 32))
    combine_row<ODT>(gathered, (size_t)rows * (kD + 2), world, row, out, tid & 31);
}

}  // namespace
}  // namespace nb200

using namespace nb200;
using namespace nb200::peer;

extern "C" size_t nb200_decode_merge_peer_workspace_bytes(int rows, int D, int world) {
  if (rows <= 0 || D != kD || world <= 0 || world > kMaxWorld) return 0;
  return buffer_floats(rows, world) * sizeof(float);
}

extern "C" int nb200_decode_merge_peer(const float *local_partial, void *const *peer_buffers, void *out, int rows, int D,
                                       int world, int rank, unsigned generation, int out_dtype, long long wait_ns,
                                       int *status, void *stream) {
  NB200_REQUIRE(local_partial && peer_buffers && out, NB200_ERR_BAD_ARG, "decode_merge_peer: null pointer");
  NB200_REQUIRE(rows > 0 && world > 0 && rank >= 0 && rank < world, NB200_ERR_BAD_ARG, "decode_merge_peer: bad extent or rank");
  NB200_REQUIRE(world <= kMaxWorld, NB200_ERR_UNSUPPORTED, "decode_merge_peer: at most %d ranks", kMaxWorld);
  NB200_REQUIRE(D == kD, NB200_ERR_UNSUPPORTED, "decode_merge_peer: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(generation != 0, NB200_ERR_BAD_ARG, "decode_merge_peer: generations start at 1 (0 is the cleared flag)");
  NB200_REQUIRE(wait_ns > 0, NB200_ERR_BAD_ARG, "decode_merge_peer: the wait limit must be positive");
  NB200_REQUIRE(aligned16(local_partial) && (reinterpret_cast<uintptr_t>(out) & (out_dtype == NB200_F32 ? 3u : 7u)) == 0,
                NB200_ERR_BAD_ARG, "decode_merge_peer: local_partial must be 16-byte and out 8-byte aligned");
  Ptrs peers{};
  for (int r = 0; r < world; ++r) {
    NB200_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), NB200_ERR_BAD_ARG,
                  "decode_merge_peer: buffer of rank %d is null or not 16-byte aligned", r);
    peers.buf[r] = static_cast<float *>(peer_buffers[r]);
  }
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 grid(world), block(kPeerThreads);
  switch (out_dtype) {
    case NB200_BF16: decode_merge_peer_kernel<NB200_BF16><<<grid, block, 0, st>>>(local_partial, peers, out, rows, world, rank, generation, wait_ns, status); break;
    case NB200_F16: decode_merge_peer_kernel<NB200_F16><<<grid, block, 0, st>>>(local_partial, peers, out, rows, world, rank, generation, wait_ns, status); break;
    case NB200_F32: decode_merge_peer_kernel<NB200_F32><<<grid, block, 0, st>>>(local_partial, peers, out, rows, world, rank, generation, wait_ns, status); break;
    default: return fail(NB200_ERR_UNSUPPORTED, "decode_merge_peer: out_dtype %d", out_dtype);
  }
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

// ---- the symmetric buffer: allocation and CUDA IPC mapping ---------------------------------------------
// These are the only entry points of the library that allocate device memory, and they say so by name; a host
// that has its own way of mapping peer memory can pass its pointers to nb200_decode_merge_peer instead.
extern "C" int nb200_peer_buffer_alloc(size_t bytes, void **ptr, unsigned char *handle64) {
  NB200_REQUIRE(ptr && handle64 && bytes > 0, NB200_ERR_BAD_ARG, "peer_buffer_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void *p = nullptr;
  NB200_CHECK_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(NB200_ERR_LAUNCH, "peer_buffer_alloc: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return NB200_OK;
}

extern "C" int nb200_peer_buffer_open(const unsigned char *handle64, void **ptr) {
  NB200_REQUIRE(ptr && handle64, NB200_ERR_BAD_ARG, "peer_buffer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  NB200_CHECK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return NB200_OK;
}

extern "C" int nb200_peer_buffer_close(void *ptr) {
  NB200_REQUIRE(ptr, NB200_ERR_BAD_ARG, "peer_buffer_close: null pointer");
  NB200_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return NB200_OK;
}

extern "C" int nb200_peer_buffer_free(void *ptr) {
  NB200_REQUIRE(ptr, NB200_ERR_BAD_ARG, "peer_buffer_free: null pointer");
  NB200_CHECK_CUDA(cudaFree(ptr));
  return NB200_OK;
}
