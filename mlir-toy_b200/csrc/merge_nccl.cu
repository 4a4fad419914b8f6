// Single-sequence decode sharded along the KV length over the GPUs of one node: the one exchange
// step of the whole operator set.  Every rank has reduced its slice of the cache to one partial
// (o[D], m, l) per query head; this entry point all-gathers those partials with NCCL and merges
// them with the same log-sum-exp combine kernel that merges the splits of one GPU, the rank index
// playing the role of the split index.  The message is tiny (rows * (D + 2) * 4 bytes per rank,
// 16 640 B for 32 heads of 128), so the cost is two launch latencies, not bandwidth; the all-gather
// lands in this GPU's own memory before any kernel of this library reads it.
//
// NCCL is not linked: the communicator handed in belongs to whatever NCCL build the host process
// uses, so the two functions needed are resolved at first use from the NCCL library that is already
// loaded in the process (or from $NEPTUNE_B200_NCCL, or libnccl.so.2 on the loader path).
#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

#include "nb200_common.cuh"

namespace nb200 {
namespace {

// ncclResult_t (*)(const void* send, void* recv, size_t sendcount, ncclDataType_t, ncclComm_t, cudaStream_t)
using AllGatherFn = int (*)(const void *, void *, size_t, int, void *, cudaStream_t);
using ErrorStringFn = const char *(*)(int);
using CommCountFn = int (*)(void *, int *);
constexpr int kNcclFloat32 = 7;  // ncclFloat32 in nccl.h's ncclDataType_t

struct NcclApi {
  AllGatherFn all_gather = nullptr;
  ErrorStringFn error_string = nullptr;
  CommCountFn comm_count = nullptr;
  char why[256] = "";
};

NcclApi &nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host process already uses
    if (!h) {
      if (const char *env = std::getenv("NEPTUNE_B200_NCCL")) h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      snprintf(api.why, sizeof(api.why), "no NCCL library could be loaded (%s)", dlerror());
      return;
    }
    api.all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
    api.error_string = reinterpret_cast<ErrorStringFn>(dlsym(h, "ncclGetErrorString"));
    api.comm_count = reinterpret_cast<CommCountFn>(dlsym(h, "ncclCommCount"));
    if (!api.all_gather || !api.comm_count)
      snprintf(api.why, sizeof(api.why), "the loaded NCCL library lacks ncclAllGather / ncclCommCount");
  });
  return api;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_decode_merge_workspace_bytes(int rows, int D, int world) {
  if (rows <= 0 || D <= 0 || world <= 0) return 0;
  return (size_t)world * rows * (D + 2) * sizeof(float);
}

extern "C" int nb200_decode_merge_nccl(const float *local_partial, float *gathered, void *out, int rows,
                                       int D, int world, int out_dtype, void *nccl_comm, void *stream) {
  NB200_REQUIRE(local_partial && gathered && out, NB200_ERR_BAD_ARG, "decode_merge_nccl: null pointer");
  NB200_REQUIRE(nccl_comm, NB200_ERR_BAD_ARG, "decode_merge_nccl: null communicator");
  NB200_REQUIRE(rows > 0 && world > 0, NB200_ERR_BAD_ARG, "decode_merge_nccl: non-positive extent");
  NB200_REQUIRE(D == 128, NB200_ERR_UNSUPPORTED, "decode_merge_nccl: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(aligned16(local_partial) && aligned16(gathered), NB200_ERR_BAD_ARG,
                "decode_merge_nccl: buffers must be 16-byte aligned");
  NcclApi &api = nccl_api();
  if (!api.all_gather || !api.comm_count) return fail(NB200_ERR_NCCL, "decode_merge_nccl: %s", api.why);
  int count = 0;
  int rc = api.comm_count(nccl_comm, &count);
  if (rc != 0)
    return fail(NB200_ERR_NCCL, "decode_merge_nccl: ncclCommCount failed: %s",
                api.error_string ? api.error_string(rc) : "?");
  NB200_REQUIRE(count == world, NB200_ERR_BAD_ARG,
                "decode_merge_nccl: the communicator has %d ranks, the call says %d", count, world);
  const size_t per_rank = (size_t)rows * (D + 2);
  rc = api.all_gather(local_partial, gathered, per_rank, kNcclFloat32, nccl_comm, static_cast<cudaStream_t>(stream));
  if (rc != 0)
    return fail(NB200_ERR_NCCL, "decode_merge_nccl: ncclAllGather failed: %s",
                api.error_string ? api.error_string(rc) : "?");
  // gathered is [world, rows, D + 2]: row stride D + 2, "split" (= rank) stride rows * (D + 2)
  return nb200_decode_combine(gathered, out, rows, D, world, D + 2, (long long)per_rank, out_dtype, stream);
}
