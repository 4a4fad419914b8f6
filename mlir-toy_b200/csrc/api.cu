// Library-wide pieces of the C ABI: version, thread-local error text, status-word read-back.
#include "nb200_common.cuh"

#include <cstring>

namespace nb200 {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace nb200

extern "C" int nb200_version(void) { return 100; }  // 0.1.0

extern "C" const char *nb200_last_error(void) { return nb200::g_error; }

extern "C" int nb200_status_read(const int *status, int *host_out, void *stream) {
  NB200_REQUIRE(status, NB200_ERR_BAD_ARG, "status_read: null status buffer");
  int host[NB200_STATUS_WORDS] = {0, 0, 0, 0};
  auto st = static_cast<cudaStream_t>(stream);
  NB200_CHECK_CUDA(cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, st));
  NB200_CHECK_CUDA(cudaStreamSynchronize(st));
  if (host_out) std::memcpy(host_out, host, sizeof(host));
  if (host[0] == 22)  // the paged decode met a block-table entry outside the pool and did not dereference it
    return nb200::fail(NB200_ERR_BAD_ARG, "paged decode: block table entry %d is outside the page pool (block %d, thread %d)",
                       host[2], host[1], host[3]);
  if (host[0] != 0)
    return nb200::fail(NB200_ERR_DEVICE_TIMEOUT,
                       "device-side wait expired: code %d, block %d, detail %d/%d", host[0], host[1],
                       host[2], host[3]);
  return NB200_OK;
}
