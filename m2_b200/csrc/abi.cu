// Library-level entry points: version, error message, device status word.
#include "common.cuh"
#include <string.h>

static thread_local char g_err[512] = "";

int m2_set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

extern "C" int m2_version(void) { return M2_B200_ABI_VERSION; }

extern "C" const char* m2_last_error(void) { return g_err; }

extern "C" int m2_device_status(int* status_out) {
  M2_REQUIRE(status_out != nullptr, M2_ERR_ARG, "m2_device_status: status_out is NULL");
  int v = 0, zero = 0;
  M2_CUDA(cudaDeviceSynchronize());
  M2_CUDA(cudaMemcpyFromSymbol(&v, m2_dev_status_word, sizeof(int)));
  M2_CUDA(cudaMemcpyToSymbol(m2_dev_status_word, &zero, sizeof(int)));
  *status_out = v;
  return M2_OK;
}
