// Thread-local error text, the library version and the per-device status word that
// bounded device-side waits report into.
#include "common.cuh"

namespace rab {

namespace {
thread_local char g_err[512] = "";
// {code, which wait, block, tile}; zero = healthy. Every GPU that loads the library
// holds these 16 bytes.
__device__ int g_device_status[4];
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

const char* last_error() { return g_err; }

int* device_status_ptr() {
  // cudaGetSymbolAddress resolves the symbol for the CURRENT device; cache per device.
  static int* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

int read_device_status(int out[4], bool clear) {
  int* p = device_status_ptr();
  RAB_REQUIRE(p != nullptr, RA_ERR_CUDA, "device status word unavailable");
  RAB_CUDA(cudaDeviceSynchronize());
  RAB_CUDA(cudaMemcpy(out, p, 4 * sizeof(int), cudaMemcpyDeviceToHost));
  if (clear && out[0] != 0) RAB_CUDA(cudaMemset(p, 0, 4 * sizeof(int)));
  return RA_OK;
}

}  // namespace rab

extern "C" {
const char* ra_last_error(void) { return rab::last_error(); }
int ra_version(void) { return 100; }
int ra_device_status(int out[4]) {
  RAB_REQUIRE(out != nullptr, RA_ERR_INVALID, "ra_device_status: null argument");
  return rab::read_device_status(out, true);
}
}
