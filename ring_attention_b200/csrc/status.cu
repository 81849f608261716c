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

// Pinned host mirror of the status word, one per device, for entry points that already end
// with a stream synchronisation: they enqueue a 16-byte copy in front of that synchronisation
// and look at the mirror afterwards, so the check costs no extra round trip.
int* status_mirror() {
  static int* mirror[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!mirror[dev]) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 4 * sizeof(int), cudaHostAllocDefault) != cudaSuccess) return nullptr;
    std::memset(p, 0, 4 * sizeof(int));
    mirror[dev] = static_cast<int*>(p);
  }
  return mirror[dev];
}

int enqueue_status_read(cudaStream_t stream) {
  int* d = device_status_ptr();
  int* h = status_mirror();
  RAB_REQUIRE(d && h, RA_ERR_CUDA, "device status word unavailable");
  RAB_CUDA(cudaMemcpyAsync(h, d, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream));
  return RA_OK;
}

int status_after_sync() {
  const int* h = status_mirror();
  if (h && h[0] != 0) {
    set_error("a bounded device-side wait ran out (code %d, wait %d, block %d, tile %d): the "
              "results of this call are invalid; ra_device_status() reads and clears the word",
              h[0], h[1], h[2], h[3]);
    return RA_ERR_DEVICE_WAIT;
  }
  return RA_OK;
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
