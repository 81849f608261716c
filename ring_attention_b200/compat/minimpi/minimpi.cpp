// minimpi implementation: see mpi.h. All ranks map one file under /dev/shm holding a
// sense-reversing barrier and a staging area with one slot per rank; every collective is
// "write my slot, barrier, read, barrier". Sizes here are tiny (timings, a 128-byte NCCL id),
// so simplicity wins over speed. Waits are bounded: a rank that never arrives (it died) makes
// the others abort after MINIMPI_TIMEOUT_S seconds (default 600) instead of hanging.
#include "mpi.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

constexpr int kMaxRanks = 64;
constexpr size_t kSlotBytes = 64 * 1024;

struct Shared {
  std::atomic<int> arrived;
  std::atomic<int> generation;
  std::atomic<int> aborted;
  int pad[13];
  unsigned char slot[kMaxRanks][kSlotBytes];
};

int g_rank = 0, g_size = 1;
Shared* g_shm = nullptr;
double g_timeout_s = 600.0;

double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

size_t type_size(MPI_Datatype t) {
  switch (t) {
    case MPI_BYTE:
    case MPI_CHAR:
      return 1;
    case MPI_INT:
    case MPI_UNSIGNED:
    case MPI_FLOAT:
      return 4;
    default:
      return 8;
  }
}

[[noreturn]] void fail(const char* what) {
  std::fprintf(stderr, "minimpi rank %d: %s\n", g_rank, what);
  if (g_shm) g_shm->aborted.store(1);
  std::_Exit(1);
}

void barrier() {
  if (g_size == 1) return;
  const int gen = g_shm->generation.load();
  if (g_shm->arrived.fetch_add(1) + 1 == g_size) {
    g_shm->arrived.store(0);
    g_shm->generation.fetch_add(1);
    return;
  }
  const double t0 = now_s();
  unsigned spins = 0;
  while (g_shm->generation.load() == gen) {
    if (g_shm->aborted.load()) std::_Exit(1);
    if ((++spins & 1023u) == 0) {
      if (now_s() - t0 > g_timeout_s) fail("barrier timed out (a rank is missing)");
      usleep(50);
    }
  }
}

template <typename T>
void combine(T* acc, const T* x, int n, MPI_Op op) {
  for (int i = 0; i < n; ++i) {
    if (op == MPI_MAX) acc[i] = x[i] > acc[i] ? x[i] : acc[i];
    else if (op == MPI_MIN) acc[i] = x[i] < acc[i] ? x[i] : acc[i];
    else acc[i] = acc[i] + x[i];
  }
}

int reduce_impl(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, int root,
                bool all) {
  const size_t bytes = count * type_size(type);
  if (bytes > kSlotBytes) fail("reduce payload larger than a slot");
  const void* src = (send == MPI_IN_PLACE) ? recv : send;
  if (g_size == 1) {
    if (recv != src) std::memcpy(recv, src, bytes);
    return MPI_SUCCESS;
  }
  std::memcpy(g_shm->slot[g_rank], src, bytes);
  barrier();
  if (all || g_rank == root) {
    unsigned char tmp[kSlotBytes];
    std::memcpy(tmp, g_shm->slot[0], bytes);
    for (int r = 1; r < g_size; ++r) {
      if (type == MPI_FLOAT) combine(reinterpret_cast<float*>(tmp), reinterpret_cast<const float*>(g_shm->slot[r]), count, op);
      else if (type == MPI_DOUBLE) combine(reinterpret_cast<double*>(tmp), reinterpret_cast<const double*>(g_shm->slot[r]), count, op);
      else if (type == MPI_INT) combine(reinterpret_cast<int*>(tmp), reinterpret_cast<const int*>(g_shm->slot[r]), count, op);
      else if (type == MPI_LONG || type == MPI_LONG_LONG) combine(reinterpret_cast<long long*>(tmp), reinterpret_cast<const long long*>(g_shm->slot[r]), count, op);
      else fail("reduce: unsupported datatype");
    }
    std::memcpy(recv, tmp, bytes);
  }
  barrier();
  return MPI_SUCCESS;
}

}  // namespace

extern "C" {

int MPI_Init(int*, char***) {
  const char* r = std::getenv("MINIMPI_RANK");
  const char* n = std::getenv("MINIMPI_SIZE");
  const char* f = std::getenv("MINIMPI_SHM");
  if (const char* t = std::getenv("MINIMPI_TIMEOUT_S")) g_timeout_s = std::atof(t);
  if (!r || !n || !f || std::atoi(n) <= 1) return MPI_SUCCESS;  // singleton
  g_rank = std::atoi(r);
  g_size = std::atoi(n);
  if (g_size > kMaxRanks || g_rank < 0 || g_rank >= g_size) fail("bad MINIMPI_RANK / MINIMPI_SIZE");
  const int fd = open(f, O_RDWR);
  if (fd < 0) fail("cannot open MINIMPI_SHM");
  void* p = mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) fail("mmap of MINIMPI_SHM failed");
  g_shm = static_cast<Shared*>(p);
  barrier();
  return MPI_SUCCESS;
}

int MPI_Finalize(void) {
  barrier();
  return MPI_SUCCESS;
}
int MPI_Comm_rank(MPI_Comm, int* rank) {
  *rank = g_rank;
  return MPI_SUCCESS;
}
int MPI_Comm_size(MPI_Comm, int* size) {
  *size = g_size;
  return MPI_SUCCESS;
}
int MPI_Comm_split_type(MPI_Comm, int, int, MPI_Info, MPI_Comm* out) {
  *out = MPI_COMM_WORLD;  // one node: the shared-memory domain is the world
  return MPI_SUCCESS;
}
int MPI_Comm_split(MPI_Comm, int color, int, MPI_Comm* out) {
  // only the trivial split (every rank the same colour) is supported
  int lo = color, hi = color;
  reduce_impl(&color, &lo, 1, MPI_INT, MPI_MIN, 0, true);
  reduce_impl(&color, &hi, 1, MPI_INT, MPI_MAX, 0, true);
  if (lo != hi) fail("MPI_Comm_split with different colours is not supported by minimpi");
  *out = MPI_COMM_WORLD;
  return MPI_SUCCESS;
}
int MPI_Comm_free(MPI_Comm* comm) {
  *comm = MPI_COMM_NULL;
  return MPI_SUCCESS;
}
int MPI_Barrier(MPI_Comm) {
  barrier();
  return MPI_SUCCESS;
}
int MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm) {
  if (g_size == 1) return MPI_SUCCESS;
  size_t left = count * type_size(type);
  unsigned char* p = static_cast<unsigned char*>(buf);
  while (left > 0) {
    const size_t n = left < kSlotBytes ? left : kSlotBytes;
    if (g_rank == root) std::memcpy(g_shm->slot[root], p, n);
    barrier();
    if (g_rank != root) std::memcpy(p, g_shm->slot[root], n);
    barrier();
    p += n;
    left -= n;
  }
  return MPI_SUCCESS;
}
int MPI_Reduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, int root,
               MPI_Comm) {
  return reduce_impl(send, recv, count, type, op, root, false);
}
int MPI_Allreduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, MPI_Comm) {
  return reduce_impl(send, recv, count, type, op, 0, true);
}
int MPI_Allgather(const void* send, int scount, MPI_Datatype stype, void* recv, int, MPI_Datatype,
                  MPI_Comm) {
  const size_t bytes = scount * type_size(stype);
  if (bytes > kSlotBytes) fail("allgather payload larger than a slot");
  if (g_size == 1) {
    if (send != MPI_IN_PLACE) std::memcpy(recv, send, bytes);
    return MPI_SUCCESS;
  }
  const void* src = (send == MPI_IN_PLACE) ? static_cast<unsigned char*>(recv) + g_rank * bytes : send;
  std::memcpy(g_shm->slot[g_rank], src, bytes);
  barrier();
  for (int r = 0; r < g_size; ++r)
    std::memcpy(static_cast<unsigned char*>(recv) + r * bytes, g_shm->slot[r], bytes);
  barrier();
  return MPI_SUCCESS;
}
double MPI_Wtime(void) { return now_s(); }
int MPI_Abort(MPI_Comm, int code) {
  if (g_shm) g_shm->aborted.store(1);
  std::_Exit(code ? code : 1);
}
int MPI_Error_string(int code, char* str, int* len) {
  *len = std::snprintf(str, MPI_MAX_ERROR_STRING, "minimpi error %d", code);
  return MPI_SUCCESS;
}
}
