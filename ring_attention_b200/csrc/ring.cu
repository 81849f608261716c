// Multi-GPU drivers: the overlapped ring prefill pass and the all-gather decode step, one
// rank per GPU over NCCL (NVLink 5 / NVSwitch inside one box).
//
// Prefill replaces run_ring_overlap_fp16 (src/ring_loop_fp16.cu:522-818) with three changes
// that matter on this hardware: the communicator lives as long as the ring handle instead of
// being rebuilt per run (src/ring_loop_fp16.cu:587), a ring step is ONE kernel launch over
// the whole shard (segment maps) instead of n_seg^2 launches (src/ring_loop_fp16.cu:642-655),
// and init / finalize are folded into the first / last step's epilogue. The rotation itself
// is the reference's: ncclSend to rank+1 and ncclRecv from rank-1 in one group on a side
// stream, double-buffered in local HBM, with an event fence so a buffer is not overwritten
// while the previous step still reads it (src/ring_loop_fp16.cu:658-701).
//
// Small shards take a second schedule (see use_gather below): one all-gather instead of P-1
// latency-bound hops.
//
// Decode replaces run_ring_decode_step (src/ring_decode.cu:85-226): the local partial is
// computed straight into the all-gather send buffer (no pack copies), one ncclAllGather of
// B*H*(D+2) floats per rank, then merge + normalise in one kernel.
//
// NCCL is loaded with dlopen at ring creation, so the rest of the library works without it.
#include <dlfcn.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace rab {
namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclId {
  char internal[128];
};
enum { kNcclInt8 = 0, kNcclFloat = 7 };

struct Nccl {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

Nccl g_nccl;
std::once_flag g_nccl_once;

bool load_nccl() {
  std::call_once(g_nccl_once, []() {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) return;
    void* h = g_nccl.handle;
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    g_nccl.CommInitRank =
        reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    g_nccl.Send = reinterpret_cast<decltype(g_nccl.Send)>(dlsym(h, "ncclSend"));
    g_nccl.Recv = reinterpret_cast<decltype(g_nccl.Recv)>(dlsym(h, "ncclRecv"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(h, "ncclAllGather"));
    g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(dlsym(h, "ncclGroupStart"));
    g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
    g_nccl.GetErrorString =
        reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  });
  return g_nccl.handle && g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy &&
         g_nccl.Send && g_nccl.Recv && g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd;
}

#define RAB_NCCL(expr)                                                                      \
  do {                                                                                      \
    int _r = (expr);                                                                        \
    if (_r != 0) {                                                                          \
      ::rab::set_error("NCCL error %d (%s) at %s:%d in %s", _r,                             \
                       g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "?", __FILE__,   \
                       __LINE__, #expr);                                                    \
      return RA_ERR_NCCL;                                                                   \
    }                                                                                       \
  } while (0)

constexpr int kMaxRanks = 16;  // one NVSwitch box

// NVTX range around one ring / decode step (visible in Nsight timelines; a no-op without a tool).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

// NCCL calls between GroupStart and GroupEnd: remember the first failure but always close the
// group, so that a failed call cannot leave the thread's NCCL group open (every later NCCL call
// of the thread, the caller's own included, would silently queue into it).
struct NcclGroup {
  int first = 0;
  const char* what = "";
  NcclGroup() { note(g_nccl.GroupStart(), "ncclGroupStart"); }
  void note(int r, const char* w) {
    if (r != 0 && first == 0) {
      first = r;
      what = w;
    }
  }
  int end() {
    note(g_nccl.GroupEnd(), "ncclGroupEnd");
    if (first != 0) {
      ::rab::set_error("NCCL error %d (%s) in %s", first,
                       g_nccl.GetErrorString ? g_nccl.GetErrorString(first) : "?", what);
      return RA_ERR_NCCL;
    }
    return RA_OK;
  }
};
constexpr int kAuxStreams = 3;
constexpr int kMaxKeyParts = 7;  // + the own-shard state = the 8 states one merge takes

}  // namespace
}  // namespace rab

using namespace rab;

constexpr int kHostGroupsMax = 2;  // head groups of the pipelined host pass

struct ra_ring {
  int rank, cp;
  ncclComm_t comm;
  bool own_comm;
  cudaStream_t comm_stream;
  cudaStream_t aux_stream[kAuxStreams];  // key-split launches of the gather schedule
  cudaEvent_t ev_aux[kAuxStreams];
  int sm_count;
  cudaEvent_t ev_start, ev_end;
  cudaEvent_t ev_comm[kMaxRanks], ev_comm_begin[kMaxRanks];
  cudaEvent_t ev_comp[kMaxRanks], ev_comp_begin[kMaxRanks];
  // decode buffers, grown on demand: send [O|m|l] block and cp * block receive area
  float* dec_buf;
  size_t dec_bytes;
  // host-buffer pass (ra_ring_prefill_host): device staging, grown on demand
  void* host_buf;
  size_t host_bytes;
  cudaStream_t host_stream, host_q_stream, host_out_stream;
  cudaEvent_t ev_host_q, ev_host_begin, ev_host_end;
  cudaEvent_t ev_host_up[kHostGroupsMax], ev_host_done[kHostGroupsMax], ev_host_pass;  // head-group pipeline of the host pass
};

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

static int ring_finish_create(int rank, int cp, ncclComm_t comm, bool own, ra_ring** out) {
  ra_ring* r = new ra_ring();
  r->rank = rank;
  r->cp = cp;
  r->comm = comm;
  r->own_comm = own;
  r->dec_buf = nullptr;
  r->dec_bytes = 0;
  r->host_buf = nullptr;
  r->host_bytes = 0;
  RAB_CUDA(cudaStreamCreateWithFlags(&r->host_stream, cudaStreamNonBlocking));
  RAB_CUDA(cudaStreamCreateWithFlags(&r->host_q_stream, cudaStreamNonBlocking));
  RAB_CUDA(cudaEventCreateWithFlags(&r->ev_host_q, cudaEventDisableTiming));
  RAB_CUDA(cudaEventCreate(&r->ev_host_begin));
  RAB_CUDA(cudaEventCreate(&r->ev_host_end));
  RAB_CUDA(cudaStreamCreateWithFlags(&r->host_out_stream, cudaStreamNonBlocking));
  RAB_CUDA(cudaEventCreate(&r->ev_host_pass));
  for (int i = 0; i < kHostGroupsMax; ++i) {
    RAB_CUDA(cudaEventCreateWithFlags(&r->ev_host_up[i], cudaEventDisableTiming));
    RAB_CUDA(cudaEventCreateWithFlags(&r->ev_host_done[i], cudaEventDisableTiming));
  }
  // The transfer stream gets the highest priority: the step kernel keeps every SM full (one
  // block per SM, all registers), so the few blocks of a send/recv kernel can only run on SMs
  // the block scheduler hands them first. Without the priority they queue behind the step
  // kernel's blocks and the "overlapped" transfer runs after the compute it should hide under.
  int prio_lo = 0, prio_hi = 0;
  RAB_CUDA(cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi));
  RAB_CUDA(cudaStreamCreateWithPriority(&r->comm_stream, cudaStreamNonBlocking, prio_hi));
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  RAB_CUDA(cudaDeviceGetAttribute(&r->sm_count, cudaDevAttrMultiProcessorCount, dev));
  for (int i = 0; i < kAuxStreams; ++i) {
    RAB_CUDA(cudaStreamCreateWithFlags(&r->aux_stream[i], cudaStreamNonBlocking));
    RAB_CUDA(cudaEventCreateWithFlags(&r->ev_aux[i], cudaEventDisableTiming));
  }
  RAB_CUDA(cudaEventCreate(&r->ev_start));
  RAB_CUDA(cudaEventCreate(&r->ev_end));
  for (int i = 0; i < kMaxRanks; ++i) {
    RAB_CUDA(cudaEventCreate(&r->ev_comm[i]));
    RAB_CUDA(cudaEventCreate(&r->ev_comm_begin[i]));
    RAB_CUDA(cudaEventCreate(&r->ev_comp[i]));
    RAB_CUDA(cudaEventCreate(&r->ev_comp_begin[i]));
  }
  *out = r;
  return RA_OK;
}

extern "C" {

int ra_nccl_unique_id(char id[128]) {
  RAB_REQUIRE(id != nullptr, RA_ERR_INVALID, "ra_nccl_unique_id: null argument");
  RAB_REQUIRE(load_nccl(), RA_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
  NcclId nid;
  RAB_NCCL(g_nccl.GetUniqueId(&nid));
  std::memcpy(id, nid.internal, 128);
  return RA_OK;
}

int ra_ring_create(int rank, int cp_size, const char id[128], ra_ring** out) {
  RAB_REQUIRE(out != nullptr, RA_ERR_INVALID, "ra_ring_create: null argument");
  RAB_REQUIRE(cp_size >= 1 && cp_size <= kMaxRanks && rank >= 0 && rank < cp_size, RA_ERR_INVALID,
              "ra_ring_create: bad rank %d / cp_size %d", rank, cp_size);
  ncclComm_t comm = nullptr;
  if (cp_size > 1) {
    RAB_REQUIRE(id != nullptr, RA_ERR_INVALID, "ra_ring_create: null unique id");
    RAB_REQUIRE(load_nccl(), RA_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
    NcclId nid;
    std::memcpy(nid.internal, id, 128);
    RAB_NCCL(g_nccl.CommInitRank(&comm, cp_size, nid, rank));
  }
  return ring_finish_create(rank, cp_size, comm, true, out);
}

int ra_ring_create_from_comm(int rank, int cp_size, void* nccl_comm, ra_ring** out) {
  RAB_REQUIRE(out != nullptr, RA_ERR_INVALID, "ra_ring_create_from_comm: null argument");
  RAB_REQUIRE(cp_size >= 1 && cp_size <= kMaxRanks && rank >= 0 && rank < cp_size, RA_ERR_INVALID,
              "ra_ring_create_from_comm: bad rank %d / cp_size %d", rank, cp_size);
  if (cp_size > 1) {
    RAB_REQUIRE(nccl_comm != nullptr, RA_ERR_INVALID, "ra_ring_create_from_comm: null comm");
    RAB_REQUIRE(load_nccl(), RA_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
  }
  return ring_finish_create(rank, cp_size, static_cast<ncclComm_t>(nccl_comm), false, out);
}

void ra_ring_destroy(ra_ring* r) {
  if (!r) return;
  cudaStreamSynchronize(r->comm_stream);
  if (r->comm && r->own_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(r->comm);
  cudaStreamDestroy(r->comm_stream);
  for (int i = 0; i < kAuxStreams; ++i) {
    cudaStreamSynchronize(r->aux_stream[i]);
    cudaStreamDestroy(r->aux_stream[i]);
    cudaEventDestroy(r->ev_aux[i]);
  }
  cudaEventDestroy(r->ev_start);
  cudaEventDestroy(r->ev_end);
  for (int i = 0; i < kMaxRanks; ++i) {
    cudaEventDestroy(r->ev_comm[i]);
    cudaEventDestroy(r->ev_comm_begin[i]);
    cudaEventDestroy(r->ev_comp[i]);
    cudaEventDestroy(r->ev_comp_begin[i]);
  }
  if (r->dec_buf) cudaFree(r->dec_buf);
  cudaStreamSynchronize(r->host_stream);
  cudaStreamSynchronize(r->host_q_stream);
  cudaStreamSynchronize(r->host_out_stream);
  if (r->host_buf) cudaFree(r->host_buf);
  cudaStreamDestroy(r->host_stream);
  cudaStreamDestroy(r->host_q_stream);
  cudaStreamDestroy(r->host_out_stream);
  cudaEventDestroy(r->ev_host_pass);
  for (int i = 0; i < kHostGroupsMax; ++i) {
    cudaEventDestroy(r->ev_host_up[i]);
    cudaEventDestroy(r->ev_host_done[i]);
  }
  cudaEventDestroy(r->ev_host_q);
  cudaEventDestroy(r->ev_host_begin);
  cudaEventDestroy(r->ev_host_end);
  delete r;
}

static int check_cfg(const ra_ring* r, const ra_ring_config* c) {
  RAB_REQUIRE(r && c, RA_ERR_INVALID, "ring prefill: null argument");
  RAB_REQUIRE(c->dtype == RA_F16 || c->dtype == RA_BF16 || c->dtype == RA_F32, RA_ERR_INVALID,
              "ring prefill: unknown dtype %d", c->dtype);
  RAB_REQUIRE(c->batch > 0 && c->heads > 0 && c->seq > 0, RA_ERR_INVALID,
              "ring prefill: bad shape");
  RAB_REQUIRE(c->layout >= 0 && c->layout <= 2, RA_ERR_INVALID, "ring prefill: bad layout %d",
              c->layout);
  // the reference's validation (src/ring_loop.cu:1584-1593, src/ring_partition.cpp:43-49)
  RAB_REQUIRE(c->seq % r->cp == 0, RA_ERR_INVALID, "seq=%d must be divisible by cp_size=%d",
              c->seq, r->cp);
  if (c->layout == 1) {
    RAB_REQUIRE(c->n_splits >= 2 && c->n_splits <= RA_MAX_SEG, RA_ERR_INVALID,
                "zig-zag needs 2 <= n_splits <= %d (got %d)", RA_MAX_SEG, c->n_splits);
    RAB_REQUIRE(c->seq % (c->n_splits * r->cp) == 0, RA_ERR_INVALID,
                "seq=%d must be divisible by n_splits*cp_size=%d", c->seq, c->n_splits * r->cp);
  }
  RAB_REQUIRE(c->schedule >= RA_SCHEDULE_AUTO && c->schedule <= RA_SCHEDULE_RING2D, RA_ERR_INVALID,
              "ring prefill: unknown schedule %d", c->schedule);
  if (c->schedule == RA_SCHEDULE_RING2D)
    RAB_REQUIRE(c->ring2d_nodes >= 1 && r->cp % c->ring2d_nodes == 0, RA_ERR_INVALID,
                "ring-2d: cp_size=%d must be a multiple of ring2d_nodes=%d", r->cp, c->ring2d_nodes);
  return RA_OK;
}

// Which schedule a pass uses. The hop-by-hop ring costs P-1 dependent NCCL exchanges; with
// small shards each exchange is latency-bound (well over 100 us on NVSwitch whatever the size)
// and cannot hide under a step kernel of a few tens of microseconds. One all-gather costs a
// single such latency, so below kGatherMaxBytes per shard tensor the pass gathers every shard
// once (overlapped with the step on the rank's own shard) and runs the other P-1 steps back to
// back. Large shards keep the ring: its transfers hide completely and its workspace does not
// grow with P.
constexpr size_t kGatherMaxBytes = static_cast<size_t>(32) << 20;

static bool use_gather(const ra_ring* r, const ra_ring_config* c, size_t kv_raw) {
  if (r->cp <= 1) return false;
  if (c->schedule == RA_SCHEDULE_RING || c->schedule == RA_SCHEDULE_BLOCKING ||
      c->schedule == RA_SCHEDULE_RING2D)
    return false;
  if (c->schedule == RA_SCHEDULE_GATHER) return true;
  return kv_raw <= kGatherMaxBytes;
}

// How the gather schedule folds the other ranks' shards. Their key segments ("entries": shard
// s hops away, sub-group i) are dealt round-robin to `parts` launches that run side by side on
// their own streams, each into its own partial state, merged at the end. More than one part is
// used when one launch cannot name all entries (RA_MAX_SEG) or when the query blocks alone do
// not fill the GPU twice over: a block's loop over every gathered key is then the critical
// path of the pass, and splitting the keys shortens it.
struct GatherPlan {
  bool stacked;        // false: one plain step per shard (fp32, head_dim 256)
  int nsg;             // key segments per shard
  int entries;         // (cp - 1) * nsg
  int parts;           // launches over the entries
  int chunks;          // head groups gathered (and folded) one after the other
  size_t part_floats;  // floats of one partial state [O | m | l]
};

static GatherPlan gather_plan(const ra_ring* r, const ra_ring_config* c) {
  GatherPlan g;
  g.nsg = (c->layout == 1 && c->n_splits >= 1) ? c->n_splits : 1;  // bad configs are rejected later
  g.entries = (r->cp - 1) * g.nsg;
  const int sloc = c->seq / r->cp;
  const int seg_len = sloc / g.nsg;
  const size_t rows = static_cast<size_t>(c->batch) * c->heads * sloc;
  g.part_floats = (rows * c->head_dim + 2 * rows + 3) & ~static_cast<size_t>(3);
  g.parts = 1;
  g.stacked = step_stacked_supported(c->dtype, c->head_dim);
  if (g.stacked) {
    const int need = (g.entries + RA_MAX_SEG - 1) / RA_MAX_SEG;
    const long long blocks =
        static_cast<long long>(c->batch) * c->heads * g.nsg * ((seg_len + 255) / 256);
    // Measured on one GPU playing a rank of 8 (config 2: 128 query blocks, 14 entries): one part
    // 180-331 us depending on the rank, two parts 184-188, three 195-230, four 190-195, seven
    // 225 (more launches, each with its own prologue and partial state to merge). So: split in
    // two as soon as the query blocks alone leave SMs idle, and no further.
    long long want = blocks > 0 && blocks < 2ll * r->sm_count ? 2 : 1;
    g.parts = need > want ? need : static_cast<int>(want);
    if (g.parts > g.entries) g.parts = g.entries > 0 ? g.entries : 1;
    if (g.parts > kMaxKeyParts) g.stacked = false;
  }
  if (!g.stacked) g.parts = 1;
  // Gathering in head groups, each folded as it lands, was measured and dropped: a fold fills
  // the GPU with one wave of long-running blocks, so the next group's all-gather kernel gets no
  // SM until they retire and the "overlapped" transfer runs after the fold (4 GPUs, config 2:
  // 0.54 ms per pass against 0.52 with a single gather). The plumbing stays general (chunks).
  g.chunks = 1;
  return g;
}

size_t ra_ring_prefill_workspace_bytes(const ra_ring* r, const ra_ring_config* c) {
  if (!r || !c || r->cp <= 0) return 0;
  const int kvH = c->kv_heads > 0 ? c->kv_heads : c->heads;
  const size_t es = c->dtype == RA_F32 ? 4 : 2;
  const size_t sloc = static_cast<size_t>(c->seq / r->cp);
  const size_t kv_raw = static_cast<size_t>(c->batch) * kvH * sloc * c->head_dim * es;
  const size_t kv_bytes = align256(kv_raw);
  const size_t ml = align256(static_cast<size_t>(c->batch) * c->heads * sloc * sizeof(float));
  size_t kv = 0;
  if (r->cp > 1 && use_gather(r, c, kv_raw)) {
    kv = 2 * align256(static_cast<size_t>(r->cp) * kv_raw);
    const GatherPlan g = gather_plan(r, c);
    if (g.parts >= 2) kv += align256((g.parts + 1) * g.part_floats * sizeof(float));
  } else if (r->cp > 1) {
    // ring: two K/V pairs (double buffer); 2-D ring: two for the inner and two for the outer ring
    kv = (c->schedule == RA_SCHEDULE_RING2D ? 8 : 4) * kv_bytes;
  }
  return kv + 2 * ml + 256;
}

int ra_ring_prefill_plan(const ra_ring* r, const ra_ring_config* c, int* schedule, int* key_parts,
                         int* launches) {
  const int rc = check_cfg(r, c);
  if (rc != RA_OK) return rc;
  const int kvH = c->kv_heads > 0 ? c->kv_heads : c->heads;
  const size_t es = c->dtype == RA_F32 ? 4 : 2;
  const size_t kv_raw =
      static_cast<size_t>(c->batch) * kvH * (c->seq / r->cp) * c->head_dim * es;
  int sched = (c->schedule == RA_SCHEDULE_BLOCKING || c->schedule == RA_SCHEDULE_RING2D)
                  ? c->schedule
                  : RA_SCHEDULE_RING;
  int parts = 1, n = r->cp;
  if (use_gather(r, c, kv_raw)) {
    sched = RA_SCHEDULE_GATHER;
    const GatherPlan g = gather_plan(r, c);
    if (g.stacked) {
      parts = g.parts;
      n = 1 + g.chunks * g.parts + (g.parts >= 2 ? 1 : 0);  // own shard, the parts, the merge
    }
  }
  if (schedule) *schedule = sched;
  if (key_parts) *key_parts = parts;
  if (launches) *launches = n;
  return RA_OK;
}

}  // extern "C"

// The pass itself. `q_ready`, when set, is an event the compute stream waits for after the
// transfers of the pass have been started and before the first step (the host-buffer entry
// point uploads Q on another stream while K/V already travel).
static int ring_prefill_impl(ra_ring* r, const ra_ring_config* c, const void* q, const void* k,
                             const void* v, float* out, float* lse, void* kv_work,
                             size_t kv_work_bytes, ra_stream stream_, ra_ring_result* result,
                             cudaEvent_t q_ready) {
  int rc = check_cfg(r, c);
  if (rc != RA_OK) return rc;
  RAB_REQUIRE(q && k && v && out && kv_work, RA_ERR_INVALID, "ring prefill: null argument");
  RAB_REQUIRE(kv_work_bytes >= ra_ring_prefill_workspace_bytes(r, c), RA_ERR_OVERFLOW,
              "ring prefill: workspace too small");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int P = r->cp;
  const int kvH = c->kv_heads > 0 ? c->kv_heads : c->heads;
  const size_t es = c->dtype == RA_F32 ? 4 : 2;
  const int sloc = c->seq / P;
  const size_t kv_raw = static_cast<size_t>(c->batch) * kvH * sloc * c->head_dim * es;
  const size_t kv_bytes = align256(kv_raw);
  const size_t rows = static_cast<size_t>(c->batch) * c->heads * sloc;
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(kv_work) + 255) & ~static_cast<uintptr_t>(255));
  const bool gather = use_gather(r, c, kv_raw);
  unsigned char* buf_k[2] = {nullptr, nullptr};
  unsigned char* buf_v[2] = {nullptr, nullptr};
  unsigned char* outer_k[2] = {nullptr, nullptr};  // 2-D ring: receive buffers of the outer ring
  unsigned char* outer_v[2] = {nullptr, nullptr};
  GatherPlan plan{};
  float* part_base = nullptr;
  if (P > 1 && gather) {
    buf_k[0] = base;  // every rank's K shard, rank-major
    buf_v[0] = base + align256(static_cast<size_t>(P) * kv_raw);
    base += 2 * align256(static_cast<size_t>(P) * kv_raw);
    plan = gather_plan(r, c);
    if (plan.parts >= 2) {
      part_base = reinterpret_cast<float*>(base);
      base += align256((plan.parts + 1) * plan.part_floats * sizeof(float));
    }
  } else if (P > 1) {
    buf_k[0] = base;
    buf_v[0] = base + kv_bytes;
    buf_k[1] = base + 2 * kv_bytes;
    buf_v[1] = base + 3 * kv_bytes;
    base += 4 * kv_bytes;
    if (c->schedule == RA_SCHEDULE_RING2D) {
      for (int i = 0; i < 2; ++i) {
        outer_k[i] = base + (2 * i) * kv_bytes;
        outer_v[i] = base + (2 * i + 1) * kv_bytes;
      }
      base += 4 * kv_bytes;
    }
  }
  float* m = reinterpret_cast<float*>(base);
  float* l = reinterpret_cast<float*>(base + align256(rows * sizeof(float)));

  ra_shape shape{c->batch, c->heads, sloc, sloc, c->head_dim, kvH};
  const int next = (r->rank + 1) % P, prev = (r->rank - 1 + P) % P;

  RAB_CUDA(cudaEventRecord(r->ev_start, stream));
  RAB_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_start, 0));
  if (gather) {
    NvtxRange range("ring prefill: all-gather K/V");
    // chunk g = heads [g * kvH / chunks, ...): a contiguous slice of the rank's K and V; the
    // gathered chunk is (P, kvH / chunks, sloc, D), chunks one after the other in the buffer
    const size_t chunk_raw = kv_raw / plan.chunks;
    RAB_CUDA(cudaEventRecord(r->ev_comm_begin[0], r->comm_stream));
    for (int g = 0; g < plan.chunks; ++g) {
      NcclGroup grp;
      grp.note(g_nccl.AllGather(static_cast<const unsigned char*>(k) + g * chunk_raw,
                                buf_k[0] + static_cast<size_t>(g) * P * chunk_raw, chunk_raw, kNcclInt8,
                                r->comm, r->comm_stream),
               "ncclAllGather(K)");
      grp.note(g_nccl.AllGather(static_cast<const unsigned char*>(v) + g * chunk_raw,
                                buf_v[0] + static_cast<size_t>(g) * P * chunk_raw, chunk_raw, kNcclInt8,
                                r->comm, r->comm_stream),
               "ncclAllGather(V)");
      rc = grp.end();
      if (rc != RA_OK) {
        cudaStreamSynchronize(r->comm_stream);
        return rc;
      }
      if (plan.chunks > 1) RAB_CUDA(cudaEventRecord(r->ev_comm[1 + g], r->comm_stream));
    }
    RAB_CUDA(cudaEventRecord(r->ev_comm[0], r->comm_stream));
  }
  if (q_ready) RAB_CUDA(cudaStreamWaitEvent(stream, q_ready, 0));
  int n_launch = 0;  // timed compute intervals of this pass
  int n_comm = gather ? 1 : P - 1;  // timed transfer intervals
  if (gather) {
    const bool split = plan.parts >= 2;
    auto part_out = [&](int p) { return part_base + static_cast<size_t>(p) * plan.part_floats; };
    auto part_m = [&](int p) { return part_out(p) + rows * c->head_dim; };
    auto part_l = [&](int p) { return part_m(p) + rows; };
    // step 0 on the rank's own shard while the all-gather runs
    ra_segmap qmap, kmap;
    int stride = ra_ring_step_maps(P, r->rank, c->seq, c->layout, c->n_splits, 0, &qmap, &kmap);
    RAB_REQUIRE(stride >= 1 && kmap.n_seg == plan.nsg, RA_ERR_INVALID,
                "ring prefill: bad partition");
    const unsigned causal_flag = c->causal ? RA_STEP_CAUSAL : 0u;
    RAB_CUDA(cudaEventRecord(r->ev_comp_begin[0], stream));
    rc = ra_attention_step_ex(c->dtype, q, k, v, split ? part_out(0) : out, split ? part_m(0) : m,
                              split ? part_l(0) : l, &shape, &qmap, &kmap, stride,
                              causal_flag | RA_STEP_FRESH, c->doc_len, 0, stream);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaEventRecord(r->ev_comp[0], stream));
    if (plan.chunks == 1) RAB_CUDA(cudaStreamWaitEvent(stream, r->ev_comm[0], 0));
    RAB_CUDA(cudaEventRecord(r->ev_comp_begin[1], stream));
    if (!plan.stacked) {
      // one plain step per shard, in ring order
      for (int s = 1; s < P; ++s) {
        const size_t src = static_cast<size_t>((r->rank - s + P) % P);
        ra_segmap kq, ks;
        stride = ra_ring_step_maps(P, r->rank, c->seq, c->layout, c->n_splits, s, &kq, &ks);
        RAB_REQUIRE(stride >= 1, RA_ERR_INVALID, "ring prefill: bad partition");
        rc = ra_attention_step_ex(c->dtype, q, buf_k[0] + src * kv_raw, buf_v[0] + src * kv_raw, out,
                                  m, l, &shape, &kq, &ks, stride,
                                  causal_flag | (s == P - 1 ? RA_STEP_FINALIZE : 0u), c->doc_len, 0,
                                  stream);
        if (rc != RA_OK) return rc;
      }
    } else {
      // entry e = (s - 1) * nsg + i: sub-group i of the shard s hops away; part z takes the
      // entries e = z, z + parts, ... so every part sees keys from all over the sequence
      bool aux_used[kAuxStreams] = {false, false, false};
      const int heads_c = c->heads / plan.chunks;  // query (= KV) heads per chunk
      const size_t chunk_raw = kv_raw / plan.chunks;
      for (int g = 0; g < plan.chunks; ++g) {
        cudaEvent_t landed = plan.chunks > 1 ? r->ev_comm[1 + g] : r->ev_comm[0];
        if (plan.chunks > 1) RAB_CUDA(cudaStreamWaitEvent(stream, landed, 0));
        const size_t q_off = static_cast<size_t>(g) * heads_c * sloc * c->head_dim;  // elements
        const size_t r_off = static_cast<size_t>(g) * heads_c * sloc;               // rows
        const unsigned char* gk = buf_k[0] + static_cast<size_t>(g) * P * chunk_raw;
        const unsigned char* gv = buf_v[0] + static_cast<size_t>(g) * P * chunk_raw;
        for (int z = 0; z < plan.parts; ++z) {
          ra_segmap ks;
          int seg_shard[RA_MAX_SEG], seg_row[RA_MAX_SEG];
          stride = ra_ring_gather_part_maps(P, r->rank, c->seq, c->layout, c->n_splits, plan.parts, z,
                                            &ks, seg_shard, seg_row);
          RAB_REQUIRE(stride >= 1 && ks.n_seg >= 1 && ks.seg_len == kmap.seg_len, RA_ERR_INVALID,
                      "ring prefill: bad partition");
          const PosMap km = make_posmap(ks);
          ra_shape sh = shape;
          sh.seq_k = km.n_seg * km.seg_len;
          if (plan.chunks > 1) sh.heads = sh.kv_heads = heads_c;
          cudaStream_t st = stream;
          if (z > 0) {
            const int a = (z - 1) % kAuxStreams;
            st = r->aux_stream[a];
            if (!aux_used[a]) {
              RAB_CUDA(cudaStreamWaitEvent(st, r->ev_start, 0));
              aux_used[a] = true;
            }
            RAB_CUDA(cudaStreamWaitEvent(st, landed, 0));
          }
          const unsigned flags = split ? (causal_flag | RA_STEP_FRESH) : (causal_flag | RA_STEP_FINALIZE);
          float* o_z = (split ? part_out(z + 1) : out) + q_off;
          float* m_z = (split ? part_m(z + 1) : m) + r_off;
          float* l_z = (split ? part_l(z + 1) : l) + r_off;
          rc = step_stacked(c->dtype, static_cast<const unsigned char*>(q) + q_off * es, gk, gv, o_z, m_z,
                            l_z, sh, make_posmap(qmap), km, seg_shard, seg_row, P, sloc, stride, flags,
                            c->doc_len, st);
          if (rc != RA_OK) return rc;
        }
      }
      if (split) {
        for (int a = 0; a < kAuxStreams; ++a) {
          if (!aux_used[a]) continue;
          RAB_CUDA(cudaEventRecord(r->ev_aux[a], r->aux_stream[a]));
          RAB_CUDA(cudaStreamWaitEvent(stream, r->ev_aux[a], 0));
        }
        rc = launch_state_merge(part_base, plan.part_floats, plan.parts + 1, rows, c->head_dim, out,
                                m, l, 1, stream);
        if (rc != RA_OK) return rc;
      }
    }
    RAB_CUDA(cudaEventRecord(r->ev_comp[1], stream));
    n_launch = 2;
  }
  // RA_SCHEDULE_BLOCKING (the reference's ring-blocking, src/ring_loop.cu:259-592): the same
  // rotation with nothing overlapped. The exchange of a step is enqueued on the compute stream
  // behind the step kernel, so every step is transfer, then compute.
  const bool blocking = c->schedule == RA_SCHEDULE_BLOCKING;
  const bool ring2d = c->schedule == RA_SCHEDULE_RING2D && P > 1;
  auto exchange = [&](cudaStream_t cs, const void* src_k, const void* src_v, void* dst_k, void* dst_v,
                      int to, int from) {
    NcclGroup grp;
    grp.note(g_nccl.Send(src_k, kv_raw, kNcclInt8, to, r->comm, cs), "ncclSend(K)");
    grp.note(g_nccl.Recv(dst_k, kv_raw, kNcclInt8, from, r->comm, cs), "ncclRecv(K)");
    grp.note(g_nccl.Send(src_v, kv_raw, kNcclInt8, to, r->comm, cs), "ncclSend(V)");
    grp.note(g_nccl.Recv(dst_v, kv_raw, kNcclInt8, from, r->comm, cs), "ncclRecv(V)");
    return grp.end();
  };
  // RA_SCHEDULE_RING2D (the reference's ring-2d, src/ring_loop.cu:1071-1550, visitation order of
  // Ring2DSchedule, src/ring2d_schedule.cpp:28-42): the ranks form `ring2d_nodes` groups of
  // G = cp / nodes. In macro-step m a rank first sends the shard it starts the macro-step with
  // (its "seed") to the same slot of the next group on the side stream, which overlaps the whole
  // inner loop; the inner loop computes against the seed and rotates it around the group's own
  // ring G - 1 times on the compute stream (as the reference does); the shard received from the
  // previous group is the next seed.
  auto ring2d_pass = [&]() -> int {
    const int N = c->ring2d_nodes, G = P / N;
    const int n = r->rank / G, g = r->rank % G;
    const int intra_next = n * G + (g + 1) % G, intra_prev = n * G + (g - 1 + G) % G;
    const int outer_next = ((n + 1) % N) * G + g, outer_prev = ((n - 1 + N) % N) * G + g;
    const void* seed_k = k;
    const void* seed_v = v;
    int idx = 0;
    n_comm = N - 1;
    for (int mstep = 0; mstep < N; ++mstep) {
      NvtxRange range("ring prefill: 2-D macro-step");
      if (mstep < N - 1) {
        // the buffer received into was the seed of the macro-step before the last one: everything
        // enqueued on the compute stream so far has to be through with it
        RAB_CUDA(cudaEventRecord(r->ev_aux[0], stream));
        RAB_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_aux[0], 0));
        RAB_CUDA(cudaEventRecord(r->ev_comm_begin[mstep], r->comm_stream));
        int rc2 = exchange(r->comm_stream, seed_k, seed_v, outer_k[mstep & 1], outer_v[mstep & 1],
                           outer_next, outer_prev);
        if (rc2 != RA_OK) {
          cudaStreamSynchronize(r->comm_stream);
          return rc2;
        }
        RAB_CUDA(cudaEventRecord(r->ev_comm[mstep], r->comm_stream));
      }
      const void* cur_k = seed_k;
      const void* cur_v = seed_v;
      for (int i = 0; i < G; ++i, ++idx) {
        const int src = ((n - mstep + N) % N) * G + (g - i + G) % G;
        const int step = (r->rank - src + P) % P;
        ra_segmap qmap, kmap;
        const int stride =
            ra_ring_step_maps(P, r->rank, c->seq, c->layout, c->n_splits, step, &qmap, &kmap);
        RAB_REQUIRE(stride >= 1, RA_ERR_INVALID, "ring prefill: bad partition");
        unsigned flags = c->causal ? RA_STEP_CAUSAL : 0u;
        if (idx == 0) flags |= RA_STEP_FRESH;
        if (idx == P - 1) flags |= RA_STEP_FINALIZE;
        if (idx == 0 && q_ready) RAB_CUDA(cudaStreamWaitEvent(stream, q_ready, 0));
        RAB_CUDA(cudaEventRecord(r->ev_comp_begin[idx], stream));
        int rc2 = ra_attention_step_ex(c->dtype, q, cur_k, cur_v, out, m, l, &shape, &qmap, &kmap,
                                       stride, flags, c->doc_len, 0, stream);
        if (rc2 == RA_OK && i < G - 1) {
          rc2 = exchange(stream, cur_k, cur_v, buf_k[i & 1], buf_v[i & 1], intra_next, intra_prev);
          cur_k = buf_k[i & 1];
          cur_v = buf_v[i & 1];
        }
        if (rc2 != RA_OK) {
          cudaStreamSynchronize(r->comm_stream);
          return rc2;
        }
        RAB_CUDA(cudaEventRecord(r->ev_comp[idx], stream));
      }
      if (mstep < N - 1) {
        RAB_CUDA(cudaStreamWaitEvent(stream, r->ev_comm[mstep], 0));
        seed_k = outer_k[mstep & 1];
        seed_v = outer_v[mstep & 1];
      }
    }
    n_launch = P;
    return RA_OK;
  };
  for (int s = 0; s < P && !gather && !ring2d; ++s) {
    NvtxRange range("ring prefill: step");
    const void* cur_k = s == 0 ? k : buf_k[(s - 1) & 1];
    const void* cur_v = s == 0 ? v : buf_v[(s - 1) & 1];
    if (s < P - 1 && !blocking) {
      // the buffer about to be received into was the source of compute step s-1
      if (s >= 1) RAB_CUDA(cudaStreamWaitEvent(r->comm_stream, r->ev_comp[s - 1], 0));
      RAB_CUDA(cudaEventRecord(r->ev_comm_begin[s], r->comm_stream));
      NcclGroup grp;
      grp.note(g_nccl.Send(cur_k, kv_raw, kNcclInt8, next, r->comm, r->comm_stream), "ncclSend(K)");
      grp.note(g_nccl.Recv(buf_k[s & 1], kv_raw, kNcclInt8, prev, r->comm, r->comm_stream), "ncclRecv(K)");
      grp.note(g_nccl.Send(cur_v, kv_raw, kNcclInt8, next, r->comm, r->comm_stream), "ncclSend(V)");
      grp.note(g_nccl.Recv(buf_v[s & 1], kv_raw, kNcclInt8, prev, r->comm, r->comm_stream), "ncclRecv(V)");
      rc = grp.end();
      if (rc != RA_OK) {
        cudaStreamSynchronize(r->comm_stream);  // nothing of this pass may still write the workspace
        return rc;
      }
      RAB_CUDA(cudaEventRecord(r->ev_comm[s], r->comm_stream));
    }
    if (s == 0 && q_ready) RAB_CUDA(cudaStreamWaitEvent(stream, q_ready, 0));
    if (s > 0 && !blocking) RAB_CUDA(cudaStreamWaitEvent(stream, r->ev_comm[s - 1], 0));
    ra_segmap qmap, kmap;
    const int stride =
        ra_ring_step_maps(P, r->rank, c->seq, c->layout, c->n_splits, s, &qmap, &kmap);
    RAB_REQUIRE(stride >= 1, RA_ERR_INVALID, "ring prefill: bad partition");
    unsigned flags = c->causal ? RA_STEP_CAUSAL : 0u;
    if (s == 0) flags |= RA_STEP_FRESH;
    if (s == P - 1) flags |= RA_STEP_FINALIZE;
    RAB_CUDA(cudaEventRecord(r->ev_comp_begin[s], stream));
    rc = ra_attention_step_ex(c->dtype, q, cur_k, cur_v, out, m, l, &shape, &qmap, &kmap, stride,
                              flags, c->doc_len, 0, stream);
    if (rc != RA_OK) {
      cudaStreamSynchronize(r->comm_stream);  // transfers already queued write the workspace
      return rc;
    }
    RAB_CUDA(cudaEventRecord(r->ev_comp[s], stream));
    n_launch = s + 1;
    if (s < P - 1 && blocking) {
      RAB_CUDA(cudaEventRecord(r->ev_comm_begin[s], stream));
      rc = exchange(stream, cur_k, cur_v, buf_k[s & 1], buf_v[s & 1], next, prev);
      if (rc != RA_OK) return rc;
      RAB_CUDA(cudaEventRecord(r->ev_comm[s], stream));
    }
  }
  if (ring2d) {
    rc = ring2d_pass();
    if (rc != RA_OK) return rc;
  }
  if (lse) {
    rc = ra_attention_lse(m, l, lse, rows, stream);
    if (rc != RA_OK) return rc;
  }
  RAB_CUDA(cudaEventRecord(r->ev_end, stream));
  if (result) {
    rc = enqueue_status_read(stream);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaStreamSynchronize(stream));
    RAB_CUDA(cudaStreamSynchronize(r->comm_stream));
    rc = status_after_sync();
    if (rc != RA_OK) return rc;
    float ms = 0.f;
    double comp = 0.0, comm = 0.0;
    for (int s = 0; s < n_launch; ++s) {
      RAB_CUDA(cudaEventElapsedTime(&ms, r->ev_comp_begin[s], r->ev_comp[s]));
      comp += ms;
    }
    for (int s = 0; s < n_comm; ++s) {
      RAB_CUDA(cudaEventElapsedTime(&ms, r->ev_comm_begin[s], r->ev_comm[s]));
      comm += ms;
    }
    RAB_CUDA(cudaEventElapsedTime(&ms, r->ev_start, r->ev_end));
    result->total_ms = ms;
    result->comp_ms = comp;
    result->comm_ms = comm;
    // time the compute stream spent not computing: transfers that were not hidden
    result->wait_ms = ms - comp > 0.0 ? ms - comp : 0.0;
  }
  return RA_OK;
}

extern "C" {

int ra_ring_prefill(ra_ring* r, const ra_ring_config* c, const void* q, const void* k,
                    const void* v, float* out, float* lse, void* kv_work, size_t kv_work_bytes,
                    ra_stream stream, ra_ring_result* result) {
  return ring_prefill_impl(r, c, q, k, v, out, lse, kv_work, kv_work_bytes, stream, result, nullptr);
}

int ra_ring_prefill_host(ra_ring* r, const ra_ring_config* c, const void* q_host,
                         const void* k_host, const void* v_host, float* out_host, float* lse_host,
                         ra_ring_result* result) {
  int rc = check_cfg(r, c);
  if (rc != RA_OK) return rc;
  RAB_REQUIRE(q_host && k_host && v_host && out_host, RA_ERR_INVALID,
              "ring prefill (host): null argument");
  NvtxRange range("ring prefill (host buffers)");
  const int kvH = c->kv_heads > 0 ? c->kv_heads : c->heads;
  const size_t es = c->dtype == RA_F32 ? 4 : 2;
  const size_t sloc = static_cast<size_t>(c->seq / r->cp);
  const size_t rows = static_cast<size_t>(c->batch) * c->heads * sloc;
  const size_t q_bytes = rows * c->head_dim * es;
  const size_t kv_raw = static_cast<size_t>(c->batch) * kvH * sloc * c->head_dim * es;
  const size_t out_bytes = rows * c->head_dim * sizeof(float);
  const size_t lse_bytes = rows * sizeof(float);
  // (see below) two half passes over head groups, when the heads are independent slices
  // Measured on config 2 (75 MB up per pass over the P links, 8 heads): N = 2 2.45 -> 1.94 ms with
  // two groups (three or four: 2.00), N = 4 no difference (1.72-1.83 against 1.77-1.84, 25 MB per
  // rank); below 16 MB per rank the second pass's own latency is not worth it.
  const int n_groups =
      (c->batch == 1 && kvH == c->heads && c->heads >= 2 && q_bytes + 2 * kv_raw >= (16u << 20))
          ? kHostGroupsMax
          : 1;
  const bool two_groups = n_groups >= 2;
  int h_split[kHostGroupsMax + 1];
  for (int g = 0; g <= n_groups; ++g) h_split[g] = static_cast<int>(static_cast<long long>(c->heads) * g / n_groups);
  size_t work_bytes = ra_ring_prefill_workspace_bytes(r, c);
  if (two_groups) {
    // a half pass may pick another plan (more key parts for fewer blocks): take the largest need
    work_bytes = 0;
    for (int g = 0; g < n_groups; ++g) {
      ra_ring_config cg = *c;
      cg.heads = cg.kv_heads = h_split[g + 1] - h_split[g];
      work_bytes = std::max(work_bytes, ra_ring_prefill_workspace_bytes(r, &cg));
    }
  }
  const size_t need = align256(q_bytes) + 2 * align256(kv_raw) + align256(out_bytes) +
                      align256(lse_bytes) + align256(work_bytes);
  if (r->host_bytes < need) {
    if (r->host_buf) {
      RAB_CUDA(cudaStreamSynchronize(r->host_stream));
      RAB_CUDA(cudaFree(r->host_buf));
    }
    r->host_buf = nullptr;
    r->host_bytes = 0;
    RAB_CUDA(cudaMalloc(&r->host_buf, need));
    r->host_bytes = need;
  }
  unsigned char* p = static_cast<unsigned char*>(r->host_buf);
  void* dq = p;
  p += align256(q_bytes);
  void* dk = p;
  p += align256(kv_raw);
  void* dv = p;
  p += align256(kv_raw);
  float* dout = reinterpret_cast<float*>(p);
  p += align256(out_bytes);
  float* dlse = reinterpret_cast<float*>(p);
  p += align256(lse_bytes);
  void* work = p;
  cudaStream_t st = r->host_stream;
  // One KV head per query head and one batch element: the heads are independent, contiguous
  // slices of every tensor, so the pass runs as two half passes (head groups) in a pipeline -
  // upload of the second half under the first half's pass, download of the first half under
  // the second half's pass. Each half pass pays its own transfers' latency, which the copies
  // it hides outweigh when a rank moves tens of megabytes.
  if (two_groups) {
    cudaStream_t up = r->host_q_stream, down = r->host_out_stream;
    const size_t head_elems = sloc * c->head_dim;
    RAB_CUDA(cudaEventRecord(r->ev_host_begin, st));
    RAB_CUDA(cudaStreamWaitEvent(up, r->ev_host_begin, 0));
    for (int g = 0; g < n_groups; ++g) {
      const size_t off = h_split[g] * head_elems * es, n = (h_split[g + 1] - h_split[g]) * head_elems * es;
      RAB_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(dk) + off, static_cast<const unsigned char*>(k_host) + off, n, cudaMemcpyHostToDevice, up));
      RAB_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(dv) + off, static_cast<const unsigned char*>(v_host) + off, n, cudaMemcpyHostToDevice, up));
      RAB_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(dq) + off, static_cast<const unsigned char*>(q_host) + off, n, cudaMemcpyHostToDevice, up));
      RAB_CUDA(cudaEventRecord(r->ev_host_up[g], up));
    }
    for (int g = 0; g < n_groups; ++g) {
      const int hg = h_split[g + 1] - h_split[g];
      const size_t off = h_split[g] * head_elems, row_off = h_split[g] * sloc;
      ra_ring_config cg = *c;
      cg.heads = hg;
      cg.kv_heads = hg;
      RAB_CUDA(cudaStreamWaitEvent(st, r->ev_host_up[g], 0));
      if (g == 0) RAB_CUDA(cudaEventRecord(r->ev_host_pass, st));
      rc = ring_prefill_impl(r, &cg, static_cast<unsigned char*>(dq) + off * es,
                             static_cast<unsigned char*>(dk) + off * es,
                             static_cast<unsigned char*>(dv) + off * es, dout + off,
                             lse_host ? dlse + row_off : nullptr, work, work_bytes, st, nullptr, nullptr);
      if (rc != RA_OK) {
        cudaStreamSynchronize(up);
        cudaStreamSynchronize(st);
        cudaStreamSynchronize(r->comm_stream);
        cudaStreamSynchronize(down);
        return rc;
      }
      RAB_CUDA(cudaEventRecord(r->ev_host_done[g], st));
      RAB_CUDA(cudaStreamWaitEvent(down, r->ev_host_done[g], 0));
      RAB_CUDA(cudaMemcpyAsync(out_host + off, dout + off, hg * head_elems * sizeof(float),
                               cudaMemcpyDeviceToHost, down));
      if (lse_host)
        RAB_CUDA(cudaMemcpyAsync(lse_host + row_off, dlse + row_off, hg * sloc * sizeof(float),
                                 cudaMemcpyDeviceToHost, down));
    }
    RAB_CUDA(cudaEventRecord(r->ev_host_end, down));
    rc = enqueue_status_read(st);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaStreamSynchronize(down));
    RAB_CUDA(cudaStreamSynchronize(st));
    RAB_CUDA(cudaStreamSynchronize(r->comm_stream));
    rc = status_after_sync();
    if (rc != RA_OK) return rc;
    if (result) {
      float ms = 0.f, pass_ms = 0.f;
      RAB_CUDA(cudaEventElapsedTime(&ms, r->ev_host_begin, r->ev_host_end));
      RAB_CUDA(cudaEventElapsedTime(&pass_ms, r->ev_host_pass, r->ev_end));
      result->total_ms = ms;           // upload + both half passes + download
      result->comp_ms = pass_ms;       // first half pass's start to second half pass's end
      result->comm_ms = 0.0;
      result->wait_ms = ms - pass_ms;  // time on the host link not covered by the passes
    }
    return RA_OK;
  }
  // Otherwise one pass. K and V go first: the transfers of the pass (all-gather or first hop)
  // need only them and start while Q is still on its way up on a second stream; the first step
  // waits for Q.
  RAB_CUDA(cudaEventRecord(r->ev_host_begin, st));
  RAB_CUDA(cudaMemcpyAsync(dk, k_host, kv_raw, cudaMemcpyHostToDevice, st));
  RAB_CUDA(cudaMemcpyAsync(dv, v_host, kv_raw, cudaMemcpyHostToDevice, st));
  RAB_CUDA(cudaStreamWaitEvent(r->host_q_stream, r->ev_host_begin, 0));
  RAB_CUDA(cudaMemcpyAsync(dq, q_host, q_bytes, cudaMemcpyHostToDevice, r->host_q_stream));
  RAB_CUDA(cudaEventRecord(r->ev_host_q, r->host_q_stream));
  ra_ring_result pass{};
  rc = ring_prefill_impl(r, c, dq, dk, dv, dout, lse_host ? dlse : nullptr, work, work_bytes, st,
                         nullptr, r->ev_host_q);
  if (rc != RA_OK) {
    cudaStreamSynchronize(r->host_q_stream);
    cudaStreamSynchronize(st);
    return rc;
  }
  RAB_CUDA(cudaMemcpyAsync(out_host, dout, out_bytes, cudaMemcpyDeviceToHost, st));
  if (lse_host) RAB_CUDA(cudaMemcpyAsync(lse_host, dlse, lse_bytes, cudaMemcpyDeviceToHost, st));
  RAB_CUDA(cudaEventRecord(r->ev_host_end, st));
  rc = enqueue_status_read(st);
  if (rc != RA_OK) return rc;
  RAB_CUDA(cudaStreamSynchronize(st));
  RAB_CUDA(cudaStreamSynchronize(r->comm_stream));
  rc = status_after_sync();
  if (rc != RA_OK) return rc;
  if (result) {
    float ms = 0.f, pass_ms = 0.f;
    RAB_CUDA(cudaEventElapsedTime(&ms, r->ev_host_begin, r->ev_host_end));
    RAB_CUDA(cudaEventElapsedTime(&pass_ms, r->ev_start, r->ev_end));
    result->total_ms = ms;           // upload + pass + download
    result->comp_ms = pass_ms;       // the ring pass alone
    result->comm_ms = 0.0;
    result->wait_ms = ms - pass_ms;  // time spent on the host link outside the pass
  }
  return RA_OK;
}

int ra_ring_decode_step_raw(ra_ring* r, int dtype, int batch, int heads, int kv_heads,
                            int head_dim, const void* q, const void* k_cache, const void* v_cache,
                            int local_len, int s_max, float* out, ra_stream stream_,
                            ra_ring_result* result) {
  RAB_REQUIRE(r && q && k_cache && v_cache && out, RA_ERR_INVALID, "ring decode: null argument");
  RAB_REQUIRE(batch > 0 && heads > 0 && local_len >= 0 && local_len <= s_max, RA_ERR_INVALID,
              "ring decode: bad sizes (local_len=%d, s_max=%d)", local_len, s_max);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  NvtxRange range("ring decode step");
  const int D = head_dim;
  const size_t bh = static_cast<size_t>(batch) * heads;
  const size_t block = bh * D + 2 * bh;  // floats per rank: [O | m | l]
  const size_t need = (1 + static_cast<size_t>(r->cp)) * block * sizeof(float);
  if (r->dec_bytes < need) {
    if (r->dec_buf) RAB_CUDA(cudaFree(r->dec_buf));
    r->dec_buf = nullptr;
    r->dec_bytes = 0;
    RAB_CUDA(cudaMalloc(reinterpret_cast<void**>(&r->dec_buf), need));
    r->dec_bytes = need;
  }
  float* send = r->dec_buf;
  float* recv = r->dec_buf + block;
  float* o_p = send;
  float* m_p = send + bh * D;
  float* l_p = m_p + bh;
  RAB_CUDA(cudaEventRecord(r->ev_start, stream));
  int rc = RA_OK;
  if (local_len > 0) {
    ra_shape s{batch, heads, 1, local_len, D, kv_heads};
    // causality is implicit: the cache only ever holds past tokens (src/ring_decode.cu:173-175);
    // the partial is written into the empty send block by the fold itself (no init launch)
    rc = decode_step(dtype, q, k_cache, v_cache, o_p, m_p, l_p, s, 0, 0, 0, stream, s_max, nullptr,
                     0, RA_STEP_FRESH);
  } else {
    rc = launch_init(o_p, m_p, l_p, bh * D, bh, stream);
  }
  if (rc != RA_OK) return rc;
  RAB_CUDA(cudaEventRecord(r->ev_comp[0], stream));
  const float* gathered = send;
  if (r->cp > 1) {
    RAB_NCCL(g_nccl.AllGather(send, recv, block, kNcclFloat, r->comm, stream));
    gathered = recv;
  }
  RAB_CUDA(cudaEventRecord(r->ev_comm[0], stream));
  rc = ra_decode_partial_merge(gathered, out, nullptr, nullptr, r->cp, static_cast<int>(bh), D, 1,
                               stream_);
  if (rc != RA_OK) return rc;
  RAB_CUDA(cudaEventRecord(r->ev_end, stream));
  if (result) {
    rc = enqueue_status_read(stream);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaStreamSynchronize(stream));
    rc = status_after_sync();
    if (rc != RA_OK) return rc;
    float a = 0.f, b = 0.f, t = 0.f;
    RAB_CUDA(cudaEventElapsedTime(&a, r->ev_start, r->ev_comp[0]));
    RAB_CUDA(cudaEventElapsedTime(&b, r->ev_comp[0], r->ev_comm[0]));
    RAB_CUDA(cudaEventElapsedTime(&t, r->ev_start, r->ev_end));
    result->comp_ms = a;
    result->comm_ms = b;
    result->wait_ms = b;
    result->total_ms = t;
  }
  return RA_OK;
}

int ra_ring_decode_step(ra_ring* r, int batch, int heads, const void* q, const void* k_new,
                        const void* v_new, int owner_rank, ra_kv_cache* cache,
                        const int* current_len_per_rank, float* out, ra_stream stream_,
                        ra_ring_result* result) {
  RAB_REQUIRE(r && q && cache && current_len_per_rank && out, RA_ERR_INVALID,
              "ring decode: null argument");
  RAB_REQUIRE(owner_rank >= 0 && owner_rank < r->cp, RA_ERR_INVALID,
              "ring decode: owner_rank %d out of range", owner_rank);
  RAB_REQUIRE(batch == cache->batch, RA_ERR_INVALID, "ring decode: batch %d != cache batch %d",
              batch, cache->batch);
  if (r->rank == owner_rank) {
    RAB_REQUIRE(k_new && v_new, RA_ERR_INVALID, "ring decode: owner needs k_new / v_new");
    const int rc = ra_kv_cache_append(cache, k_new, v_new, stream_);
    if (rc != RA_OK) return rc;
  }
  // the caller's bookkeeping must agree with the cache (src/ring_decode.cu:108-125)
  RAB_REQUIRE(current_len_per_rank[r->rank] == cache->current_len, RA_ERR_INVALID,
              "ring_decode: current_len_per_rank[%d]=%d but cache.current_len=%d", r->rank,
              current_len_per_rank[r->rank], cache->current_len);
  return ra_ring_decode_step_raw(r, cache->dtype, batch, heads, cache->kv_heads, cache->head_dim, q,
                                 cache->k, cache->v, cache->current_len, cache->s_max, out, stream_,
                                 result);
}

}  // extern "C"
