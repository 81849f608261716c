// Second half of the C++ shim: the reference's multi-rank drivers (src/ring_loop.hpp,
// src/ring_decode.hpp) on top of the C ABI, so that the reference's MPI command-line driver
// (apps/ring_attention_cli/main.cu) builds and runs unchanged. MPI here is whatever <mpi.h>
// the build finds: a real MPI, or the minimpi beside this file.
//
// What is kept from the reference's contract (src/ring_loop_fp16.cu:522-818): inputs from
// gen_elem with cfg.seed, one warm-up pass, `iters` timed passes between barriers,
// total_ms = wall / iters, comm / comp / wait from device events, all MAX-reduced to rank 0,
// --verify against cpu_attention on every rank's own rows (max absolute error, -1 where not
// verified), the flag validation and its messages, and abort-on-error.
// What differs, on purpose: --mode=allgather gathers the shards once and then runs one masked
// step per source shard, every other --mode runs the overlapped ring or, for small shards, the
// same gather (on one NVSwitch box the blocking and 2-D schedules have nothing to offer;
// results are identical), a ring step is one launch over the whole shard (so --segmented changes nothing), the
// communicator of nccl_init is wrapped, not rebuilt inside the timed region, and the initial
// K/V shard is uploaded once, not once per pass (the ring never overwrites it).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mpi.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#ifndef RING_USE_NCCL
#define RING_USE_NCCL 1
#endif
#include "attention.hpp"
#include "cpu_attention.hpp"
#include "device_tensor.hpp"
#include "nccl_utils.hpp"
#include "ring_decode.hpp"
#include "ring_gen.hpp"
#include "ring_loop.hpp"
#include "ring_partition.hpp"

#include "../../include/ring_attention_b200.h"

namespace ring_attention {

namespace {

[[noreturn]] void mpi_die(const std::string& msg) {
  int rank = 0;
  MPI_Comm_rank(MPI_COMM_WORLD, &rank);
  if (rank == 0) std::fprintf(stderr, "ERROR: %s\n", msg.c_str());
  MPI_Abort(MPI_COMM_WORLD, EXIT_FAILURE);
  std::abort();
}
void must(int rc, const char* what) {
  if (rc != RA_OK) mpi_die(std::string(what) + ": " + ra_last_error());
}
void cuda_must(cudaError_t e, const char* what) {
  if (e != cudaSuccess) mpi_die(std::string(what) + ": " + cudaGetErrorString(e));
}

struct Layout {
  int mode;      // 0 contiguous, 1 zig-zag, 2 striped (RingPartition::Mode order)
  int n_splits;  // zig-zag sub-groups
};
Layout layout_of(const RingConfig& c) {
  if (c.zigzag_n > 0) return {1, zigzag_sub_groups(c.zigzag_n)};
  if (c.striped) return {2, 2};
  return {0, 2};
}

// Global positions of this rank's rows, sub-groups concatenated (the shard order of the library).
std::vector<int> local_rows(const RingConfig& c, const Layout& lay) {
  const RingPartition part(c.cp_size, c.rank, c.seq, static_cast<RingPartition::Mode>(lay.mode),
                           lay.n_splits);
  std::vector<int> rows;
  const int n = part.local_chunk_len(), st = part.position_stride();
  for (int sg = 0; sg < part.num_sub_groups(); ++sg)
    for (int i = 0; i < n; ++i) rows.push_back(part.q_offset(sg) + i * st);
  return rows;
}

// (b, h, rows[i], d) of tensor `id` from the coordinate hash (src/ring_gen.hpp:18-29).
void fill_local(std::vector<float>& dst, const RingConfig& c, int id, int heads,
                const std::vector<int>& rows) {
  const size_t n = rows.size();
  dst.resize(static_cast<size_t>(c.batch) * heads * n * c.head_dim);
  size_t o = 0;
  for (int b = 0; b < c.batch; ++b)
    for (int h = 0; h < heads; ++h)
      for (size_t i = 0; i < n; ++i)
        for (int d = 0; d < c.head_dim; ++d) dst[o++] = gen_elem(c.seed, id, b, h, rows[i], d);
}

}  // namespace

RingMode mode_from_string(const std::string& s) {
  if (s == "allgather") return RingMode::AllGather;
  if (s == "ring-blocking") return RingMode::RingBlocking;
  if (s == "ring-overlap") return RingMode::RingOverlap;
  if (s == "ring-2d") return RingMode::Ring2D;
  mpi_die("Unknown --mode=" + s + " (valid: allgather ring-blocking ring-overlap ring-2d)");
}

RingDtype dtype_from_string(const std::string& s) {
  if (s == "fp32" || s == "float") return RingDtype::Float;
  if (s == "fp16" || s == "half") return RingDtype::Half;
  mpi_die("Unknown --dtype=" + s + " (valid: fp32 fp16)");
}

RingResult run_ring_attention(const RingConfig& cfg) {
  // the reference's flag validation (src/ring_loop.cu:1584-1593)
  if (cfg.zigzag_n > 0 && cfg.striped)
    mpi_die("--zigzag-n and --striped are mutually exclusive (pick one partition scheme)");
  if (cfg.zigzag_n > 0 && cfg.mode == RingMode::AllGather)
    mpi_die("--zigzag-n is not supported with --mode=allgather (use ring-blocking or ring-overlap)");
  if (cfg.striped && cfg.mode == RingMode::AllGather)
    mpi_die("--striped is not supported with --mode=allgather (use ring-blocking or ring-overlap)");
  if (cfg.segmented && ((cfg.mode != RingMode::RingOverlap && cfg.mode != RingMode::Ring2D) ||
                        cfg.dtype == RingDtype::Half || cfg.zigzag_n <= 0 || cfg.striped))
    mpi_die("--segmented requires fp32 ring-overlap or ring-2d with --zigzag-n N (not --striped)");
  if (cfg.dtype == RingDtype::Half && cfg.mode == RingMode::Ring2D)
    mpi_die("--mode=ring-2d is not supported with --dtype=fp16");

  const Layout lay = layout_of(cfg);
  const int kvH = cfg.kv_heads > 0 ? cfg.kv_heads : cfg.heads;
  const std::vector<int> rows = local_rows(cfg, lay);
  const size_t sloc = rows.size();
  const bool half = cfg.dtype == RingDtype::Half;

  std::vector<float> hq, hk, hv;
  fill_local(hq, cfg, 0, cfg.heads, rows);
  fill_local(hk, cfg, 1, kvH, rows);
  fill_local(hv, cfg, 2, kvH, rows);

  DeviceTensor<float> q32(hq.size()), k32(hk.size()), v32(hv.size());
  q32.copy_from_host(hq);
  k32.copy_from_host(hk);
  v32.copy_from_host(hv);
  DeviceTensor<__half> q16(half ? hq.size() : 0), k16(half ? hk.size() : 0),
      v16(half ? hv.size() : 0);
  if (half) {
    launch_float_to_half(q32.data(), q16.data(), hq.size());
    launch_float_to_half(k32.data(), k16.data(), hk.size());
    launch_float_to_half(v32.data(), v16.data(), hv.size());
  }
  const void* dq = half ? static_cast<const void*>(q16.data()) : q32.data();
  const void* dk = half ? static_cast<const void*>(k16.data()) : k32.data();
  const void* dv = half ? static_cast<const void*>(v16.data()) : v32.data();
  DeviceTensor<float> out(hq.size());

  ncclComm_t comm = nullptr;
  if (cfg.cp_size > 1) comm = nccl_init(cfg.rank, cfg.cp_size);
  ra_ring* ring = nullptr;
  must(ra_ring_create_from_comm(cfg.rank, cfg.cp_size, comm, &ring), "ra_ring_create_from_comm");

  ra_ring_config rc{};
  rc.batch = cfg.batch;
  rc.heads = cfg.heads;
  rc.kv_heads = kvH;
  rc.seq = cfg.seq;
  rc.head_dim = cfg.head_dim;
  rc.dtype = half ? RA_F16 : RA_F32;
  rc.causal = cfg.causal ? 1 : 0;
  rc.layout = lay.mode;
  rc.n_splits = lay.n_splits;
  rc.doc_len = 0;
  // every --mode runs the schedule it names (AUTO, which picks by shard size, is for the library
  // API). ring-2d groups ranks by node as the reference does (src/ring_loop.cu:1079-1091): one
  // node here, unless RA_RING2D_NODES asks for more groups to exercise the two-tier order.
  rc.ring2d_nodes = 1;
  switch (cfg.mode) {
    case RingMode::AllGather: rc.schedule = RA_SCHEDULE_GATHER; break;
    case RingMode::RingBlocking: rc.schedule = RA_SCHEDULE_BLOCKING; break;
    case RingMode::Ring2D: {
      rc.schedule = RA_SCHEDULE_RING2D;
      const char* e = std::getenv("RA_RING2D_NODES");
      const int nodes = e ? std::atoi(e) : 1;
      if (nodes >= 1 && cfg.cp_size % nodes == 0) rc.ring2d_nodes = nodes;
    } break;
    default: rc.schedule = RA_SCHEDULE_RING; break;
  }
  const size_t work_bytes = ra_ring_prefill_workspace_bytes(ring, &rc);
  DeviceTensor<signed char> work(work_bytes);

  cudaStream_t stream = nullptr;
  cuda_must(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
  auto one_pass = [&](ra_ring_result* t) {
    must(ra_ring_prefill(ring, &rc, dq, dk, dv, out.data(), nullptr, work.data(), work_bytes,
                         stream, t),
         "ra_ring_prefill");
  };

  ra_ring_result t{};
  one_pass(&t);  // warm-up, untimed (src/ring_loop_fp16.cu:724-726)
  double comm_ms = 0, comp_ms = 0, wait_ms = 0;
  const int iters = std::max(1, cfg.iters);
  MPI_Barrier(MPI_COMM_WORLD);
  const double t0 = MPI_Wtime();
  for (int i = 0; i < iters; ++i) {
    one_pass(&t);
    comm_ms += t.comm_ms;
    comp_ms += t.comp_ms;
    wait_ms += t.wait_ms;
  }
  MPI_Barrier(MPI_COMM_WORLD);
  const double total_ms = (MPI_Wtime() - t0) * 1e3 / iters;

  double mine[4] = {comm_ms / iters, comp_ms / iters, wait_ms / iters, total_ms};
  double top[4] = {0, 0, 0, 0};
  MPI_Reduce(mine, top, 4, MPI_DOUBLE, MPI_MAX, 0, MPI_COMM_WORLD);

  RingResult res;
  res.comm_ms = cfg.rank == 0 ? top[0] : mine[0];
  res.comp_ms = cfg.rank == 0 ? top[1] : mine[1];
  res.wait_ms = cfg.rank == 0 ? top[2] : mine[2];
  res.total_ms = cfg.rank == 0 ? top[3] : mine[3];

  if (cfg.verify) {
    // full tensors on every rank, the reference's cpu_attention, own rows compared
    // (src/ring_loop_fp16.cu:755-796)
    RingConfig full = cfg;
    std::vector<int> all(cfg.seq);
    for (int i = 0; i < cfg.seq; ++i) all[i] = i;
    std::vector<float> fq, fk, fv;
    fill_local(fq, full, 0, cfg.heads, all);
    fill_local(fk, full, 1, kvH, all);
    fill_local(fv, full, 2, kvH, all);
    std::vector<float> want(fq.size());
    AttentionShape shape{cfg.batch, cfg.heads, cfg.seq, cfg.seq, cfg.head_dim, kvH};
    cpu_attention(fq.data(), fk.data(), fv.data(), want.data(), shape, cfg.causal);
    std::vector<float> got;
    out.copy_to_host(got);
    float err = 0.f;
    const int D = cfg.head_dim;
    for (int b = 0; b < cfg.batch; ++b)
      for (int h = 0; h < cfg.heads; ++h)
        for (size_t i = 0; i < sloc; ++i)
          for (int d = 0; d < D; ++d) {
            const size_t gi = ((static_cast<size_t>(b) * cfg.heads + h) * sloc + i) * D + d;
            const size_t wi =
                ((static_cast<size_t>(b) * cfg.heads + h) * cfg.seq + rows[i]) * D + d;
            err = std::max(err, std::fabs(got[gi] - want[wi]));
          }
    float top_err = 0.f;
    MPI_Reduce(&err, &top_err, 1, MPI_FLOAT, MPI_MAX, 0, MPI_COMM_WORLD);
    res.max_err = cfg.rank == 0 ? top_err : -1.f;
  }

  cudaStreamDestroy(stream);
  ra_ring_destroy(ring);
  if (comm) ncclCommDestroy(comm);
  return res;
}

RingResult run_ring_decode_step(const RingDecodeConfig& cfg, const float* q, const float* k_new,
                                const float* v_new, int owner_rank, DeviceKVCache<float>& cache,
                                const std::vector<int>& current_len_per_rank, float* out) {
  if (static_cast<int>(current_len_per_rank.size()) != cfg.cp_size) {
    std::fprintf(stderr,
                 "run_ring_decode_step: current_len_per_rank.size()=%zu does not match cp_size=%d\n",
                 current_len_per_rank.size(), cfg.cp_size);
    MPI_Abort(MPI_COMM_WORLD, EXIT_FAILURE);
  }
  if (cfg.rank == owner_rank) cache.append(k_new, v_new);
  if (cache.current_len() != current_len_per_rank[cfg.rank]) {
    std::fprintf(stderr,
                 "run_ring_decode_step: cache.current_len()=%d on rank %d disagrees with "
                 "current_len_per_rank[rank]=%d\n",
                 cache.current_len(), cfg.rank, current_len_per_rank[cfg.rank]);
    MPI_Abort(MPI_COMM_WORLD, EXIT_FAILURE);
  }
  // One ring handle per communicator, kept for the life of the process (the caller reuses
  // the communicator across steps, src/ring_decode.hpp:31-44).
  static ra_ring* ring = nullptr;
  static ncclComm_t ring_comm = nullptr;
  if (ring == nullptr || ring_comm != cfg.nccl_comm) {
    if (ring) ra_ring_destroy(ring);
    must(ra_ring_create_from_comm(cfg.rank, cfg.cp_size, cfg.nccl_comm, &ring),
         "ra_ring_create_from_comm");
    ring_comm = cfg.nccl_comm;
  }
  MPI_Barrier(MPI_COMM_WORLD);
  const double t0 = MPI_Wtime();
  ra_ring_result t{};
  must(ra_ring_decode_step_raw(ring, RA_F32, cfg.batch, cfg.heads, cache.kv_heads(),
                               cache.head_dim(), q, cache.k_data(), cache.v_data(),
                               cache.current_len(), cache.s_max(), out, nullptr, &t),
       "ra_ring_decode_step_raw");
  cuda_must(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  MPI_Barrier(MPI_COMM_WORLD);
  RingResult res;
  res.comm_ms = t.comm_ms;
  res.comp_ms = t.comp_ms;
  res.wait_ms = t.wait_ms;
  res.total_ms = (MPI_Wtime() - t0) * 1e3;
  return res;
}

}  // namespace ring_attention
