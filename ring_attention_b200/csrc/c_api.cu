// C-ABI entry points that dispatch to the kernels: ring steps (affine, segmented, general),
// whole single-GPU attention on device and on host buffers, the KV cache, the local decode
// op and the partition index maps.
#include <algorithm>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace rab {

void set_tc_wait_limit_ns(unsigned long long ns);
void set_tc_stall_after(int items);
void set_tc_block_order(int order);

namespace {

size_t elem_size(int dtype) { return dtype == RA_F32 ? 4 : 2; }

// Validate and launch one general step (the funnel of every step entry point).
int step_ex(int dtype, const void* q, const void* k, const void* v, float* out, float* m, float* l,
            const ra_shape& s, const PosMap& qmap, const PosMap& kmap, int pos_stride,
            unsigned flags, long long doc_len, int kv_row_stride, cudaStream_t stream) {
  RAB_REQUIRE(q && k && v && out && m && l, RA_ERR_INVALID, "attention step: null argument");
  RAB_REQUIRE(dtype == RA_F32 || dtype == RA_F16 || dtype == RA_BF16, RA_ERR_INVALID,
              "attention step: unknown dtype %d", dtype);
  RAB_REQUIRE(s.batch > 0 && s.heads > 0 && s.seq_q >= 0 && s.seq_k >= 0, RA_ERR_INVALID,
              "attention step: bad shape");
  if (s.head_dim != 32 && s.head_dim != 64 && s.head_dim != 128 && s.head_dim != 256) {
    set_error("attention_step: unsupported head_dim=%d (supported: 32, 64, 128, 256)", s.head_dim);
    return RA_ERR_UNSUPPORTED;
  }
  RAB_REQUIRE(pos_stride >= 1, RA_ERR_INVALID, "attention step: pos_stride must be >= 1");
  RAB_REQUIRE(qmap.n_seg >= 1 && qmap.n_seg <= RA_MAX_SEG && kmap.n_seg >= 1 &&
                  kmap.n_seg <= RA_MAX_SEG,
              RA_ERR_INVALID, "attention step: segment count out of range");
  RAB_REQUIRE(static_cast<long long>(qmap.n_seg) * qmap.seg_len == s.seq_q &&
                  static_cast<long long>(kmap.n_seg) * kmap.seg_len == s.seq_k,
              RA_ERR_INVALID, "attention step: n_seg * seg_len must equal the sequence length");
  if (s.seq_q == 0) return RA_OK;
  StepArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.m = m;
  a.l = l;
  a.B = s.batch;
  a.H = s.heads;
  a.kvH = kv_heads_of(s);
  a.Sq = s.seq_q;
  a.Sk = s.seq_k;
  a.D = s.head_dim;
  a.kv_head_stride =
      static_cast<long long>(kv_row_stride > 0 ? kv_row_stride : s.seq_k) * s.head_dim;
  a.qmap = qmap;
  a.kmap = kmap;
  for (int i = 0; i < RA_MAX_SEG; ++i) {
    a.kseg_head[i] = 0;
    a.kseg_row[i] = i * kmap.seg_len;
  }
  a.k_heads_total = static_cast<long long>(a.B) * a.kvH;
  a.k_rows = s.seq_k;
  a.k_stacked = false;
  a.stride = pos_stride;
  a.flags = flags;
  a.doc_len = doc_len;
  a.status = device_status_ptr();
  if (s.seq_k == 0) {
    // nothing to fold; honour FRESH / FINALIZE on the state alone
    const size_t rows = static_cast<size_t>(s.batch) * s.heads * s.seq_q;
    if (flags & RA_STEP_FRESH) return launch_init(out, m, l, rows * s.head_dim, rows, stream);
    if (flags & RA_STEP_FINALIZE) return launch_finalize(out, l, rows, s.head_dim, stream);
    return RA_OK;
  }
  if (!(flags & RA_STEP_FORCE_SIMT) && step_tc_supported(dtype, a))
    return launch_step_tc(dtype, a, stream);
  if (!(flags & RA_STEP_FORCE_SIMT) && step_tf32_supported(dtype, a))
    return launch_step_tf32(a, stream);
  return launch_step_simt(dtype, a, stream);
}

}  // namespace

bool step_stacked_supported(int dtype, int head_dim) {
  return (dtype == RA_F16 || dtype == RA_BF16) &&
         (head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256);
}

int step_stacked(int dtype, const void* q, const void* k, const void* v, float* out, float* m,
                 float* l, const ra_shape& s, const PosMap& qmap, const PosMap& kmap,
                 const int* seg_shard, const int* seg_row, int n_shards, int shard_rows,
                 int pos_stride, unsigned flags, long long doc_len, cudaStream_t stream) {
  RAB_REQUIRE(q && k && v && out && m && l && seg_shard && seg_row, RA_ERR_INVALID,
              "stacked step: null argument");
  RAB_REQUIRE(step_stacked_supported(dtype, s.head_dim), RA_ERR_INVALID,
              "stacked step: needs a 16-bit dtype and head_dim 32, 64, 128 or 256");
  RAB_REQUIRE(kmap.n_seg >= 1 && kmap.n_seg <= RA_MAX_SEG && kmap.seg_len >= 1 &&
                  kmap.n_seg * kmap.seg_len == s.seq_k && n_shards >= 1 && shard_rows >= 1,
              RA_ERR_INVALID, "stacked step: bad key map");
  RAB_REQUIRE(qmap.n_seg >= 1 && qmap.n_seg <= RA_MAX_SEG && qmap.n_seg * qmap.seg_len == s.seq_q,
              RA_ERR_INVALID, "stacked step: bad query map");
  StepArgs a;
  a.q = q;
  a.k = k;
  a.v = v;
  a.out = out;
  a.m = m;
  a.l = l;
  a.B = s.batch;
  a.H = s.heads;
  a.kvH = kv_heads_of(s);
  a.Sq = s.seq_q;
  a.Sk = s.seq_k;
  a.D = s.head_dim;
  a.kv_head_stride = static_cast<long long>(shard_rows) * s.head_dim;
  a.qmap = qmap;
  a.kmap = kmap;
  const int heads_per_shard = a.B * a.kvH;
  for (int i = 0; i < RA_MAX_SEG; ++i) {
    a.kseg_head[i] = 0;
    a.kseg_row[i] = 0;
    if (i >= kmap.n_seg) continue;
    RAB_REQUIRE(seg_shard[i] >= 0 && seg_shard[i] < n_shards && seg_row[i] >= 0 &&
                    seg_row[i] + kmap.seg_len <= shard_rows,
                RA_ERR_INVALID, "stacked step: segment %d outside its shard", i);
    a.kseg_head[i] = seg_shard[i] * heads_per_shard;
    a.kseg_row[i] = seg_row[i];
  }
  a.k_heads_total = static_cast<long long>(n_shards) * heads_per_shard;
  a.k_rows = shard_rows;
  a.k_stacked = true;
  a.stride = pos_stride;
  a.flags = flags;
  a.doc_len = doc_len;
  a.status = device_status_ptr();
  RAB_REQUIRE(step_tc_supported(dtype, a), RA_ERR_INVALID,
              "stacked step: the tensor-core kernel cannot take these arguments");
  return launch_step_tc(dtype, a, stream);
}

namespace {

int affine_step(int dtype, const void* q, const void* k, const void* v, float* out, float* m,
                float* l, const ra_shape* shape, int q_offset, int k_offset, int causal,
                cudaStream_t stream, int pos_stride) {
  RAB_REQUIRE(shape != nullptr, RA_ERR_INVALID, "attention step: null shape");
  if (shape->seq_q == 1) {
    // same dispatch as the reference: one query row goes to the decode kernel, which
    // ignores pos_stride (src/attention_step.cu:494-497)
    return decode_step(dtype, q, k, v, out, m, l, *shape, q_offset, k_offset, causal, stream, 0,
                       nullptr, 0);
  }
  return step_ex(dtype, q, k, v, out, m, l, *shape, affine_posmap(q_offset, shape->seq_q),
                 affine_posmap(k_offset, shape->seq_k), pos_stride > 0 ? pos_stride : 1,
                 causal ? RA_STEP_CAUSAL : 0u, 0, 0, stream);
}

}  // namespace
}  // namespace rab

using namespace rab;

extern "C" {

int ra_attention_step(const float* q, const float* k, const float* v, float* out, float* m,
                      float* l, const ra_shape* shape, int q_offset, int k_offset, int causal,
                      ra_stream stream, int pos_stride) {
  return affine_step(RA_F32, q, k, v, out, m, l, shape, q_offset, k_offset, causal,
                     static_cast<cudaStream_t>(stream), pos_stride);
}

int ra_attention_step_fp16(const void* q, const void* k, const void* v, float* out, float* m,
                           float* l, const ra_shape* shape, int q_offset, int k_offset, int causal,
                           ra_stream stream, int pos_stride) {
  RAB_REQUIRE(shape != nullptr, RA_ERR_INVALID, "attention step: null shape");
  // The reference's fp16 entry point has no seq_q == 1 dispatch (src/attention_step_fp16.cu:
  // 256-326 always runs the tiled kernel); one row is simply a short tile here too.
  return step_ex(RA_F16, q, k, v, out, m, l, *shape, affine_posmap(q_offset, shape->seq_q),
                 affine_posmap(k_offset, shape->seq_k), pos_stride > 0 ? pos_stride : 1,
                 causal ? RA_STEP_CAUSAL : 0u, 0, 0, static_cast<cudaStream_t>(stream));
}

int ra_attention_step_segmented(const float* q, const float* k, const float* v, float* out,
                                float* m, float* l, const ra_shape* shape, const ra_segmap* qmap,
                                const ra_segmap* kmap, int causal, ra_stream stream) {
  RAB_REQUIRE(shape && qmap && kmap, RA_ERR_INVALID, "attention step: null argument");
  return step_ex(RA_F32, q, k, v, out, m, l, *shape, make_posmap(*qmap), make_posmap(*kmap), 1,
                 causal ? RA_STEP_CAUSAL : 0u, 0, 0, static_cast<cudaStream_t>(stream));
}

int ra_attention_step_ex(int dtype, const void* q, const void* k, const void* v, float* out,
                         float* m, float* l, const ra_shape* shape, const ra_segmap* qmap,
                         const ra_segmap* kmap, int pos_stride, unsigned flags, long long doc_len,
                         int kv_row_stride, ra_stream stream) {
  RAB_REQUIRE(shape && qmap && kmap, RA_ERR_INVALID, "attention step: null argument");
  RAB_REQUIRE(doc_len >= 0, RA_ERR_INVALID, "attention step: doc_len must be >= 0");
  return step_ex(dtype, q, k, v, out, m, l, *shape, make_posmap(*qmap), make_posmap(*kmap),
                 pos_stride, flags, doc_len, kv_row_stride, static_cast<cudaStream_t>(stream));
}

int ra_attention_step_stacked(int dtype, const void* q, const void* k, const void* v, float* out,
                              float* m, float* l, const ra_shape* shape, const ra_segmap* qmap,
                              const ra_segmap* kmap, const int* seg_shard, const int* seg_row,
                              int n_shards, int shard_rows, int pos_stride, unsigned flags,
                              long long doc_len, ra_stream stream) {
  RAB_REQUIRE(shape && qmap && kmap, RA_ERR_INVALID, "stacked step: null argument");
  RAB_REQUIRE(doc_len >= 0 && pos_stride >= 1, RA_ERR_INVALID,
              "stacked step: doc_len must be >= 0 and pos_stride >= 1");
  RAB_REQUIRE(shape->batch > 0 && shape->heads > 0 && shape->seq_q > 0 && shape->seq_k > 0,
              RA_ERR_INVALID, "stacked step: bad shape");
  RAB_REQUIRE(qmap->n_seg >= 1 && qmap->n_seg <= RA_MAX_SEG && kmap->n_seg >= 1 &&
                  kmap->n_seg <= RA_MAX_SEG,
              RA_ERR_INVALID, "stacked step: segment count out of range");
  return step_stacked(dtype, q, k, v, out, m, l, *shape, make_posmap(*qmap), make_posmap(*kmap),
                      seg_shard, seg_row, n_shards, shard_rows, pos_stride, flags, doc_len,
                      static_cast<cudaStream_t>(stream));
}

RA_API int ra_attention_step_path(int dtype, int head_dim) {
  if (head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256) return -1;
  if (dtype == RA_F16 || dtype == RA_BF16) return 1;
  if (dtype == RA_F32) return head_dim <= 128 ? 2 : 0;
  return -1;
}
RA_API void ra_debug_set_wait_limit_ns(unsigned long long ns) { rab::set_tc_wait_limit_ns(ns); }
RA_API void ra_debug_stall_producer_after(int items) { rab::set_tc_stall_after(items); }
RA_API void ra_debug_set_block_order(int order) { rab::set_tc_block_order(order); }


/* ------------------------------------------------ whole attention, device buffers ---- */

size_t ra_flash_workspace_bytes(const ra_shape* s, int half_precision) {
  if (!s) return 0;
  const size_t rows = static_cast<size_t>(s->batch) * s->heads * s->seq_q;
  size_t bytes = 2 * rows * sizeof(float);  // m, l
  if (half_precision) {
    const int kvH = s->kv_heads > 0 ? s->kv_heads : s->heads;
    const size_t qn = rows * s->head_dim;
    const size_t kn = static_cast<size_t>(s->batch) * kvH * s->seq_k * s->head_dim;
    bytes += (qn + 2 * kn) * 2 + 64;
  }
  return bytes + 256;
}

int ra_flash_attention(const float* q, const float* k, const float* v, float* out,
                       const ra_shape* s, int causal, int half_precision, void* workspace,
                       size_t workspace_bytes, ra_stream stream_) {
  RAB_REQUIRE(q && k && v && out && s && workspace, RA_ERR_INVALID,
              "ra_flash_attention: null argument");
  RAB_REQUIRE(workspace_bytes >= ra_flash_workspace_bytes(s, half_precision), RA_ERR_OVERFLOW,
              "ra_flash_attention: workspace too small");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int kvH = kv_heads_of(*s);
  const size_t rows = static_cast<size_t>(s->batch) * s->heads * s->seq_q;
  uintptr_t p = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~static_cast<uintptr_t>(255);
  float* m = reinterpret_cast<float*>(p);
  float* l = m + rows;
  // end-aligned causal mask: key j visible to query i iff j <= i + (seq_k - seq_q)
  // (src/cpu_attention.cpp:32-34) == global positions q_offset = seq_k - seq_q, k_offset = 0
  const PosMap qmap = affine_posmap(s->seq_k - s->seq_q, s->seq_q);
  const PosMap kmap = affine_posmap(0, s->seq_k);
  const unsigned flags = (causal ? RA_STEP_CAUSAL : 0u) | RA_STEP_FRESH | RA_STEP_FINALIZE;
  if (!half_precision) {
    return step_ex(RA_F32, q, k, v, out, m, l, *s, qmap, kmap, 1, flags, 0, 0, stream);
  }
  const size_t qn = rows * s->head_dim;
  const size_t kn = static_cast<size_t>(s->batch) * kvH * s->seq_k * s->head_dim;
  uintptr_t hp = (reinterpret_cast<uintptr_t>(l + rows) + 15) & ~static_cast<uintptr_t>(15);
  __half* qh = reinterpret_cast<__half*>(hp);
  __half* kh = qh + ((qn + 7) & ~static_cast<size_t>(7));
  __half* vh = kh + ((kn + 7) & ~static_cast<size_t>(7));
  int rc = ra_float_to_half(q, qh, qn, stream_);
  if (rc == RA_OK) rc = ra_float_to_half(k, kh, kn, stream_);
  if (rc == RA_OK) rc = ra_float_to_half(v, vh, kn, stream_);
  if (rc != RA_OK) return rc;
  return step_ex(RA_F16, qh, kh, vh, out, m, l, *s, qmap, kmap, 1, flags, 0, 0, stream);
}

/* --------------------------------------------------- whole attention, host buffers ---- */

int ra_prefill_host(int dtype, const void* q_host, const void* k_host, const void* v_host,
                    float* out_host, float* lse_host, const ra_shape* s, const ra_segmap* qmap,
                    const ra_segmap* kmap, int pos_stride, unsigned flags, long long doc_len) {
  RAB_REQUIRE(q_host && k_host && v_host && out_host && s && qmap && kmap, RA_ERR_INVALID,
              "ra_prefill_host: null argument");
  const int kvH = kv_heads_of(*s);
  const size_t es = elem_size(dtype);
  const size_t rows = static_cast<size_t>(s->batch) * s->heads * s->seq_q;
  const size_t qn = rows * s->head_dim;
  const size_t kn = static_cast<size_t>(s->batch) * kvH * s->seq_k * s->head_dim;
  // Per-thread device buffers that grow on demand and are reused across calls, so a
  // benchmark loop measures copies and kernels, not cudaMalloc.
  constexpr int kHostPipeEvents = 16;
  struct Scratch {
    void* p = nullptr;
    size_t bytes = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr, s_in = nullptr, s_out = nullptr;
    cudaEvent_t e_in[kHostPipeEvents], e_done[kHostPipeEvents];
  };
  // one per device and host thread: streams, events and the buffer always belong to `dev`
  thread_local Scratch scratch_of_device[64];
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  RAB_REQUIRE(dev >= 0 && dev < 64, RA_ERR_INVALID, "device index %d out of range", dev);
  Scratch& sc = scratch_of_device[dev];
  const size_t a256 = 255;
  const size_t need = ((qn * es + a256) & ~a256) + 2 * ((kn * es + a256) & ~a256) +
                      ((qn * 4 + a256) & ~a256) + 3 * ((rows * 4 + a256) & ~a256);
  if (sc.stream == nullptr) {
    RAB_CUDA(cudaStreamCreateWithFlags(&sc.stream, cudaStreamNonBlocking));
    RAB_CUDA(cudaDeviceGetAttribute(&sc.sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  if (sc.bytes < need) {
    if (sc.p) {
      RAB_CUDA(cudaStreamSynchronize(sc.stream));
      RAB_CUDA(cudaFree(sc.p));
    }
    sc.p = nullptr;
    sc.bytes = 0;
    RAB_CUDA(cudaMalloc(&sc.p, need));
    sc.bytes = need;
  }
  unsigned char* base = static_cast<unsigned char*>(sc.p);
  void* dq = base;
  base += (qn * es + a256) & ~a256;
  void* dk = base;
  base += (kn * es + a256) & ~a256;
  void* dv = base;
  base += (kn * es + a256) & ~a256;
  float* dout = reinterpret_cast<float*>(base);
  base += (qn * 4 + a256) & ~a256;
  float* dm = reinterpret_cast<float*>(base);
  base += (rows * 4 + a256) & ~a256;
  float* dl = reinterpret_cast<float*>(base);
  base += (rows * 4 + a256) & ~a256;
  float* dlse = reinterpret_cast<float*>(base);
  cudaStream_t st = sc.stream;
  const unsigned f = (flags & (RA_STEP_CAUSAL | RA_STEP_FORCE_SIMT)) | RA_STEP_FRESH |
                     RA_STEP_FINALIZE;
  const PosMap qm = make_posmap(*qmap), km = make_posmap(*kmap);
  const int stride = pos_stride > 0 ? pos_stride : 1;

  // With one KV head per query head the (batch, head) slices are independent and contiguous,
  // so the pass is pipelined over groups of them: upload of group c+1, kernel of group c and
  // download of group c-1 run on three streams, which hides most of the PCIe time behind
  // the other direction and the kernel. Groups are sized to keep the kernel's grid at about
  // two waves of the SM count (benchmark shape, 100 MB up at 54.8 GB/s = 1.84 ms and 67 MB down
  // = 1.2 ms when each runs alone: 3 / 3 / 2 heads 2.76 ms per pass, 2 heads per group 2.80,
  // 4 heads 3.21, 1 head 3.31 - the two directions share the link, so finer groups only add
  // copies that get in each other's way).
  const int bh_total = s->batch * s->heads;
  int groups = 1, bh_per_group = bh_total;
  if (kvH == s->heads && bh_total >= 2 && s->seq_q > 0) {
    const int qblocks = (s->seq_q + 255) / 256;
    bh_per_group = std::max(1, (2 * sc.sm_count + qblocks - 1) / qblocks);
    groups = (bh_total + bh_per_group - 1) / bh_per_group;
    if (groups > kHostPipeEvents) {
      bh_per_group = (bh_total + kHostPipeEvents - 1) / kHostPipeEvents;
      groups = (bh_total + bh_per_group - 1) / bh_per_group;
    }
  }
  if (groups < 2) {
    RAB_CUDA(cudaMemcpyAsync(dq, q_host, qn * es, cudaMemcpyHostToDevice, st));
    RAB_CUDA(cudaMemcpyAsync(dk, k_host, kn * es, cudaMemcpyHostToDevice, st));
    RAB_CUDA(cudaMemcpyAsync(dv, v_host, kn * es, cudaMemcpyHostToDevice, st));
    int rc = step_ex(dtype, dq, dk, dv, dout, dm, dl, *s, qm, km, stride, f, doc_len, 0, st);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaMemcpyAsync(out_host, dout, qn * 4, cudaMemcpyDeviceToHost, st));
    if (lse_host) {
      rc = ra_attention_lse(dm, dl, dlse, rows, st);
      if (rc != RA_OK) return rc;
      RAB_CUDA(cudaMemcpyAsync(lse_host, dlse, rows * 4, cudaMemcpyDeviceToHost, st));
    }
    rc = enqueue_status_read(st);
    if (rc != RA_OK) return rc;
    RAB_CUDA(cudaStreamSynchronize(st));
    return status_after_sync();
  }
  if (sc.s_in == nullptr) {
    RAB_CUDA(cudaStreamCreateWithFlags(&sc.s_in, cudaStreamNonBlocking));
    RAB_CUDA(cudaStreamCreateWithFlags(&sc.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < kHostPipeEvents; ++i) {
      RAB_CUDA(cudaEventCreateWithFlags(&sc.e_in[i], cudaEventDisableTiming));
      RAB_CUDA(cudaEventCreateWithFlags(&sc.e_done[i], cudaEventDisableTiming));
    }
  }
  const size_t q_head = static_cast<size_t>(s->seq_q) * s->head_dim;  // elements per (b,h)
  const size_t k_head = static_cast<size_t>(s->seq_k) * s->head_dim;
  for (int g = 0; g < groups; ++g) {
    const int bh0 = g * bh_per_group;
    const int nbh = std::min(bh_per_group, bh_total - bh0);
    const size_t qo = bh0 * q_head, ko = bh0 * k_head, ro = static_cast<size_t>(bh0) * s->seq_q;
    unsigned char* gq = static_cast<unsigned char*>(dq) + qo * es;
    unsigned char* gk = static_cast<unsigned char*>(dk) + ko * es;
    unsigned char* gv = static_cast<unsigned char*>(dv) + ko * es;
    RAB_CUDA(cudaMemcpyAsync(gq, static_cast<const unsigned char*>(q_host) + qo * es,
                             nbh * q_head * es, cudaMemcpyHostToDevice, sc.s_in));
    RAB_CUDA(cudaMemcpyAsync(gk, static_cast<const unsigned char*>(k_host) + ko * es,
                             nbh * k_head * es, cudaMemcpyHostToDevice, sc.s_in));
    RAB_CUDA(cudaMemcpyAsync(gv, static_cast<const unsigned char*>(v_host) + ko * es,
                             nbh * k_head * es, cudaMemcpyHostToDevice, sc.s_in));
    RAB_CUDA(cudaEventRecord(sc.e_in[g], sc.s_in));
    RAB_CUDA(cudaStreamWaitEvent(st, sc.e_in[g], 0));
    ra_shape gs{1, nbh, s->seq_q, s->seq_k, s->head_dim, nbh};
    int rc = step_ex(dtype, gq, gk, gv, dout + qo, dm + ro, dl + ro, gs, qm, km, stride, f,
                     doc_len, 0, st);
    if (rc == RA_OK && lse_host)
      rc = ra_attention_lse(dm + ro, dl + ro, dlse + ro, static_cast<size_t>(nbh) * s->seq_q, st);
    if (rc != RA_OK) {
      // leave no copy in flight on the caller's buffers
      cudaStreamSynchronize(sc.s_in);
      cudaStreamSynchronize(st);
      cudaStreamSynchronize(sc.s_out);
      return rc;
    }
    RAB_CUDA(cudaEventRecord(sc.e_done[g], st));
    RAB_CUDA(cudaStreamWaitEvent(sc.s_out, sc.e_done[g], 0));
    RAB_CUDA(cudaMemcpyAsync(out_host + qo, dout + qo, nbh * q_head * 4, cudaMemcpyDeviceToHost,
                             sc.s_out));
    if (lse_host)
      RAB_CUDA(cudaMemcpyAsync(lse_host + ro, dlse + ro, static_cast<size_t>(nbh) * s->seq_q * 4,
                               cudaMemcpyDeviceToHost, sc.s_out));
  }
  const int rc_status = enqueue_status_read(st);
  if (rc_status != RA_OK) return rc_status;
  RAB_CUDA(cudaStreamSynchronize(sc.s_out));
  RAB_CUDA(cudaStreamSynchronize(st));
  return status_after_sync();
}

/* ------------------------------------------------------------------------ KV cache ---- */

int ra_kv_cache_create(int dtype, int batch, int kv_heads, int s_max, int head_dim,
                       ra_kv_cache** out) {
  RAB_REQUIRE(out != nullptr, RA_ERR_INVALID, "ra_kv_cache_create: null argument");
  RAB_REQUIRE(batch > 0 && kv_heads > 0 && s_max > 0 && head_dim > 0, RA_ERR_INVALID,
              "ra_kv_cache_create: bad sizes");
  RAB_REQUIRE(dtype == RA_F32 || dtype == RA_F16 || dtype == RA_BF16, RA_ERR_INVALID,
              "ra_kv_cache_create: unknown dtype %d", dtype);
  ra_kv_cache* c = new ra_kv_cache{dtype, batch, kv_heads, s_max, head_dim, 0, nullptr, nullptr};
  const size_t bytes =
      static_cast<size_t>(batch) * kv_heads * s_max * head_dim * elem_size(dtype);
  if (cudaMalloc(&c->k, bytes) != cudaSuccess || cudaMalloc(&c->v, bytes) != cudaSuccess) {
    set_error("ra_kv_cache_create: cudaMalloc of %zu bytes failed", bytes);
    if (c->k) cudaFree(c->k);
    delete c;
    cudaGetLastError();
    return RA_ERR_CUDA;
  }
  *out = c;
  return RA_OK;
}

void ra_kv_cache_destroy(ra_kv_cache* c) {
  if (!c) return;
  cudaFree(c->k);
  cudaFree(c->v);
  delete c;
}
void* ra_kv_cache_k(ra_kv_cache* c) { return c ? c->k : nullptr; }
void* ra_kv_cache_v(ra_kv_cache* c) { return c ? c->v : nullptr; }
int ra_kv_cache_len(const ra_kv_cache* c) { return c ? c->current_len : 0; }
int ra_kv_cache_s_max(const ra_kv_cache* c) { return c ? c->s_max : 0; }
void ra_kv_cache_reset(ra_kv_cache* c) {
  if (c) c->current_len = 0;
}

// Strided copy of `rows` rows per (batch, kv head) into the cache starting at row `at`
// (reference: cudaMemcpy2DAsync with pitch s_max * D * sizeof(T), src/kv_cache.cu:41-44,60-63).
static int cache_copy(ra_kv_cache* c, const void* k_src, const void* v_src, int rows, int at,
                      cudaStream_t stream) {
  const size_t es = elem_size(c->dtype);
  const size_t width = static_cast<size_t>(rows) * c->head_dim * es;
  const size_t dpitch = static_cast<size_t>(c->s_max) * c->head_dim * es;
  const size_t height = static_cast<size_t>(c->batch) * c->kv_heads;
  const size_t off = static_cast<size_t>(at) * c->head_dim * es;
  if (width == 0) return RA_OK;
  RAB_CUDA(cudaMemcpy2DAsync(static_cast<unsigned char*>(c->k) + off, dpitch, k_src, width, width,
                             height, cudaMemcpyDeviceToDevice, stream));
  RAB_CUDA(cudaMemcpy2DAsync(static_cast<unsigned char*>(c->v) + off, dpitch, v_src, width, width,
                             height, cudaMemcpyDeviceToDevice, stream));
  return RA_OK;
}

int ra_kv_cache_copy_prefill(ra_kv_cache* c, const void* k_src, const void* v_src, int prefill_len,
                             ra_stream stream) {
  RAB_REQUIRE(c && k_src && v_src, RA_ERR_INVALID, "ra_kv_cache_copy_prefill: null argument");
  RAB_REQUIRE(prefill_len >= 0 && prefill_len <= c->s_max, RA_ERR_OVERFLOW,
              "DeviceKVCache::copy_prefill: prefill_len=%d exceeds s_max=%d", prefill_len,
              c->s_max);
  const int rc = cache_copy(c, k_src, v_src, prefill_len, 0, static_cast<cudaStream_t>(stream));
  if (rc == RA_OK) c->current_len = prefill_len;
  return rc;
}

int ra_kv_cache_append(ra_kv_cache* c, const void* k_step, const void* v_step, ra_stream stream) {
  RAB_REQUIRE(c && k_step && v_step, RA_ERR_INVALID, "ra_kv_cache_append: null argument");
  RAB_REQUIRE(c->current_len < c->s_max, RA_ERR_OVERFLOW,
              "DeviceKVCache::append: cache full (current_len=%d, s_max=%d)", c->current_len,
              c->s_max);
  const int rc =
      cache_copy(c, k_step, v_step, 1, c->current_len, static_cast<cudaStream_t>(stream));
  if (rc == RA_OK) c->current_len += 1;
  return rc;
}

/* -------------------------------------------------------------------- local decode ---- */

int ra_local_decode_step(const void* q, const ra_kv_cache* cache, int heads, int q_pos_global,
                         int cache_k_offset, int causal, float* out, ra_stream stream_) {
  RAB_REQUIRE(q && cache && out, RA_ERR_INVALID, "ra_local_decode_step: null argument");
  RAB_REQUIRE(heads > 0 && heads <= 4096, RA_ERR_INVALID, "ra_local_decode_step: bad heads");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  ra_shape s{cache->batch, heads, 1, cache->current_len, cache->head_dim, cache->kv_heads};
  const size_t rows = static_cast<size_t>(cache->batch) * heads;
  // m and l of this one-shot state live in a per-device scratch that is allocated once and
  // grows on demand (not safe for concurrent streams, like the decode workspace itself)
  float* ml = nullptr;
  int rc = decode_ml_scratch(2 * rows, &ml);
  if (rc != RA_OK) return rc;
  // init and the division by l ride on the fold of the split partials: two launches in all
  if (cache->current_len > 0) {
    rc = decode_step(cache->dtype, q, cache->k, cache->v, out, ml, ml + rows, s, q_pos_global,
                     cache_k_offset, causal, stream, cache->s_max, nullptr, 0,
                     RA_STEP_FRESH | RA_STEP_FINALIZE);
  } else {
    rc = launch_init(out, ml, ml + rows, rows * cache->head_dim, rows, stream);
  }
  return rc;
}

/* ----------------------------------------------------------------------- partition ---- */

int ra_partition_k_offset_for_source(int cp, int rank, int seq, int mode, int n_splits, int source,
                                     int sg) {
  (void)rank;
  if (mode == 0) return source * (seq / cp);
  if (mode == 2) return source;
  const int chunk = seq / (n_splits * cp);
  const int pass = sg / 2;
  return (sg % 2 == 0) ? (pass * cp + source) * chunk
                       : ((n_splits - 1 - pass) * cp + (cp - 1 - source)) * chunk;
}
int ra_partition_q_offset(int cp, int rank, int seq, int mode, int n_splits, int sg) {
  return ra_partition_k_offset_for_source(cp, rank, seq, mode, n_splits, rank, sg);
}
int ra_partition_k_offset_for_step(int cp, int rank, int seq, int mode, int n_splits, int step,
                                   int sg) {
  const int source = (rank - step % cp + cp) % cp;
  return ra_partition_k_offset_for_source(cp, rank, seq, mode, n_splits, source, sg);
}
int ra_partition_local_chunk_len(int cp, int seq, int mode, int n_splits) {
  return mode == 1 ? seq / (n_splits * cp) : seq / cp;
}
int ra_partition_num_sub_groups(int mode, int n_splits) { return mode == 1 ? n_splits : 1; }
int ra_partition_position_stride(int cp, int mode) { return mode == 2 ? cp : 1; }
int ra_partition_next_rank(int cp, int rank) { return (rank + 1) % cp; }
int ra_partition_prev_rank(int cp, int rank) { return (rank - 1 + cp) % cp; }

int ra_ring2d_source(int num_nodes, int gpus_per_node, int node, int local, int m, int i) {
  if (num_nodes <= 0 || gpus_per_node <= 0 || node < 0 || node >= num_nodes || local < 0 ||
      local >= gpus_per_node || m < 0 || m >= num_nodes || i < 0 || i >= gpus_per_node)
    return -1;
  // a node's band of shards moves on one node per macro-step; inside a macro-step the shards
  // of the band move on one local index per inner round
  const int band = (node + num_nodes - m) % num_nodes;
  const int slot = (local + gpus_per_node - i) % gpus_per_node;
  return band * gpus_per_node + slot;
}

int ra_ring_step_maps(int cp, int rank, int seq, int mode, int n_splits, int step,
                      ra_segmap* qmap, ra_segmap* kmap) {
  if (!qmap || !kmap || cp <= 0 || rank < 0 || rank >= cp) return -1;
  const int nsg = ra_partition_num_sub_groups(mode, n_splits);
  if (nsg > RA_MAX_SEG) return -1;
  const int len = ra_partition_local_chunk_len(cp, seq, mode, n_splits);
  std::memset(qmap, 0, sizeof(*qmap));
  std::memset(kmap, 0, sizeof(*kmap));
  qmap->n_seg = kmap->n_seg = nsg;
  qmap->seg_len = kmap->seg_len = len;
  for (int sg = 0; sg < nsg; ++sg) {
    qmap->base[sg] = ra_partition_q_offset(cp, rank, seq, mode, n_splits, sg);
    kmap->base[sg] = ra_partition_k_offset_for_step(cp, rank, seq, mode, n_splits, step, sg);
  }
  return ra_partition_position_stride(cp, mode);
}

int ra_ring_gather_part_maps(int cp, int rank, int seq, int mode, int n_splits, int parts,
                             int part, ra_segmap* kmap, int* seg_shard, int* seg_row) {
  if (!kmap || !seg_shard || !seg_row || cp <= 1 || rank < 0 || rank >= cp || parts < 1 ||
      part < 0 || part >= parts)
    return -1;
  const int nsg = ra_partition_num_sub_groups(mode, n_splits);
  if (nsg < 1 || nsg > RA_MAX_SEG) return -1;
  const int entries = (cp - 1) * nsg;
  std::memset(kmap, 0, sizeof(*kmap));
  kmap->seg_len = ra_partition_local_chunk_len(cp, seq, mode, n_splits);
  for (int e = part; e < entries; e += parts) {
    if (kmap->n_seg >= RA_MAX_SEG) return -1;
    const int s = 1 + e / nsg, i = e % nsg;
    const int owner = (rank - s + cp) % cp;  // the shard s hops away
    kmap->base[kmap->n_seg] = ra_partition_k_offset_for_source(cp, rank, seq, mode, n_splits, owner, i);
    seg_shard[kmap->n_seg] = owner;
    seg_row[kmap->n_seg] = i * kmap->seg_len;
    ++kmap->n_seg;
  }
  return ra_partition_position_stride(cp, mode);
}

double ra_ring_step_visible_pairs(const ra_segmap* qmap, const ra_segmap* kmap, int stride,
                                  int causal, long long doc_len) {
  if (!qmap || !kmap) return 0.0;
  // Exact count by walking query rows of each segment pair in closed form per row would be
  // O(rows); segments are affine, so count per (q segment, k segment) with arithmetic series.
  double total = 0.0;
  for (int a = 0; a < qmap->n_seg; ++a)
    for (int b = 0; b < kmap->n_seg; ++b) {
      const long long qb = qmap->base[a], kb = kmap->base[b];
      const long long Lq = qmap->seg_len, Lk = kmap->seg_len;
      if (!causal && doc_len <= 0) {
        total += static_cast<double>(Lq) * static_cast<double>(Lk);
        continue;
      }
      // Row i sees keys j in [lo_i, hi_i]. Walk rows in runs where the document is constant;
      // inside a run hi_i is affine in i and clamps at both ends, so sum with at most three
      // pieces. For clarity (segment counts are tiny, rows up to ~1e6) use a direct loop with
      // O(1) work per row.
      for (long long i = 0; i < Lq; ++i) {
        const long long qp = qb + i * stride;
        long long lo = 0, hi = Lk - 1;
        if (causal) {
          if (qp < kb) continue;
          hi = std::min(hi, (qp - kb) / stride);
        }
        if (doc_len > 0) {
          const long long p_lo = (qp / doc_len) * doc_len, p_hi = p_lo + doc_len - 1;
          if (p_hi < kb) continue;
          hi = std::min(hi, (p_hi - kb) / stride);
          if (p_lo > kb) lo = (p_lo - kb + stride - 1) / stride;
        }
        if (hi >= lo) total += static_cast<double>(hi - lo + 1);
      }
    }
  return total;
}

}  // extern "C"
