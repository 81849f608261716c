/*
 * ring_attention_b200 — C ABI of the B200 (sm_100a) ring-attention hot path.
 *
 * Every entry point is a plain-C function over raw device (or, where the name
 * says `_host`, host) pointers, sizes and an explicit CUDA stream handle. There
 * are no C++ or torch types in any signature, so the library can be bound from
 * C, C++, ctypes, cgo or JNI alike. Each declaration cites the interface of the
 * reference implementation (h1ppox99/ring-attention, paths relative to that
 * project) that it replaces.
 *
 * Conventions
 *  - Tensors are row-major (batch, heads, seq, head_dim), contiguous
 *    (src/attention.hpp:6). K/V carry `kv_heads` heads; query head h reads KV
 *    head h % kv_heads (src/cpu_attention.cpp:41-42).
 *  - All launches are asynchronous on `stream` (NULL = the default stream) and
 *    never synchronise (src/attention.hpp:7-9).
 *  - Functions return 0 (RA_OK) or a non-zero ra_status; ra_last_error() gives a
 *    thread-local message. The reference aborts the process instead
 *    (src/common.cuh:16-24); the C++ shim turns a non-zero status back into that.
 *  - The online-softmax state (out unnormalised fp32, m, l) has the reference's
 *    semantics (src/attention_step.cu:71-77): out = sum_j exp(s_j - m) v_j,
 *    l = sum_j exp(s_j - m), s_j = q.k_j / sqrt(head_dim) in natural-log units;
 *    a row that has seen no visible key keeps m = -inf, l = 0, out = 0.
 */
#ifndef RING_ATTENTION_B200_H_
#define RING_ATTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RA_API __attribute__((visibility("default")))

typedef enum ra_status {
  RA_OK = 0,
  RA_ERR_INVALID = 1,      /* bad argument / unsupported combination of flags */
  RA_ERR_CUDA = 2,         /* a CUDA runtime or driver call failed */
  RA_ERR_UNSUPPORTED = 3,  /* e.g. head_dim outside {32, 64, 128, 256} */
  RA_ERR_NCCL = 4,
  RA_ERR_DEVICE_WAIT = 5,  /* a bounded device-side wait ran out (see ra_device_status) */
  RA_ERR_OVERFLOW = 6      /* KV cache full / workspace too small */
} ra_status;

/* Element types of Q/K/V buffers. */
typedef enum ra_dtype { RA_F32 = 0, RA_F16 = 1, RA_BF16 = 2 } ra_dtype;

/* Problem shape of one attention call: mirrors AttentionShape (src/attention.hpp:19-26);
 * kv_heads == 0 means kv_heads = heads. */
typedef struct ra_shape {
  int batch;
  int heads;
  int seq_q;
  int seq_k;
  int head_dim;
  int kv_heads;
} ra_shape;

/* Piecewise-affine position map: mirrors SegMap (src/attention.hpp:102-107). Local
 * row i sits at global position base[i / seg_len] + (i % seg_len) * pos_stride. */
#define RA_MAX_SEG 16
typedef struct ra_segmap {
  int n_seg;
  int seg_len;
  int base[RA_MAX_SEG];
} ra_segmap;

typedef void* ra_stream; /* a cudaStream_t */

RA_API const char* ra_last_error(void);
RA_API int ra_version(void);

/* Reads and clears the device-side status word of the current device. Kernels with
 * bounded waits (mbarrier spins) record a non-zero code there instead of hanging:
 * out[0] = code (0 = none), out[1] = which wait, out[2] = block index, out[3] = tile.
 * Synchronises the device. No counterpart in the reference (its kernels have no waits). */
RA_API int ra_device_status(int out[4]);

/* Test hooks for the bounded waits; no counterpart in the reference. The limit of every
 * device-side wait of the tcgen05 step kernel (default 2 s; 0 restores the default), and a
 * switch that makes that kernel's TMA producer stop after `items` K/V tiles (negative = off),
 * so that a test can watch a wait run out: the kernel returns, ra_device_status reports
 * RA_ERR_DEVICE_WAIT, nothing is accessed out of bounds. Process-wide; not for production use. */
RA_API void ra_debug_set_wait_limit_ns(unsigned long long ns);
RA_API void ra_debug_stall_producer_after(int items);
/* Block order of the tcgen05 step kernel: -1 = chosen by shape (default), 0 = (batch, head)
 * fastest, k > 0 = waves of k KV heads (all query blocks of their query heads before the next
 * k; ignored unless k divides batch * kv_heads). Lets a test run every order on a small shape.
 * Process-wide; not for production use. */
RA_API void ra_debug_set_block_order(int order);

/* ------------------------------------------------------------------ prefill ---- */

/* out = 0, l = 0, m = -inf. Replaces launch_attention_init (src/attention.hpp:73,
 * src/attention_step.cu:478-486). */
RA_API int ra_attention_init(float* out, float* m, float* l, const ra_shape* shape,
                             size_t m_count, ra_stream stream);

/* One ring step, fp32 Q/K/V. Replaces launch_attention_step (src/attention.hpp:92-94,
 * src/attention_step.cu:488-525). Head_dim 32, 64 and 128 run on the tensor cores with every
 * operand split into two TF32 terms (about 2^-22 per product, inside the reference's fp32
 * tolerance of 1e-5 for its test and benchmark inputs; RA_STEP_FORCE_SIMT of
 * ra_attention_step_ex selects plain fp32), 256 on the SIMT kernel; seq_q == 1 dispatches to the decode kernel exactly as
 * the reference does (src/attention_step.cu:494-497). */
RA_API int ra_attention_step(const float* q, const float* k, const float* v, float* out, float* m,
                             float* l, const ra_shape* shape, int q_offset, int k_offset,
                             int causal, ra_stream stream, int pos_stride);

/* One ring step, fp16 Q/K/V, fp32 state. Replaces launch_attention_step_fp16
 * (src/attention.hpp:147-150, src/attention_step_fp16.cu:256-326). Runs the tcgen05 kernel
 * for head_dim 32, 64, 128 and 256 (32 on the 64-wide kernel, the loads zero-filling the upper
 * half of every row; 256 with one query tile per block). */
RA_API int ra_attention_step_fp16(const void* q, const void* k, const void* v, float* out,
                                  float* m, float* l, const ra_shape* shape, int q_offset,
                                  int k_offset, int causal, ra_stream stream, int pos_stride);

/* Single-launch segmented step, fp32. Replaces launch_attention_step_segmented
 * (src/attention.hpp:115-119, src/attention_step.cu:527-554). */
RA_API int ra_attention_step_segmented(const float* q, const float* k, const float* v, float* out,
                                       float* m, float* l, const ra_shape* shape,
                                       const ra_segmap* qmap, const ra_segmap* kmap, int causal,
                                       ra_stream stream);

/* Flags of ra_attention_step_ex. */
#define RA_STEP_CAUSAL 1u    /* visible iff k_pos <= q_pos */
#define RA_STEP_FRESH 2u     /* the state is known to be empty: overwrite, do not read it */
#define RA_STEP_FINALIZE 4u  /* after folding this step, divide out by l (as ra_attention_finalize) */
#define RA_STEP_FORCE_SIMT 8u /* run the SIMT kernel whatever the head_dim (cross-checks) */
#define RA_STEP_P_IN_SMEM 16u /* tcgen05 kernel: stage P through shared memory instead of tensor
                               * memory (the second, cross-checking form of the same kernel) */
#define RA_STEP_CTA_PAIR 32u /* tcgen05 kernel, head_dim 128 / 256 with P in tensor memory: cluster
                              * pairs with M = 256 MMAs (cta_group::2), each block holding half of
                              * every K / V tile; the third, cross-checking form of the kernel */

/* The general step every other step entry point funnels into: any dtype, segmented
 * positions with a stride, optional document mask (visible only if
 * q_pos / doc_len == k_pos / doc_len; 0 = off), optional strided K/V rows
 * (kv_row_stride = rows between consecutive KV heads; 0 = seq_k). One launch covers a
 * whole zig-zag shard, replacing the n_seg^2 launches per ring step of
 * src/ring_loop_fp16.cu:642-655, with fully masked tiles skipped. The document mask and
 * bf16 are additions the reference does not have. */
RA_API int ra_attention_step_ex(int dtype, const void* q, const void* k, const void* v, float* out,
                                float* m, float* l, const ra_shape* shape, const ra_segmap* qmap,
                                const ra_segmap* kmap, int pos_stride, unsigned flags,
                                long long doc_len, int kv_row_stride, ra_stream stream);

/* Which kernel the step entry points run for a dtype and head_dim (given 16-byte aligned
 * tensors): 1 = the tcgen05 / TMA / tensor-memory kernel (fp16 and bf16, head_dim 32, 64, 128,
 * 256), 2 = the same on split TF32 operands (fp32, head_dim 32, 64, 128), 0 = the SIMT fp32
 * kernel (fp32 head_dim 256, or any shape with RA_STEP_FORCE_SIMT), -1 = unsupported. Host only. The reference dispatches on
 * head_dim alone (src/attention_step_fp16.cu:275-292). */
RA_API int ra_attention_step_path(int dtype, int head_dim);

/* The general step over key segments that sit in n_shards stacked shards instead of one tensor:
 * k / v point at shard 0, every shard is (batch * kv_heads, shard_rows, head_dim) and shard s
 * starts s * batch * kv_heads * shard_rows * head_dim elements later (the receive buffer of an
 * all-gather of per-rank shards). Key segment i of kmap is rows seg_row[i] .. seg_row[i] +
 * seg_len of shard seg_shard[i]; shape->seq_k = kmap->n_seg * kmap->seg_len. 16-bit dtypes and
 * head_dim 32 / 64 / 128 only (RA_ERR_INVALID otherwise). One launch then folds the shards of
 * several ring steps; the reference has no counterpart (its all-gather mode copies the shards
 * into one tensor first, src/ring_loop.cu:273-420). */
RA_API int ra_attention_step_stacked(int dtype, const void* q, const void* k, const void* v,
                                     float* out, float* m, float* l, const ra_shape* shape,
                                     const ra_segmap* qmap, const ra_segmap* kmap,
                                     const int* seg_shard, const int* seg_row, int n_shards,
                                     int shard_rows, int pos_stride, unsigned flags,
                                     long long doc_len, ra_stream stream);

/* out_i *= 1 / l_i (0 where l_i <= 0). Replaces launch_attention_finalize
 * (src/attention.hpp:136, src/attention_step.cu:556-562). */
RA_API int ra_attention_finalize(float* out, const float* l, const ra_shape* shape,
                                 ra_stream stream);

/* lse_i = m_i + log(l_i) (-inf where l_i <= 0). The reference computes this quantity
 * inside cpu_attention and discards it (src/cpu_attention.cpp:50-66). */
RA_API int ra_attention_lse(const float* m, const float* l, float* lse, size_t count,
                            ra_stream stream);

/* Element-wise casts. Replace launch_float_to_half / launch_half_to_float /
 * launch_float_to_int8 / launch_int8_to_float (src/attention.hpp:154-166,
 * src/attention_step_fp16.cu:217-254; int8 uses the fixed scale 127 with clamping). */
RA_API int ra_float_to_half(const float* src, void* dst, size_t n, ra_stream stream);
RA_API int ra_half_to_float(const void* src, float* dst, size_t n, ra_stream stream);
RA_API int ra_float_to_bf16(const float* src, void* dst, size_t n, ra_stream stream);
RA_API int ra_float_to_int8(const float* src, signed char* dst, size_t n, ra_stream stream);
RA_API int ra_int8_to_float(const signed char* src, float* dst, size_t n, ra_stream stream);

/* Whole single-GPU attention, fp32 in and out, end-aligned causal mask
 * (j <= i + seq_k - seq_q). Replaces launch_flash_attention and launch_flash_attention_fp16
 * (src/attention.hpp:48-65). `workspace` must hold
 * ra_flash_workspace_bytes(shape, half_precision) bytes of device memory. */
RA_API size_t ra_flash_workspace_bytes(const ra_shape* shape, int half_precision);
RA_API int ra_flash_attention(const float* q, const float* k, const float* v, float* out,
                              const ra_shape* shape, int causal, int half_precision,
                              void* workspace, size_t workspace_bytes, ra_stream stream);

/* Whole single-GPU attention for ANY head_dim (1..1024), fp32 end to end, same mask as
 * ra_flash_attention. Replaces launch_naive_attention (src/attention.hpp:42-46,
 * src/naive_attention.cu), the reference's correctness baseline, which its tests call with
 * head sizes the tiled kernels do not take (16, 24). Not a fast path. */
RA_API int ra_naive_attention(const float* q, const float* k, const float* v, float* out,
                              const ra_shape* shape, int causal, ra_stream stream);

/* Whole attention on HOST buffers (pinned or pageable), fp16/bf16/fp32 Q/K/V in, fp32 out:
 * uploads, runs init + step + finalize on the current device, downloads and
 * synchronises. This is the host-buffer form of what run_ring_attention does at
 * cp_size = 1 (src/ring_loop_fp16.cu:522-818: upload, init, steps, finalize). Positions
 * are given by the segment maps (one segment of seq rows at base 0 = plain causal).
 * `lse_host` may be NULL. */
RA_API int ra_prefill_host(int dtype, const void* q_host, const void* k_host, const void* v_host,
                           float* out_host, float* lse_host, const ra_shape* shape,
                           const ra_segmap* qmap, const ra_segmap* kmap, int pos_stride,
                           unsigned flags, long long doc_len);

/* ------------------------------------------------------------------- decode ---- */

/* Split-K decode step (seq_q == 1) folding seq_k cached rows into the persistent state.
 * Replaces launch_attention_decode_step (src/attention.hpp:128-131,
 * src/attention_decode.cu:279-347). `dtype` is the type of q, k and v (the reference is
 * fp32 only). The causal cut-off is q_offset - k_offset + 1 rows
 * (src/attention_decode.cu:110-116). Partials go through `workspace`
 * (ra_decode_workspace_bytes bytes); NULL uses a per-device buffer the library grows on
 * demand, like the reference's process-static workspace (src/attention_decode.cu:55-65). */
RA_API size_t ra_decode_workspace_bytes(const ra_shape* shape);
RA_API int ra_attention_decode_step(int dtype, const void* q, const void* k, const void* v,
                                    float* out, float* m, float* l, const ra_shape* shape,
                                    int q_offset, int k_offset, int causal, ra_stream stream,
                                    int kv_row_stride, void* workspace, size_t workspace_bytes);

/* The same decode step for callers that cannot allocate device memory: processes that gave
 * all of it to their own arena, callers inside a section where the CUDA allocator must not
 * be entered, embedders that forbid hidden allocations. It has no counterpart in the
 * reference. The split partials go to a 1 MiB array built into the library image (each GPU
 * that loads the library holds it until exit); the call makes no cudaMalloc / cudaFree or
 * any other allocating call. Limit: batch * heads * (head_dim + 2) floats must fit the array
 * (262144 floats); larger problems are refused with RA_ERR_OVERFLOW and a message naming the
 * limit, and fewer splits are used when the usual split count would not fit. The first call
 * on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current), so make that first call outside any stream capture. All calls on a device share
 * the one array: two calls whose kernels may overlap on the GPU (different streams) race;
 * serialise them. The array keeps the previous call's contents, which is harmless because
 * each call writes every slot before reading it. Arguments as ra_attention_decode_step. */
RA_API int ra_attention_decode_step_noalloc(int dtype, const void* q, const void* k,
                                            const void* v, float* out, float* m, float* l,
                                            const ra_shape* shape, int q_offset, int k_offset,
                                            int causal, ra_stream stream, int kv_row_stride);

/* Merge cp_size rank partials laid out as cp_size blocks [O (BH*D) | m (BH) | l (BH)]
 * into (out, m_out, l_out); with normalise != 0 also divides out by l. Replaces
 * decode_partial_merge_kernel (+ the finalize after it) (src/ring_decode.cu:50-81,192-203). */
RA_API int ra_decode_partial_merge(const float* gathered, float* out, float* m_out, float* l_out,
                                   int cp_size, int bh, int head_dim, int normalise,
                                   ra_stream stream);

/* KV cache (batch, kv_heads, s_max, head_dim) for K and V. Replaces DeviceKVCache<T>
 * (src/kv_cache.hpp:22-73, src/kv_cache.cu:20-68); dtype RA_F32 or RA_F16/RA_BF16. */
typedef struct ra_kv_cache ra_kv_cache;
RA_API int ra_kv_cache_create(int dtype, int batch, int kv_heads, int s_max, int head_dim,
                              ra_kv_cache** out);
RA_API void ra_kv_cache_destroy(ra_kv_cache* c);
RA_API void* ra_kv_cache_k(ra_kv_cache* c);
RA_API void* ra_kv_cache_v(ra_kv_cache* c);
RA_API int ra_kv_cache_len(const ra_kv_cache* c);
RA_API int ra_kv_cache_s_max(const ra_kv_cache* c);
RA_API int ra_kv_cache_copy_prefill(ra_kv_cache* c, const void* k_src, const void* v_src,
                                    int prefill_len, ra_stream stream);
RA_API int ra_kv_cache_append(ra_kv_cache* c, const void* k_step, const void* v_step,
                              ra_stream stream);
RA_API void ra_kv_cache_reset(ra_kv_cache* c);

/* Decode one token against the local cache: init + decode step (in place, no repack) +
 * finalize. Replaces run_local_decode_step / run_local_decode_step_fp16
 * (src/decode_op.hpp:34-42, src/decode_op.cu:44-90). q has the cache's dtype. */
RA_API int ra_local_decode_step(const void* q, const ra_kv_cache* cache, int heads,
                                int q_pos_global, int cache_k_offset, int causal, float* out,
                                ra_stream stream);

/* ---------------------------------------------------------------- partition ---- */

/* Index maps of RingPartition (src/ring_partition.hpp:11-75, src/ring_partition.cpp:41-108).
 * mode: 0 contiguous, 1 zig-zag (n_splits sub-groups), 2 striped. Pure integer host code. */
RA_API int ra_partition_q_offset(int cp_size, int rank, int seq, int mode, int n_splits, int sg);
RA_API int ra_partition_k_offset_for_step(int cp_size, int rank, int seq, int mode, int n_splits,
                                          int step, int sg);
RA_API int ra_partition_k_offset_for_source(int cp_size, int rank, int seq, int mode, int n_splits,
                                            int source_rank, int sg);
RA_API int ra_partition_local_chunk_len(int cp_size, int seq, int mode, int n_splits);
RA_API int ra_partition_num_sub_groups(int mode, int n_splits);
RA_API int ra_partition_position_stride(int cp_size, int mode);
RA_API int ra_partition_next_rank(int cp_size, int rank);
RA_API int ra_partition_prev_rank(int cp_size, int rank);

/* Hierarchical (2-D) ring visitation order: the global rank whose shard GPU (node, local) of a
 * num_nodes x gpus_per_node cluster holds at macro-step m (0..num_nodes-1), inner round i
 * (0..gpus_per_node-1); global rank = node * gpus_per_node + local. Replaces
 * Ring2DSchedule::source (src/ring2d_schedule.hpp:42-44, src/ring2d_schedule.cpp:30-42).
 * Pure integer arithmetic, host only; -1 on arguments out of range. */
RA_API int ra_ring2d_source(int num_nodes, int gpus_per_node, int node, int local, int m, int i);

/* Fills the segment maps a rank uses at one ring step: qmap = its own sub-groups, kmap =
 * the sub-groups of the shard it holds at `step` (source (rank - step) mod cp_size,
 * src/ring_partition.cpp:64-68). Returns the position stride. Host only. */
RA_API int ra_ring_step_maps(int cp_size, int rank, int seq, int mode, int n_splits, int step,
                             ra_segmap* qmap, ra_segmap* kmap);

/* Gather schedule, host only: the key segments of the other cp_size - 1 ranks' shards that part
 * `part` of `parts` folds for `rank` (entry e = (s - 1) * n_sub_groups + i is sub-group i of the
 * shard s hops away; part z takes e = z, z + parts, ...). Fills kmap (one base per segment) and,
 * per segment, the owning rank (= shard index in the gathered buffer) and the first row inside
 * that shard. Returns the position stride, or -1 on bad arguments or more than RA_MAX_SEG
 * segments. Over all parts, plus the rank's own shard, every key of the sequence appears once. */
RA_API int ra_ring_gather_part_maps(int cp_size, int rank, int seq, int mode, int n_splits,
                                    int parts, int part, ra_segmap* kmap, int* seg_shard,
                                    int* seg_row);

/* Causal-adjusted work of one rank at one ring step, in (query, key) pairs that are
 * visible (the FLOP model of apps/bench_attention/bench_attention.cu:46-51 is
 * 4 * head_dim * heads * batch * pairs). Host only; exact, O(n_seg^2). */
RA_API double ra_ring_step_visible_pairs(const ra_segmap* qmap, const ra_segmap* kmap,
                                         int pos_stride, int causal, long long doc_len);

/* --------------------------------------------------------------------- ring ---- */

/* A ring of cp_size ranks, one process (or thread) per GPU, over NCCL. The communicator
 * is made once and reused; the reference makes one per run (src/nccl_utils.hpp:30-37,
 * src/ring_loop_fp16.cu:587). ra_nccl_unique_id fills 128 bytes on rank 0 which the caller
 * broadcasts by its own means (MPI_Bcast in the reference). */
typedef struct ra_ring ra_ring;
RA_API int ra_nccl_unique_id(char id[128]);
RA_API int ra_ring_create(int rank, int cp_size, const char id[128], ra_ring** out);
RA_API int ra_ring_create_from_comm(int rank, int cp_size, void* nccl_comm, ra_ring** out);
RA_API void ra_ring_destroy(ra_ring* r);

/* Mirrors RingConfig (src/ring_loop.hpp:38-62) for the ring-overlap mode. */
typedef struct ra_ring_config {
  int batch, heads, kv_heads, seq, head_dim; /* seq = GLOBAL sequence length */
  int dtype;                                 /* RA_F16 / RA_BF16 */
  int causal;
  int layout;    /* 0 contiguous, 1 zig-zag, 2 striped */
  int n_splits;  /* zig-zag sub-groups per rank (2 * zigzag_n) */
  long long doc_len; /* 0 = no document mask */
  int schedule;      /* RA_SCHEDULE_*; 0 (auto) picks by shard size */
  int ring2d_nodes;  /* RA_SCHEDULE_RING2D: number of rank groups N (cp_size = N * G); else unused */
} ra_ring_config;

/* How the K/V shards reach every rank. RING is the reference's overlapped hop-by-hop rotation
 * (RingMode::RingOverlap, src/ring_loop.hpp:16); GATHER is one all-gather overlapped with the
 * step on the rank's own shard, then the remaining steps back to back (what the reference's
 * RingMode::AllGather does, src/ring_loop.cu:273-420, but still one masked step per source
 * shard). AUTO takes GATHER while a shard tensor is at most 32 MiB, where a hop's latency
 * cannot hide under a step, and RING above. Results are identical. */
enum {
  RA_SCHEDULE_AUTO = 0,
  RA_SCHEDULE_RING = 1,
  RA_SCHEDULE_GATHER = 2,
  /* RingMode::RingBlocking (src/ring_loop.cu:259-592): the rotation with nothing overlapped,
   * every exchange on the compute stream behind its step. The baseline the overlap is measured
   * against. */
  RA_SCHEDULE_BLOCKING = 3,
  /* RingMode::Ring2D (src/ring_loop.cu:1071-1550) in the visitation order of Ring2DSchedule
   * (src/ring2d_schedule.cpp:28-42): ring2d_nodes groups of ranks; the outer exchange of a
   * macro-step runs on the side stream under the inner ring's steps. On one NVSwitch box all
   * links are alike, so this is for comparison and for parity with the reference's CLI. */
  RA_SCHEDULE_RING2D = 4
};

/* Mirrors RingResult (src/ring_loop.hpp:30-36); times of this rank, milliseconds. */
typedef struct ra_ring_result {
  double comm_ms, comp_ms, wait_ms, total_ms;
} ra_ring_result;

/* One overlapped ring pass over device shards: q (B,H,Sloc,D), k/v (B,kvH,Sloc,D) in
 * the rank's local order (sub-groups concatenated along seq), out fp32 (B,H,Sloc,D)
 * normalised, lse (B,H,Sloc) or NULL. K/V rotate rank -> rank+1 on a side stream,
 * double-buffered, while the step kernel runs (src/ring_loop_fp16.cu:638-708).
 * `kv_work` must hold ra_ring_prefill_workspace_bytes bytes. Returns after enqueueing
 * unless `result` is non-NULL, in which case it synchronises, fills the timings and returns
 * RA_ERR_DEVICE_WAIT if a bounded device-side wait ran out. Callers that do not synchronise
 * here poll ra_device_status themselves. */
RA_API size_t ra_ring_prefill_workspace_bytes(const ra_ring* r, const ra_ring_config* cfg);
RA_API int ra_ring_prefill(ra_ring* r, const ra_ring_config* cfg, const void* q, const void* k,
                           const void* v, float* out, float* lse, void* kv_work,
                           size_t kv_work_bytes, ra_stream stream, ra_ring_result* result);

/* What ra_ring_prefill will do for cfg on this rank: the schedule taken (RA_SCHEDULE_RING or
 * _GATHER), the number of key parts the gather schedule folds side by side (1 otherwise), and
 * how many kernels of this library one pass launches (step kernels plus the merge of partial
 * states). Host only. The reference prints its mode per run (apps/ring_attention_cli/main.cu:371-377). */
RA_API int ra_ring_prefill_plan(const ra_ring* r, const ra_ring_config* cfg, int* schedule,
                                int* key_parts, int* launches);

/* The same pass from HOST buffers holding this rank's shards (pinned memory recommended): K and
 * V are uploaded first so that the pass's transfers start while Q is still on its way, the
 * output (and lse, if not NULL) comes back to the host, and the call returns after everything
 * has completed. With one KV head per query head, batch 1 and at least 16 MB of Q, K, V per rank
 * the pass runs as two half passes over head groups instead, so that the second half's upload
 * and the first half's download overlap a pass (every rank takes the same decision from cfg).
 * Device staging lives in the ring handle and grows on demand. The reference
 * uploads inside its timed pass too (src/ring_loop_fp16.cu:624-626). `result`, if not NULL,
 * gets total_ms = upload + pass + download, comp_ms = the pass alone, wait_ms = the rest.
 * Returns RA_ERR_DEVICE_WAIT when a bounded device-side wait ran out during the pass. */
RA_API int ra_ring_prefill_host(ra_ring* r, const ra_ring_config* cfg, const void* q_host,
                                const void* k_host, const void* v_host, float* out_host,
                                float* lse_host, ra_ring_result* result);

/* One multi-rank decode step. Replaces run_ring_decode_step (src/ring_decode.hpp:67-69,
 * src/ring_decode.cu:85-226): owner appends, every rank folds its local shard, partials
 * are all-gathered and merged, every rank ends with the same normalised out (B,H,1,D). */
RA_API int ra_ring_decode_step(ra_ring* r, int batch, int heads, const void* q, const void* k_new,
                               const void* v_new, int owner_rank, ra_kv_cache* cache,
                               const int* current_len_per_rank, float* out, ra_stream stream,
                               ra_ring_result* result);

/* The same step on raw cache pointers (K, V of shape (batch, kv_heads, s_max, head_dim), the
 * first local_len rows of every head valid), for callers that own the cache themselves, such
 * as the reference's DeviceKVCache<T> (src/kv_cache.hpp:22-73); the append on the owner rank
 * is then the caller's (src/ring_decode.cu:116-118). */
RA_API int ra_ring_decode_step_raw(ra_ring* r, int dtype, int batch, int heads, int kv_heads,
                                   int head_dim, const void* q, const void* k_cache,
                                   const void* v_cache, int local_len, int s_max, float* out,
                                   ra_stream stream, ra_ring_result* result);

#ifdef __cplusplus
}
#endif
#endif /* RING_ATTENTION_B200_H_ */
