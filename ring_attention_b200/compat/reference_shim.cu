// C++ shim: the reference project's own headers (namespace ring_attention, included from
// the reference tree, never copied here) implemented on top of the C ABI of
// libring_attention_b200.so. With this one file in place of the reference's kernel and
// container translation units, the reference's own test programs build unchanged and run
// against the B200 kernels. Errors keep the reference's behaviour: message on stderr, abort
// (src/common.cuh:16-24).
//
// Build: see oracle/Makefile (target reftests); needs the reference tree for its headers.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <utility>
#include <vector>

#include "attention.hpp"
#include "decode_op.hpp"
#include "device_tensor.hpp"
#include "kv_cache.hpp"
#include "ring2d_schedule.hpp"
#include "ring_partition.hpp"

#include "../../include/ring_attention_b200.h"

namespace ring_attention {

namespace {

[[noreturn]] void die(const char* what) {
  std::fprintf(stderr, "%s: %s\n", what, ra_last_error());
  std::abort();
}
void must(int rc, const char* what) {
  if (rc != RA_OK) die(what);
}
void cuda_must(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "CUDA error %s in %s\n", cudaGetErrorString(e), what);
    std::abort();
  }
}
ra_shape to_c(const AttentionShape& s) {
  ra_shape c;
  c.batch = s.batch;
  c.heads = s.heads;
  c.seq_q = s.seq_q;
  c.seq_k = s.seq_k;
  c.head_dim = s.head_dim;
  c.kv_heads = s.kv_heads;
  return c;
}
ra_segmap to_c(const SegMap& m) {
  ra_segmap c;
  c.n_seg = m.n_seg;
  c.seg_len = m.seg_len;
  for (int i = 0; i < RA_MAX_SEG; ++i) c.base[i] = i < SegMap::kMaxSeg ? m.base[i] : 0;
  return c;
}

// One device scratch per process for the whole-attention entry points (grown on demand).
void* flash_scratch(size_t bytes) {
  static void* ptr = nullptr;
  static size_t have = 0;
  if (have < bytes) {
    if (ptr) cudaFree(ptr);
    cuda_must(cudaMalloc(&ptr, bytes), "flash scratch");
    have = bytes;
  }
  return ptr;
}
void flash(const float* q, const float* k, const float* v, float* out, const AttentionShape& s,
           bool causal, bool half_precision, cudaStream_t stream, const char* who) {
  const ra_shape c = to_c(s);
  const size_t need = ra_flash_workspace_bytes(&c, half_precision);
  must(ra_flash_attention(q, k, v, out, &c, causal, half_precision, flash_scratch(need), need,
                          stream),
       who);
}

}  // namespace

// ---- src/attention.hpp ---------------------------------------------------------------

void launch_naive_attention(const float* q, const float* k, const float* v, float* out,
                            const AttentionShape& s, bool causal, cudaStream_t stream) {
  const ra_shape c = to_c(s);
  must(ra_naive_attention(q, k, v, out, &c, causal ? 1 : 0, stream), "launch_naive_attention");
}
void launch_flash_attention(const float* q, const float* k, const float* v, float* out,
                            const AttentionShape& s, bool causal, cudaStream_t stream) {
  flash(q, k, v, out, s, causal, false, stream, "launch_flash_attention");
}
void launch_flash_attention_fp16(const float* q, const float* k, const float* v, float* out,
                                 const AttentionShape& s, bool causal, cudaStream_t stream) {
  flash(q, k, v, out, s, causal, true, stream, "launch_flash_attention_fp16");
}
void launch_attention_init(float* out, float* m, float* l, const AttentionShape& s,
                           std::size_t m_count, cudaStream_t stream) {
  const ra_shape c = to_c(s);
  must(ra_attention_init(out, m, l, &c, m_count, stream), "launch_attention_init");
}
void launch_attention_step(const float* q, const float* k, const float* v, float* out, float* m,
                           float* l, const AttentionShape& s, int q_offset, int k_offset,
                           bool causal, cudaStream_t stream, int pos_stride) {
  const ra_shape c = to_c(s);
  must(ra_attention_step(q, k, v, out, m, l, &c, q_offset, k_offset, causal, stream, pos_stride),
       "launch_attention_step");
}
void launch_attention_step_segmented(const float* q, const float* k, const float* v, float* out,
                                     float* m, float* l, const AttentionShape& s,
                                     const SegMap& qmap, const SegMap& kmap, bool causal,
                                     cudaStream_t stream) {
  const ra_shape c = to_c(s);
  const ra_segmap a = to_c(qmap), b = to_c(kmap);
  must(ra_attention_step_segmented(q, k, v, out, m, l, &c, &a, &b, causal, stream),
       "launch_attention_step_segmented");
}
void launch_attention_decode_step(const float* q, const float* k, const float* v, float* out,
                                  float* m, float* l, const AttentionShape& s, int q_offset,
                                  int k_offset, bool causal, cudaStream_t stream,
                                  int kv_row_stride) {
  const ra_shape c = to_c(s);
  must(ra_attention_decode_step(RA_F32, q, k, v, out, m, l, &c, q_offset, k_offset, causal, stream,
                                kv_row_stride, nullptr, 0),
       "launch_attention_decode_step");
}
void launch_attention_finalize(float* out, const float* l, const AttentionShape& s,
                               cudaStream_t stream) {
  const ra_shape c = to_c(s);
  must(ra_attention_finalize(out, l, &c, stream), "launch_attention_finalize");
}
void launch_attention_step_fp16(const __half* q, const __half* k, const __half* v, float* out,
                                float* m, float* l, const AttentionShape& s, int q_offset,
                                int k_offset, bool causal, cudaStream_t stream, int pos_stride) {
  const ra_shape c = to_c(s);
  must(ra_attention_step_fp16(q, k, v, out, m, l, &c, q_offset, k_offset, causal, stream,
                              pos_stride),
       "launch_attention_step_fp16");
}
void launch_float_to_half(const float* src, __half* dst, std::size_t n, cudaStream_t stream) {
  must(ra_float_to_half(src, dst, n, stream), "launch_float_to_half");
}
void launch_half_to_float(const __half* src, float* dst, std::size_t n, cudaStream_t stream) {
  must(ra_half_to_float(src, dst, n, stream), "launch_half_to_float");
}
void launch_float_to_int8(const float* src, signed char* dst, std::size_t n, cudaStream_t stream) {
  must(ra_float_to_int8(src, dst, n, stream), "launch_float_to_int8");
}
void launch_int8_to_float(const signed char* src, float* dst, std::size_t n, cudaStream_t stream) {
  must(ra_int8_to_float(src, dst, n, stream), "launch_int8_to_float");
}

// ---- src/device_tensor.hpp -----------------------------------------------------------

template <typename T>
DeviceTensor<T>::DeviceTensor(std::size_t count) : ptr_(nullptr), count_(count) {
  if (count != 0) cuda_must(cudaMalloc(reinterpret_cast<void**>(&ptr_), bytes()), "DeviceTensor");
}
template <typename T>
DeviceTensor<T>::~DeviceTensor() {
  if (ptr_) cudaFree(ptr_);
}
template <typename T>
DeviceTensor<T>::DeviceTensor(DeviceTensor&& o) noexcept : ptr_(o.ptr_), count_(o.count_) {
  o.ptr_ = nullptr;
  o.count_ = 0;
}
template <typename T>
DeviceTensor<T>& DeviceTensor<T>::operator=(DeviceTensor&& o) noexcept {
  if (this == &o) return *this;
  std::swap(ptr_, o.ptr_);
  std::swap(count_, o.count_);
  if (o.ptr_) cudaFree(o.ptr_);  // what this object held before
  o.ptr_ = nullptr;
  o.count_ = 0;
  return *this;
}
template <typename T>
void DeviceTensor<T>::copy_from_host(const T* host) {
  cuda_must(cudaMemcpy(ptr_, host, bytes(), cudaMemcpyHostToDevice), "copy_from_host");
}
template <typename T>
void DeviceTensor<T>::copy_to_host(T* host) const {
  cuda_must(cudaMemcpy(host, ptr_, bytes(), cudaMemcpyDeviceToHost), "copy_to_host");
  // This is where results reach the caller: the reference would have aborted in cudaCheck had a
  // kernel failed (src/common.cuh:16-24). A bounded device-side wait that ran out is this
  // library's equivalent, so it aborts here too instead of handing back what the kernel left.
  int st[4] = {0, 0, 0, 0};
  if (ra_device_status(st) == RA_OK && st[0] != 0) {
    std::fprintf(stderr, "copy_to_host: a device-side wait ran out (code %d, wait %d, block %d, tile %d)\n",
                 st[0], st[1], st[2], st[3]);
    std::abort();
  }
}
template <typename T>
void DeviceTensor<T>::copy_from_host(const std::vector<T>& host) {
  if (host.size() != count_) {
    std::fprintf(stderr, "DeviceTensor::copy_from_host: size %zu != %zu\n", host.size(), count_);
    std::abort();
  }
  copy_from_host(host.data());
}
template <typename T>
void DeviceTensor<T>::copy_to_host(std::vector<T>& host) const {
  host.resize(count_);
  copy_to_host(host.data());
}
template class DeviceTensor<float>;
template class DeviceTensor<int>;
template class DeviceTensor<unsigned int>;
template class DeviceTensor<__half>;
template class DeviceTensor<signed char>;

// ---- src/kv_cache.hpp ------------------------------------------------------------------

template <typename T>
DeviceKVCache<T>::DeviceKVCache(int batch, int kv_heads, int s_max, int head_dim)
    : k_(static_cast<std::size_t>(batch) * kv_heads * s_max * head_dim),
      v_(static_cast<std::size_t>(batch) * kv_heads * s_max * head_dim),
      batch_(batch),
      kv_heads_(kv_heads),
      s_max_(s_max),
      head_dim_(head_dim) {}

namespace {
// `rows` rows per (batch, kv head) from a packed source into cache rows [at, at + rows)
template <typename T>
void rows_into_cache(T* dst, const T* src, int rows, int at, int s_max, int head_dim,
                     std::size_t heads, cudaStream_t stream) {
  const std::size_t width = static_cast<std::size_t>(rows) * head_dim * sizeof(T);
  if (width == 0) return;
  cuda_must(cudaMemcpy2DAsync(dst + static_cast<std::size_t>(at) * head_dim,
                              static_cast<std::size_t>(s_max) * head_dim * sizeof(T), src, width,
                              width, heads, cudaMemcpyDeviceToDevice, stream),
            "DeviceKVCache copy");
}
}  // namespace

template <typename T>
void DeviceKVCache<T>::copy_prefill(const T* k_src, const T* v_src, int prefill_len,
                                    cudaStream_t stream) {
  if (prefill_len > s_max_ || prefill_len < 0) {
    std::fprintf(stderr, "DeviceKVCache::copy_prefill: prefill_len=%d exceeds s_max=%d\n",
                 prefill_len, s_max_);
    std::abort();
  }
  const std::size_t heads = static_cast<std::size_t>(batch_) * kv_heads_;
  rows_into_cache(k_.data(), k_src, prefill_len, 0, s_max_, head_dim_, heads, stream);
  rows_into_cache(v_.data(), v_src, prefill_len, 0, s_max_, head_dim_, heads, stream);
  current_len_ = prefill_len;
}
template <typename T>
void DeviceKVCache<T>::append(const T* k_step, const T* v_step, cudaStream_t stream) {
  if (current_len_ >= s_max_) {
    std::fprintf(stderr, "DeviceKVCache::append: cache full (current_len=%d, s_max=%d)\n",
                 current_len_, s_max_);
    std::abort();
  }
  const std::size_t heads = static_cast<std::size_t>(batch_) * kv_heads_;
  rows_into_cache(k_.data(), k_step, 1, current_len_, s_max_, head_dim_, heads, stream);
  rows_into_cache(v_.data(), v_step, 1, current_len_, s_max_, head_dim_, heads, stream);
  ++current_len_;
}
template class DeviceKVCache<float>;
template class DeviceKVCache<__half>;

// ---- src/decode_op.hpp -----------------------------------------------------------------

namespace {
template <typename T>
void local_decode(int dtype, const T* q, const DeviceKVCache<T>& cache, int heads, int q_pos,
                  int k_off, bool causal, float* out, cudaStream_t stream) {
  const int B = cache.batch(), D = cache.head_dim();
  const std::size_t rows = static_cast<std::size_t>(B) * heads;
  DeviceTensor<float> ml(2 * rows);
  ra_shape s{B, heads, 1, cache.current_len(), D, cache.kv_heads()};
  must(ra_attention_init(out, ml.data(), ml.data() + rows, &s, rows, stream), "decode init");
  if (cache.current_len() > 0) {
    // the cache is read in place: row stride s_max, no repack (src/decode_op.cu:25-42 repacks)
    must(ra_attention_decode_step(dtype, q, cache.k_data(), cache.v_data(), out, ml.data(),
                                  ml.data() + rows, &s, q_pos, k_off, causal, stream,
                                  cache.s_max(), nullptr, 0),
         "decode step");
  }
  must(ra_attention_finalize(out, ml.data() + rows, &s, stream), "decode finalize");
  cuda_must(cudaStreamSynchronize(stream), "decode sync");  // ml is freed on return
}
}  // namespace

void run_local_decode_step(const float* q, const DeviceKVCache<float>& cache, int heads,
                           int q_pos_global, int cache_k_offset, bool causal, float* out,
                           cudaStream_t stream) {
  local_decode<float>(RA_F32, q, cache, heads, q_pos_global, cache_k_offset, causal, out, stream);
}
void run_local_decode_step_fp16(const __half* q, const DeviceKVCache<__half>& cache, int heads,
                                int q_pos_global, int cache_k_offset, bool causal, float* out,
                                cudaStream_t stream) {
  local_decode<__half>(RA_F16, q, cache, heads, q_pos_global, cache_k_offset, causal, out, stream);
}

// ---- src/ring2d_schedule.hpp -------------------------------------------------------------

Ring2DSchedule::Ring2DSchedule(int num_nodes, int gpus_per_node, int node, int local)
    : num_nodes_(num_nodes), gpus_per_node_(gpus_per_node), node_(node), local_(local) {
  if (num_nodes <= 0 || gpus_per_node <= 0 || node < 0 || node >= num_nodes || local < 0 ||
      local >= gpus_per_node) {
    std::fprintf(stderr, "Ring2DSchedule: invalid arguments\n");
    std::abort();
  }
  trace_.reserve(static_cast<std::size_t>(num_nodes) * gpus_per_node);
  for (int m = 0; m < num_nodes; ++m)
    for (int i = 0; i < gpus_per_node; ++i)
      trace_.push_back(ra_ring2d_source(num_nodes, gpus_per_node, node, local, m, i));
}

// ---- src/ring_partition.hpp --------------------------------------------------------------

RingPartition::RingPartition(int cp_size, int rank, int seq, Mode mode, int n_splits)
    : cp_size_(cp_size), rank_(rank), seq_(seq), n_splits_(n_splits), mode_(mode) {
  const bool ok = cp_size > 0 && rank >= 0 && rank < cp_size && seq % cp_size == 0 &&
                  (mode != Mode::Zigzag || (n_splits >= 2 && seq % (n_splits * cp_size) == 0));
  if (!ok) {
    std::fprintf(stderr, "RingPartition: invalid arguments\n");
    std::abort();
  }
}
int RingPartition::q_offset(int sg) const {
  return ra_partition_q_offset(cp_size_, rank_, seq_, static_cast<int>(mode_), n_splits_, sg);
}
int RingPartition::k_offset_for_step(int step, int sg) const {
  return ra_partition_k_offset_for_step(cp_size_, rank_, seq_, static_cast<int>(mode_), n_splits_,
                                        step, sg);
}
int RingPartition::k_offset_for_source(int source_rank, int sg) const {
  return ra_partition_k_offset_for_source(cp_size_, rank_, seq_, static_cast<int>(mode_),
                                          n_splits_, source_rank, sg);
}
int RingPartition::local_chunk_len(int) const {
  return ra_partition_local_chunk_len(cp_size_, seq_, static_cast<int>(mode_), n_splits_);
}
int RingPartition::next_rank() const { return ra_partition_next_rank(cp_size_, rank_); }
int RingPartition::prev_rank() const { return ra_partition_prev_rank(cp_size_, rank_); }
int RingPartition::num_sub_groups() const {
  return ra_partition_num_sub_groups(static_cast<int>(mode_), n_splits_);
}
int RingPartition::position_stride() const {
  return ra_partition_position_stride(cp_size_, static_cast<int>(mode_));
}

}  // namespace ring_attention
