// Shared host/device helpers of the library: status handling, the device status word
// that bounded waits report into, and the position maps every step kernel uses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/ring_attention_b200.h"

// The cache handle of the C ABI: K and V of shape (batch, kv_heads, s_max, head_dim).
struct ra_kv_cache {
  int dtype, batch, kv_heads, s_max, head_dim, current_len;
  void* k;
  void* v;
};

namespace rab {

// ---- host-side error reporting -------------------------------------------------
void set_error(const char* fmt, ...);
const char* last_error();

#define RAB_CUDA(expr)                                                                  \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) {                                                            \
      ::rab::set_error("CUDA error '%s' at %s:%d in %s", cudaGetErrorString(_e), __FILE__, \
                       __LINE__, #expr);                                                \
      return RA_ERR_CUDA;                                                               \
    }                                                                                   \
  } while (0)

#define RAB_REQUIRE(cond, code, ...)  \
  do {                                \
    if (!(cond)) {                    \
      ::rab::set_error(__VA_ARGS__);  \
      return (code);                  \
    }                                 \
  } while (0)

inline int kv_heads_of(const ra_shape& s) { return s.kv_heads > 0 ? s.kv_heads : s.heads; }

// ---- device status word ----------------------------------------------------------
// One per device (a __device__ array in status.cu). A kernel whose bounded wait runs out
// records {code, which wait, block, tile} and every later block of any kernel in this
// library returns at once, so a protocol bug costs seconds, never a hung GPU.
int* device_status_ptr();  // device address of the 4-int status word of the current device
int read_device_status(int out[4], bool clear);
// For entry points that end with a synchronisation of `stream`: enqueue_status_read in front
// of it, status_after_sync behind it (RA_ERR_DEVICE_WAIT when a wait ran out; the word stays
// set, so every later launch returns at once, until ra_device_status reads and clears it).
int enqueue_status_read(cudaStream_t stream);
int status_after_sync();
// Scratch for the (m, l) of the local decode op, per device, grown on demand.
int decode_ml_scratch(size_t floats, float** out);

// ---- position maps ------------------------------------------------------------------
// Kernel-side copy of a segment map: local row i -> base[i / seg_len] + (i % seg_len) * stride.
struct PosMap {
  int n_seg;
  int seg_len;
  int base[RA_MAX_SEG];
};

inline PosMap make_posmap(const ra_segmap& s) {
  PosMap p;
  p.n_seg = s.n_seg;
  p.seg_len = s.seg_len;
  for (int i = 0; i < RA_MAX_SEG; ++i) p.base[i] = i < s.n_seg ? s.base[i] : 0;
  return p;
}

inline PosMap affine_posmap(int offset, int len) {
  PosMap p;
  std::memset(&p, 0, sizeof(p));
  p.n_seg = 1;
  p.seg_len = len > 0 ? len : 1;
  p.base[0] = offset;
  return p;
}

// Arguments shared by the SIMT and the tcgen05 step kernels.
struct StepArgs {
  const void* q;
  const void* k;
  const void* v;
  float* out;
  float* m;
  float* l;
  int B, H, kvH, Sq, Sk, D;
  long long kv_head_stride;  // elements between consecutive KV heads (rows * D)
  // Where key segment i sits in the K / V allocation, seen as (k_heads_total, k_rows, D): head
  // coordinate kseg_head[i] + (b * kvH + kv head), first row kseg_row[i]. One tensor with the
  // segments concatenated along the sequence is kseg_head = 0, kseg_row[i] = i * seg_len; a
  // stack of gathered shards puts every shard's heads after the previous shard's.
  int kseg_head[RA_MAX_SEG];
  int kseg_row[RA_MAX_SEG];
  long long k_heads_total;
  int k_rows;
  bool k_stacked;  // true when the segment placement is not the concatenated default
  PosMap qmap, kmap;
  int stride;
  unsigned flags;
  long long doc_len;
  int* status;
};

int launch_step_simt(int dtype, const StepArgs& a, cudaStream_t stream);
int launch_step_tc(int dtype, const StepArgs& a, cudaStream_t stream);
bool step_tc_supported(int dtype, const StepArgs& a);
// fp32 on the tensor cores through split TF32 operands (step_tf32.cu): head_dim 32 and 64
int launch_step_tf32(const StepArgs& a, cudaStream_t stream);
bool step_tf32_supported(int dtype, const StepArgs& a);

// One step over key segments that live in several stacked shards (see StepArgs::kseg_head):
// k / v point at shard 0, every shard is (B * kvH, shard_rows, D) and shard s starts
// s * B * kvH heads later. kmap has one entry per key segment; seg_shard[i] and seg_row[i] place
// it. Only the tensor-core kernel reads this layout: returns RA_ERR_INVALID where it cannot run.
int step_stacked(int dtype, const void* q, const void* k, const void* v, float* out, float* m,
                 float* l, const ra_shape& shape, const PosMap& qmap, const PosMap& kmap,
                 const int* seg_shard, const int* seg_row, int n_shards, int shard_rows,
                 int pos_stride, unsigned flags, long long doc_len, cudaStream_t stream);
bool step_stacked_supported(int dtype, int head_dim);

// seq_q == 1 split-K decode step (decode.cu); workspace NULL = per-device buffer.
int decode_step(int dtype, const void* q, const void* k, const void* v, float* out, float* m,
                float* l, const ra_shape& s, int q_offset, int k_offset, int causal,
                cudaStream_t stream, int kv_row_stride, void* ws, size_t ws_bytes,
                unsigned flags = 0);  // RA_STEP_FRESH / RA_STEP_FINALIZE fused into the fold

int launch_init(float* out, float* m, float* l, size_t out_count, size_t m_count,
                cudaStream_t stream);
int launch_finalize(float* out, const float* l, size_t rows, int D, cudaStream_t stream);
// Merge up to 8 online-softmax states of the same rows ([O | m | l] blocks part_stride floats
// apart, rows * D + rows even multiples of 4 floats so every O stays 16-byte aligned).
int launch_state_merge(const float* parts, size_t part_stride, int n_parts, size_t rows, int D,
                       float* out, float* m_out, float* l_out, int normalise, cudaStream_t stream);

}  // namespace rab
