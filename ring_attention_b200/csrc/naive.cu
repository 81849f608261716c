// Whole attention for ANY head_dim, fp32 end to end: the counterpart of the reference's
// baseline kernel (launch_naive_attention, src/attention.hpp:42-46, src/naive_attention.cu),
// which its tests call with head sizes the tiled kernels do not take (16, 24). It is a
// correctness baseline, not a fast path: one block per (batch, head, query row); keys are
// scored 128 at a time (one key per thread), the block agrees on the running maximum, and the
// threads then switch roles and each accumulates output columns over the chunk's weights.
#include <cfloat>

#include "common.cuh"

namespace rab {
namespace {

constexpr int kNaiveThreads = 128;

__device__ inline float block_reduce(float x, float* scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float y = __shfl_xor_sync(0xffffffffu, x, o);
    x = is_max ? fmaxf(x, y) : x + y;
  }
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < kNaiveThreads / 32; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
  return r;
}

// Dynamic shared memory: q row (D floats) | chunk weights (kNaiveThreads floats).
__global__ void __launch_bounds__(kNaiveThreads)
    naive_attention_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                           const float* __restrict__ V, float* __restrict__ O, int H, int kvH,
                           int Sq, int Sk, int D, int causal) {
  extern __shared__ float naive_smem[];
  __shared__ float scratch[kNaiveThreads / 32];
  float* q_s = naive_smem;
  float* p_s = naive_smem + D;
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const float* q = Q + ((static_cast<size_t>(b) * H + h) * Sq + i) * D;
  const size_t kv_head = (static_cast<size_t>(b) * kvH + (h % kvH)) * static_cast<size_t>(Sk) * D;
  for (int d = tid; d < D; d += kNaiveThreads) q_s[d] = q[d];
  __syncthreads();
  // end-aligned causal mask: key j is visible iff j <= i + (Sk - Sq) (src/cpu_attention.cpp:32-34)
  const int last = causal ? min(Sk - 1, i + (Sk - Sq)) : Sk - 1;
  const float scale = rsqrtf(static_cast<float>(D));
  // output columns tid, tid + 128, ... (at most 8 per thread: head_dim <= 1024)
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  for (int j0 = 0; j0 <= last; j0 += kNaiveThreads) {
    const int j = j0 + tid;
    float s = -INFINITY;
    if (j <= last) {
      const float* kr = K + kv_head + static_cast<size_t>(j) * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot += q_s[d] * kr[d];
      s = dot * scale;
    }
    const float m_new = fmaxf(m_run, block_reduce(s, scratch, true));
    const float p = (j <= last) ? expf(s - m_new) : 0.f;
    const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    l_run = alpha * l_run + block_reduce(p, scratch, false);
    p_s[tid] = p;
    __syncthreads();
    const int n = min(kNaiveThreads, last + 1 - j0);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int d = tid + c * kNaiveThreads;
      if (d < D) {
        float a = acc[c] * alpha;
        const float* vr = V + kv_head + static_cast<size_t>(j0) * D + d;
        for (int jj = 0; jj < n; ++jj) a += p_s[jj] * vr[static_cast<size_t>(jj) * D];
        acc[c] = a;
      }
    }
    m_run = m_new;
    __syncthreads();  // p_s is rewritten by the next chunk
  }
  float* o = O + ((static_cast<size_t>(b) * H + h) * Sq + i) * D;
  const float inv = l_run > 0.f ? 1.f / l_run : 0.f;  // a row that sees no key gives zeros
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int d = tid + c * kNaiveThreads;
    if (d < D) o[d] = acc[c] * inv;
  }
}

}  // namespace
}  // namespace rab

using namespace rab;

extern "C" int ra_naive_attention(const float* q, const float* k, const float* v, float* out,
                                  const ra_shape* s, int causal, ra_stream stream) {
  RAB_REQUIRE(q && k && v && out && s, RA_ERR_INVALID, "ra_naive_attention: null argument");
  const int kvH = s->kv_heads > 0 ? s->kv_heads : s->heads;
  RAB_REQUIRE(s->batch > 0 && s->heads > 0 && s->seq_q >= 0 && s->seq_k >= 0 && s->head_dim >= 1 &&
                  s->head_dim <= 8 * kNaiveThreads && s->heads <= 65535 && s->batch <= 65535,
              RA_ERR_INVALID, "ra_naive_attention: bad shape (head_dim 1..%d)", 8 * kNaiveThreads);
  RAB_REQUIRE(s->heads % kvH == 0, RA_ERR_INVALID,
              "ra_naive_attention: heads=%d not a multiple of kv_heads=%d", s->heads, kvH);
  if (s->seq_q == 0) return RA_OK;
  const dim3 grid(static_cast<unsigned>(s->seq_q), static_cast<unsigned>(s->heads),
                  static_cast<unsigned>(s->batch));
  const size_t smem = (static_cast<size_t>(s->head_dim) + kNaiveThreads) * sizeof(float);
  naive_attention_kernel<<<grid, kNaiveThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      q, k, v, out, s->heads, kvH, s->seq_q, s->seq_k, s->head_dim, causal ? 1 : 0);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}
