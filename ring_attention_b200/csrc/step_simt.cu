// SIMT online-softmax ring step: fp32 arithmetic end to end, for fp32 / fp16 / bf16 inputs
// and every supported head_dim (32, 64, 128, 256). It is the fp32 path of the library
// (1e-5 agreement with cpu_attention needs fp32 products, which tensor cores do not give)
// and the path for the head sizes the tcgen05 kernel does not take.
//
// Same recurrence and state semantics as the reference's attention_step_kernel
// (src/attention_step.cu:114-282): per row, m/l/out are read, folded with one K/V chunk and
// written back unnormalised; a row with no visible key keeps its state. Positions come from
// piecewise-affine maps, which covers the affine call (one segment), the segmented call
// (src/attention_step.cu:305-460) and striped layouts (stride > 1).
//
// Layout of the work: a block owns 64 query rows; 4 threads share a row, each holding a
// quarter of the head dimension of Q and of the output accumulator in registers. K/V tiles
// of 4096/D keys are staged in shared memory as fp32; a score is a quarter dot product per
// thread plus two shuffles.
#include <cfloat>

#include "common.cuh"

namespace rab {

namespace {

constexpr int kRows = 64;
constexpr int kThreadsPerRow = 4;
constexpr int kThreads = kRows * kThreadsPerRow;
constexpr int kChunk = 16;  // keys folded per online-softmax update

template <typename T>
__device__ inline float load_as_float(const T* p);
template <>
__device__ inline float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ inline float load_as_float<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ inline float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

// Four consecutive elements as float4 (16-byte load for fp32, 8-byte for 16-bit types).
template <typename T>
__device__ inline float4 load4(const T* p);
template <>
__device__ inline float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ inline float4 load4<__half>(const __half* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
template <>
__device__ inline float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}

__device__ inline int pos_of(const PosMap& pm, int i, int stride) {
  const int seg = i / pm.seg_len;
  return pm.base[seg] + (i - seg * pm.seg_len) * stride;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
    step_simt_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                     float* __restrict__ O, float* __restrict__ M, float* __restrict__ L, int H,
                     int kvH, int Sq, int Sk, long long kv_head_stride, PosMap qmap, PosMap kmap,
                     int stride, unsigned flags, long long doc_len) {
  constexpr int DQ = D / kThreadsPerRow;  // elements of the head dimension per thread
  constexpr int BC = 4096 / D;            // keys per shared-memory tile
  static_assert(BC % kChunk == 0, "tile must be a whole number of chunks");
  __shared__ __align__(16) float Ks[BC * D];
  __shared__ __align__(16) float Vs[BC * D];
  __shared__ int kpos_s[BC];
  __shared__ int qmax_s;

  const bool causal = (flags & RA_STEP_CAUSAL) != 0;
  const bool fresh = (flags & RA_STEP_FRESH) != 0;
  const int tid = threadIdx.x;
  const int r = tid / kThreadsPerRow;
  const int c = tid % kThreadsPerRow;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int i = blockIdx.x * kRows + r;
  const bool active = i < Sq;
  const float scale = rsqrtf(static_cast<float>(D));

  const size_t q_head = (static_cast<size_t>(b) * H + h) * static_cast<size_t>(Sq) * D;
  const size_t kv_head = (static_cast<size_t>(b) * kvH + (h % kvH)) * kv_head_stride;
  const size_t row_idx = (static_cast<size_t>(b) * H + h) * Sq + (active ? i : 0);

  const int qpos = active ? pos_of(qmap, i, stride) : INT_MIN;
  const long long qdoc = (doc_len > 0 && active) ? qpos / doc_len : 0;

  if (tid == 0) qmax_s = INT_MIN;
  __syncthreads();
  if (active && c == 0) atomicMax(&qmax_s, qpos);

  float q_reg[DQ], o_reg[DQ];
  float m_i = -INFINITY, l_i = 0.f;
#pragma unroll
  for (int d = 0; d < DQ; ++d) {
    q_reg[d] = 0.f;
    o_reg[d] = 0.f;
  }
  if (active) {
    const T* qp = Q + q_head + static_cast<size_t>(i) * D + c * DQ;
#pragma unroll
    for (int d = 0; d < DQ; d += 4) {
      const float4 x = load4<T>(qp + d);
      q_reg[d] = x.x;
      q_reg[d + 1] = x.y;
      q_reg[d + 2] = x.z;
      q_reg[d + 3] = x.w;
    }
    if (!fresh) {
      const float* op = O + q_head + static_cast<size_t>(i) * D + c * DQ;
#pragma unroll
      for (int d = 0; d < DQ; d += 4) {
        const float4 x = *reinterpret_cast<const float4*>(op + d);
        o_reg[d] = x.x;
        o_reg[d + 1] = x.y;
        o_reg[d + 2] = x.z;
        o_reg[d + 3] = x.w;
      }
      m_i = M[row_idx];
      l_i = L[row_idx];
    }
  }
  __syncthreads();
  const int qmax = qmax_s;

  for (int j0 = 0; j0 < Sk; j0 += BC) {
    // Global position of each key of the tile (INT_MAX marks rows past the chunk).
    int any = 0;
    if (tid < BC) {
      const int j = j0 + tid;
      const int kp = j < Sk ? pos_of(kmap, j, stride) : INT_MAX;
      any = (j < Sk) && (!causal || kp <= qmax);
      // written after the previous tile's readers passed the barrier at the end of the loop
      kpos_s[tid] = kp;
    }
    // Skip tiles no row of this block can see (also publishes kpos_s).
    if (!__syncthreads_or(any)) continue;

    // Stage K and V as fp32, zero-filled past the chunk.
    for (int e = tid * 4; e < BC * D; e += kThreads * 4) {
      const int jl = e / D;
      const int d = e - jl * D;
      const int j = j0 + jl;
      float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
      if (j < Sk) {
        const size_t off = kv_head + static_cast<size_t>(j) * D + d;
        kx = load4<T>(K + off);
        vx = load4<T>(V + off);
      }
      *reinterpret_cast<float4*>(&Ks[e]) = kx;
      *reinterpret_cast<float4*>(&Vs[e]) = vx;
    }
    __syncthreads();

#pragma unroll 1
    for (int jc = 0; jc < BC; jc += kChunk) {
      float s[kChunk];
#pragma unroll
      for (int jj = 0; jj < kChunk; ++jj) {
        const float* kr = &Ks[(jc + jj) * D + c * DQ];
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < DQ; d += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
          acc += q_reg[d] * k4.x + q_reg[d + 1] * k4.y + q_reg[d + 2] * k4.z +
                 q_reg[d + 3] * k4.w;
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        s[jj] = acc;
      }
      float m_new = m_i;
#pragma unroll
      for (int jj = 0; jj < kChunk; ++jj) {
        const int kp = kpos_s[jc + jj];
        bool vis = (kp != INT_MAX) && (!causal || kp <= qpos);
        if (doc_len > 0 && vis) vis = (kp / doc_len) == qdoc;
        if (vis) {
          s[jj] *= scale;
          m_new = fmaxf(m_new, s[jj]);
        } else {
          s[jj] = -INFINITY;
        }
      }
      if (m_new == -INFINITY) continue;  // nothing visible so far: state unchanged
      const float alpha = expf(m_i - m_new);
      float row_sum = 0.f;
#pragma unroll
      for (int jj = 0; jj < kChunk; ++jj) {
        s[jj] = (s[jj] == -INFINITY) ? 0.f : expf(s[jj] - m_new);
        row_sum += s[jj];
      }
#pragma unroll
      for (int d = 0; d < DQ; ++d) o_reg[d] *= alpha;
#pragma unroll
      for (int jj = 0; jj < kChunk; ++jj) {
        const float p = s[jj];
        const float* vr = &Vs[(jc + jj) * D + c * DQ];
#pragma unroll
        for (int d = 0; d < DQ; d += 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(vr + d);
          o_reg[d] += p * v4.x;
          o_reg[d + 1] += p * v4.y;
          o_reg[d + 2] += p * v4.z;
          o_reg[d + 3] += p * v4.w;
        }
      }
      l_i = alpha * l_i + row_sum;
      m_i = m_new;
    }
    __syncthreads();  // everyone is done with Ks/Vs/kpos_s before the next tile overwrites them
  }

  if (active) {
    float inv = 1.f;
    if (flags & RA_STEP_FINALIZE) inv = l_i > 0.f ? 1.f / l_i : 0.f;
    float* op = O + q_head + static_cast<size_t>(i) * D + c * DQ;
#pragma unroll
    for (int d = 0; d < DQ; d += 4) {
      *reinterpret_cast<float4*>(op + d) = make_float4(o_reg[d] * inv, o_reg[d + 1] * inv,
                                                       o_reg[d + 2] * inv, o_reg[d + 3] * inv);
    }
    if (c == 0) {
      M[row_idx] = m_i;
      L[row_idx] = l_i;
    }
  }
}

template <typename T>
int launch_typed(const StepArgs& a, cudaStream_t stream) {
  const dim3 grid((a.Sq + kRows - 1) / kRows, a.H, a.B);
  const dim3 block(kThreads);
  const T* q = static_cast<const T*>(a.q);
  const T* k = static_cast<const T*>(a.k);
  const T* v = static_cast<const T*>(a.v);
#define RAB_SIMT_CASE(DD)                                                                      \
  case DD:                                                                                     \
    step_simt_kernel<T, DD><<<grid, block, 0, stream>>>(q, k, v, a.out, a.m, a.l, a.H, a.kvH,  \
                                                        a.Sq, a.Sk, a.kv_head_stride, a.qmap,  \
                                                        a.kmap, a.stride, a.flags, a.doc_len); \
    break;
  switch (a.D) {
    RAB_SIMT_CASE(32)
    RAB_SIMT_CASE(64)
    RAB_SIMT_CASE(128)
    RAB_SIMT_CASE(256)
    default:
      set_error("attention step: unsupported head_dim=%d (supported: 32, 64, 128, 256)", a.D);
      return RA_ERR_UNSUPPORTED;
  }
#undef RAB_SIMT_CASE
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

}  // namespace

int launch_step_simt(int dtype, const StepArgs& a, cudaStream_t stream) {
  if (a.Sq <= 0 || a.B <= 0 || a.H <= 0) return RA_OK;
  RAB_REQUIRE(a.H <= 65535 && a.B <= 65535, RA_ERR_INVALID,
              "attention step: heads/batch exceed the grid limit");
  switch (dtype) {
    case RA_F32:
      return launch_typed<float>(a, stream);
    case RA_F16:
      return launch_typed<__half>(a, stream);
    case RA_BF16:
      return launch_typed<__nv_bfloat16>(a, stream);
  }
  set_error("attention step: unknown dtype %d", dtype);
  return RA_ERR_INVALID;
}

}  // namespace rab
