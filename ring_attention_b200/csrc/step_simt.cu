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
// Layout of the work: 256 threads per block, 4 to 16 threads share a query row (16 elements of
// the head dimension each, 8 at head_dim 32) and every thread carries TWO rows, so a K or V
// value read from shared memory feeds two multiply-adds and the inner loops are bound by the
// FMA pipe (packed fp32x2 multiply-adds) instead of by shared-memory reads. K/V tiles of
// 8192/D keys are staged in shared memory as fp32; a score is a partial dot product per thread
// plus a transposing shuffle reduction over the row's threads, which leaves each complete
// score on exactly one lane: that lane masks and exponentiates it, and the weights travel back
// by shuffle for the second product.
#include <cfloat>

#include "common.cuh"

namespace rab {

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 8;   // keys folded per online-softmax update
constexpr int kR = 2;       // query rows per thread

template <int D>
struct SimtCfg {
  static constexpr int kTPR = D <= 64 ? 4 : D / 16;  // threads per row
  static constexpr int kDQ = D / kTPR;               // head-dimension elements per thread
  static constexpr int kGroups = kThreads / kTPR;    // row groups per block
  static constexpr int kRows = kGroups * kR;         // query rows per block
  static constexpr int kBC = 8192 / D;               // keys per shared-memory tile (32 KiB each of K, V)
  static constexpr int kSmemBytes = 2 * kBC * D * 4 + kBC * 4;
};

// packed fp32x2 multiply-add: one instruction for two lanes
__device__ inline float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)),
        "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}

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
__global__ void __launch_bounds__(kThreads, 2)
    step_simt_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                     float* __restrict__ O, float* __restrict__ M, float* __restrict__ L, int H,
                     int kvH, int Sq, int Sk, long long kv_head_stride, PosMap qmap, PosMap kmap,
                     int stride, unsigned flags, long long doc_len) {
  using C = SimtCfg<D>;
  constexpr int DQ = C::kDQ, BC = C::kBC, TPR = C::kTPR;
  constexpr int CH = kChunk > TPR ? kChunk : TPR;  // keys folded per online-softmax update
  constexpr int KPL = CH / TPR;                    // of which this lane scores KPL
  static_assert(BC % CH == 0, "tile must be a whole number of chunks");
  static_assert(DQ % 4 == 0, "float4 loads");
  extern __shared__ __align__(16) unsigned char simt_smem[];
  float* Ks = reinterpret_cast<float*>(simt_smem);
  float* Vs = Ks + BC * D;
  int* kpos_s = reinterpret_cast<int*>(Vs + BC * D);
  __shared__ int qmax_s;
  static_assert(BC <= kThreads, "one thread per key computes the tile's positions");

  const bool causal = (flags & RA_STEP_CAUSAL) != 0;
  const bool fresh = (flags & RA_STEP_FRESH) != 0;
  const int tid = threadIdx.x;
  const int g = tid / TPR;  // row group; its rows are g and g + kGroups of the block
  const int c = tid % TPR;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const float scale = rsqrtf(static_cast<float>(D));

  const size_t q_head = (static_cast<size_t>(b) * H + h) * static_cast<size_t>(Sq) * D;
  const size_t kv_head = (static_cast<size_t>(b) * kvH + (h % kvH)) * kv_head_stride;

  int row[kR], qpos[kR];
  long long qdoc[kR];
  bool active[kR];
  size_t row_idx[kR];
  float2 q2[kR][DQ / 2], o2[kR][DQ / 2];
  float m_i[kR], l_i[kR];

  if (tid == 0) qmax_s = INT_MIN;
  __syncthreads();
#pragma unroll
  for (int rr = 0; rr < kR; ++rr) {
    row[rr] = blockIdx.x * C::kRows + rr * C::kGroups + g;
    active[rr] = row[rr] < Sq;
    row_idx[rr] = (static_cast<size_t>(b) * H + h) * Sq + (active[rr] ? row[rr] : 0);
    qpos[rr] = active[rr] ? pos_of(qmap, row[rr], stride) : INT_MIN;
    qdoc[rr] = (doc_len > 0 && active[rr]) ? qpos[rr] / doc_len : 0;
    m_i[rr] = -INFINITY;
    l_i[rr] = 0.f;
#pragma unroll
    for (int d = 0; d < DQ / 2; ++d) {
      q2[rr][d] = make_float2(0.f, 0.f);
      o2[rr][d] = make_float2(0.f, 0.f);
    }
    if (active[rr]) {
      if (c == 0) atomicMax(&qmax_s, qpos[rr]);
      const T* qp = Q + q_head + static_cast<size_t>(row[rr]) * D + c * DQ;
#pragma unroll
      for (int d = 0; d < DQ; d += 4) {
        const float4 x = load4<T>(qp + d);
        q2[rr][d / 2] = make_float2(x.x, x.y);
        q2[rr][d / 2 + 1] = make_float2(x.z, x.w);
      }
      if (!fresh) {
        const float* op = O + q_head + static_cast<size_t>(row[rr]) * D + c * DQ;
#pragma unroll
        for (int d = 0; d < DQ; d += 4) {
          const float4 x = *reinterpret_cast<const float4*>(op + d);
          o2[rr][d / 2] = make_float2(x.x, x.y);
          o2[rr][d / 2 + 1] = make_float2(x.z, x.w);
        }
        m_i[rr] = M[row_idx[rr]];
        l_i[rr] = c == 0 ? L[row_idx[rr]] : 0.f;  // the row sum is kept as per-lane shares
      }
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
    for (int jc = 0; jc < BC; jc += CH) {
      // Scores of CH keys for both rows. The partial dot products of a group of TPR keys are
      // summed with a transposing reduction (TPR - 1 shuffles per group and row): afterwards
      // lane c of the row holds the complete score of key c of the group, so the mask, the
      // maximum and the exponential of a key are computed once, not once per lane.
      float sc[kR][KPL];  // this lane's keys: group gi, key gi * TPR + c of the chunk
#pragma unroll
      for (int gi = 0; gi < KPL; ++gi) {
        float part[kR][TPR];
#pragma unroll
        for (int t = 0; t < TPR; ++t) {
          const float* kr = &Ks[(jc + gi * TPR + t) * D + c * DQ];
          float2 acc[kR];
#pragma unroll
          for (int rr = 0; rr < kR; ++rr) acc[rr] = make_float2(0.f, 0.f);
#pragma unroll
          for (int d = 0; d < DQ; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
            const float2 ka = make_float2(k4.x, k4.y), kb = make_float2(k4.z, k4.w);
#pragma unroll
            for (int rr = 0; rr < kR; ++rr) {
              acc[rr] = ffma2(q2[rr][d / 2], ka, acc[rr]);
              acc[rr] = ffma2(q2[rr][d / 2 + 1], kb, acc[rr]);
            }
          }
#pragma unroll
          for (int rr = 0; rr < kR; ++rr) part[rr][t] = acc[rr].x + acc[rr].y;
        }
#pragma unroll
        for (int rr = 0; rr < kR; ++rr) {
#pragma unroll
          for (int o = TPR / 2; o >= 1; o >>= 1) {
            const bool upper = (c & o) != 0;  // this lane keeps the upper half of the values
#pragma unroll
            for (int t = 0; t < o; ++t) {
              const float keep = upper ? part[rr][t + o] : part[rr][t];
              const float send = upper ? part[rr][t] : part[rr][t + o];
              part[rr][t] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
          }
          sc[rr][gi] = part[rr][0];
        }
      }
      bool live[kR];
#pragma unroll
      for (int rr = 0; rr < kR; ++rr) {
        float m_new = -INFINITY;
#pragma unroll
        for (int gi = 0; gi < KPL; ++gi) {
          const int kp = kpos_s[jc + gi * TPR + c];
          bool vis = (kp != INT_MAX) && (!causal || kp <= qpos[rr]);
          if (doc_len > 0 && vis) vis = (kp / doc_len) == qdoc[rr];
          sc[rr][gi] = vis ? sc[rr][gi] * scale : -INFINITY;
          m_new = fmaxf(m_new, sc[rr][gi]);
        }
#pragma unroll
        for (int o = 1; o < TPR; o <<= 1) m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, o));
        m_new = fmaxf(m_new, m_i[rr]);
        live[rr] = m_new != -INFINITY;  // false: nothing visible so far, state unchanged
        const float alpha = live[rr] ? expf(m_i[rr] - m_new) : 1.f;
        float part_sum = 0.f;
#pragma unroll
        for (int gi = 0; gi < KPL; ++gi) {
          sc[rr][gi] = (sc[rr][gi] == -INFINITY) ? 0.f : expf(sc[rr][gi] - m_new);
          part_sum += sc[rr][gi];
        }
        if (live[rr]) {
          l_i[rr] = alpha * l_i[rr] + part_sum;  // per-lane share of the row sum
          m_i[rr] = m_new;
#pragma unroll
          for (int d = 0; d < DQ / 2; ++d)
            o2[rr][d] = make_float2(o2[rr][d].x * alpha, o2[rr][d].y * alpha);
        }
      }
      bool any_live = false;
#pragma unroll
      for (int rr = 0; rr < kR; ++rr) any_live |= live[rr];
      // the weights are fetched from their owner lanes with warp shuffles below, so the whole
      // warp takes this branch together
      if (!__any_sync(0xffffffffu, any_live)) continue;
#pragma unroll
      for (int jj = 0; jj < CH; ++jj) {
        const float* vr = &Vs[(jc + jj) * D + c * DQ];
        float2 p2[kR];
#pragma unroll
        for (int rr = 0; rr < kR; ++rr) {
          const float pw = __shfl_sync(0xffffffffu, sc[rr][jj / TPR], jj % TPR, TPR);
          p2[rr] = make_float2(pw, pw);
        }
#pragma unroll
        for (int d = 0; d < DQ; d += 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(vr + d);
          const float2 va = make_float2(v4.x, v4.y), vb = make_float2(v4.z, v4.w);
#pragma unroll
          for (int rr = 0; rr < kR; ++rr) {
            o2[rr][d / 2] = ffma2(p2[rr], va, o2[rr][d / 2]);
            o2[rr][d / 2 + 1] = ffma2(p2[rr], vb, o2[rr][d / 2 + 1]);
          }
        }
      }
    }
    __syncthreads();  // everyone is done with Ks/Vs/kpos_s before the next tile overwrites them
  }

#pragma unroll
  for (int rr = 0; rr < kR; ++rr) {
#pragma unroll
    for (int o = 1; o < TPR; o <<= 1) l_i[rr] += __shfl_xor_sync(0xffffffffu, l_i[rr], o);
  }
#pragma unroll
  for (int rr = 0; rr < kR; ++rr) {
    if (!active[rr]) continue;
    float inv = 1.f;
    if (flags & RA_STEP_FINALIZE) inv = l_i[rr] > 0.f ? 1.f / l_i[rr] : 0.f;
    float* op = O + q_head + static_cast<size_t>(row[rr]) * D + c * DQ;
#pragma unroll
    for (int d = 0; d < DQ; d += 4) {
      *reinterpret_cast<float4*>(op + d) =
          make_float4(o2[rr][d / 2].x * inv, o2[rr][d / 2].y * inv, o2[rr][d / 2 + 1].x * inv,
                      o2[rr][d / 2 + 1].y * inv);
    }
    if (c == 0) {
      M[row_idx[rr]] = m_i[rr];
      L[row_idx[rr]] = l_i[rr];
    }
  }
}

template <typename T>
int launch_typed(const StepArgs& a, cudaStream_t stream) {
  const dim3 block(kThreads);
  const T* q = static_cast<const T*>(a.q);
  const T* k = static_cast<const T*>(a.k);
  const T* v = static_cast<const T*>(a.v);
#define RAB_SIMT_CASE(DD)                                                                      \
  case DD: {                                                                                   \
    const dim3 grid((a.Sq + SimtCfg<DD>::kRows - 1) / SimtCfg<DD>::kRows, a.H, a.B);           \
    RAB_CUDA(cudaFuncSetAttribute(step_simt_kernel<T, DD>,                                     \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                  SimtCfg<DD>::kSmemBytes));                                   \
    step_simt_kernel<T, DD><<<grid, block, SimtCfg<DD>::kSmemBytes, stream>>>(                 \
        q, k, v, a.out, a.m, a.l, a.H, a.kvH, a.Sq, a.Sk, a.kv_head_stride, a.qmap, a.kmap,    \
        a.stride, a.flags, a.doc_len);                                                         \
    break;                                                                                     \
  }
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
