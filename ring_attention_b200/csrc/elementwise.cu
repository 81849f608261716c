// Streaming kernels around the step kernels: state init / finalize / lse, dtype casts and
// the decode partial merge. All are HBM-bound, so they move 16 bytes per thread per
// access where alignment allows and size their grid-stride launch as a multiple of the
// SM count.
#include <cmath>
#include <mutex>

#include "common.cuh"

namespace rab {

namespace {

int grid_for(size_t work_items, int block) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      sms = v;
  }
  size_t need = (work_items + block - 1) / block;
  size_t cap = static_cast<size_t>(sms) * 8;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// out = 0, m = -inf, l = 0 (reference: src/attention_step.cu:42-53).
__global__ void init_kernel(float* __restrict__ out, float* __restrict__ m, float* __restrict__ l,
                            size_t out_count, size_t m_count, int vec_ok) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t n4 = vec_ok ? out_count / 4 : 0;
  float4* o4 = reinterpret_cast<float4*>(out);
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t i = tid; i < n4; i += nth) o4[i] = z;
  for (size_t i = n4 * 4 + tid; i < out_count; i += nth) out[i] = 0.f;
  for (size_t i = tid; i < m_count; i += nth) {
    m[i] = -INFINITY;
    l[i] = 0.f;
  }
}

// out_row *= 1 / l_row, 0 where l_row <= 0 (reference: src/attention_step.cu:56-69).
// One thread per 4 consecutive elements; D is a multiple of 4.
__global__ void finalize_kernel(float* __restrict__ out, const float* __restrict__ l, size_t rows,
                                int D) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  const int d4 = D / 4;
  const size_t n4 = rows * d4;
  float4* o4 = reinterpret_cast<float4*>(out);
  for (size_t i = tid; i < n4; i += nth) {
    const float lv = l[i / d4];
    const float inv = lv > 0.f ? 1.f / lv : 0.f;
    float4 x = o4[i];
    x.x *= inv;
    x.y *= inv;
    x.z *= inv;
    x.w *= inv;
    o4[i] = x;
  }
}

__global__ void finalize_scalar_kernel(float* __restrict__ out, const float* __restrict__ l,
                                       size_t rows, int D) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < rows * D; i += nth) {
    const float lv = l[i / D];
    out[i] *= lv > 0.f ? 1.f / lv : 0.f;
  }
}

__global__ void lse_kernel(const float* __restrict__ m, const float* __restrict__ l,
                           float* __restrict__ lse, size_t n) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < n; i += nth) lse[i] = l[i] > 0.f ? m[i] + logf(l[i]) : -INFINITY;
}

template <typename Dst>
__device__ inline Dst cvt_from_float(float x);
template <>
__device__ inline __half cvt_from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ inline __nv_bfloat16 cvt_from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// fp32 -> 16-bit, 8 elements (32 B in, 16 B out) per thread per trip when both pointers are
// 16-byte aligned (reference: src/attention_step_fp16.cu:217-224).
template <typename Dst>
__global__ void narrow_kernel(const float* __restrict__ src, Dst* __restrict__ dst, size_t n,
                              int vec_ok) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t done = 0;
  if (vec_ok) {
    const size_t n8 = n / 8;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (size_t i = tid; i < n8; i += nth) {
      const float4 a = s4[2 * i], b = s4[2 * i + 1];
      union {
        uint4 u;
        Dst h[8];
      } pk;
      pk.h[0] = cvt_from_float<Dst>(a.x);
      pk.h[1] = cvt_from_float<Dst>(a.y);
      pk.h[2] = cvt_from_float<Dst>(a.z);
      pk.h[3] = cvt_from_float<Dst>(a.w);
      pk.h[4] = cvt_from_float<Dst>(b.x);
      pk.h[5] = cvt_from_float<Dst>(b.y);
      pk.h[6] = cvt_from_float<Dst>(b.z);
      pk.h[7] = cvt_from_float<Dst>(b.w);
      d4[i] = pk.u;
    }
    done = n8 * 8;
  }
  for (size_t i = done + tid; i < n; i += nth) dst[i] = cvt_from_float<Dst>(src[i]);
}

// fp16 -> fp32 (reference: src/attention_step_fp16.cu:226-233).
__global__ void widen_kernel(const __half* __restrict__ src, float* __restrict__ dst, size_t n,
                             int vec_ok) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t done = 0;
  if (vec_ok) {
    const size_t n8 = n / 8;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (size_t i = tid; i < n8; i += nth) {
      union {
        uint4 u;
        __half h[8];
      } pk;
      pk.u = s4[i];
      d4[2 * i] = make_float4(__half2float(pk.h[0]), __half2float(pk.h[1]), __half2float(pk.h[2]),
                              __half2float(pk.h[3]));
      d4[2 * i + 1] = make_float4(__half2float(pk.h[4]), __half2float(pk.h[5]),
                                  __half2float(pk.h[6]), __half2float(pk.h[7]));
    }
    done = n8 * 8;
  }
  for (size_t i = done + tid; i < n; i += nth) dst[i] = __half2float(src[i]);
}

// Fixed symmetric scale 127, clamped to [-127, 127], round to nearest
// (reference: src/attention_step_fp16.cu:238-254).
__global__ void to_int8_kernel(const float* __restrict__ src, signed char* __restrict__ dst,
                               size_t n) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < n; i += nth) {
    float x = src[i] * 127.f;
    x = fminf(fmaxf(x, -127.f), 127.f);
    dst[i] = static_cast<signed char>(__float2int_rn(x));
  }
}

__global__ void from_int8_kernel(const signed char* __restrict__ src, float* __restrict__ dst,
                                 size_t n) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < n; i += nth) dst[i] = static_cast<float>(src[i]) * (1.f / 127.f);
}

// Merge cp_size rank partials [O (BH*D) | m (BH) | l (BH)] per rank
// (reference: src/ring_decode.cu:50-81). One block per (b,h) row, D threads. With
// `normalise` the division by l that the reference does in a second launch
// (src/ring_decode.cu:199-203) happens here.
__global__ void partial_merge_kernel(const float* __restrict__ gathered, float* __restrict__ out,
                                     float* __restrict__ m_out, float* __restrict__ l_out,
                                     int cp_size, int BH, int D, int normalise) {
  const int bh = blockIdx.x;
  const int d = threadIdx.x;
  if (bh >= BH || d >= D) return;
  const size_t block = static_cast<size_t>(BH) * D + 2 * static_cast<size_t>(BH);
  const size_t m_off = static_cast<size_t>(BH) * D + bh;
  const size_t l_off = static_cast<size_t>(BH) * D + BH + bh;
  float m_max = -INFINITY;
  for (int r = 0; r < cp_size; ++r) m_max = fmaxf(m_max, gathered[r * block + m_off]);
  float o_acc = 0.f, l_acc = 0.f;
  for (int r = 0; r < cp_size; ++r) {
    const float m_r = gathered[r * block + m_off];
    const float sc = (m_r == -INFINITY) ? 0.f : expf(m_r - m_max);
    o_acc += sc * gathered[r * block + static_cast<size_t>(bh) * D + d];
    l_acc += sc * gathered[r * block + l_off];
  }
  if (normalise) o_acc *= l_acc > 0.f ? 1.f / l_acc : 0.f;
  out[static_cast<size_t>(bh) * D + d] = o_acc;
  if (d == 0) {
    if (m_out) m_out[bh] = m_max;
    if (l_out) l_out[bh] = l_acc;
  }
}

// Merge n_parts online-softmax states of the same rows, each laid out [O rows*D | m rows | l rows]
// and part_stride floats apart, into out / m_out / l_out. One thread per float4 of a row.
constexpr int kMaxStateParts = 8;
__global__ void state_merge_kernel(const float* __restrict__ parts, size_t part_stride, int n_parts,
                                   size_t rows, int D, float* __restrict__ out,
                                   float* __restrict__ m_out, float* __restrict__ l_out,
                                   int normalise) {
  const int vec = D / 4;
  const size_t total = rows * vec;
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += step) {
    const size_t row = idx / vec;
    const int c = static_cast<int>(idx - row * vec);
    float sc[kMaxStateParts];
    float m_max = -INFINITY;
    for (int p = 0; p < n_parts; ++p) {
      sc[p] = parts[p * part_stride + rows * D + row];
      m_max = fmaxf(m_max, sc[p]);
    }
    float l_acc = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_parts; ++p) {
      const float w = (sc[p] == -INFINITY) ? 0.f : expf(sc[p] - m_max);
      l_acc += w * parts[p * part_stride + rows * D + rows + row];
      const float4 o = *reinterpret_cast<const float4*>(parts + p * part_stride + row * D + 4 * c);
      acc.x += w * o.x;
      acc.y += w * o.y;
      acc.z += w * o.z;
      acc.w += w * o.w;
    }
    if (normalise) {
      const float inv = l_acc > 0.f ? 1.f / l_acc : 0.f;
      acc.x *= inv;
      acc.y *= inv;
      acc.z *= inv;
      acc.w *= inv;
    }
    *reinterpret_cast<float4*>(out + row * D + 4 * c) = acc;
    if (c == 0) {
      if (m_out) m_out[row] = m_max;
      if (l_out) l_out[row] = l_acc;
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int launch_init(float* out, float* m, float* l, size_t out_count, size_t m_count,
                cudaStream_t stream) {
  const int vec_ok = aligned16(out);  // float4 stores need 16-byte alignment
  const size_t o_work = vec_ok ? out_count / 4 : out_count;
  const size_t work = o_work > m_count ? o_work : m_count;
  init_kernel<<<grid_for(work, 256), 256, 0, stream>>>(out, m, l, out_count, m_count, vec_ok);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int launch_state_merge(const float* parts, size_t part_stride, int n_parts, size_t rows, int D,
                       float* out, float* m_out, float* l_out, int normalise, cudaStream_t stream) {
  RAB_REQUIRE(parts && out && n_parts >= 1 && n_parts <= kMaxStateParts && D % 4 == 0 &&
                  part_stride % 4 == 0 && aligned16(parts) && aligned16(out),
              RA_ERR_INVALID, "state merge: bad arguments");
  if (rows == 0) return RA_OK;
  state_merge_kernel<<<grid_for(rows * (D / 4), 256), 256, 0, stream>>>(
      parts, part_stride, n_parts, rows, D, out, m_out, l_out, normalise);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int launch_finalize(float* out, const float* l, size_t rows, int D, cudaStream_t stream) {
  if (rows == 0) return RA_OK;
  if (D % 4 == 0 && aligned16(out)) {
    finalize_kernel<<<grid_for(rows * (D / 4), 256), 256, 0, stream>>>(out, l, rows, D);
  } else {
    finalize_scalar_kernel<<<grid_for(rows * D, 256), 256, 0, stream>>>(out, l, rows, D);
  }
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

}  // namespace rab

using namespace rab;

extern "C" {

int ra_attention_init(float* out, float* m, float* l, const ra_shape* shape, size_t m_count,
                      ra_stream stream) {
  RAB_REQUIRE(out && m && l && shape, RA_ERR_INVALID, "ra_attention_init: null argument");
  const size_t out_count = static_cast<size_t>(shape->batch) * shape->heads * shape->seq_q *
                           static_cast<size_t>(shape->head_dim);
  return launch_init(out, m, l, out_count, m_count, static_cast<cudaStream_t>(stream));
}

int ra_attention_finalize(float* out, const float* l, const ra_shape* shape, ra_stream stream) {
  RAB_REQUIRE(out && l && shape, RA_ERR_INVALID, "ra_attention_finalize: null argument");
  const size_t rows = static_cast<size_t>(shape->batch) * shape->heads * shape->seq_q;
  return launch_finalize(out, l, rows, shape->head_dim, static_cast<cudaStream_t>(stream));
}

int ra_attention_lse(const float* m, const float* l, float* lse, size_t count, ra_stream stream) {
  RAB_REQUIRE(m && l && lse, RA_ERR_INVALID, "ra_attention_lse: null argument");
  if (count == 0) return RA_OK;
  lse_kernel<<<grid_for(count, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(m, l, lse,
                                                                                   count);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_float_to_half(const float* src, void* dst, size_t n, ra_stream stream) {
  if (n == 0) return RA_OK;
  RAB_REQUIRE(src && dst, RA_ERR_INVALID, "ra_float_to_half: null argument");
  const int vec = aligned16(src) && aligned16(dst);
  narrow_kernel<__half><<<grid_for(n / 8 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__half*>(dst), n, vec);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_float_to_bf16(const float* src, void* dst, size_t n, ra_stream stream) {
  if (n == 0) return RA_OK;
  RAB_REQUIRE(src && dst, RA_ERR_INVALID, "ra_float_to_bf16: null argument");
  const int vec = aligned16(src) && aligned16(dst);
  narrow_kernel<__nv_bfloat16>
      <<<grid_for(n / 8 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
          src, static_cast<__nv_bfloat16*>(dst), n, vec);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_half_to_float(const void* src, float* dst, size_t n, ra_stream stream) {
  if (n == 0) return RA_OK;
  RAB_REQUIRE(src && dst, RA_ERR_INVALID, "ra_half_to_float: null argument");
  const int vec = aligned16(src) && aligned16(dst);
  widen_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(src), dst, n, vec);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_float_to_int8(const float* src, signed char* dst, size_t n, ra_stream stream) {
  if (n == 0) return RA_OK;
  RAB_REQUIRE(src && dst, RA_ERR_INVALID, "ra_float_to_int8: null argument");
  to_int8_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst, n);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_int8_to_float(const signed char* src, float* dst, size_t n, ra_stream stream) {
  if (n == 0) return RA_OK;
  RAB_REQUIRE(src && dst, RA_ERR_INVALID, "ra_int8_to_float: null argument");
  from_int8_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst, n);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

int ra_decode_partial_merge(const float* gathered, float* out, float* m_out, float* l_out,
                            int cp_size, int bh, int head_dim, int normalise, ra_stream stream) {
  RAB_REQUIRE(gathered && out, RA_ERR_INVALID, "ra_decode_partial_merge: null argument");
  RAB_REQUIRE(cp_size > 0 && bh > 0 && head_dim > 0 && head_dim <= 1024, RA_ERR_INVALID,
              "ra_decode_partial_merge: bad sizes cp=%d bh=%d D=%d", cp_size, bh, head_dim);
  partial_merge_kernel<<<bh, head_dim, 0, static_cast<cudaStream_t>(stream)>>>(
      gathered, out, m_out, l_out, cp_size, bh, head_dim, normalise);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

}  // extern "C"
