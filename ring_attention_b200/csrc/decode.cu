// Split-K decode (seq_q == 1) against a KV cache read in place: the HBM-bound half of the
// hot path. Replaces the reference's split + reduce kernels (src/attention_decode.cu:73-277).
//
// What bounds it: every K and V row of the local shard is read exactly once from HBM, so
// the kernels are built around bytes in flight, not arithmetic.
//  - One block per (split, KV head, batch row) serves ALL query heads that map to that KV
//    head (h % kv_heads), so grouped-query attention reads each cached row once instead of
//    once per query head (the reference re-reads it per head, src/attention_decode.cu:88).
//  - The split count is chosen so the grid is about three waves of the SM count.
//  - decode_mma_kernel (fp16 / bf16 caches, head_dim >= 64) is the fast path: K/V rows stream
//    through a 5-8-stage shared-memory ring of 64-key stages filled with 16-byte cp.async
//    copies (fully coalesced, XOR-swizzled), and per 16-key block a warp does both
//    contractions on mma.sync m16n8k16 with the up to 16 grouped query heads as M rows
//    (ldmatrix / ldmatrix.trans), online softmax with warp-shuffle row maxima and a lazy
//    rescale; warps are merged through shared memory. The tensor cores are there to get under
//    the instruction-issue bound (about 5 instead of about 80 warp instructions per cached
//    row), the kernel is bound by the copy (0.87 of the measured HBM copy bandwidth).
//  - decode_split_kernel (fp32 caches, head_dim 32) is the SIMT form of the same structure
//    with a 4-stage ring: a group of `LPR` lanes owns a row, each lane keeps its slice of q
//    (pre-scaled) for every head of the group, the dot product finishes with log2(LPR)
//    shuffles, each lane group carries its own running (m, l, out), and a warp-shuffle
//    log-sum-exp merge plus one shared-memory pass combine lane groups and warps.
// Partials (m, l, out) per (split, batch, head) go to a workspace; a second tiny kernel
// folds them into the persistent state (src/attention_decode.cu:228-277 does the same for
// its fixed 8 splits).
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace rab {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kMaxSplits = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ inline float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ inline void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc),
               "r"(src_bytes)
               : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Unpack one 16-byte piece into floats.
template <typename T>
struct Piece;
template <>
struct Piece<float> {
  static constexpr int kElems = 4;
  __device__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
};
template <>
struct Piece<__half> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
};
template <>
struct Piece<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // bf16 -> fp32 is a 16-bit shift
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T, int D>
struct DecodeCfg {
  static constexpr int kRowBytes = D * static_cast<int>(sizeof(T));
  static constexpr int kPieces = kRowBytes / 16;  // 16-byte pieces per row
  // lanes per row: every lane owns 1..4 pieces
  static constexpr int kLPR = kPieces >= 32 ? 16 : (kPieces >= 8 ? 8 : 4);
  static constexpr int kVPT = kPieces / kLPR;               // pieces per lane
  static constexpr int kEPL = kVPT * Piece<T>::kElems;      // elements per lane
  static constexpr int kRowsPerWarpStep = 32 / kLPR;
  static constexpr int kRowsPerStep = kWarps * kRowsPerWarpStep;
  static constexpr int kSteps =
      (8192 / (kRowsPerStep * kRowBytes)) > 0 ? (8192 / (kRowsPerStep * kRowBytes)) : 1;
  static constexpr int kRowsPerStage = kRowsPerStep * kSteps;
  static constexpr int kStageBytes = kRowsPerStage * kRowBytes;  // per tensor
  static constexpr int kSmemBytes = 2 * kStages * kStageBytes;
};

// grid = (n_split, kv_heads * head_batches, batch). GB = query heads handled per block.
template <typename T, int D, int GB>
__global__ void __launch_bounds__(kThreads)
    decode_split_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                        float* __restrict__ Mp, float* __restrict__ Lp, float* __restrict__ Op,
                        int B, int H, int kvH, int sk_eff, long long kv_head_stride,
                        int rows_per_split, int head_batches, float scale_log2) {
  using C = DecodeCfg<T, D>;
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* k_ring = smem;
  unsigned char* v_ring = smem + kStages * C::kStageBytes;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int lr = lane % C::kLPR;       // lane within the row group
  const int grp = lane / C::kLPR;      // row group within the warp
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / head_batches;
  const int hb = blockIdx.y % head_batches;
  const int b = blockIdx.z;

  // Query heads of this block: h = kvh + kvH * (hb * GB + g), while h < H.
  float q_reg[GB][C::kEPL];
  float o_reg[GB][C::kEPL];
  float m_run[GB], l_run[GB];
#pragma unroll
  for (int g = 0; g < GB; ++g) {
    const int h = kvh + kvH * (hb * GB + g);
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int v = 0; v < C::kVPT; ++v) {
      float f[Piece<T>::kElems];
      if (h < H) {
        const uint4 u = *reinterpret_cast<const uint4*>(
            reinterpret_cast<const unsigned char*>(Q + (static_cast<size_t>(b) * H + h) * D) +
            (v * C::kLPR + lr) * 16);
        Piece<T>::unpack(u, f);
      } else {
#pragma unroll
        for (int e = 0; e < Piece<T>::kElems; ++e) f[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < Piece<T>::kElems; ++e) {
        q_reg[g][v * Piece<T>::kElems + e] = f[e] * scale_log2;
        o_reg[g][v * Piece<T>::kElems + e] = 0.f;
      }
    }
  }

  const int row_begin = split * rows_per_split;
  const int row_end = min(sk_eff, row_begin + rows_per_split);
  const int n_rows = max(0, row_end - row_begin);
  const int n_stages = (n_rows + C::kRowsPerStage - 1) / C::kRowsPerStage;
  const unsigned char* k_base = reinterpret_cast<const unsigned char*>(
      K + (static_cast<size_t>(b) * kvH + kvh) * kv_head_stride);
  const unsigned char* v_base = reinterpret_cast<const unsigned char*>(
      V + (static_cast<size_t>(b) * kvH + kvh) * kv_head_stride);

  auto issue = [&](int st) {
    if (st < n_stages) {
      const int slot = st % kStages;
      const long long first = static_cast<long long>(row_begin) + st * C::kRowsPerStage;
      const long long valid_bytes =
          (static_cast<long long>(row_end) - first) * C::kRowBytes;  // > 0
      const size_t goff = static_cast<size_t>(first) * C::kRowBytes;
      for (int p = tid; p < C::kStageBytes / 16; p += kThreads) {
        const long long off = static_cast<long long>(p) * 16;
        const bool ok = off < valid_bytes;
        // past the split: src-size 0 zero-fills the destination, the source is not read
        cp_async16(k_ring + slot * C::kStageBytes + off, ok ? k_base + goff + off : k_base,
                   ok ? 16 : 0);
        cp_async16(v_ring + slot * C::kStageBytes + off, ok ? v_base + goff + off : v_base,
                   ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);

  for (int st = 0; st < n_stages; ++st) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    issue(st + kStages - 1);
    const int slot = st % kStages;
    const int stage_row0 = st * C::kRowsPerStage;
#pragma unroll 1
    for (int step = 0; step < C::kSteps; ++step) {
      const int rl = step * C::kRowsPerStep + warp * C::kRowsPerWarpStep + grp;
      const bool valid = stage_row0 + rl < n_rows;
      const unsigned char* krow = k_ring + slot * C::kStageBytes + rl * C::kRowBytes;
      const unsigned char* vrow = v_ring + slot * C::kStageBytes + rl * C::kRowBytes;
      float kf[C::kEPL];
#pragma unroll
      for (int v = 0; v < C::kVPT; ++v) {
        const uint4 u = *reinterpret_cast<const uint4*>(krow + (v * C::kLPR + lr) * 16);
        Piece<T>::unpack(u, &kf[v * Piece<T>::kElems]);
      }
      float s[GB];
#pragma unroll
      for (int g = 0; g < GB; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < C::kEPL; ++e) acc = fmaf(q_reg[g][e], kf[e], acc);
        s[g] = acc;
      }
#pragma unroll
      for (int off = 1; off < C::kLPR; off <<= 1) {
#pragma unroll
        for (int g = 0; g < GB; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
      }
      float vf[C::kEPL];
#pragma unroll
      for (int v = 0; v < C::kVPT; ++v) {
        const uint4 u = *reinterpret_cast<const uint4*>(vrow + (v * C::kLPR + lr) * 16);
        Piece<T>::unpack(u, &vf[v * Piece<T>::kElems]);
      }
      if (valid) {
#pragma unroll
        for (int g = 0; g < GB; ++g) {
          if (s[g] > m_run[g]) {  // rare after the first rows: rescale only when the max moves
            const float alpha = ex2(m_run[g] - s[g]);  // ex2(-inf) = 0 on the first row
            l_run[g] *= alpha;
#pragma unroll
            for (int e = 0; e < C::kEPL; ++e) o_reg[g][e] *= alpha;
            m_run[g] = s[g];
          }
          const float p = ex2(s[g] - m_run[g]);
          l_run[g] += p;
#pragma unroll
          for (int e = 0; e < C::kEPL; ++e) o_reg[g][e] = fmaf(p, vf[e], o_reg[g][e]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // Merge the row groups of the warp (log-sum-exp merge through shuffles) ...
#pragma unroll
  for (int off = C::kLPR; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < GB; ++g) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run[g], off);
      const float m_n = fmaxf(m_run[g], m_o);
      const float a = (m_run[g] == -INFINITY) ? 0.f : ex2(m_run[g] - m_n);
      const float c = (m_o == -INFINITY) ? 0.f : ex2(m_o - m_n);
      l_run[g] = a * l_run[g] + c * l_o;
#pragma unroll
      for (int e = 0; e < C::kEPL; ++e) {
        const float o_o = __shfl_xor_sync(0xffffffffu, o_reg[g][e], off);
        o_reg[g][e] = a * o_reg[g][e] + c * o_o;
      }
      m_run[g] = m_n;
    }
  }
  // ... then the warps of the block through shared memory (the ring is idle now).
  __syncthreads();
  float* red_m = reinterpret_cast<float*>(smem);            // [kWarps][GB]
  float* red_l = red_m + kWarps * GB;                        // [kWarps][GB]
  float* red_o = red_l + kWarps * GB;                        // [kWarps][GB][D]
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < GB; ++g) {
      if (lr == 0) {
        red_m[warp * GB + g] = m_run[g];
        red_l[warp * GB + g] = l_run[g];
      }
#pragma unroll
      for (int v = 0; v < C::kVPT; ++v)
#pragma unroll
        for (int e = 0; e < Piece<T>::kElems; ++e)
          red_o[(warp * GB + g) * D + (v * C::kLPR + lr) * Piece<T>::kElems + e] =
              o_reg[g][v * Piece<T>::kElems + e];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < GB * D; idx += kThreads) {
    const int g = idx / D;
    const int d = idx - g * D;
    const int h = kvh + kvH * (hb * GB + g);
    if (h >= H) continue;
    float m_n = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m_n = fmaxf(m_n, red_m[w * GB + g]);
    float o_acc = 0.f, l_acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = red_m[w * GB + g];
      const float sc = (mw == -INFINITY) ? 0.f : ex2(mw - m_n);
      o_acc += sc * red_o[(w * GB + g) * D + d];
      l_acc += sc * red_l[w * GB + g];
    }
    const size_t prow = (static_cast<size_t>(split) * B + b) * H + h;
    Op[prow * D + d] = o_acc;
    if (d == 0) {
      Mp[prow] = m_n * kLn2;  // back to natural-log units, the unit of the persistent state
      Lp[prow] = l_acc;
    }
  }
}

// ---- tensor-core variant for 16-bit caches ---------------------------------------------
//
// The SIMT kernel above spends ~80 warp instructions per cached row (a convert and one FMA
// per element per query head), which makes it issue-bound at well under HBM speed. For
// fp16 / bf16 caches both contractions of a block of 16 keys run on mma.sync m16n8k16
// instead: the (up to 16) query heads that share the KV head are the M rows, so a key row
// costs ~5 instructions and the kernel is bound by the copy into shared memory again.
// K/V rows go to shared memory with the same 16-byte cp.async copies, but each 16-byte
// piece c of row r is stored at piece c ^ (r & 7), so that the ldmatrix reads (8 rows at a
// fixed column) touch all banks once.
constexpr int kMmaWarps = 4;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaKeysPerWarp = 16;
constexpr int kMmaStageRows = kMmaWarps * kMmaKeysPerWarp;  // 64 keys per stage

template <typename T>
__device__ inline void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1);
template <>
__device__ inline void mma16816<__half>(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                        unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ inline void mma16816<__nv_bfloat16>(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                               unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ inline void ldmatrix_x4(unsigned (&r)[4], unsigned saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ inline void ldmatrix_x4_trans(unsigned (&r)[4], unsigned saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
template <typename T>
__device__ inline unsigned pack_pair(float lo, float hi);
template <>
__device__ inline unsigned pack_pair<__half>(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&h);
}
template <>
__device__ inline unsigned pack_pair<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&h);
}

template <int D>
struct MmaCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kPieces = kRowBytes / 16;
  static constexpr int kStageBytes = kMmaStageRows * kRowBytes;  // per tensor
  static constexpr int kStagesRaw = (160 * 1024) / (2 * kStageBytes);
  static constexpr int kStages = kStagesRaw > 8 ? 8 : (kStagesRaw < 3 ? 3 : kStagesRaw);
  static constexpr int kSmemBytes = 2 * kStages * kStageBytes;
};

// grid = (n_split, kv_heads * head_batches, batch); a block serves up to 16 query heads of one
// KV head (rows of the MMA tile; row r is head kvh + kv_heads * (16 * hb + r)).
template <typename T, int D>
__global__ void __launch_bounds__(kMmaThreads)
    decode_mma_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                      float* __restrict__ Mp, float* __restrict__ Lp, float* __restrict__ Op, int B,
                      int H, int kvH, int sk_eff, long long kv_head_stride, int rows_per_split,
                      int head_batches, float scale_log2) {
  using C = MmaCfg<D>;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* k_ring = smem;
  unsigned char* v_ring = smem + C::kStages * C::kStageBytes;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;   // fragment row (and row + 8)
  const int tq = lane & 3;   // fragment column pair
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / head_batches;
  const int hb = blockIdx.y % head_batches;
  const int b = blockIdx.z;

  // Q as A fragments: reg0 (row g, k 2tq..), reg1 (row g+8, same k), reg2 / reg3 the same at k+8.
  const int h0 = kvh + kvH * (hb * 16 + g);
  const int h1 = kvh + kvH * (hb * 16 + g + 8);
  unsigned qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int d0 = ks * 16 + 2 * tq;
    const T* q0 = Q + (static_cast<size_t>(b) * H + (h0 < H ? h0 : 0)) * D + d0;
    const T* q1 = Q + (static_cast<size_t>(b) * H + (h1 < H ? h1 : 0)) * D + d0;
    qa[ks][0] = h0 < H ? *reinterpret_cast<const unsigned*>(q0) : 0u;
    qa[ks][1] = h1 < H ? *reinterpret_cast<const unsigned*>(q1) : 0u;
    qa[ks][2] = h0 < H ? *reinterpret_cast<const unsigned*>(q0 + 8) : 0u;
    qa[ks][3] = h1 < H ? *reinterpret_cast<const unsigned*>(q1 + 8) : 0u;
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};  // this lane's share of the row sums (its four columns per block)

  const int row_begin = split * rows_per_split;
  const int row_end = min(sk_eff, row_begin + rows_per_split);
  const int n_rows = max(0, row_end - row_begin);
  const int n_stages = (n_rows + kMmaStageRows - 1) / kMmaStageRows;
  const unsigned char* k_base = reinterpret_cast<const unsigned char*>(
      K + (static_cast<size_t>(b) * kvH + kvh) * kv_head_stride);
  const unsigned char* v_base = reinterpret_cast<const unsigned char*>(
      V + (static_cast<size_t>(b) * kvH + kvh) * kv_head_stride);

  auto issue = [&](int st) {
    if (st < n_stages) {
      const int slot = st % C::kStages;
      const long long first = static_cast<long long>(row_begin) + st * kMmaStageRows;
      const long long valid_bytes = (static_cast<long long>(row_end) - first) * C::kRowBytes;
      const size_t goff = static_cast<size_t>(first) * C::kRowBytes;
      for (int p = tid; p < C::kStageBytes / 16; p += kMmaThreads) {
        const int r = p / C::kPieces;
        const int c = p - r * C::kPieces;
        const long long off = static_cast<long long>(p) * 16;
        const int dst = slot * C::kStageBytes + r * C::kRowBytes + ((c ^ (r & 7)) << 4);
        const bool ok = off < valid_bytes;
        cp_async16(k_ring + dst, ok ? k_base + goff + off : k_base, ok ? 16 : 0);
        cp_async16(v_ring + dst, ok ? v_base + goff + off : v_base, ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < C::kStages - 1; ++s) issue(s);

  const int mi = lane >> 3, r8 = lane & 7;
  const int key0 = warp * kMmaKeysPerWarp;
  // per-lane row offsets of the ldmatrix addresses (piece index is XORed with r8 = key & 7)
  const unsigned k_row_off = static_cast<unsigned>((key0 + (mi >> 1) * 8 + r8) * C::kRowBytes);
  const unsigned v_row_off = static_cast<unsigned>((key0 + (mi & 1) * 8 + r8) * C::kRowBytes);

  for (int st = 0; st < n_stages; ++st) {
    cp_async_wait<C::kStages - 2>();
    __syncthreads();
    issue(st + C::kStages - 1);
    const int slot = st % C::kStages;
    const int n_valid = n_rows - (st * kMmaStageRows + key0);  // valid keys of this warp's block
    if (n_valid <= 0) continue;
    const unsigned kt = static_cast<unsigned>(__cvta_generic_to_shared(k_ring + slot * C::kStageBytes));
    const unsigned vt = static_cast<unsigned>(__cvta_generic_to_shared(v_ring + slot * C::kStageBytes));

    // S = Q K^T for 16 keys: s0 = keys 0..7, s1 = keys 8..15
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      unsigned kb[4];
      ldmatrix_x4(kb, kt + k_row_off + (((2 * ks + (mi & 1)) ^ r8) << 4));
      mma16816<T>(s0, qa[ks], kb[0], kb[1]);
      mma16816<T>(s1, qa[ks], kb[2], kb[3]);
    }
    // scale, hide the keys past the end, row maxima (rows g and g + 8)
    float v[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = ((i >> 1) & 1) * 8 + 2 * tq + (i & 1);
      v[i] = (col < n_valid) ? v[i] * scale_log2 : -INFINITY;
    }
    float mx0 = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    float mx1 = fmaxf(fmaxf(v[4], v[5]), fmaxf(v[6], v[7]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const bool moved = mx0 > m_run[0] || mx1 > m_run[1];
    if (__any_sync(0xffffffffu, moved)) {  // rare after the first blocks
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float a0 = (m_run[0] == -INFINITY) ? 0.f : ex2(m_run[0] - mn0);
      const float a1 = (m_run[1] == -INFINITY) ? 0.f : ex2(m_run[1] - mn1);
      l_run[0] *= a0;
      l_run[1] *= a1;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= a0;
        o[n][1] *= a0;
        o[n][2] *= a1;
        o[n][3] *= a1;
      }
      m_run[0] = mn0;
      m_run[1] = mn1;
    }
    const float ms0 = (m_run[0] == -INFINITY) ? 0.f : m_run[0];
    const float ms1 = (m_run[1] == -INFINITY) ? 0.f : m_run[1];
    float p[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      p[i] = ex2(v[i] - ms0);
      p[4 + i] = ex2(v[4 + i] - ms1);
    }
    l_run[0] += (p[0] + p[1]) + (p[2] + p[3]);
    l_run[1] += (p[4] + p[5]) + (p[6] + p[7]);
    // P as the A fragment of the second product
    unsigned pa[4];
    pa[0] = pack_pair<T>(p[0], p[1]);  // row g,     keys 2tq, 2tq+1
    pa[1] = pack_pair<T>(p[4], p[5]);  // row g + 8, same keys
    pa[2] = pack_pair<T>(p[2], p[3]);  // row g,     keys 8 + 2tq, ...
    pa[3] = pack_pair<T>(p[6], p[7]);  // row g + 8
#pragma unroll
    for (int c2 = 0; c2 < D / 16; ++c2) {
      unsigned vb[4];
      ldmatrix_x4_trans(vb, vt + v_row_off + (((2 * c2 + (mi >> 1)) ^ r8) << 4));
      mma16816<T>(o[2 * c2], pa, vb[0], vb[1]);
      mma16816<T>(o[2 * c2 + 1], pa, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();

  // row sums over the four lanes of a row, then the warps of the block through shared memory
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  __syncthreads();
  float* red_m = reinterpret_cast<float*>(smem);  // [warps][16]
  float* red_l = red_m + kMmaWarps * 16;          // [warps][16]
  float* red_o = red_l + kMmaWarps * 16;          // [warps][16][D]
  if (tq == 0) {
    red_m[warp * 16 + g] = m_run[0];
    red_m[warp * 16 + g + 8] = m_run[1];
    red_l[warp * 16 + g] = l_run[0];
    red_l[warp * 16 + g + 8] = l_run[1];
  }
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    float* r0 = red_o + (warp * 16 + g) * D + n * 8 + 2 * tq;
    float* r1 = red_o + (warp * 16 + g + 8) * D + n * 8 + 2 * tq;
    r0[0] = o[n][0];
    r0[1] = o[n][1];
    r1[0] = o[n][2];
    r1[1] = o[n][3];
  }
  __syncthreads();
  for (int idx = tid; idx < 16 * D; idx += kMmaThreads) {
    const int r = idx / D;
    const int d = idx - r * D;
    const int h = kvh + kvH * (hb * 16 + r);
    if (h >= H) continue;
    float m_n = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) m_n = fmaxf(m_n, red_m[w * 16 + r]);
    float o_acc = 0.f, l_acc = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float mw = red_m[w * 16 + r];
      const float sc = (mw == -INFINITY) ? 0.f : ex2(mw - m_n);
      o_acc += sc * red_o[(w * 16 + r) * D + d];
      l_acc += sc * red_l[w * 16 + r];
    }
    const size_t prow = (static_cast<size_t>(split) * B + b) * H + h;
    Op[prow * D + d] = o_acc;
    if (d == 0) {
      Mp[prow] = m_n * kLn2;
      Lp[prow] = l_acc;
    }
  }
}

// Fold n_split partials into the persistent (out, m, l). grid = (H, B), block = D threads.
// RA_STEP_FRESH: the state is known to be empty (it is written, never read, which saves the
// caller an init launch); RA_STEP_FINALIZE: divide by l after folding (saves the finalize
// launch).
__global__ void decode_reduce_kernel(const float* __restrict__ Mp, const float* __restrict__ Lp,
                                     const float* __restrict__ Op, float* __restrict__ M,
                                     float* __restrict__ L, float* __restrict__ O, int B, int H,
                                     int D, int n_split, unsigned flags) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const size_t row = static_cast<size_t>(b) * H + h;
  const bool fresh = (flags & RA_STEP_FRESH) != 0, finalize = (flags & RA_STEP_FINALIZE) != 0;
  const float m_old = fresh ? -INFINITY : M[row];
  float m_n = m_old;
  for (int s = 0; s < n_split; ++s) m_n = fmaxf(m_n, Mp[(static_cast<size_t>(s) * B + b) * H + h]);
  if (m_n == -INFINITY) {
    // nothing visible anywhere: the state stays as it is (or is written empty)
    if (fresh || finalize) {
      O[row * D + d] = 0.f;
      if (fresh && d == 0) {
        M[row] = -INFINITY;
        L[row] = 0.f;
      }
    }
    return;
  }
  const float a = (m_old == -INFINITY) ? 0.f : expf(m_old - m_n);
  float o_acc = (m_old == -INFINITY) ? 0.f : a * O[row * D + d];
  float l_acc = (m_old == -INFINITY) ? 0.f : a * L[row];
  for (int s = 0; s < n_split; ++s) {
    const size_t prow = (static_cast<size_t>(s) * B + b) * H + h;
    const float ms = Mp[prow];
    const float sc = (ms == -INFINITY) ? 0.f : expf(ms - m_n);
    o_acc += sc * Op[prow * D + d];
    l_acc += sc * Lp[prow];
  }
  if (finalize) o_acc *= l_acc > 0.f ? 1.f / l_acc : 0.f;
  O[row * D + d] = o_acc;
  __syncthreads();  // every thread has read M/L before thread 0 overwrites them
  if (d == 0) {
    M[row] = m_n;
    L[row] = l_acc;
  }
}

struct Plan {
  int n_split;
  int rows_per_split;
  int gb;
  int head_batches;
};

int sm_count() {
  int dev = 0, v = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
  return v > 0 ? v : 148;
}

Plan make_plan(int B, int H, int kvH, int sk_eff, int rows_per_stage, int sms,
               int split_cap = kMaxSplits) {
  Plan p;
  const int group = (H + kvH - 1) / kvH;  // query heads per KV head (largest group)
  p.gb = group > 4 ? 8 : (group > 2 ? 4 : (group > 1 ? 2 : 1));  // smallest of 1/2/4/8 that fits
  p.head_batches = (group + p.gb - 1) / p.gb;
  const int blocks_per_split = B * kvH * p.head_batches;
  int want = (3 * sms + blocks_per_split - 1) / blocks_per_split;
  const int max_by_rows = std::max(1, sk_eff / (2 * rows_per_stage));
  want = std::max(1, std::min(std::min(want, max_by_rows), split_cap));
  int rps = (sk_eff + want - 1) / want;
  rps = ((rps + rows_per_stage - 1) / rows_per_stage) * rows_per_stage;
  if (rps < rows_per_stage) rps = rows_per_stage;
  p.rows_per_split = rps;
  p.n_split = std::max(1, (sk_eff + rps - 1) / rps);
  return p;
}

// Per-device workspace that grows on demand, like the reference's process-static buffer
// (src/attention_decode.cu:55-65). Not safe for concurrent streams, as the reference's.
struct DevWorkspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};
DevWorkspace g_ws[64];
std::mutex g_ws_mu;

int ensure_workspace(size_t need, void** out) {
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  RAB_REQUIRE(dev >= 0 && dev < 64, RA_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_ws_mu);
  DevWorkspace& w = g_ws[dev];
  if (w.bytes < need) {
    if (w.ptr) RAB_CUDA(cudaFree(w.ptr));
    w.ptr = nullptr;
    w.bytes = 0;
    RAB_CUDA(cudaMalloc(&w.ptr, need));
    w.bytes = need;
  }
  *out = w.ptr;
  return RA_OK;
}

}  // namespace

int decode_ml_scratch(size_t floats, float** out) {
  static DevWorkspace ml[64];
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  RAB_REQUIRE(dev >= 0 && dev < 64, RA_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_ws_mu);
  DevWorkspace& w = ml[dev];
  const size_t need = floats * sizeof(float);
  if (w.bytes < need) {
    if (w.ptr) RAB_CUDA(cudaFree(w.ptr));
    w.ptr = nullptr;
    w.bytes = 0;
    RAB_CUDA(cudaMalloc(&w.ptr, need));
    w.bytes = need;
  }
  *out = static_cast<float*>(w.ptr);
  return RA_OK;
}

namespace {

template <typename T, int D>
int launch_decode_typed(const void* q, const void* k, const void* v, float* out, float* m,
                        float* l, const ra_shape& s, int sk_eff, long long kv_head_stride,
                        void* workspace, size_t workspace_bytes, cudaStream_t stream,
                        int split_cap = kMaxSplits, unsigned flags = 0) {
  if constexpr (sizeof(T) == 2 && D >= 64) {
    // 16-bit caches: the tensor-core kernel (16 query heads per block, 64-key stages)
    using M = MmaCfg<D>;
    const int kvH = kv_heads_of(s);
    const int group = (s.heads + kvH - 1) / kvH;
    const int head_batches = (group + 15) / 16;
    const int blocks_per_split = s.batch * kvH * head_batches;
    int want = (3 * sm_count() + blocks_per_split - 1) / blocks_per_split;
    want = std::max(1, std::min(std::min(want, std::max(1, sk_eff / (2 * kMmaStageRows))),
                                split_cap));
    int rps = (sk_eff + want - 1) / want;
    rps = ((rps + kMmaStageRows - 1) / kMmaStageRows) * kMmaStageRows;
    const int n_split = std::max(1, (sk_eff + rps - 1) / rps);
    const size_t prow = static_cast<size_t>(n_split) * s.batch * s.heads;
    const size_t need = prow * (D + 2) * sizeof(float);
    if (workspace == nullptr) {
      const int rc = ensure_workspace(need, &workspace);
      if (rc != RA_OK) return rc;
    } else {
      RAB_REQUIRE(workspace_bytes >= need, RA_ERR_OVERFLOW,
                  "decode workspace too small: %zu < %zu bytes", workspace_bytes, need);
    }
    float* Mp = static_cast<float*>(workspace);
    float* Lp = Mp + prow;
    float* Op = Lp + prow;
    const float scale_log2 = kLog2e / sqrtf(static_cast<float>(D));
    const size_t red_bytes = static_cast<size_t>(kMmaWarps) * 16 * (D + 2) * sizeof(float);
    const size_t smem = std::max(static_cast<size_t>(M::kSmemBytes), red_bytes);
    auto kern = decode_mma_kernel<T, D>;
    RAB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    kern<<<dim3(n_split, kvH * head_batches, s.batch), kMmaThreads, smem, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), Mp, Lp, Op,
        s.batch, s.heads, kvH, sk_eff, kv_head_stride, rps, head_batches, scale_log2);
    RAB_CUDA(cudaGetLastError());
    decode_reduce_kernel<<<dim3(s.heads, s.batch), D, 0, stream>>>(Mp, Lp, Op, m, l, out, s.batch,
                                                                   s.heads, D, n_split, flags);
    RAB_CUDA(cudaGetLastError());
    return RA_OK;
  }
  using C = DecodeCfg<T, D>;
  const int kvH = kv_heads_of(s);
  const Plan p =
      make_plan(s.batch, s.heads, kvH, sk_eff, C::kRowsPerStage, sm_count(), split_cap);
  const size_t prow = static_cast<size_t>(p.n_split) * s.batch * s.heads;
  const size_t need = prow * (D + 2) * sizeof(float);
  if (workspace == nullptr) {
    const int rc = ensure_workspace(need, &workspace);
    if (rc != RA_OK) return rc;
  } else {
    RAB_REQUIRE(workspace_bytes >= need, RA_ERR_OVERFLOW,
                "decode workspace too small: %zu < %zu bytes", workspace_bytes, need);
  }
  float* Mp = static_cast<float*>(workspace);
  float* Lp = Mp + prow;
  float* Op = Lp + prow;
  const float scale_log2 = kLog2e / sqrtf(static_cast<float>(D));
  const dim3 grid(p.n_split, kvH * p.head_batches, s.batch);
  const size_t red_bytes = static_cast<size_t>(kWarps) * 8 * (D + 2) * sizeof(float);
  const size_t smem = std::max(static_cast<size_t>(C::kSmemBytes), red_bytes);
#define RAB_DECODE_GB(GBV)                                                                     \
  case GBV: {                                                                                  \
    auto kern = decode_split_kernel<T, D, GBV>;                                                \
    RAB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                  static_cast<int>(smem)));                                    \
    kern<<<grid, kThreads, smem, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k), \
                                           static_cast<const T*>(v), Mp, Lp, Op, s.batch,      \
                                           s.heads, kvH, sk_eff, kv_head_stride,               \
                                           p.rows_per_split, p.head_batches, scale_log2);      \
  } break;
  switch (p.gb) {
    RAB_DECODE_GB(1)
    RAB_DECODE_GB(2)
    RAB_DECODE_GB(4)
    RAB_DECODE_GB(8)
  }
#undef RAB_DECODE_GB
  RAB_CUDA(cudaGetLastError());
  decode_reduce_kernel<<<dim3(s.heads, s.batch), D, 0, stream>>>(Mp, Lp, Op, m, l, out, s.batch,
                                                                 s.heads, D, p.n_split, flags);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

template <typename T>
int launch_decode_dtype(const void* q, const void* k, const void* v, float* out, float* m,
                        float* l, const ra_shape& s, int sk_eff, long long kv_head_stride,
                        void* ws, size_t ws_bytes, cudaStream_t stream,
                        int split_cap = kMaxSplits, unsigned flags = 0) {
  switch (s.head_dim) {
    case 32:
      return launch_decode_typed<T, 32>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                        ws_bytes, stream, split_cap, flags);
    case 64:
      return launch_decode_typed<T, 64>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                        ws_bytes, stream, split_cap, flags);
    case 128:
      return launch_decode_typed<T, 128>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                         ws_bytes, stream, split_cap, flags);
    case 256:
      return launch_decode_typed<T, 256>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                         ws_bytes, stream, split_cap, flags);
  }
  set_error("attention_decode_step: unsupported head_dim=%d (supported: 32, 64, 128, 256)",
            s.head_dim);
  return RA_ERR_UNSUPPORTED;
}

}  // namespace

int decode_step(int dtype, const void* q, const void* k, const void* v, float* out, float* m,
                float* l, const ra_shape& s, int q_offset, int k_offset, int causal,
                cudaStream_t stream, int kv_row_stride, void* ws, size_t ws_bytes,
                unsigned flags) {
  RAB_REQUIRE(q && k && v && out && m && l, RA_ERR_INVALID, "decode step: null argument");
  RAB_REQUIRE(s.seq_q == 1, RA_ERR_INVALID, "decode step: seq_q must be 1 (got %d)", s.seq_q);
  RAB_REQUIRE(s.batch > 0 && s.heads > 0 && s.batch <= 65535, RA_ERR_INVALID,
              "decode step: bad batch/heads");
  RAB_REQUIRE((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
               reinterpret_cast<uintptr_t>(v)) % 16 == 0,
              RA_ERR_INVALID, "decode step: q, k and v must be 16-byte aligned");
  int sk_eff = s.seq_k;
  if (causal) {
    // rows [0, q_offset - k_offset] are visible (reference: src/attention_decode.cu:110-116)
    const long long vis = static_cast<long long>(q_offset) - k_offset + 1;
    if (vis < sk_eff) sk_eff = vis < 0 ? 0 : static_cast<int>(vis);
  }
  if (sk_eff <= 0) {
    // nothing visible: the state stays as it is, or is written empty / normalised on request
    const size_t rows = static_cast<size_t>(s.batch) * s.heads;
    if (flags & RA_STEP_FRESH) return launch_init(out, m, l, rows * s.head_dim, rows, stream);
    if (flags & RA_STEP_FINALIZE) return launch_finalize(out, l, rows, s.head_dim, stream);
    return RA_OK;
  }
  const int stride_rows = kv_row_stride > 0 ? kv_row_stride : s.seq_k;
  const long long kv_head_stride = static_cast<long long>(stride_rows) * s.head_dim;
  switch (dtype) {
    case RA_F32:
      return launch_decode_dtype<float>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                        ws_bytes, stream, kMaxSplits, flags);
    case RA_F16:
      return launch_decode_dtype<__half>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                         ws_bytes, stream, kMaxSplits, flags);
    case RA_BF16:
      return launch_decode_dtype<__nv_bfloat16>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, ws,
                                                ws_bytes, stream, kMaxSplits, flags);
  }
  set_error("decode step: unknown dtype %d", dtype);
  return RA_ERR_INVALID;
}

// ---- decode step that never allocates --------------------------------------------------
//
// Some hosts of this library may not call cudaMalloc at all: a serving process that handed
// its whole memory budget to one arena at start-up, a caller inside a region where the
// allocator is locked (a stream being captured, a real-time loop that must not take the
// driver's allocation lock), or an embedder whose policy forbids a library to allocate behind
// its back. For them the split partials live in a fixed array that is part of the library
// image: every GPU that loads the library holds these kStaticScratchFloats * 4 bytes (1 MiB)
// until the process exits.
constexpr size_t kStaticScratchFloats = 262144;  // 1 MiB
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

// Device address of the array on the CURRENT device. In host code the array's name is only a
// host-side handle for the symbol, never a device pointer, so the address is asked for once
// per device (with that device current) and cached.
int static_scratch_ptr(float** out) {
  static float* cache[64] = {};
  static std::mutex mu;
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  RAB_REQUIRE(dev >= 0 && dev < 64, RA_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    RAB_CUDA(cudaGetSymbolAddress(&p, g_decode_static_scratch));
    RAB_REQUIRE(p != nullptr, RA_ERR_CUDA, "no device address for the static decode scratch");
    cache[dev] = static_cast<float*>(p);
  }
  *out = cache[dev];
  return RA_OK;
}

int decode_step_noalloc(int dtype, const void* q, const void* k, const void* v, float* out,
                        float* m, float* l, const ra_shape& s, int q_offset, int k_offset,
                        int causal, cudaStream_t stream, int kv_row_stride) {
  RAB_REQUIRE(q && k && v && out && m && l, RA_ERR_INVALID, "decode step: null argument");
  RAB_REQUIRE(s.seq_q == 1, RA_ERR_INVALID, "decode step: seq_q must be 1 (got %d)", s.seq_q);
  RAB_REQUIRE(s.batch > 0 && s.heads > 0 && s.batch <= 65535, RA_ERR_INVALID,
              "decode step: bad batch/heads");
  RAB_REQUIRE(s.head_dim == 32 || s.head_dim == 64 || s.head_dim == 128 || s.head_dim == 256,
              RA_ERR_UNSUPPORTED,
              "attention_decode_step: unsupported head_dim=%d (supported: 32, 64, 128, 256)",
              s.head_dim);
  RAB_REQUIRE((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
               reinterpret_cast<uintptr_t>(v)) % 16 == 0,
              RA_ERR_INVALID, "decode step: q, k and v must be 16-byte aligned");
  // One split needs batch * heads * (head_dim + 2) floats; the array must hold at least one.
  const size_t per_split = static_cast<size_t>(s.batch) * s.heads * (s.head_dim + 2);
  RAB_REQUIRE(per_split <= kStaticScratchFloats, RA_ERR_OVERFLOW,
              "ra_attention_decode_step_noalloc: batch*heads*(head_dim+2) = %zu floats exceeds the "
              "built-in scratch of %zu floats (1 MiB); use ra_attention_decode_step with a "
              "caller-provided workspace",
              per_split, kStaticScratchFloats);
  const int split_cap =
      static_cast<int>(std::min<size_t>(kMaxSplits, kStaticScratchFloats / per_split));
  float* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != RA_OK) return rc;
  int sk_eff = s.seq_k;
  if (causal) {
    const long long vis = static_cast<long long>(q_offset) - k_offset + 1;
    if (vis < sk_eff) sk_eff = vis < 0 ? 0 : static_cast<int>(vis);
  }
  if (sk_eff <= 0) return RA_OK;
  const int stride_rows = kv_row_stride > 0 ? kv_row_stride : s.seq_k;
  const long long kv_head_stride = static_cast<long long>(stride_rows) * s.head_dim;
  const size_t bytes = kStaticScratchFloats * sizeof(float);
  // Nothing in the array has to start at zero: every (split, batch, head) slot the reduce
  // kernel reads is written by the split kernel of the same call first.
  switch (dtype) {
    case RA_F32:
      return launch_decode_dtype<float>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, scratch,
                                        bytes, stream, split_cap);
    case RA_F16:
      return launch_decode_dtype<__half>(q, k, v, out, m, l, s, sk_eff, kv_head_stride, scratch,
                                         bytes, stream, split_cap);
    case RA_BF16:
      return launch_decode_dtype<__nv_bfloat16>(q, k, v, out, m, l, s, sk_eff, kv_head_stride,
                                                scratch, bytes, stream, split_cap);
  }
  set_error("decode step: unknown dtype %d", dtype);
  return RA_ERR_INVALID;
}

}  // namespace rab

extern "C" {

int ra_attention_decode_step_noalloc(int dtype, const void* q, const void* k, const void* v,
                                     float* out, float* m, float* l, const ra_shape* shape,
                                     int q_offset, int k_offset, int causal, ra_stream stream,
                                     int kv_row_stride) {
  RAB_REQUIRE(shape != nullptr, RA_ERR_INVALID, "ra_attention_decode_step_noalloc: null shape");
  return rab::decode_step_noalloc(dtype, q, k, v, out, m, l, *shape, q_offset, k_offset, causal,
                                  static_cast<cudaStream_t>(stream), kv_row_stride);
}

size_t ra_decode_workspace_bytes(const ra_shape* shape) {
  if (!shape) return 0;
  return static_cast<size_t>(rab::kMaxSplits) * shape->batch * shape->heads *
         (static_cast<size_t>(shape->head_dim) + 2) * sizeof(float);
}

int ra_attention_decode_step(int dtype, const void* q, const void* k, const void* v, float* out,
                             float* m, float* l, const ra_shape* shape, int q_offset, int k_offset,
                             int causal, ra_stream stream, int kv_row_stride, void* workspace,
                             size_t workspace_bytes) {
  RAB_REQUIRE(shape != nullptr, RA_ERR_INVALID, "ra_attention_decode_step: null shape");
  return rab::decode_step(dtype, q, k, v, out, m, l, *shape, q_offset, k_offset, causal,
                          static_cast<cudaStream_t>(stream), kv_row_stride, workspace,
                          workspace_bytes);
}

}  // extern "C"
