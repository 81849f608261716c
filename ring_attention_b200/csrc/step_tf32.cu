// Blackwell (sm_100a) ring step for fp32 Q/K/V on the tensor cores: the same FlashAttention-style
// forward as step_tc.cu (TMA, tcgen05.mma, tensor memory) with every operand split into two TF32
// terms, x ~ hi + lo (hi = x rounded to TF32, lo = x - hi rounded to TF32), and every product
// taken as hi*hi + lo*hi + hi*lo with fp32 accumulation. What is dropped (lo*lo and the rounding
// of lo) is about 2^-22 of each product, unbiased, against the 2^-24 of an fp32 multiply-add: for
// inputs of the reference's tests and benchmarks (N(0,1), U[-1,1)) the result meets the fp32
// tolerance (1e-5) of the reference's fp32 step (src/attention_step.cu:114-282), which this
// replaces for head_dim 32, 64 and 128 at ~15x the speed of the SIMT kernel. Scores whose single
// products reach the hundreds lose that margin (error ~ 2^-22 * sum |q_d k_d| / sqrt(D) in the
// exponent); RA_STEP_FORCE_SIMT selects the plain-fp32 kernel. Head_dim 256 keeps the SIMT kernel
// (its Q tile and lo copy alone exceed shared memory).
//
// Work decomposition: grid = (batch * heads, 128-row query blocks); a block owns one 128-row
// query tile and walks the visible 64-key tiles (32-key at head_dim 128) of every key segment,
// heaviest blocks first.
//
// Roles inside a block (384 threads)
//   warp 0        TMA producer: Q once, then K_t, V_t, K_t+1, ... as 128B-swizzled fp32 tiles into
//                 a 4-slot (head_dim 128: 3-slot) shared-memory ring (no multicast).
//   warp 1        MMA issuer (converged warp, one elected lane): S = Qh Kh^T + Ql Kh^T + Qh Kl^T
//                 and O += Ph V_h + Pl V_h + Ph V_l, kind::tf32, accumulators in tensor memory.
//   warps 4-7     splitter: when a raw tile has landed, rounds it to TF32 in place (hi) and writes
//                 the lo tile next to it, element for element in the same swizzled layout.
//   warps 8-11    softmax, one thread per row: P = 2^(s * scale - m_ref) with the lazily moved
//                 reference point of step_tc.cu, written to tensor memory as Ph and Pl; epilogue.
//   S and P are double-buffered, so the scores of tile t+1 are computed while the softmax of
//   tile t runs and the softmax of tile t+1 never waits for P.V of tile t.
//
// Tensor memory (columns, n = keys per tile): S0 S1 [0,2n) Ph0 Pl0 Ph1 Pl1 [2n,6n) O [6n,6n+D).
// Every wait on an mbarrier is bounded (see tc_common.cuh); a wait that runs out reports into
// the device status word and the block unwinds.
#include "tc_common.cuh"

namespace rab {

using namespace tcgen;

namespace {

constexpr int kThreadsF = 384;

template <int D>
struct F32Cfg {
  // head_dim 128: Q with its lo copy is 128 KiB, so the key tile shrinks to 32 keys and the ring
  // to three slots (K_t, V_t and the K of the next tile) to fit beside it
  static constexpr int kBN = D == 128 ? 32 : 64;        // keys per tile
  static constexpr int kStages = D == 128 ? 3 : 4;      // ring slots (raw + lo of one K or V tile)
  static constexpr int kBoxes = D / 32;                 // 32 fp32 = one 128-byte box row
  static constexpr int kQBytes = kBM * D * 4;           // one Q tile (hi or lo)
  static constexpr int kKvBytes = kBN * D * 4;          // one K or V tile (hi or lo)
  static constexpr int kOffQ = 0;                       // hi, then lo
  static constexpr int kOffKV = 2 * kQBytes;            // slot: hi, then lo
  static constexpr int kOffBar = kOffKV + kStages * 2 * kKvBytes;
  static constexpr int kNumBars = 2 + 3 * kStages + 8;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
  // tensor memory: S0 S1 (kBN columns each), Ph0 Pl0 Ph1 Pl1 (kBN each), O (D)
  static constexpr int kColS = 0, kColP = 2 * kBN, kColO = 6 * kBN;
  static_assert(kColO + D <= 512, "tensor memory budget");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// x rounded to the nearest TF32 value (sign, exponent, 10 mantissa bits; the low 13 bits of the
// word are zero, so the tensor core, which ignores them, reads exactly this number). Rounding
// instead of letting the hardware truncate keeps the split free of a systematic bias.
__device__ inline float tf32_round(float x) {
  unsigned u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

__device__ inline void mma_ss_tf32(unsigned d_tmem, unsigned long long a_desc,
                                   unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ inline void mma_ts_tf32(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                   unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(kThreadsF, 1)
    step_tf32_kernel(const __grid_constant__ CUtensorMap tmap_q,
                     const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const TcArgs a) {
  using C = F32Cfg<D>;
  constexpr int kBNf = C::kBN;
  constexpr int kStagesF = C::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const unsigned s_base = smem_u32(smem);
  const unsigned s_q = s_base + C::kOffQ;
  const unsigned s_kv = s_base + C::kOffKV;
  const unsigned s_bar = s_base + C::kOffBar;
  const unsigned bar_q_raw = s_bar;                              // TMA bytes of Q
  const unsigned bar_q_full = s_bar + 8;                         // Q lo written
  const unsigned bar_kv_raw = s_bar + 16;                        // [kStagesF] TMA bytes
  const unsigned bar_kv_full = bar_kv_raw + 8 * kStagesF;        // [kStagesF] lo written
  const unsigned bar_kv_empty = bar_kv_full + 8 * kStagesF;      // [kStagesF] MMAs done
  const unsigned bar_s_full = bar_kv_empty + 8 * kStagesF;       // [2]
  const unsigned bar_s_free = bar_s_full + 16;                   // [2] S held in registers
  const unsigned bar_p_full = bar_s_free + 16;                   // [2]
  const unsigned bar_o_done = bar_p_full + 16;                   // [2] P.V of the buffer done
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + C::kOffBar + C::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;

  if (__syncthreads_or(*reinterpret_cast<volatile int*>(a.status) != 0)) return;

  const bool causal = (a.flags & RA_STEP_CAUSAL) != 0;
  const bool fresh = (a.flags & RA_STEP_FRESH) != 0;
  const bool finalize = (a.flags & RA_STEP_FINALIZE) != 0;

  const int bh = blockIdx.x;
  const int qb_lin = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  const int sq = qb_lin / a.n_qblocks_per_seg;
  const int tq = qb_lin - sq * a.n_qblocks_per_seg;
  const int h = bh % a.H;
  const int b = bh / a.H;
  const int kv_bh = b * a.kvH + (h % a.kvH);
  const int q_seg_len = a.qmap.seg_len;
  const int row0 = tq * kBM;
  const int rows_in_block = min(kBM, q_seg_len - row0);
  const int qmin = a.qmap.base[sq] + row0 * a.stride;
  const int qmax = a.qmap.base[sq] + (row0 + rows_in_block - 1) * a.stride;

  int n_tiles = 0;
  for (int sk = 0; sk < a.kmap.n_seg; ++sk) {
    const TileRange r = tile_range<kBNf>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
    n_tiles += r.hi - r.lo;
  }

  if (tid == 0) {
    mbar_init(bar_q_raw, 1);
    mbar_init(bar_q_full, 128);
    for (int s = 0; s < kStagesF; ++s) {
      mbar_init(bar_kv_raw + 8 * s, 1);
      mbar_init(bar_kv_full + 8 * s, 128);
      mbar_init(bar_kv_empty + 8 * s, 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar_s_full + 8 * w, 1);
      mbar_init(bar_s_free + 8 * w, kBM);
      mbar_init(bar_p_full + 8 * w, kBM);
      mbar_init(bar_o_done + 8 * w, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                     smem_u32(tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ----
    if (lane == 0 && n_tiles > 0) {
      const int q_row = sq * q_seg_len + row0;
      mbar_expect_tx(bar_q_raw, C::kQBytes);
      for (int bx = 0; bx < C::kBoxes; ++bx)
        tma_load_3d(s_q + bx * (kBM * 128), &tmap_q, bar_q_raw, bx * 32, q_row, bh);
      int it = 0;
      bool ok = true;
      for (int sk = 0; sk < a.kmap.n_seg && ok; ++sk) {
        const TileRange r = tile_range<kBNf>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
        for (int t = r.lo; t < r.hi && ok; ++t) {
          const int k_row = a.kseg_row[sk] + t * kBNf;
          const int k_head = a.kseg_head[sk] + kv_bh;
          for (int which = 0; which < 2 && ok; ++which, ++it) {
            const int slot = it % kStagesF;
            if (it >= kStagesF)
              ok = mbar_wait(bar_kv_empty + 8 * slot, ((it / kStagesF) + 1) & 1, abort_flag, a.status,
                             1, it, a.wait_ns);
            if (!ok) break;
            if (a.stall_after >= 0 && it >= a.stall_after) {  // test hook, see step_tc.cu
              ok = false;
              break;
            }
            mbar_expect_tx(bar_kv_raw + 8 * slot, C::kKvBytes);
            const CUtensorMap* map = which == 0 ? &tmap_k : &tmap_v;
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_3d(s_kv + slot * 2 * C::kKvBytes + bx * (kBNf * 128), map,
                          bar_kv_raw + 8 * slot, bx * 32, k_row, k_head);
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer ----
    if (n_tiles > 0) {
      constexpr unsigned idesc_s = make_idesc(2u, 0, kBNf, kBM);  // tf32 x tf32 -> fp32, B K-major
      constexpr unsigned idesc_pv = make_idesc(2u, 1, D, kBM);    // B (V) MN-major
      constexpr unsigned kQBox = (kBM * 128) >> 4;                // one 32-element box of Q, 16-byte units
      constexpr unsigned kKvBox = (kBNf * 128) >> 4;
      const unsigned long long qd_hi = desc_kmajor(s_q);
      const unsigned long long qd_lo = desc_kmajor(s_q + C::kQBytes);
      auto wait = [&](unsigned bar, unsigned parity, int which, int tile) {
        return __all_sync(0xffffffffu,
                          mbar_wait(bar, parity, abort_flag, a.status, which, tile, a.wait_ns)) != 0;
      };
      // ring item of K_t: 2t, of V_t: 2t + 1
      auto do_s = [&](int t) {
        const int it = 2 * t, slot = it % kStagesF, buf = t & 1;
        if (!wait(bar_kv_full + 8 * slot, (it / kStagesF) & 1, 5, t)) return false;
        tc_fence_after();
        const unsigned kv = s_kv + slot * 2 * C::kKvBytes;
        const unsigned long long kd_hi = desc_kmajor(kv), kd_lo = desc_kmajor(kv + C::kKvBytes);
        const unsigned t_s = tmem_base + C::kColS + kBNf * buf;
        if (elect_one()) {
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const unsigned long long qd = term == 1 ? qd_lo : qd_hi;  // hi*hi, lo*hi, hi*lo
            const unsigned long long kd = term == 2 ? kd_lo : kd_hi;
#pragma unroll
            for (int ks = 0; ks < D / 8; ++ks) {  // 8 fp32 = 32 bytes per k-step, 4 steps per box
              const unsigned off_q = (ks / 4) * kQBox + (ks % 4) * 2;
              const unsigned off_k = (ks / 4) * kKvBox + (ks % 4) * 2;
              mma_ss_tf32(t_s, qd + off_q, kd + off_k, idesc_s, (term > 0 || ks > 0) ? 1u : 0u);
            }
          }
          tc_commit(bar_s_full + 8 * buf);
          tc_commit(bar_kv_empty + 8 * slot);
        }
        return true;
      };
      auto do_pv = [&](int t) {
        const int it = 2 * t + 1, slot = it % kStagesF, buf = t & 1;
        if (!wait(bar_kv_full + 8 * slot, (it / kStagesF) & 1, 4, t)) return false;
        tc_fence_after();
        const unsigned kv = s_kv + slot * 2 * C::kKvBytes;
        // MN-major V (loaded with the 32-byte-atom swizzle a 32-bit MN-major operand needs): 32
        // head_dim columns per 128-byte row, boxes kBNf * 128 bytes apart, 8 keys (two 4-row
        // groups, 1 KiB) per k-step
        const unsigned long long vd_hi = desc_mnmajor_32b(kv, kBNf * 128, 512);
        const unsigned long long vd_lo = desc_mnmajor_32b(kv + C::kKvBytes, kBNf * 128, 512);
        const unsigned t_ph = tmem_base + C::kColP + 2 * kBNf * buf, t_pl = t_ph + kBNf;
        const unsigned t_o = tmem_base + C::kColO;
        if (elect_one()) {
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            const unsigned t_p = term == 1 ? t_pl : t_ph;  // hi*hi, lo*hi, hi*lo
            const unsigned long long vd = term == 2 ? vd_lo : vd_hi;
#pragma unroll
            for (int ks = 0; ks < kBNf / 8; ++ks)
              mma_ts_tf32(t_o, t_p + ks * 8, vd + ks * (1024 >> 4), idesc_pv,
                          (t > 0 || term > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(bar_o_done + 8 * buf);
          tc_commit(bar_kv_empty + 8 * slot);
        }
        return true;
      };
      bool ok = wait(bar_q_full, 0, 3, 0) && do_s(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) {
          // S buffer (t+1) & 1 last held tile t-1: its softmax must have the scores in registers
          if (t >= 1) ok = wait(bar_s_free + 8 * ((t + 1) & 1), ((t - 1) >> 1) & 1, 9, t);
          ok = ok && do_s(t + 1);
        }
        ok = ok && wait(bar_p_full + 8 * (t & 1), (t >> 1) & 1, 6, t) && do_pv(t);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------------------------------------------------------- splitter ----
    // every element of a landed tile becomes hi = tf32(x), in place, and lo = tf32(x - hi) at the
    // same place of the (swizzled) layout in the slot's second half
    if (n_tiles > 0) {
      const int st = tid - 128;
      auto split = [&](unsigned raw, unsigned lo, int bytes) {
        for (int off = st * 16; off < bytes; off += 128 * 16) {
          float4 x;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                       : "r"(raw + off));
          float4 hi, lw;
          hi.x = tf32_round(x.x);
          hi.y = tf32_round(x.y);
          hi.z = tf32_round(x.z);
          hi.w = tf32_round(x.w);
          lw.x = tf32_round(x.x - hi.x);
          lw.y = tf32_round(x.y - hi.y);
          lw.z = tf32_round(x.z - hi.z);
          lw.w = tf32_round(x.w - hi.w);
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(raw + off), "f"(hi.x), "f"(hi.y),
                       "f"(hi.z), "f"(hi.w)
                       : "memory");
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(lo + off), "f"(lw.x), "f"(lw.y),
                       "f"(lw.z), "f"(lw.w)
                       : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      };
      bool ok = mbar_wait(bar_q_raw, 0, abort_flag, a.status, 12, 0, a.wait_ns);
      if (ok) {
        split(s_q, s_q + C::kQBytes, C::kQBytes);
        mbar_arrive(bar_q_full);
      }
      for (int it = 0; it < 2 * n_tiles && ok; ++it) {
        const int slot = it % kStagesF;
        ok = mbar_wait(bar_kv_raw + 8 * slot, (it / kStagesF) & 1, abort_flag, a.status, 13, it, a.wait_ns);
        if (!ok) break;
        const unsigned kv = s_kv + slot * 2 * C::kKvBytes;
        split(kv, kv + C::kKvBytes, C::kKvBytes);
        mbar_arrive(bar_kv_full + 8 * slot);
      }
    }
  } else if (warp >= 8) {
    // ----------------------------------------------------------------- softmax ----
    const int row = ((warp & 3) << 5) + lane;  // row of the tile = tensor-memory lane
    const unsigned lane_base = static_cast<unsigned>((warp & 3) << 5) << 16;
    const unsigned t_o = tmem_base + lane_base + C::kColO;
    const int r_in_seg = row0 + row;
    const bool row_valid = r_in_seg < q_seg_len;
    const int qpos = a.qmap.base[sq] + r_in_seg * a.stride;
    const long long qdoc = a.doc_len > 0 ? qpos / a.doc_len : 0;
    const float scale_log2 = rsqrtf(static_cast<float>(D)) * kLog2e;
    // P is fp32 here, so the reference point only has to keep the sums in range
    constexpr float kSumLimit = 1.0e12f;

    float m_ref = -INFINITY;  // reference point of P, O and l, log2 units
    float l_run = 0.f;
    bool ok = true;
    int j = 0;
    for (int sk = 0; sk < a.kmap.n_seg && ok; ++sk) {
      const TileRange tr = tile_range<kBNf>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
      // visible local key indices [rel_lo, rel_hi) of this segment for this row
      int rel_lo = 0, rel_hi = row_valid ? a.kmap.seg_len : 0;
      {
        const long long kb = a.kmap.base[sk];
        if (causal) {
          const long long d = static_cast<long long>(qpos) - kb;
          rel_hi = d < 0 ? 0 : static_cast<int>(min(static_cast<long long>(rel_hi), d / a.stride + 1));
        }
        if (a.doc_len > 0) {
          const long long p_lo = qdoc * a.doc_len, p_hi = p_lo + a.doc_len - 1;
          if (p_hi < kb) {
            rel_hi = 0;
          } else {
            rel_hi = static_cast<int>(min(static_cast<long long>(rel_hi), (p_hi - kb) / a.stride + 1));
            if (p_lo > kb)
              rel_lo = static_cast<int>(min(static_cast<long long>(a.kmap.seg_len),
                                            (p_lo - kb + a.stride - 1) / a.stride));
          }
        }
      }
      for (int t = tr.lo; t < tr.hi && ok; ++t, ++j) {
        const int buf = j & 1;
        const unsigned t_s = tmem_base + lane_base + C::kColS + kBNf * buf;
        const unsigned t_ph = tmem_base + lane_base + C::kColP + 2 * kBNf * buf, t_pl = t_ph + kBNf;
        int c_lo = min(max(rel_lo - t * kBNf, 0), kBNf);
        int c_hi = min(max(rel_hi - t * kBNf, 0), kBNf);
        if (c_hi < c_lo) c_hi = c_lo;
        const bool full = __all_sync(0xffffffffu, c_lo == 0 && c_hi == kBNf);

        ok = mbar_wait(bar_s_full + 8 * buf, (j >> 1) & 1, abort_flag, a.status, 7, j, a.wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float s[kBNf];
#pragma unroll
        for (int c = 0; c < kBNf / 32; ++c) {
          float part[32];
          tmem_ld32(t_s + 32 * c, part);
#pragma unroll
          for (int i = 0; i < 32; ++i) s[32 * c + i] = part[i];
        }
        tc_fence_before();
        mbar_arrive(bar_s_free + 8 * buf);  // the tensor core may reuse this S buffer
        if (!full) {
#pragma unroll
          for (int i = 0; i < kBNf; ++i) s[i] = (i >= c_lo && i < c_hi) ? s[i] : -INFINITY;
        }
        // wait for P.V of tile t to have completed (its P buffer / O are then free to touch)
        auto wait_pv = [&](int t_done) {
          if (t_done < 0 || !ok) return;
          ok = mbar_wait(bar_o_done + 8 * (t_done & 1), (t_done >> 1) & 1, abort_flag, a.status, 10, j,
                         a.wait_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) tc_fence_after();
        };
        float row_sum = 0.f;
        // P = 2^(s * scale - m_ref) as hi + lo in tensor memory, 32 columns at a time
        auto exponentials = [&](float neg_m) {
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int c = 0; c < kBNf / 32; ++c) {
            float ph[32], pl[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = ex2(fmaf(s[32 * c + i], scale_log2, neg_m));
              const float p1 = ex2(fmaf(s[32 * c + i + 1], scale_log2, neg_m));
              sum0 += p0;
              sum1 += p1;
              ph[i] = tf32_round(p0);
              ph[i + 1] = tf32_round(p1);
              pl[i] = tf32_round(p0 - ph[i]);
              pl[i + 1] = tf32_round(p1 - ph[i + 1]);
            }
            tmem_st32(t_ph + 32 * c, ph);
            tmem_st32(t_pl + 32 * c, pl);
          }
          row_sum = sum0 + sum1;
        };
        bool slow = __any_sync(0xffffffffu, m_ref == -INFINITY && c_hi > c_lo) != 0;
        wait_pv(j - 2);  // this P buffer was last read by P.V of tile j-2
        if (!ok) break;
        if (!slow) {
          exponentials(m_ref == -INFINITY ? 0.f : -m_ref);
          slow = __any_sync(0xffffffffu, !(row_sum <= kSumLimit)) != 0;  // also catches NaN
        }
        if (slow) {
          wait_pv(j - 1);  // O must be at rest before it is rescaled
          if (!ok) break;
          float mx = s[0];
#pragma unroll
          for (int i = 1; i < kBNf; ++i) mx = fmaxf(mx, s[i]);
          const float tile_max = mx * scale_log2;  // -inf stays -inf
          float alpha = 1.f;
          bool rescale = false;
          if (tile_max > m_ref) {
            if (m_ref > -INFINITY) {
              alpha = ex2(m_ref - tile_max);
              rescale = true;
            }
            m_ref = tile_max;
          }
          if (j > 0 && __any_sync(0xffffffffu, rescale)) {
            l_run *= alpha;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              float o[32];
              tmem_ld32(t_o + c * 32, o);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= alpha;
              tmem_st32(t_o + c * 32, o);
            }
          }
          exponentials(m_ref == -INFINITY ? 0.f : -m_ref);
        }
        l_run += row_sum;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full + 8 * buf);
      }
    }

    // ---------------------------------------------------------------- epilogue ----
    if (ok && n_tiles > 0)
      ok = mbar_wait(bar_o_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag,
                     a.status, 8, n_tiles, a.wait_ns);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const size_t grow = (static_cast<size_t>(bh) * a.Sq + static_cast<size_t>(sq) * q_seg_len +
                           (row_valid ? r_in_seg : 0));
      float* o_g = a.out + grow * D;
      const bool have = row_valid && n_tiles > 0 && m_ref > -INFINITY;
      float m_old = -INFINITY, l_old = 0.f;
      if (!fresh && row_valid) {
        m_old = a.m[grow];
        l_old = a.l[grow];
      }
      const float m_new = have ? m_ref * kLn2 : -INFINITY;  // natural-log units
      const float m_fin = fmaxf(m_old, m_new);
      const float ca = (m_old == -INFINITY) ? 0.f : expf(m_old - m_fin);
      const float cb = have ? expf(m_new - m_fin) : 0.f;
      const float l_fin = ca * l_old + cb * l_run;
      const float inv = finalize ? (l_fin > 0.f ? 1.f / l_fin : 0.f) : 1.f;
      const bool touch = row_valid && (have || fresh || finalize);
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (n_tiles > 0) {  // block-uniform: the tensor-memory load is warp-collective
          tmem_ld32(t_o + c * 32, o);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (touch) {
          float4* dst = reinterpret_cast<float4*>(o_g + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!fresh) old = dst[i];
            float4 r;
            r.x = (ca * old.x + (have ? cb * o[4 * i] : 0.f)) * inv;
            r.y = (ca * old.y + (have ? cb * o[4 * i + 1] : 0.f)) * inv;
            r.z = (ca * old.z + (have ? cb * o[4 * i + 2] : 0.f)) * inv;
            r.w = (ca * old.w + (have ? cb * o[4 * i + 3] : 0.f)) * inv;
            dst[i] = r;
          }
        }
      }
      if (touch) {
        a.m[grow] = m_fin;
        a.l[grow] = l_fin;
      }
    }
  }

  // ---------------------------------------------------------------- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies and MMAs still in flight time to land before tensor memory is released
      const unsigned long long t0 = global_ns();
      while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base)
                 : "memory");
  }
}

// ---- host side ----------------------------------------------------------------------

template <int D>
int launch_tf32(const StepArgs& a, cudaStream_t stream) {
  using C = F32Cfg<D>;
  CUtensorMap mq, mk, mv;
  int rc = make_map(&mq, RA_F32, a.q, a.D, a.Sq, static_cast<long long>(a.B) * a.H,
                    static_cast<long long>(a.Sq) * a.D, kBM);
  if (rc != RA_OK) return rc;
  rc = make_map(&mk, RA_F32, a.k, a.D, a.k_rows, a.k_heads_total, a.kv_head_stride, C::kBN);
  if (rc != RA_OK) return rc;
  rc = make_map(&mv, RA_F32, a.v, a.D, a.k_rows, a.k_heads_total, a.kv_head_stride, C::kBN, true);
  if (rc != RA_OK) return rc;
  TcArgs t;
  t.kv_per_wave = 0;
  t.out = a.out;
  t.m = a.m;
  t.l = a.l;
  t.H = a.H;
  t.kvH = a.kvH;
  t.Sq = a.Sq;
  t.n_qblocks_per_seg = (a.qmap.seg_len + kBM - 1) / kBM;
  t.qmap = a.qmap;
  t.kmap = a.kmap;
  for (int i = 0; i < RA_MAX_SEG; ++i) {
    t.kseg_head[i] = a.kseg_head[i];
    t.kseg_row[i] = a.kseg_row[i];
  }
  t.stride = a.stride;
  t.flags = a.flags;
  t.doc_len = a.doc_len;
  t.status = a.status;
  t.wait_ns = tc_wait_limit_ns();
  t.stall_after = tc_stall_after();
  const long long n_qblocks = static_cast<long long>(t.n_qblocks_per_seg) * a.qmap.n_seg;
  RAB_REQUIRE(n_qblocks <= 65535, RA_ERR_INVALID, "attention step: too many query blocks (%lld)",
              n_qblocks);
  auto kern = step_tf32_kernel<D>;
  RAB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  const dim3 grid(static_cast<unsigned>(a.B) * a.H, static_cast<unsigned>(n_qblocks));
  kern<<<grid, kThreadsF, C::kSmemBytes, stream>>>(mq, mk, mv, t);
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

}  // namespace

bool step_tf32_supported(int dtype, const StepArgs& a) {
  if (dtype != RA_F32) return false;
  if (a.D != 32 && a.D != 64 && a.D != 128) return false;
  if (a.Sq <= 0 || a.Sk <= 0) return false;
  if (a.qmap.n_seg * a.qmap.seg_len != a.Sq || a.kmap.n_seg * a.kmap.seg_len != a.Sk) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
       reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.out)) & 15u)
    return false;
  return true;
}

int launch_step_tf32(const StepArgs& a, cudaStream_t stream) {
  RAB_REQUIRE(a.status != nullptr, RA_ERR_CUDA, "attention step: no device status word");
  if (a.D == 32) return launch_tf32<32>(a, stream);
  if (a.D == 64) return launch_tf32<64>(a, stream);
  return launch_tf32<128>(a, stream);
}

}  // namespace rab
