// Blackwell (sm_100a) ring step for fp16 / bf16 Q/K/V: a FlashAttention-style forward built
// directly on TMA, tcgen05.mma and tensor memory. Replaces the reference's one-warp wmma
// kernel (src/attention_step_fp16.cu:41-212) and, because positions come from segment
// maps, also the n_seg^2 launches per ring step of its driver
// (src/ring_loop_fp16.cu:642-655): one launch covers a whole zig-zag shard and skips the
// K tiles no row of the block can see.
//
// Work decomposition
//   grid = (batch * heads, query blocks). A block owns 256 query rows of one segment as two
//   128-row tiles (head_dim 256: one tile) and walks the visible 128-key tiles of every key
//   segment. Heaviest query blocks (largest positions) are launched first; with very many query
//   blocks per KV head the grid is turned so that all query blocks of the heads sharing one KV
//   head run before the next KV head (see launch_cfg).
//
// Three selectable forms of the same kernel, tested against each other: P in tensor memory
// (default) or staged through shared memory (RA_STEP_P_IN_SMEM), and cluster pairs
// (RA_STEP_CTA_PAIR, head_dim 128 / 256): tcgen05.mma.cta_group::2 with M = 256 over the two
// blocks of a cluster, each block loading half of every K and V tile.
//
// Roles inside a block (384 threads)
//   warp 0        TMA producer: Q tiles once, then K_j, V_j, K_j+1, ... into a shared-memory
//                 ring of 128B-swizzled tiles (cp.async.bulk.tensor, no multicast).
//   warps 1, 2    MMA issuers, one per query tile: S_w = Q_w K_j^T and O_w += P_w V_j with fp32
//                 accumulators in tensor memory. The whole warp runs the loop (uniform control
//                 flow and descriptors), one elected lane executes tcgen05.mma / commit.
//                 Warp 1 also allocates / frees tensor memory.
//   warps 4-7     softmax for query tile 0: one thread per row reads S from tensor memory,
//   warps 8-11    (tile 1) writes P = 2^(s * scale - m_ref) as 16-bit back into tensor memory
//                 (or into shared memory), keeps the row sum, and runs the epilogue. m_ref is
//                 the row's reference point, set from the row maximum of the first tile the row
//                 sees and moved (with a rescale of O and l) only when a tile's row sum shows
//                 that some score ran more than 2^15 above it; the common tile needs neither
//                 a row maximum nor a rescale.
//   The two query tiles are independent streams (own issuing warp, own barriers): the tensor
//   core works on one tile's MMAs while the other tile's rows are in their exponentials.
//
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D), and
// at head_dim 64 a separate P0 / P1 of 64 columns each behind them (otherwise P overwrites S).
// Head_dim 256: S0 / S1 are the two score buffers of the one query tile, O takes [256,512).
//
// What bounds it: a timing probe of back-to-back tcgen05.mma from an elected lane gives 66 clk
// per M128 N128 K16 instruction (shared-memory operands) and 33 clk at N = 64 with A in tensor
// memory, i.e. the arithmetic rate; cta_group::2 pairs cost the same per SM. A pair of 128x128
// tiles therefore needs ~1070 clk of tensor time at head_dim 64 (~2110 at 128) but 2048 clk of
// the exp unit (16 ex2 per clock per SM) plus the rest of the softmax instructions: the
// softmax warps, not the MMA issue, set the tile period at head_dim 64.
//
// Epilogue: the step's partial (O, m_ref, l) is merged with the persistent state in HBM using
// the log-sum-exp merge, which is the same recurrence as folding the tiles one by one
// (src/attention_step_fp16.cu:155-172), so the (out, m, l) contract of the reference holds:
// unnormalised out and l relative to a natural-log m (m is a reference point at or below the
// running maximum, within 2^15; m + log(l) is the exact log-sum-exp), rows without a visible
// key untouched.
//
// Every wait on an mbarrier is bounded: when one runs out the block records where in the
// device status word, all roles leave their loops, tensor memory is freed and the kernel
// returns; later blocks see the status word and return at once.
#include <atomic>

#include "tc_common.cuh"

namespace rab {

using namespace tcgen;

namespace {

constexpr int kBN = 128;           // keys per tile

// Register split between the producer / MMA warpgroup and the two softmax warpgroups
// (128 * LO + 256 * HI <= 65536).
#ifndef RAB_REGS_LO
#define RAB_REGS_LO 72
#define RAB_REGS_HI 216
#endif
template <bool kBf16>
__device__ inline unsigned pack16(float lo, float hi) {

  if constexpr (kBf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
  } else {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
  }
}

template <int D, bool kPInTmem, bool kPair = false>
struct TcCfg {
  // head_dim 256: O alone takes 256 tensor-memory columns, so a block owns ONE 128-row query
  // tile (one MMA warp, one softmax group), and a 128-key K or V tile (64 KiB) travels through
  // the ring as four 16 KiB items of 64 head_dim columns each, consumed one by one (in a CTA
  // pair: two items per tile, 128 head_dim columns of this block's half of the tile each).
  static constexpr int kTiles = D == 256 ? 1 : 2;            // query tiles per block
  static constexpr int kThreads = 128 + 128 * kTiles;
  static constexpr int kTileBytes = kBM * D * 2;             // one 128-row tile of Q, K or V
  static constexpr int kBoxes = D / 64;                      // 64-element (128-byte) boxes per tile
  static constexpr int kItemsPerTile = D == 256 ? (kPair ? 2 : 4) : 1;  // ring items per K / V tile
  static constexpr int kBoxesPerItem = kBoxes / kItemsPerTile;
  // CTA pair (head_dim 128 / 256, P in tensor memory): the two blocks of a cluster work on one key
  // tile with M = 256 instructions. Each block loads and holds HALF of every K tile (64 of its
  // 128 keys: the N columns of S it contributes) and half of every V tile (64 of the 128
  // head_dim columns: the N columns of O), so a block's shared-memory reads per score tile drop
  // from 8 to 6 KiB per k-step, its K/V loads from L2 halve, and the ring holds twice the tiles.
  static constexpr int kKRows = kPair ? kBN / 2 : kBN;       // keys of a K tile in this block
  static constexpr int kItemBytes = kTileBytes / kItemsPerTile / (kPair ? 2 : 1);
  static constexpr int kStages = kPair ? (D == 256 ? 10 : 8)
                                 : D == 256 ? (kPInTmem ? 10 : 8)
                                            : (kPInTmem ? (D == 128 ? 4 : 6) : (D == 128 ? 3 : 6));
  static_assert(!kPair || ((D == 128 || D == 256) && kPInTmem),
                "the CTA-pair schedule is built for head_dim 128 and 256 with P in tensor memory");
  // Item-wise K/V (head_dim 256): K items and V items get a ring half each. In one shared ring
  // of 1.25 tiles the K items of tile t+1 would wait for slots that P.V of tile t-1 frees last, and
  // their load latency would sit in front of every score tile; with a half each, K(t+1) loads as
  // soon as the scores of tile t are done and V(t) as soon as P.V of tile t-1 is, both under the
  // softmax of tile t.
  static constexpr bool kSplitRing = kItemsPerTile > 1;
  static constexpr int kPBytes = kPInTmem ? 0 : kBM * kBN * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kTiles * kTileBytes;
  static constexpr int kOffP = kOffKV + kStages * kItemBytes;
  static constexpr int kOffBar = kOffP + kTiles * kPBytes;
  static constexpr int kNumBars = 2 + 2 * kStages + 8;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;  // + alignment slack
  // Three schedules of the two MMAs of a key tile.
  //  * early S (P in shared memory; head_dim 64 with P in tensor memory: S 256 + O 128 + P 128
  //    columns = 512): P does not overlap S, so the next S tile is issued as soon as the softmax
  //    threads hold the current one in registers, instead of after P is written.
  //  * double S (one query tile per block, head_dim 256 with P in tensor memory: S 2 x 128 + O 256
  //    columns): the scores of tile t land in buffer t & 1 and P(t) is written over them. The
  //    issuer runs S(t+1) a whole tile ahead and S(t+2) straight behind P.V(t) (the tensor core
  //    executes in order, so P(t) has been read by then): the softmax of tile t+1 never waits for
  //    an MMA that depends on the softmax of tile t, and no hand-shake sits on that path.
  //  * otherwise (head_dim 128: S 256 + O 256 columns) P aliases S and P.V(t), S(t+1) go out in
  //    one batch when P(t) is written.
  static constexpr bool kDoubleS = kTiles == 1 && kPInTmem;
  static constexpr bool kEarlyS = !kPInTmem || D == 64;
  static constexpr int kColS0 = 0, kColS1 = 128;
  static constexpr int kColO0 = (kTiles == 2 || kDoubleS) ? 256 : 128, kColO1 = 256 + D;
  static constexpr int kColP0 = (kPInTmem && kEarlyS) ? 384 : kColS0;
  static constexpr int kColP1 = (kPInTmem && kEarlyS) ? 448 : kColS1;
  static constexpr int kPvN = D / kItemsPerTile;  // output columns one P.V instruction covers
  static constexpr int kMmaM = kPair ? 2 * kBM : kBM;  // rows one instruction covers
  static_assert(kItemsPerTile == 1 || kEarlyS || kDoubleS,
                "item-wise K/V needs the early-S or the double-S schedule");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Where a K (which = 0) or V (which = 1) item of key tile t sits in the ring and how often that
// slot has been used before (its barrier phase).
struct RingPos {
  int slot, use;
};
template <class C>
__device__ inline RingPos ring_pos(int which, int t, int sub) {
  if constexpr (C::kSplitRing) {
    constexpr int kHalf = C::kStages / 2;
    const int n = t * C::kItemsPerTile + sub;
    return {which * kHalf + n % kHalf, n / kHalf};
  } else {
    const int it = (2 * t + which) * C::kItemsPerTile + sub;
    return {it % C::kStages, it / C::kStages};
  }
}


// DR is the head_dim of the tensors in memory: D, or 32 on the 64-wide kernel (see launch_cfg).
template <int D, bool kBf16, bool kPInTmem, int DR, bool kPair = false>
__global__ void __launch_bounds__((TcCfg<D, kPInTmem, kPair>::kThreads), 1)
    step_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const TcArgs a) {
  using C = TcCfg<D, kPInTmem, kPair>;
  extern __shared__ unsigned char smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const unsigned s_base = smem_u32(smem);
  const unsigned s_q = s_base + C::kOffQ;
  const unsigned s_kv = s_base + C::kOffKV;
  const unsigned s_p = s_base + C::kOffP;
  const unsigned s_bar = s_base + C::kOffBar;
  // barrier table
  const unsigned bar_q_full = s_bar;                            // [2]
  const unsigned bar_kv_full = s_bar + 16;                      // [kStages]
  const unsigned bar_kv_empty = bar_kv_full + 8 * C::kStages;   // [kStages]
  const unsigned bar_s_full = bar_kv_empty + 8 * C::kStages;    // [2]
  const unsigned bar_p_full = bar_s_full + 16;                  // [2]
  const unsigned bar_o_done = bar_p_full + 16;                  // [2] PV_w done
  const unsigned bar_s_free = bar_o_done + 16;                  // [2] S_w held in registers
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + C::kOffBar + C::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // provably warp-uniform
  const int lane = tid & 31;

  // Rank inside the CTA pair; rank 0 (the leader) issues the pair's MMAs.
  unsigned cta_rank = 0;
  if constexpr (kPair) cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  // An earlier block gave up: leave at once (the vote makes the decision block-uniform). The
  // two blocks of a pair could decide differently, so a pair starts in the aborted state instead
  // (every wait then returns at once) and still meets at the cluster barriers below.
  if constexpr (!kPair) {
    if (__syncthreads_or(*reinterpret_cast<volatile int*>(a.status) != 0)) return;
  }

  const bool causal = (a.flags & RA_STEP_CAUSAL) != 0;
  const bool fresh = (a.flags & RA_STEP_FRESH) != 0;
  const bool finalize = (a.flags & RA_STEP_FINALIZE) != 0;

  // Block -> (batch*head, query segment, 256-row block inside the segment); heavy first.
  // (pairs: the two blocks of a cluster are neighbours in x - the pair instructions want the
  // cluster laid out along x - so x = 2 * (batch*head) + rank and y counts pairs of query blocks)
  int bh, qb_lin;
  if (a.kv_per_wave > 0) {
    // Waves of KV heads: y = a set of kv_per_wave KV heads, x = (query block, heavy first) x (the
    // query heads of that set, fastest). The blocks in flight read the K/V streams of one set
    // only, all from their first key on and at the same pace. (Pairs: the two blocks of a
    // cluster, neighbours in x, take the query blocks 2i and 2i + 1 of one head.)
    const int group = a.H / a.kvH, per_x = group * a.kv_per_wave;
    const int n_qb = a.n_qblocks_per_seg * a.qmap.n_seg;
    const int x = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int j = x % per_x;
    qb_lin = kPair ? n_qb - 1 - (2 * (x / per_x) + static_cast<int>(blockIdx.x & 1)) : n_qb - 1 - x / per_x;
    const int kv_lin = static_cast<int>(blockIdx.y) * a.kv_per_wave + j / group;  // batch * kvH + kv head
    bh = (kv_lin / a.kvH) * a.H + (j % group) * a.kvH + kv_lin % a.kvH;
  } else {
    bh = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    qb_lin = kPair ? 2 * static_cast<int>(gridDim.y) - 1 -
                         (2 * static_cast<int>(blockIdx.y) + static_cast<int>(blockIdx.x & 1))
                   : static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  }
  const int sq = qb_lin / a.n_qblocks_per_seg;
  const int tq = qb_lin - sq * a.n_qblocks_per_seg;
  const int h = bh % a.H;
  const int b = bh / a.H;
  const int kv_bh = b * a.kvH + (h % a.kvH);
  const int q_seg_len = a.qmap.seg_len;
  constexpr int kQBlock = C::kTiles * kBM;  // query rows per block
  const int row0 = tq * kQBlock;            // first row of the block inside its segment
  // The key tiles are chosen for the rows of the block, or of both blocks of a pair (a pair
  // walks one tile list; the second block of the last pair of a segment may have no rows).
  constexpr int kSpan = kPair ? 2 * kQBlock : kQBlock;
  const int span_row0 = kPair ? (tq & ~1) * kQBlock : row0;
  const int rows_in_span = min(kSpan, q_seg_len - span_row0);
  const int qmin = a.qmap.base[sq] + span_row0 * a.stride;
  const int qmax = a.qmap.base[sq] + (span_row0 + rows_in_span - 1) * a.stride;

  // Tile list: segments in order, tiles [lo, hi) of each; identical in every role.
  int n_tiles = 0;
  for (int sk = 0; sk < a.kmap.n_seg; ++sk) {
    const TileRange r = tile_range<kBN>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
    n_tiles += r.hi - r.lo;
  }

  if (tid == 0) {
    // In a pair the leader's "full" barriers also count the peer: its relay warp arrives when
    // the peer's half of Q / K / V has landed, its softmax threads arrive when their P is written.
    const unsigned peers = (kPair && leader) ? 2 : 1;
    mbar_init(bar_q_full, peers);
    mbar_init(bar_q_full + 8, peers);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_kv_full + 8 * s, peers);
      mbar_init(bar_kv_empty + 8 * s, C::kTiles);  // one commit from each issuing warp
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar_s_full + 8 * w, 1);
      mbar_init(bar_p_full + 8 * w, kPair ? 4 * peers : kBM);  // pair: one arrival per warp
      mbar_init(bar_o_done + 8 * w, 1);
      mbar_init(bar_s_free + 8 * w, kPair ? 4 * peers : kBM);
    }

    *abort_flag = (kPair && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                       smem_u32(tmem_slot))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
                       smem_u32(tmem_slot))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  // no arrival from the peer and no multicast commit before both blocks' barriers exist
  if constexpr (kPair) cluster_sync();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  // Registers follow the work: the producer / MMA warpgroup gives most of its registers back,
  // the two softmax warpgroups (one row of 128 scores per thread) take them.
  // (with one query tile per block there are 256 threads and registers to spare: no split)
  if (warp < 4) {
    if constexpr (C::kTiles == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(RAB_REGS_LO));
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ----
    if (lane == 0 && n_tiles > 0) {
      const int q_row = sq * q_seg_len + row0;
      for (int w = 0; w < C::kTiles; ++w) {
        mbar_expect_tx(bar_q_full + 8 * w, C::kTileBytes);
        for (int bx = 0; bx < C::kBoxes; ++bx)
          tma_load_3d(s_q + w * C::kTileBytes + bx * (kBM * 128), &tmap_q, bar_q_full + 8 * w,
                      bx * 64, q_row + w * kBM, bh);
      }
      int it = 0, jt = 0;  // ring items and key tiles so far
      bool ok = true;
      // all ring items of one operand (which: 0 = K, 1 = V) of key tile `tile`
      auto load_items = [&](int which, int tile, int k_row, int k_head) {
        for (int sub = 0; sub < C::kItemsPerTile && ok; ++sub, ++it) {
          const RingPos pos = ring_pos<C>(which, tile, sub);
          const int slot = pos.slot;
          if (pos.use >= 1)
            ok = mbar_wait(bar_kv_empty + 8 * slot, (pos.use + 1) & 1, abort_flag, a.status, 1, it,
                           a.wait_ns);
          if (!ok) break;
          // test hook: stop feeding the ring so that a consumer's bounded wait runs out
          if (a.stall_after >= 0 && it >= a.stall_after) {
            ok = false;
            break;
          }
          mbar_expect_tx(bar_kv_full + 8 * slot, C::kItemBytes);
          if constexpr (kPair) {
            // this block's half: keys [64 rank, 64 rank + 64) of K in 64-row boxes, head_dim
            // columns [64 rank, 64 rank + 64) of V in one 128-row box
            if (which == 0) {
              for (int bx = 0; bx < C::kBoxesPerItem; ++bx)
                tma_load_3d(s_kv + slot * C::kItemBytes + bx * (C::kKRows * 128), &tmap_k,
                            bar_kv_full + 8 * slot, (sub * C::kBoxesPerItem + bx) * 64,
                            k_row + static_cast<int>(cta_rank) * C::kKRows, k_head);
            } else {
              tma_load_3d(s_kv + slot * C::kItemBytes, &tmap_v, bar_kv_full + 8 * slot,
                          sub * C::kPvN + static_cast<int>(cta_rank) * 64, k_row, k_head);
            }
          } else {
          const CUtensorMap* map = which == 0 ? &tmap_k : &tmap_v;
          for (int bx = 0; bx < C::kBoxesPerItem; ++bx)
            tma_load_3d(s_kv + slot * C::kItemBytes + bx * (kBN * 128), map, bar_kv_full + 8 * slot,
                        (sub * C::kBoxesPerItem + bx) * 64, k_row, k_head);
          }
        }
      };
      // Order of the loads. One ring: K(t), V(t), K(t+1), ... (the order the slots come free in).
      // Two half rings: K(0), K(1), V(0), K(2), V(1), ... - the issuer runs the scores of tile
      // t + 1 before P.V of tile t, so K(t+1) must not queue behind a V(t) that waits for P.V of
      // tile t - 1.
      int v_row = 0, v_head = 0;
      bool v_pending = false;
      for (int sk = 0; sk < a.kmap.n_seg && ok; ++sk) {
        const TileRange r = tile_range<kBN>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
        for (int t = r.lo; t < r.hi && ok; ++t, ++jt) {
          const int k_row = a.kseg_row[sk] + t * kBN;
          const int k_head = a.kseg_head[sk] + kv_bh;
          load_items(0, jt, k_row, k_head);
          if constexpr (C::kSplitRing) {
            if (v_pending) load_items(1, jt - 1, v_row, v_head);
            v_row = k_row, v_head = k_head, v_pending = true;
          } else {
            load_items(1, jt, k_row, k_head);
          }
        }
      }
      if (C::kSplitRing && v_pending && ok) load_items(1, jt - 1, v_row, v_head);
    }
  } else if (kPair && !leader) {
    // ------------------------------------------------ relay (second block of a pair) ----
    // The leader issues the MMAs that read this block's shared memory, so it has to learn when
    // this block's loads have landed: warp 1 waits on the local "full" barriers in ring order
    // and passes each completion on to the leader's barrier of the same name.
    if (warp == 1 && n_tiles > 0) {
      auto relay = [&](unsigned bar, unsigned parity, int which, int tile) {
        const bool good = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, a.status, which,
                                                            tile, a.wait_ns)) != 0;
        if (good && lane == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");
          mbar_arrive_cluster(bar, 0);
        }
        return good;
      };
      bool ok = true;
      for (int w = 0; w < C::kTiles && ok; ++w) ok = relay(bar_q_full + 8 * w, 0, 3, w);
      auto relay_items = [&](int which, int t) {
        for (int sub = 0; sub < C::kItemsPerTile && ok; ++sub) {
          const RingPos pos = ring_pos<C>(which, t, sub);
          ok = relay(bar_kv_full + 8 * pos.slot, pos.use & 1, 5 - which, t);
        }
      };
      // in the order the producer loads (and the leader consumes) them
      for (int t = 0; t < n_tiles && ok; ++t) {
        if constexpr (C::kSplitRing) {
          if (t == 0) relay_items(0, 0);
          if (t + 1 < n_tiles) relay_items(0, t + 1);
          relay_items(1, t);
        } else {
          relay_items(0, t);
          relay_items(1, t);
        }
      }
    }
  } else if (warp == 1 || (warp == 2 && C::kTiles == 2)) {
    // ------------------------------------------------------------- MMA issuers ----
    // One issuing warp per query tile (warp 1: tile 0, warp 2: tile 1). The two tiles are
    // independent instruction streams, so a tile that is still in its exponentials never holds
    // back the other one and the two softmax groups are free to run out of step (which is what
    // keeps the exp unit busy: one group's loads, maxima and stores overlap the other group's
    // exponentials). The whole warp runs the loop so that descriptors and loop state stay
    // warp-uniform; the tcgen05.mma / tcgen05.commit instructions are executed by one elected
    // lane. A K/V ring slot is released when both warps have committed their reads of it.
    if (n_tiles > 0) {
      const int w = warp - 1;
      constexpr unsigned kFmt = kBf16 ? 1u : 0u;
      constexpr unsigned idesc_s = make_idesc(kFmt, 0, kBN, C::kMmaM);
      constexpr unsigned idesc_pv = make_idesc(kFmt, 1, C::kPvN, C::kMmaM);
      const unsigned t_s = tmem_base + (w == 0 ? C::kColS0 : C::kColS1);
      const unsigned t_o = tmem_base + (w == 0 ? C::kColO0 : C::kColO1);
      [[maybe_unused]] const unsigned t_p = tmem_base + (w == 0 ? C::kColP0 : C::kColP1);
      const unsigned long long qd = desc_kmajor(s_q + w * C::kTileBytes);
      [[maybe_unused]] const unsigned long long pd = desc_kmajor(s_p + w * C::kPBytes);
      const unsigned long long dkv0_k = desc_kmajor(s_kv);
      const unsigned long long dkv0_v = desc_mnmajor(s_kv, kBN * 128, 1024);
      constexpr unsigned kItemUnits = C::kItemBytes >> 4;  // one ring slot in 16-byte units
      constexpr unsigned kBox = (kBM * 128) >> 4;          // one 64-element box in 16-byte units
      constexpr unsigned kKBox = (C::kKRows * 128) >> 4;   // the same of a K item
      constexpr int kIPT = C::kItemsPerTile;
      const unsigned b_s_full = bar_s_full + 8 * w, b_s_free = bar_s_free + 8 * w;
      const unsigned b_p_full = bar_p_full + 8 * w, b_o_done = bar_o_done + 8 * w;
      auto wait = [&](unsigned bar, unsigned parity, int which, int tile) {
        return __all_sync(0xffffffffu,
                          mbar_wait(bar, parity, abort_flag, a.status, which, tile, a.wait_ns)) != 0;
      };
      // the pair forms reach both blocks: M = 256 instructions, commits that arrive on the
      // barrier of the same name in each block
      auto mma_ss_x = [&](unsigned d, unsigned long long ad, unsigned long long bd, unsigned idesc,
                          unsigned acc) {
        if constexpr (kPair) mma_ss_pair(d, ad, bd, idesc, acc);
        else mma_ss(d, ad, bd, idesc, acc);
      };
      auto mma_ts_x = [&](unsigned d, unsigned at, unsigned long long bd, unsigned idesc,
                          unsigned acc) {
        if constexpr (kPair) mma_ts_pair(d, at, bd, idesc, acc);
        else mma_ts(d, at, bd, idesc, acc);
      };
      auto commit = [&](unsigned bar) {
        if constexpr (kPair) tc_commit_pair(bar);
        else tc_commit(bar);
      };
      auto wait_kv = [&](RingPos pos, int which, int tile) {
        return wait(bar_kv_full + 8 * pos.slot, pos.use & 1, which, tile);
      };
      // Ring items of key tile t: see ring_pos.
      // The k-steps of one K item of S_w = Q_w K^T (called by the elected lane).
      auto s_ksteps = [&](int slot, int sub, [[maybe_unused]] int sbuf) {
        const unsigned long long kd = dkv0_k + static_cast<unsigned long long>(slot * kItemUnits);
#pragma unroll
        for (int ks = 0; ks < C::kBoxesPerItem * 4; ++ks) {
          // 64-element box, 32 B per k-step; Q holds all boxes, the item only its own
          const unsigned off_q = (sub * C::kBoxesPerItem + ks / 4) * kBox + (ks % 4) * 2;
          const unsigned off_k = (ks / 4) * kKBox + (ks % 4) * 2;
          mma_ss_x(t_s + (C::kDoubleS ? sbuf * kBN : 0), qd + off_q, kd + off_k, idesc_s,
                   (sub > 0 || ks > 0) ? 1u : 0u);
        }
      };
      // The k-steps of one V item of O_w += P_w V: kPvN output columns.
      auto pv_ksteps = [&](int slot, int sub, bool acc, [[maybe_unused]] int pbuf) {
        const unsigned long long vd = dkv0_v + static_cast<unsigned long long>(slot * kItemUnits);
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          const unsigned long long bd = vd + ks * (2048 >> 4);  // 16 keys = two 8-row groups
          const unsigned accum = (acc || ks > 0) ? 1u : 0u;
          if constexpr (kPInTmem) {
            mma_ts_x(t_o + sub * C::kPvN, t_p + pbuf * kBN + ks * 8, bd, idesc_pv, accum);
          } else {
            mma_ss_x(t_o + sub * C::kPvN, pd + ((ks / 4) * kBox + (ks % 4) * 2), bd, idesc_pv, accum);
          }
        }
      };
      // S_w(t): every K item as it lands; an item's slot is released by a commit behind its last
      // k-step, the softmax group is signalled behind the last item.
      auto do_s = [&](int t) {
        bool good = true;
#pragma unroll
        for (int sub = 0; sub < kIPT && good; ++sub) {
          const RingPos pos = ring_pos<C>(0, t, sub);
          const int slot = pos.slot;
          good = wait_kv(pos, 5, t);
          if (!good) break;
          tc_fence_after();
          if (elect_one()) {
            const int sbuf = C::kDoubleS ? (t & 1) : 0;
            s_ksteps(slot, sub, sbuf);
            if (sub == kIPT - 1) commit(b_s_full + 8 * sbuf);
            commit(bar_kv_empty + 8 * slot);
          }
        }
        return good;
      };
      // O_w += P_w V_t, one V item at a time.
      auto do_pv = [&](int t) {
        bool good = true;
#pragma unroll
        for (int sub = 0; sub < kIPT && good; ++sub) {
          const RingPos pos = ring_pos<C>(1, t, sub);
          const int slot = pos.slot;
          good = wait_kv(pos, 4, t);
          if (!good) break;
          tc_fence_after();
          if (elect_one()) {
            pv_ksteps(slot, sub, t > 0, C::kDoubleS ? (t & 1) : 0);
            if (sub == kIPT - 1) commit(b_o_done);
            commit(bar_kv_empty + 8 * slot);
          }
        }
        return good;
      };
      bool ok = wait(bar_q_full + 8 * w, 0, 3, w) && do_s(0);
      if constexpr (C::kDoubleS) ok = ok && (n_tiles < 2 || do_s(1));
      for (int t = 0; t < n_tiles && ok; ++t) {
        const bool more = t + 1 < n_tiles;
        if constexpr (C::kDoubleS) {
          // P.V of tile t when its P is written, then the scores of tile t + 2 into the buffer
          // that P(t) leaves (in order behind P.V(t) on the tensor core)
          ok = wait(b_p_full, t & 1, 6, t) && do_pv(t);
          if (t + 2 < n_tiles) ok = ok && do_s(t + 2);
        } else if constexpr (C::kEarlyS) {
          // S_w(t+1) goes out as soon as the softmax threads hold S_w(t) in registers; P.V of
          // tile t follows when its P is written. The tensor core works on the next scores
          // while the exponentials of the current tile run.
          if (more) ok = wait(b_s_free, t & 1, 9, t) && do_s(t + 1);
          ok = ok && wait(b_p_full, t & 1, 6, t) && do_pv(t);
        } else {
          // P aliases S (whole tiles are single ring items here): P.V of tile t and the scores
          // of tile t+1 go out in one batch once P_w(t) is written; the scores' completion
          // tells the softmax group that P.V is done as well.
          const RingPos pos_v = ring_pos<C>(1, t, 0), pos_k = ring_pos<C>(0, t + 1, 0);
          const int slot_v = pos_v.slot, slot_k = pos_k.slot;
          ok = wait_kv(pos_v, 4, t) && (!more || wait_kv(pos_k, 5, t)) && wait(b_p_full, t & 1, 6, t);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            pv_ksteps(slot_v, 0, t > 0, 0);
            if (more) {
              s_ksteps(slot_k, 0, 0);
              commit(b_s_full);
              commit(bar_kv_empty + 8 * slot_v);
              commit(bar_kv_empty + 8 * slot_k);
            } else {
              commit(b_o_done);
              commit(bar_kv_empty + 8 * slot_v);
            }
          }
        }
      }
    }
  }
  } else {
    if constexpr (C::kTiles == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(RAB_REGS_HI));
    // ----------------------------------------------------------------- softmax ----
    const int w = (warp - 4) >> 2;                   // query tile of this warpgroup
    const int row = ((warp & 3) << 5) + lane;        // row inside the tile = TMEM lane
    const unsigned lane_base = static_cast<unsigned>((warp & 3) << 5) << 16;
    const unsigned t_s = tmem_base + lane_base + (w == 0 ? C::kColS0 : C::kColS1);
    const unsigned t_o = tmem_base + lane_base + (w == 0 ? C::kColO0 : C::kColO1);
    [[maybe_unused]] const unsigned t_p =
        tmem_base + lane_base + (w == 0 ? C::kColP0 : C::kColP1);
    const int r_in_seg = row0 + w * kBM + row;
    const bool row_valid = r_in_seg < q_seg_len;
    const int qpos = a.qmap.base[sq] + r_in_seg * a.stride;
    const long long qdoc = a.doc_len > 0 ? qpos / a.doc_len : 0;
    const float scale_log2 = rsqrtf(static_cast<float>(DR)) * kLog2e;

    float m_ref = -INFINITY;  // reference point of P, O and l, log2 units (see the tile loop)
    float l_run = 0.f;
    bool ok = true;

    int j = 0;
    for (int sk = 0; sk < a.kmap.n_seg && ok; ++sk) {
      const TileRange tr = tile_range<kBN>(a.kmap, sk, a.stride, causal, a.doc_len, qmin, qmax);
      // Keys of this segment the row can see are the local indices [rel_lo, rel_hi): causal
      // and document limits are affine in the key index, so they are worked out once per
      // segment (64-bit divisions) and the per-tile work is two 32-bit clamps.
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
        // Visible columns of this row in this tile: [c_lo, c_hi), from the segment's bounds.
        int c_lo = min(max(rel_lo - t * kBN, 0), kBN);
        int c_hi = min(max(rel_hi - t * kBN, 0), kBN);
        if (c_hi < c_lo) c_hi = c_lo;
        const bool full = __all_sync(0xffffffffu, c_lo == 0 && c_hi == kBN);

        // (double S: buffer j & 1 and its barrier, used every other tile)
        const int sbuf = C::kDoubleS ? (j & 1) : 0;
        ok = mbar_wait(bar_s_full + 8 * (C::kDoubleS ? sbuf : w), C::kDoubleS ? (j >> 1) & 1 : j & 1,
                       abort_flag, a.status, 7, j, a.wait_ns);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory accesses below are warp-collective
        if (!ok) break;
        tc_fence_after();

        // All 128 scores of the row in registers: four loads in flight, one wait.
        float s[kBN];
        tmem_ld128(t_s + sbuf * kBN, s);
        if constexpr (C::kEarlyS) {
          // the scores are in registers: the tensor core may overwrite S_w with the next tile
          tc_fence_before();
          if constexpr (kPair) {
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(bar_s_free + 8 * w, 0);
          } else {
            mbar_arrive(bar_s_free + 8 * w);
          }
        }
        if (!full) {
          // hidden columns become -inf, which the exponential below turns into exactly 0
#pragma unroll
          for (int i = 0; i < kBN; ++i) s[i] = (i >= c_lo && i < c_hi) ? s[i] : -INFINITY;
        }

        // P = 2^(s * scale - m_ref), two columns at a time (packed fp32x2 multiply-add and add),
        // row sum in two independent accumulators, 16-bit P for the second MMA. m_ref is the
        // row's reference point: the row maximum at the time it was last set. It is NOT moved on
        // every tile: as long as the row sum of a tile stays below 2^15 every P fits 16 bits and
        // the fp32 sums hold it, so the common tile costs no row maximum at all (64 three-input
        // max instructions per row saved) and no rescale of O. A tile whose sum runs over (some
        // score more than 2^15 above the reference), or the first tile a row sees, takes the
        // slow path below: true row maximum, new reference, O and l rescaled, P recomputed.
        // P is produced and stored in two halves of 64 keys so that only 32 packed registers
        // are live beside the 128 scores.
        const float2 scale2 = make_float2(scale_log2, scale_log2);
        float2 sum_a, sum_b;
        auto half_tile = [&](int h, float neg_m) {
          const float2 negm2 = make_float2(neg_m, neg_m);
          unsigned pk[kBN / 4];
#pragma unroll
          for (int i = 0; i < kBN / 2; i += 4) {
            const int c = h * (kBN / 2) + i;
            const float2 x0 = ffma2(make_float2(s[c], s[c + 1]), scale2, negm2);
            const float2 x1 = ffma2(make_float2(s[c + 2], s[c + 3]), scale2, negm2);
            const float2 p0 = make_float2(ex2(x0.x), ex2(x0.y));
            const float2 p1 = make_float2(ex2(x1.x), ex2(x1.y));
            sum_a = fadd2(sum_a, p0);
            sum_b = fadd2(sum_b, p1);
            pk[i / 2] = pack16<kBf16>(p0.x, p0.y);
            pk[i / 2 + 1] = pack16<kBf16>(p1.x, p1.y);
          }
          if constexpr (kPInTmem) {
            // keys 64h .. 64h+63 as 32 packed columns (over the consumed S columns when P aliases S)
            tmem_st32u(t_p + sbuf * kBN + h * 32, &pk[0]);
          } else {
            // K-major 128B-swizzled P tile: row r, 16-byte piece q of 64-key box h at
            // h * 16 KiB + r * 128 + ((q ^ (r & 7)) * 16)
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) {
              const unsigned box = s_p + w * C::kPBytes + h * (kBM * 128) + row * 128;
              const unsigned addr = box + ((piece ^ (row & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pk[4 * piece]), "r"(pk[4 * piece + 1]), "r"(pk[4 * piece + 2]),
                           "r"(pk[4 * piece + 3])
                           : "memory");
            }
          }
        };
        // The P buffer about to be written must have been consumed: with early S wait for
        // PV_w(j-1), issued a whole softmax ago. With P written over S the completed S_w(j)
        // already implies it; only a rescale of O (`all`) then has to wait for PV_w(j-1) under
        // the double-S schedule, where S_w(j) was issued ahead of it.
        auto wait_prev_pv = [&]([[maybe_unused]] bool all) {
          if constexpr (C::kDoubleS || C::kEarlyS) {
            if (j > 0 && (all || !C::kDoubleS)) {
              ok = mbar_wait(bar_o_done + 8 * w, (j - 1) & 1, abort_flag, a.status, 10, j, a.wait_ns);
              ok = __all_sync(0xffffffffu, ok);
              if (ok) tc_fence_after();
            }
          }
        };
        // a row without a reference yet needs one as soon as it sees a key
        bool slow = __any_sync(0xffffffffu, m_ref == -INFINITY && c_hi > c_lo) != 0;
        float row_sum = 0.f;
        if (!slow) {
          const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
          sum_a = make_float2(0.f, 0.f);
          sum_b = make_float2(0.f, 0.f);
          wait_prev_pv(false);
          if (!ok) break;
          half_tile(0, neg_m);
          half_tile(1, neg_m);
          row_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
          slow = __any_sync(0xffffffffu, !(row_sum <= kRowSumLimit)) != 0;  // also catches NaN
        }
        else {
          wait_prev_pv(true);
          if (!ok) break;
        }
        if (slow) {
          if constexpr (C::kDoubleS) {  // O must be at rest
            wait_prev_pv(true);
            if (!ok) break;
          }
          float m0 = s[0], m1 = s[1], m2 = s[2], m3 = s[3];  // four independent chains
#pragma unroll
          for (int i = 4; i < kBN; i += 8) {
            m0 = max3(m0, s[i], s[i + 1]);
            m1 = max3(m1, s[i + 2], s[i + 3]);
            if (i + 4 < kBN) {
              m2 = max3(m2, s[i + 4], s[i + 5]);
              m3 = max3(m3, s[i + 6], s[i + 7]);
            }
          }
          const float tile_max = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * scale_log2;  // -inf stays -inf
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
            // O_w is at rest here: PV_w(j-1) has completed
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
          const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
          sum_a = make_float2(0.f, 0.f);
          sum_b = make_float2(0.f, 0.f);
          half_tile(0, neg_m);
          half_tile(1, neg_m);
          row_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        }
        l_run += row_sum;
        if constexpr (C::kDoubleS) {
          // Keep step with the P.V barrier, one phase per tile (a parity wait only tells the
          // latest phase from the one before). P.V(j-1) was issued a whole softmax ago, so this
          // rarely waits.
          wait_prev_pv(true);
          if (!ok) break;
        }
        if constexpr (kPInTmem) {
          tmem_wait_st();
        } else {
          tmem_wait_st();  // the O rescale above may have stores in flight
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tc_fence_before();
        if constexpr (kPair) {
          // one arrival per warp on the leader's barrier (arrivals that cross to the other block
          // are not cheap enough for one per thread)
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(bar_p_full + 8 * w, 0);
        } else {
          mbar_arrive(bar_p_full + 8 * w);
        }
      }
    }

    // ---------------------------------------------------------------- epilogue ----
    if (ok && n_tiles > 0)
      ok = mbar_wait(bar_o_done + 8 * w, (C::kEarlyS || C::kDoubleS) ? ((n_tiles - 1) & 1) : 0,
                     abort_flag, a.status, 8, n_tiles, a.wait_ns);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const size_t grow = (static_cast<size_t>(bh) * a.Sq + static_cast<size_t>(sq) * q_seg_len +
                           (row_valid ? r_in_seg : 0));
      float* o_g = a.out + grow * DR;
      const bool have = row_valid && n_tiles > 0 && m_ref > -INFINITY;
      float m_old = -INFINITY, l_old = 0.f;
      if (!fresh && row_valid) {
        m_old = a.m[grow];
        l_old = a.l[grow];
      }
      const float m_new = have ? m_ref * kLn2 : -INFINITY;  // natural-log units
      const float m_fin = fmaxf(m_old, m_new);
      const float ca = (m_old == -INFINITY) ? 0.f : expf(m_old - m_fin);
      // O and l are relative to m_ref; bring them to m_fin
      const float cb = have ? expf(m_new - m_fin) : 0.f;
      const float l_fin = ca * l_old + cb * l_run;
      const float inv = finalize ? (l_fin > 0.f ? 1.f / l_fin : 0.f) : 1.f;
      // a row that saw nothing keeps its state unless the caller asked to overwrite / normalise
      const bool touch = row_valid && (have || fresh || finalize);
#pragma unroll 1
      for (int c = 0; c < DR / 32; ++c) {
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
  // a block of a pair keeps its shared and tensor memory until the other one is done as well
  if constexpr (kPair) cluster_sync();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies and MMAs still in flight time to land before tensor memory is released
      const unsigned long long t0 = global_ns();
      while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
    tc_fence_after();
    if constexpr (kPair)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base)
                 : "memory");
  }
}

// ---- host side ----------------------------------------------------------------------

// Test hooks (see ra_debug_set_wait_limit_ns / ra_debug_stall_producer_after).
std::atomic<unsigned long long> g_wait_ns{kWaitLimitNs};
std::atomic<int> g_stall_after{-1};
std::atomic<int> g_block_order{-1};  // -1: by shape, 0: heads fastest, k > 0: waves of k KV heads

template <int D, bool kBf16, bool kPInTmem, int DR, bool kPair = false>
int launch_cfg(const StepArgs& a, cudaStream_t stream) {
  using C = TcCfg<D, kPInTmem, kPair>;
  CUtensorMap mq, mk, mv;
  const int dtype = kBf16 ? RA_BF16 : RA_F16;
  int rc = make_map(&mq, dtype, a.q, a.D, a.Sq, static_cast<long long>(a.B) * a.H,
                    static_cast<long long>(a.Sq) * a.D);
  if (rc != RA_OK) return rc;
  rc = make_map(&mk, dtype, a.k, a.D, a.k_rows, a.k_heads_total, a.kv_head_stride, C::kKRows);
  if (rc != RA_OK) return rc;
  rc = make_map(&mv, dtype, a.v, a.D, a.k_rows, a.k_heads_total, a.kv_head_stride);
  if (rc != RA_OK) return rc;

  TcArgs t;
  t.out = a.out;
  t.m = a.m;
  t.l = a.l;
  t.H = a.H;
  t.kvH = a.kvH;
  t.Sq = a.Sq;
  constexpr int kQBlock = C::kTiles * kBM;
  t.n_qblocks_per_seg = (a.qmap.seg_len + kQBlock - 1) / kQBlock;
  if (kPair) t.n_qblocks_per_seg = (t.n_qblocks_per_seg + 1) & ~1;  // whole pairs per segment
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
  t.wait_ns = g_wait_ns.load(std::memory_order_relaxed);
  t.stall_after = g_stall_after.load(std::memory_order_relaxed);
  const long long n_qblocks = static_cast<long long>(t.n_qblocks_per_seg) * a.qmap.n_seg;
  // Block order. By default (kv_per_wave = 0) the (batch, head) index runs fastest and the query
  // blocks go heavy first over the whole grid, which balances best - as long as the K and V of
  // all heads stay in L2 together. When they do not (long sequences: 67 MB per KV head at
  // S131072 D128), every block streams its keys from DRAM, and on the long head_dim 128 passes,
  // which run under the power cap, that traffic costs clock. Then the grid is cut into waves of
  // KV heads: all query blocks (heavy first) of the query heads of a few KV heads, whose K/V
  // (the part a block sweeps: a document, if there is a mask) fit in about half of L2, before
  // the next few - but never fewer than 512 blocks per wave, or the waves' tails cost more than
  // the traffic. Measured on D128 causal, same GPU: B2 H32/kvH8 S131072 271 -> 241 ms per pass
  // (SM clock 1350 -> 1550 MHz; at S32768 DRAM reads 12.4 -> 0.81 GB per launch, the algorithmic
  // bytes), H16 MHA S131072 1110 -> 1165 TFLOP/s; one head at a time with fewer blocks loses
  // (H16 MHA S131072 in four documents 1118 -> 1095, H8 S8192 D64 589 -> 409).
  const long long kv_heads_total = static_cast<long long>(a.B) * a.kvH;
  const long long q_rows = static_cast<long long>(a.qmap.seg_len) * a.qmap.n_seg;
  const long long k_rows = static_cast<long long>(a.kmap.seg_len) * a.kmap.n_seg;
  const long long q_rows_eff = a.doc_len > 0 && a.doc_len < q_rows ? a.doc_len : q_rows;
  const long long k_rows_eff = a.doc_len > 0 && a.doc_len < k_rows ? a.doc_len : k_rows;
  const long long kv_bytes_per_head = k_rows_eff * a.D * 2 * 2;  // K and V, 16-bit
  const long long blocks_per_kv_head = (a.H / a.kvH) * ((q_rows_eff + kQBlock - 1) / kQBlock);
  int kv_per_wave = 0;
  if (kv_bytes_per_head * kv_heads_total > (96ll << 20)) {
    auto divisor_at_most = [&](long long want) {
      long long d = std::max(1ll, std::min(want, kv_heads_total));
      while (kv_heads_total % d) --d;
      return d;
    };
    long long d = divisor_at_most((64ll << 20) / std::max(1ll, kv_bytes_per_head));
    while (d < kv_heads_total && d * blocks_per_kv_head < 512) {
      ++d;
      while (kv_heads_total % d) ++d;
    }
    kv_per_wave = d < kv_heads_total ? static_cast<int>(d) : 0;
  }
  const int order = g_block_order.load(std::memory_order_relaxed);  // test hook
  if (order == 0 || (order > 0 && kv_heads_total % order == 0)) kv_per_wave = order;
  t.kv_per_wave = kv_per_wave;
  const long long bh_total = static_cast<long long>(a.B) * a.H;
  const long long per_x = kv_per_wave > 0 ? static_cast<long long>(a.H / a.kvH) * kv_per_wave : 0;
  RAB_REQUIRE(kv_per_wave > 0 ? n_qblocks * per_x < (1ll << 31) : n_qblocks <= 65535, RA_ERR_INVALID,
              "attention step: grid too large (%lld query blocks, %lld heads)", n_qblocks, bh_total);
  auto kern = step_tc_kernel<D, kBf16, kPInTmem, DR, kPair>;
  // once per device and instantiation: the attribute call costs microseconds that a pass of a
  // few short launches would otherwise pay every time
  static std::atomic<unsigned long long> smem_set{0};
  int dev = 0;
  RAB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !(smem_set.load(std::memory_order_acquire) >> dev & 1ull)) {
    RAB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    if (dev >= 0 && dev < 64) smem_set.fetch_or(1ull << dev, std::memory_order_release);
  }
  dim3 grid(static_cast<unsigned>(a.B) * a.H, static_cast<unsigned>(n_qblocks));
  if (kv_per_wave > 0)
    grid = dim3(static_cast<unsigned>(n_qblocks * per_x), static_cast<unsigned>(kv_heads_total / kv_per_wave));
  if constexpr (kPair) {
    // the two blocks of a pair are neighbours in x; they take the query blocks 2i and 2i + 1
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = kv_per_wave > 0 ? grid : dim3(2 * grid.x, grid.y / 2);
    cfg.blockDim = dim3(C::kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    RAB_CUDA(cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, t));
  } else {
    kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(mq, mk, mv, t);
  }
  RAB_CUDA(cudaGetLastError());
  return RA_OK;
}

template <int D>
int launch_d(int dtype, const StepArgs& a, cudaStream_t stream) {
  // P stays in tensor memory unless the caller asks for the shared-memory path (kept as a
  // cross-check of the first one; both are tested)
  const bool p_in_tmem = (a.flags & RA_STEP_P_IN_SMEM) == 0;
  // the 64-wide kernel also takes head_dim 32 (DR = 32)
  if constexpr (D == 64) {
    if (a.D == 32) {
      if (dtype == RA_BF16)
        return p_in_tmem ? launch_cfg<64, true, true, 32>(a, stream)
                         : launch_cfg<64, true, false, 32>(a, stream);
      return p_in_tmem ? launch_cfg<64, false, true, 32>(a, stream)
                       : launch_cfg<64, false, false, 32>(a, stream);
    }
  }
  if constexpr (D == 128 || D == 256) {
    // Cluster pairs with M = 256 MMAs (cta_group::2), on request, wherever a segment has at least
    // two query blocks to pair up. Measured on B200 the pairs are 5-15 % slower than independent
    // blocks at both head_dims: each block's operand traffic halves, but neither shared-memory nor
    // L2 bandwidth was the limit, and every tile now crosses between the blocks twice (P written
    // -> leader, commit -> peer).
    const bool want_pair = (a.flags & RA_STEP_CTA_PAIR) != 0;
    if (p_in_tmem && want_pair && a.qmap.seg_len > TcCfg<D, true>::kTiles * kBM) {
      return dtype == RA_BF16 ? launch_cfg<D, true, true, D, true>(a, stream)
                              : launch_cfg<D, false, true, D, true>(a, stream);
    }
  }
  if (dtype == RA_BF16) {
    return p_in_tmem ? launch_cfg<D, true, true, D>(a, stream) : launch_cfg<D, true, false, D>(a, stream);
  }
  return p_in_tmem ? launch_cfg<D, false, true, D>(a, stream) : launch_cfg<D, false, false, D>(a, stream);
}

}  // namespace

bool step_tc_supported(int dtype, const StepArgs& a) {
  if (dtype != RA_F16 && dtype != RA_BF16) return false;
  if (a.D != 32 && a.D != 64 && a.D != 128 && a.D != 256) return false;
  if (a.Sq <= 0 || a.Sk <= 0) return false;
  if (a.qmap.n_seg * a.qmap.seg_len != a.Sq || a.kmap.n_seg * a.kmap.seg_len != a.Sk) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
       reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.out)) & 15u)
    return false;
  return true;
}

int launch_step_tc(int dtype, const StepArgs& a, cudaStream_t stream) {
  RAB_REQUIRE(a.status != nullptr, RA_ERR_CUDA, "attention step: no device status word");
  // head_dim 32 runs on the 64-wide kernel: the loads zero-fill the upper half of every row
  // (see make_map), so the scores are exact and the upper 32 output columns are never stored
  if (a.D == 32 || a.D == 64) return launch_d<64>(dtype, a, stream);
  if (a.D == 128) return launch_d<128>(dtype, a, stream);
  return launch_d<256>(dtype, a, stream);
}


namespace tcgen {
unsigned long long tc_wait_limit_ns() { return g_wait_ns.load(std::memory_order_relaxed); }
int tc_stall_after() { return g_stall_after.load(std::memory_order_relaxed); }
}  // namespace tcgen

void set_tc_wait_limit_ns(unsigned long long ns) {
  g_wait_ns.store(ns ? ns : kWaitLimitNs, std::memory_order_relaxed);
}
void set_tc_stall_after(int items) { g_stall_after.store(items, std::memory_order_relaxed); }
void set_tc_block_order(int order) { g_block_order.store(order, std::memory_order_relaxed); }


}  // namespace rab

