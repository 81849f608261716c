/*
 * CPU oracle: a plain-C restatement of the reference's host-side algorithms for
 * the ring-attention hot path. TEST INFRASTRUCTURE ONLY: nothing in the shipped
 * library links, loads or calls this file; it is the checker the CUDA path is
 * compared against (tests, the smoke check, and the CPU-baseline leg of the
 * benchmark).
 *
 * Parity pin: every function here is compared (a) against the reference's own
 * compiled code (cpu_attention.cpp, ring_partition.cpp, ring_gen.hpp built into
 * oracle/_ref by oracle/Makefile), (b) against the analytic known answers in the
 * reference's tests/test_cpu_attention.cpp and the offset tables in
 * tests/test_ring_partition.cpp, and (c) against golden vectors generated from
 * the reference's Python package (tests/golden/).
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static size_t head_off(int b, int h, int heads, int seq, int d) {
  return (((size_t)b * heads) + h) * (size_t)seq * d;
}

/*
 * Dense attention with optional end-aligned causal mask; follows
 * src/cpu_attention.cpp:23-79 loop for loop (score row, running max, exp,
 * denominator, then the P.V sum with p = e * (1/denom)). kv head = h % kv_heads
 * (src/cpu_attention.cpp:41-42). `lse` (may be NULL) receives
 * row_max + log(denom) per row, which the reference computes but discards
 * (src/cpu_attention.cpp:50-66); rows with no visible key get -inf.
 */
ORC_API void orc_cpu_attention(const float* q, const float* k, const float* v, float* out,
                               float* lse, int B, int H, int Sq, int Sk, int D, int kv_heads,
                               int causal) {
  const int kvH = kv_heads > 0 ? kv_heads : H;
  const float scale = 1.0f / sqrtf((float)D);
  const int shift = Sk - Sq;
  float* scores = (float*)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < H; ++h) {
      const float* qh = q + head_off(b, h, H, Sq, D);
      const float* kh = k + head_off(b, h % kvH, kvH, Sk, D);
      const float* vh = v + head_off(b, h % kvH, kvH, Sk, D);
      float* oh = out + head_off(b, h, H, Sq, D);
      for (int i = 0; i < Sq; ++i) {
        const float* qr = qh + (size_t)i * D;
        int jmax = Sk;
        if (causal) {
          jmax = i + shift + 1;
          if (jmax > Sk) jmax = Sk;
        }
        float row_max = -INFINITY;
        for (int j = 0; j < jmax; ++j) {
          const float* kr = kh + (size_t)j * D;
          float s = 0.0f;
          for (int d = 0; d < D; ++d) s += qr[d] * kr[d];
          s *= scale;
          scores[j] = s;
          if (s > row_max) row_max = s;
        }
        float denom = 0.0f;
        for (int j = 0; j < jmax; ++j) {
          scores[j] = expf(scores[j] - row_max);
          denom += scores[j];
        }
        const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
        float* orow = oh + (size_t)i * D;
        for (int d = 0; d < D; ++d) orow[d] = 0.0f;
        for (int j = 0; j < jmax; ++j) {
          const float p = scores[j] * inv;
          const float* vr = vh + (size_t)j * D;
          for (int d = 0; d < D; ++d) orow[d] += p * vr[d];
        }
        if (lse) {
          lse[(((size_t)b * H) + h) * Sq + i] = denom > 0.0f ? row_max + logf(denom) : -INFINITY;
        }
      }
    }
  }
  free(scores);
}

/*
 * One row of causal attention at global position `pos` against keys [0, pos]:
 * the sampled-row form used at sequence lengths where the full O(S^2) oracle
 * is too slow. Identical arithmetic to orc_cpu_attention with seq_q = 1,
 * seq_k = n_keys (src/cpu_attention.cpp:45-75). q_row: D floats; k, v:
 * (n_keys, D) rows of ONE kv head. `visible` (may be NULL): per-key 0/1 mask
 * applied on top (document masks).
 */
ORC_API void orc_attention_row(const float* q_row, const float* k, const float* v, int n_keys,
                               int D, const unsigned char* visible, float* out_row,
                               float* lse) {
  const float scale = 1.0f / sqrtf((float)D);
  float* scores = (float*)malloc(sizeof(float) * (size_t)(n_keys > 0 ? n_keys : 1));
  float row_max = -INFINITY;
  for (int j = 0; j < n_keys; ++j) {
    if (visible && !visible[j]) {
      scores[j] = -INFINITY;
      continue;
    }
    const float* kr = k + (size_t)j * D;
    float s = 0.0f;
    for (int d = 0; d < D; ++d) s += q_row[d] * kr[d];
    s *= scale;
    scores[j] = s;
    if (s > row_max) row_max = s;
  }
  float denom = 0.0f;
  for (int j = 0; j < n_keys; ++j) {
    scores[j] = (scores[j] == -INFINITY) ? 0.0f : expf(scores[j] - row_max);
    denom += scores[j];
  }
  const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
  for (int d = 0; d < D; ++d) out_row[d] = 0.0f;
  for (int j = 0; j < n_keys; ++j) {
    const float p = scores[j] * inv;
    if (p == 0.0f) continue;
    const float* vr = v + (size_t)j * D;
    for (int d = 0; d < D; ++d) out_row[d] += p * vr[d];
  }
  if (lse) *lse = denom > 0.0f ? row_max + logf(denom) : -INFINITY;
  free(scores);
}

/*
 * Persistent-state ring step on the CPU: the online-softmax recurrence of
 * src/attention_step.cu:205-282 applied to a whole K/V chunk at once (one
 * "tile" = the chunk, which is the same recurrence because it is associative
 * up to rounding). State (out unnormalised, m, l) is read-modify-written; a row
 * with no visible key keeps its state (src/attention_step.cu:238). Visibility:
 * j < Sk and (!causal or k_pos <= q_pos) with positions from piecewise-affine
 * maps: pos(i) = base[i / seg_len] + (i % seg_len) * stride
 * (src/attention.hpp:96-107 for the segmented form, src/attention_step.cu:165,
 * 228-229 for the affine one, which is n_seg = 1). doc_len > 0 additionally
 * requires q_pos / doc_len == k_pos / doc_len (document mask; an extension the
 * reference does not have).
 */
ORC_API void orc_attention_step(const float* q, const float* k, const float* v, float* out,
                                float* m, float* l, int B, int H, int Sq, int Sk, int D,
                                int kv_heads, const int* q_base, int q_nseg, int q_seg_len,
                                const int* k_base, int k_nseg, int k_seg_len, int stride,
                                int causal, long long doc_len) {
  const int kvH = kv_heads > 0 ? kv_heads : H;
  const float scale = 1.0f / sqrtf((float)D);
  float* s = (float*)malloc(sizeof(float) * (size_t)(Sk > 0 ? Sk : 1));
  (void)q_nseg;
  (void)k_nseg;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < H; ++h) {
      const float* qh = q + head_off(b, h, H, Sq, D);
      const float* kh = k + head_off(b, h % kvH, kvH, Sk, D);
      const float* vh = v + head_off(b, h % kvH, kvH, Sk, D);
      float* oh = out + head_off(b, h, H, Sq, D);
      for (int i = 0; i < Sq; ++i) {
        const size_t row = (((size_t)b * H) + h) * Sq + i;
        const long long qpos = (long long)q_base[i / q_seg_len] + (long long)(i % q_seg_len) * stride;
        float m_i = m[row], l_i = l[row];
        float m_new = m_i;
        for (int j = 0; j < Sk; ++j) {
          const long long kpos =
              (long long)k_base[j / k_seg_len] + (long long)(j % k_seg_len) * stride;
          int vis = !causal || kpos <= qpos;
          if (doc_len > 0 && (kpos / doc_len) != (qpos / doc_len)) vis = 0;
          if (vis) {
            float acc = 0.0f;
            const float* kr = kh + (size_t)j * D;
            const float* qr = qh + (size_t)i * D;
            for (int d = 0; d < D; ++d) acc += qr[d] * kr[d];
            acc *= scale;
            s[j] = acc;
            if (acc > m_new) m_new = acc;
          } else {
            s[j] = -INFINITY;
          }
        }
        if (m_new == -INFINITY) continue;
        const float alpha = expf(m_i - m_new);
        float row_sum = 0.0f;
        float* orow = oh + (size_t)i * D;
        for (int d = 0; d < D; ++d) orow[d] *= alpha;
        for (int j = 0; j < Sk; ++j) {
          if (s[j] == -INFINITY) continue;
          const float p = expf(s[j] - m_new);
          row_sum += p;
          const float* vr = vh + (size_t)j * D;
          for (int d = 0; d < D; ++d) orow[d] += p * vr[d];
        }
        l[row] = alpha * l_i + row_sum;
        m[row] = m_new;
      }
    }
  free(s);
}

/* out = 0, l = 0, m = -inf (src/attention_step.cu:42-53). */
ORC_API void orc_attention_init(float* out, float* m, float* l, size_t out_count, size_t m_count) {
  for (size_t i = 0; i < out_count; ++i) out[i] = 0.0f;
  for (size_t i = 0; i < m_count; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.0f;
  }
}

/* out_i *= 1/l_i, 0 when l_i <= 0 (src/attention_step.cu:56-69). */
ORC_API void orc_attention_finalize(float* out, const float* l, size_t rows, int D) {
  for (size_t r = 0; r < rows; ++r) {
    const float inv = l[r] > 0.0f ? 1.0f / l[r] : 0.0f;
    for (int d = 0; d < D; ++d) out[r * D + d] *= inv;
  }
}

/*
 * Merge cp_size rank partials laid out as cp_size blocks of
 * [O (BH*D) | m (BH) | l (BH)] (src/ring_decode.cu:50-81): global max, then
 * exp(m_r - m_max)-weighted sums; a rank with m_r = -inf contributes 0.
 */
ORC_API void orc_decode_partial_merge(const float* gathered, float* out, float* m_out,
                                      float* l_out, int cp_size, int BH, int D) {
  const size_t block = (size_t)BH * D + 2 * (size_t)BH;
  for (int bh = 0; bh < BH; ++bh) {
    float m_max = -INFINITY;
    for (int r = 0; r < cp_size; ++r) {
      const float m_r = gathered[r * block + (size_t)BH * D + bh];
      if (m_r > m_max) m_max = m_r;
    }
    float l_acc = 0.0f;
    for (int d = 0; d < D; ++d) out[(size_t)bh * D + d] = 0.0f;
    for (int r = 0; r < cp_size; ++r) {
      const float m_r = gathered[r * block + (size_t)BH * D + bh];
      const float sc = (m_r == -INFINITY) ? 0.0f : expf(m_r - m_max);
      for (int d = 0; d < D; ++d)
        out[(size_t)bh * D + d] += sc * gathered[r * block + (size_t)bh * D + d];
      l_acc += sc * gathered[r * block + (size_t)BH * D + BH + bh];
    }
    m_out[bh] = m_max;
    l_out[bh] = l_acc;
  }
}

/* xorshift32 stream, uniform [-1, 1) (src/cpu_attention.cpp:81-99; a zero seed
 * is replaced by 0x9E3779B9, src/cpu_attention.hpp:32). */
ORC_API uint32_t orc_xorshift32_fill(uint32_t seed, float* out, size_t n) {
  uint32_t x = seed ? seed : 0x9E3779B9u;
  for (size_t i = 0; i < n; ++i) {
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    const uint32_t mant = x >> 8;
    const float u = (float)mant * (1.0f / 16777216.0f);
    out[i] = 2.0f * u - 1.0f;
  }
  return x; /* state, so consecutive fills continue the same stream */
}

/* Coordinate hash in [-1, 1) (src/ring_gen.hpp:18-29). */
ORC_API float orc_gen_elem(uint32_t seed, int tensor_id, int b, int h, int s, int d) {
  uint32_t v = seed;
  v ^= (uint32_t)tensor_id * 2654435761u;
  v ^= (uint32_t)b * 2246822519u;
  v ^= (uint32_t)h * 3266489917u;
  v ^= (uint32_t)s * 668265263u;
  v ^= (uint32_t)d * 374761393u;
  v ^= v << 13;
  v ^= v >> 17;
  v ^= v << 5;
  return (float)(int32_t)v * (1.0f / 2147483648.0f);
}

/* Partition index maps (src/ring_partition.cpp:51-108). mode: 0 contiguous,
 * 1 zig-zag (coarse, n_splits sub-groups), 2 striped. */
ORC_API int orc_part_k_offset_for_source(int cp, int rank, int seq, int mode, int n_splits,
                                         int source, int sg) {
  (void)rank;
  if (mode == 0) return source * (seq / cp);
  if (mode == 2) return source;
  const int chunk = seq / (n_splits * cp);
  const int kk = sg / 2;
  if (sg % 2 == 0) return (kk * cp + source) * chunk;
  return ((n_splits - 1 - kk) * cp + (cp - 1 - source)) * chunk;
}
ORC_API int orc_part_q_offset(int cp, int rank, int seq, int mode, int n_splits, int sg) {
  return orc_part_k_offset_for_source(cp, rank, seq, mode, n_splits, rank, sg);
}
ORC_API int orc_part_k_offset_for_step(int cp, int rank, int seq, int mode, int n_splits,
                                       int step, int sg) {
  const int source = (rank - step % cp + cp) % cp;
  return orc_part_k_offset_for_source(cp, rank, seq, mode, n_splits, source, sg);
}
ORC_API int orc_part_local_chunk_len(int cp, int seq, int mode, int n_splits) {
  return mode == 1 ? seq / (n_splits * cp) : seq / cp;
}
ORC_API int orc_part_num_sub_groups(int mode, int n_splits) { return mode == 1 ? n_splits : 1; }
ORC_API int orc_part_position_stride(int cp, int mode) { return mode == 2 ? cp : 1; }
ORC_API int orc_part_next_rank(int cp, int rank) { return (rank + 1) % cp; }
ORC_API int orc_part_prev_rank(int cp, int rank) { return (rank - 1 + cp) % cp; }

/* Hierarchical (2-D) ring visitation order (src/ring2d_schedule.cpp:30-42): the shard that
 * GPU (node, local) of a num_nodes x gpus_per_node cluster holds at macro-step m, inner round
 * i. The band of a node moves one node on per macro-step, and inside a macro-step shards move
 * one local index on per inner round. Global rank = node * gpus_per_node + local. */
ORC_API int orc_ring2d_source(int num_nodes, int gpus_per_node, int node, int local, int m, int i) {
  const int from_node = ((node - m) % num_nodes + num_nodes) % num_nodes;
  const int from_local = ((local - i) % gpus_per_node + gpus_per_node) % gpus_per_node;
  return from_node * gpus_per_node + from_local;
}
