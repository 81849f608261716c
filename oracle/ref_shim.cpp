// extern "C" doorway onto the reference's OWN host code, compiled from the
// reference source tree where it lies (never copied here): cpu_attention /
// XorShift32 (src/cpu_attention.cpp), RingPartition (src/ring_partition.cpp),
// gen_elem (src/ring_gen.hpp), Ring2DSchedule (src/ring2d_schedule.cpp). Built into oracle/_ref/libref_oracle.so by
// oracle/Makefile. TEST INFRASTRUCTURE ONLY: used to validate the C restatement
// in oracle.c and as the timed CPU baseline; the shipped library never loads it.
#include <cstddef>
#include <cstdint>
#include <thread>
#include <vector>

#include "cpu_attention.hpp"
#include "ring_gen.hpp"
#include "ring2d_schedule.hpp"
#include "ring_partition.hpp"

using ring_attention::AttentionShape;
using ring_attention::RingPartition;

extern "C" {

void ref_cpu_attention(const float* q, const float* k, const float* v, float* out, int B, int H,
                       int Sq, int Sk, int D, int kv_heads, int causal) {
  AttentionShape s{B, H, Sq, Sk, D, kv_heads};
  ring_attention::cpu_attention(q, k, v, out, s, causal != 0);
}

// The unchanged single-threaded function, one call per (batch, query head) on a
// one-head shape, spread over `threads` host threads. kv head = h % kv_heads as
// in src/cpu_attention.cpp:41-42.
void ref_cpu_attention_mt(const float* q, const float* k, const float* v, float* out, int B, int H,
                          int Sq, int Sk, int D, int kv_heads, int causal, int threads) {
  const int kvH = kv_heads > 0 ? kv_heads : H;
  const int jobs = B * H;
  if (threads < 1) threads = 1;
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    pool.emplace_back([=]() {
      for (int job = t; job < jobs; job += threads) {
        const int b = job / H, h = job % H;
        const std::size_t qo = (static_cast<std::size_t>(b) * H + h) * Sq * D;
        const std::size_t ko = (static_cast<std::size_t>(b) * kvH + (h % kvH)) * Sk * D;
        AttentionShape s{1, 1, Sq, Sk, D, 0};
        ring_attention::cpu_attention(q + qo, k + ko, v + ko, out + qo, s, causal != 0);
      }
    });
  }
  for (auto& th : pool) th.join();
}

std::uint32_t ref_xorshift32_fill(std::uint32_t seed, float* out, std::size_t n) {
  ring_attention::XorShift32 rng(seed);
  for (std::size_t i = 0; i < n; ++i) out[i] = rng.next_uniform();
  return rng.next_u32();  // the value after the last one drawn (lets a caller check the stream position)
}

float ref_gen_elem(std::uint32_t seed, int tensor_id, int b, int h, int s, int d) {
  return ring_attention::gen_elem(seed, tensor_id, b, h, s, d);
}

static RingPartition make(int cp, int rank, int seq, int mode, int n_splits) {
  return RingPartition(cp, rank, seq, static_cast<RingPartition::Mode>(mode), n_splits);
}
int ref_part_q_offset(int cp, int rank, int seq, int mode, int n_splits, int sg) {
  return make(cp, rank, seq, mode, n_splits).q_offset(sg);
}
int ref_part_k_offset_for_step(int cp, int rank, int seq, int mode, int n_splits, int step,
                               int sg) {
  return make(cp, rank, seq, mode, n_splits).k_offset_for_step(step, sg);
}
int ref_part_k_offset_for_source(int cp, int rank, int seq, int mode, int n_splits, int source,
                                 int sg) {
  return make(cp, rank, seq, mode, n_splits).k_offset_for_source(source, sg);
}
int ref_part_local_chunk_len(int cp, int rank, int seq, int mode, int n_splits) {
  return make(cp, rank, seq, mode, n_splits).local_chunk_len();
}
int ref_part_num_sub_groups(int cp, int rank, int seq, int mode, int n_splits) {
  return make(cp, rank, seq, mode, n_splits).num_sub_groups();
}
int ref_part_position_stride(int cp, int rank, int seq, int mode, int n_splits) {
  return make(cp, rank, seq, mode, n_splits).position_stride();
}
int ref_part_next_rank(int cp, int rank, int seq) { return make(cp, rank, seq, 0, 2).next_rank(); }
int ref_part_prev_rank(int cp, int rank, int seq) { return make(cp, rank, seq, 0, 2).prev_rank(); }

int ref_ring2d_source(int num_nodes, int gpus_per_node, int node, int local, int m, int i) {
  return ring_attention::Ring2DSchedule(num_nodes, gpus_per_node, node, local).source(m, i);
}
}
