// Timing probe behind the design notes of step_tc.cu (a measurement tool, not part of the library):
// the cost of back-to-back tcgen05.mma instructions (M = 128 per CTA, K = 16, kind::f16, zeroed
// operands, 64 instructions per measurement, clock64 from the first issue to the arrival of the
// commit) for N = 64 / 128 / 256, operands from shared memory (SS) or A from tensor memory (TS),
// B K-major or MN-major, issued by an elected lane of a converged warp or by a single thread in a
// divergent branch, and the same for cta_group::2 pairs (M = 256 over two CTAs). Every wait is
// bounded. Build: python -m ring_attention_b200.build --probes; run: csrc/probe/_bin/mma_issue_probe
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>
__device__ inline unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ inline void mbar_init(unsigned bar, unsigned c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(c)); }
__device__ inline bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ inline bool elect_one() {
  unsigned pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ inline void tc_commit(unsigned bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ inline void mma_ss(unsigned d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ inline void mma_ts(unsigned d, unsigned a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ inline unsigned long long desc_kmajor(unsigned saddr) {
  const unsigned lo = ((saddr & 0x3FFFFu) >> 4) | (1u << 16);
  const unsigned hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((unsigned long long)hi << 32) | lo;
}
__host__ __device__ constexpr unsigned make_idesc(unsigned fmt, unsigned b_mn, unsigned n, unsigned m) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ long long g_out[16][3];
constexpr int kIters = 64;

__device__ inline unsigned long long desc_mnmajor(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes) {
  const unsigned lo = ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
  const unsigned hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  return ((unsigned long long)hi << 32) | lo;
}
template <int N, bool TS>
__device__ inline void run_mn(unsigned tm, unsigned sbase, unsigned bar, unsigned& parity, int mode) {
  // B is MN-major (the V operand of P.V): 8 k-steps of 16 keys through a 128-key tile, like the product kernel
  const unsigned long long da = desc_kmajor(sbase);
  const unsigned long long db = desc_mnmajor(sbase + 16384, 128 * 128, 1024);
  constexpr unsigned idesc = make_idesc(0, 1, N, 128);
  const long long t0 = clock64();
#pragma unroll 8
  for (int it = 0; it < kIters; ++it) {
    const unsigned ks = it % 8;
    if (elect_one()) {
      if (TS) mma_ts(tm, tm + 448 + ks * 8, db + ks * (2048 >> 4), idesc, it > 0 ? 1u : 0u);
      else mma_ss(tm, da + (ks % 4) * 2, db + ks * (2048 >> 4), idesc, it > 0 ? 1u : 0u);
    }
  }
  const long long t1 = clock64();
  if (elect_one()) tc_commit(bar);
  long long spins = 0;
  while (!mbar_try_wait(bar, parity) && spins < 20000000) ++spins;
  const long long t2 = clock64();
  parity ^= 1;
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { g_out[mode][0] = t1 - t0; g_out[mode][1] = t2 - t0; g_out[mode][2] = spins; }
}

// ---- kind::tf32 (K = 8 per instruction, 32-bit operands) ----
__device__ inline void mma_ss_tf32(unsigned d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ inline void mma_ts_tf32(unsigned d, unsigned a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
template <int N, bool TS>
__device__ inline void run_tf32(unsigned tm, unsigned sbase, unsigned bar, unsigned& parity, int mode) {
  const unsigned long long da = desc_kmajor(sbase);
  const unsigned long long db = desc_kmajor(sbase + 16384);
  constexpr unsigned idesc = make_idesc(2, 0, N, 128);
  const long long t0 = clock64();
#pragma unroll 8
  for (int it = 0; it < kIters; ++it) {
    const unsigned off = (it % 4) * 2;
    if (elect_one()) {
      if (TS) mma_ts_tf32(tm, tm + 448 + (it % 4) * 8, db + off, idesc, it > 0 ? 1u : 0u);
      else mma_ss_tf32(tm, da + off, db + off, idesc, it > 0 ? 1u : 0u);
    }
  }
  const long long t1 = clock64();
  if (elect_one()) tc_commit(bar);
  long long spins = 0;
  while (!mbar_try_wait(bar, parity) && spins < 20000000) ++spins;
  const long long t2 = clock64();
  parity ^= 1;
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { g_out[mode][0] = t1 - t0; g_out[mode][1] = t2 - t0; g_out[mode][2] = spins; }
}
template <int N, bool TS>
__device__ inline void run_uniform(unsigned tm, unsigned sbase, unsigned bar, unsigned& parity, int mode) {
  // executed by all 32 lanes of one warp
  const unsigned long long da = desc_kmajor(sbase);
  const unsigned long long db = desc_kmajor(sbase + 16384);
  constexpr unsigned idesc = make_idesc(0, 0, N, 128);
  const long long t0 = clock64();
#pragma unroll 8
  for (int it = 0; it < kIters; ++it) {
    const unsigned off = (it % 4) * 2;
    if (elect_one()) {
      if (TS) mma_ts(tm, tm + 448 + (it % 4) * 8, db + off, idesc, it > 0 ? 1u : 0u);
      else mma_ss(tm, da + off, db + off, idesc, it > 0 ? 1u : 0u);
    }
  }
  const long long t1 = clock64();
  if (elect_one()) tc_commit(bar);
  long long spins = 0;
  while (!mbar_try_wait(bar, parity) && spins < 20000000) ++spins;
  const long long t2 = clock64();
  parity ^= 1;
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { g_out[mode][0] = t1 - t0; g_out[mode][1] = t2 - t0; g_out[mode][2] = spins; }
}
template <int N, bool TS>
__device__ inline void run_single(unsigned tm, unsigned sbase, unsigned bar, unsigned& parity, int mode) {
  // executed by one thread (divergent branch), fully unrolled by 8 like the product kernel
  const unsigned long long da = desc_kmajor(sbase);
  const unsigned long long db = desc_kmajor(sbase + 16384);
  constexpr unsigned idesc = make_idesc(0, 0, N, 128);
  const long long t0 = clock64();
#pragma unroll 8
  for (int it = 0; it < kIters; ++it) {
    const unsigned off = (it % 4) * 2;
    if (TS) mma_ts(tm, tm + 448 + (it % 4) * 8, db + off, idesc, it > 0 ? 1u : 0u);
    else mma_ss(tm, da + off, db + off, idesc, it > 0 ? 1u : 0u);
  }
  const long long t1 = clock64();
  tc_commit(bar);
  long long spins = 0;
  while (!mbar_try_wait(bar, parity) && spins < 20000000) ++spins;
  const long long t2 = clock64();
  parity ^= 1;
  if (blockIdx.x == 0) { g_out[mode][0] = t1 - t0; g_out[mode][1] = t2 - t0; g_out[mode][2] = spins; }
}

__global__ void __launch_bounds__(128, 1) probe4(int dummy) {
  extern __shared__ unsigned char raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ unsigned tmem_slot;
  __shared__ unsigned long long bar;
  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  for (int i = tid; i < 96 * 1024 / 4; i += 128) ((unsigned*)smem)[i] = 0;
  if (tid == 0) { mbar_init(smem_u32(&bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tm = tmem_slot;
  const unsigned sbase = smem_u32(smem);
  const unsigned b = smem_u32(&bar);
  unsigned parity = 0;
  if (warp == 1) {
    run_uniform<64, false>(tm, sbase, b, parity, 0);
    run_uniform<128, false>(tm, sbase, b, parity, 1);
    run_uniform<256, false>(tm, sbase, b, parity, 2);
    run_uniform<64, true>(tm, sbase, b, parity, 3);
    run_uniform<128, true>(tm, sbase, b, parity, 4);
    run_uniform<256, true>(tm, sbase, b, parity, 5);
    run_tf32<64, false>(tm, sbase, b, parity, 14);
    run_tf32<128, false>(tm, sbase, b, parity, 15);
    run_mn<64, true>(tm, sbase, b, parity, 10);
    run_mn<128, true>(tm, sbase, b, parity, 11);
    run_mn<64, false>(tm, sbase, b, parity, 12);
    run_mn<128, false>(tm, sbase, b, parity, 13);
    if ((tid & 31) == 0) {
      run_single<64, false>(tm, sbase, b, parity, 6);
      run_single<128, false>(tm, sbase, b, parity, 7);
      run_single<64, true>(tm, sbase, b, parity, 8);
      run_single<128, true>(tm, sbase, b, parity, 9);
    }
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
  }
}

// ---- cta_group::2: one instruction drives the tensor cores of a CTA pair (M = 256) ----
__device__ inline void tc_commit2(unsigned bar) { asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ inline void mma_ss2(unsigned d, unsigned long long a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ inline void mma_ts2(unsigned d, unsigned a, unsigned long long b, unsigned idesc, unsigned acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ inline void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int N, bool TS>
__device__ inline void run_pair(unsigned tm, unsigned sbase, unsigned bar, unsigned& parity, int mode) {
  const unsigned long long da = desc_kmajor(sbase);
  const unsigned long long db = desc_kmajor(sbase + 16384);
  constexpr unsigned idesc = make_idesc(0, 0, N, 256);
  const long long t0 = clock64();
#pragma unroll 8
  for (int it = 0; it < kIters; ++it) {
    const unsigned off = (it % 4) * 2;
    if (elect_one()) {
      if (TS) mma_ts2(tm, tm + 448 + (it % 4) * 8, db + off, idesc, it > 0 ? 1u : 0u);
      else mma_ss2(tm, da + off, db + off, idesc, it > 0 ? 1u : 0u);
    }
  }
  const long long t1 = clock64();
  if (elect_one()) tc_commit2(bar);
  long long spins = 0;
  while (!mbar_try_wait(bar, parity) && spins < 20000000) ++spins;
  const long long t2 = clock64();
  parity ^= 1;
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { g_out[mode][0] = t1 - t0; g_out[mode][1] = t2 - t0; g_out[mode][2] = spins; }
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) probe_pair(int dummy) {
  extern __shared__ unsigned char raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ unsigned tmem_slot;
  __shared__ unsigned long long bar;
  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  for (int i = tid; i < 96 * 1024 / 4; i += 128) ((unsigned*)smem)[i] = 0;
  if (tid == 0) { mbar_init(smem_u32(&bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tm = tmem_slot;
  const unsigned sbase = smem_u32(smem);
  const unsigned b = smem_u32(&bar);
  unsigned parity = 0;
  if (warp == 1 && rank == 0) {  // the leader CTA issues for the pair
    run_pair<64, false>(tm, sbase, b, parity, 0);
    run_pair<128, false>(tm, sbase, b, parity, 1);
    run_pair<256, false>(tm, sbase, b, parity, 2);
    run_pair<64, true>(tm, sbase, b, parity, 3);
    run_pair<128, true>(tm, sbase, b, parity, 4);
    run_pair<256, true>(tm, sbase, b, parity, 5);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
  }
}
int main() {
  cudaFuncSetAttribute(probe4, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  probe4<<<148, 128, 100 * 1024>>>(0);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
  long long h[16][3];
  cudaMemcpyFromSymbol(h, g_out, sizeof(h));
  const char* names[] = {"uniform SS N64", "uniform SS N128", "uniform SS N256", "uniform TS N64", "uniform TS N128", "uniform TS N256", "single SS N64", "single SS N128", "single TS N64", "single TS N128", "MN-major B TS N64", "MN-major B TS N128", "MN-major B SS N64", "MN-major B SS N128", "tf32 SS N64 (K=8)", "tf32 SS N128 (K=8)"};
  for (int m = 0; m < 16; ++m)
    printf("  %-18s issue %6lld clk  done %6lld clk  = %.1f clk per MMA%s\n", names[m], h[m][0], h[m][1], h[m][1] / 64.0, h[m][2] >= 20000000 ? "  TIMEOUT" : "");
  cudaFuncSetAttribute(probe_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  probe_pair<<<148, 128, 100 * 1024>>>(0);
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
  cudaMemcpyFromSymbol(h, g_out, sizeof(h));
  const char* pair_names[] = {"pair SS N64", "pair SS N128", "pair SS N256", "pair TS N64", "pair TS N128", "pair TS N256"};
  for (int m = 0; m < 6; ++m)
    printf("  %-18s issue %6lld clk  done %6lld clk  = %.1f clk per MMA (M = 256 over two CTAs)%s\n", pair_names[m], h[m][0], h[m][1], h[m][1] / 64.0, h[m][2] >= 20000000 ? "  TIMEOUT" : "");
  return 0;
}
