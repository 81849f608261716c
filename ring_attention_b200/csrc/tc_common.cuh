// Device-side building blocks shared by the tcgen05 step kernels (step_tc.cu: fp16 / bf16,
// step_tf32.cu: fp32 through split TF32 operands): mbarrier / TMA / tcgen05 wrappers with bounded
// waits, shared-memory and instruction descriptors, the visible key-tile range of a query
// block, the kernel argument block and the host-side tensor-map encoder.
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace rab {
namespace tcgen {

constexpr int kBM = 128;           // query rows per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRowSumLimit = 32768.f;  // a tile's row sum of P above this moves the reference
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // default limit of every wait: 2 s

// ---- PTX wrappers -------------------------------------------------------------------
__device__ inline unsigned smem_u32(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ inline void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ inline void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ inline void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ inline bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with acquire semantics at cluster scope: for a barrier that threads of the peer CTA of
// a pair arrive on.
__device__ inline bool mbar_try_wait_cluster(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking form: has the phase with this parity completed?
__device__ inline bool mbar_test_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// One lane of a converged warp (the same lane every time for a full mask).
__device__ inline bool elect_one() {
  unsigned pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ inline unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait. Returns false when the block is aborting (own limit reached or another
// role flagged it). `which` identifies the wait in the status word.
template <bool kClusterScope = false>
__device__ inline bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag,
                                 int* status, int which, int tile, unsigned long long limit_ns) {
  auto try_wait = [&]() {
    return kClusterScope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity);
  };
  if (try_wait()) return true;
  const unsigned long long t0 = global_ns();
  unsigned spins = 0;
  while (true) {
    if (try_wait()) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (atomicCAS(&status[0], 0, RA_ERR_DEVICE_WAIT) == 0) {
          status[1] = which;
          status[2] = static_cast<int>(blockIdx.x + blockIdx.y * gridDim.x);
          status[3] = tile;
        }
        return false;
      }
    }
  }
}

__device__ inline void tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0,
                                   int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ inline void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ inline void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ inline void tc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ inline void mma_ss(unsigned d_tmem, unsigned long long a_desc,
                              unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ inline void mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                              unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}


// ---- CTA pairs (cta_group::2): one instruction drives the tensor cores of two CTAs of a cluster,
// M = 256 (128 rows from each CTA's A operand and into each CTA's tensor memory), each CTA
// holding half of the B operand's N columns in its own shared memory at the same offset.
__device__ inline unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ inline void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ inline void mbar_arrive_cluster(unsigned bar, unsigned rank) {
  asm volatile(
      "{\n\t.reg .b32 r;\n\t"
      "mapa.shared::cluster.u32 r, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [r];\n\t}" ::"r"(bar),
      "r"(rank)
      : "memory");
}
// The barrier at this offset in BOTH CTAs of the pair gets the arrival.
__device__ inline void tc_commit_pair(unsigned bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(static_cast<unsigned short>(3))
      : "memory");
}
__device__ inline void mma_ss_pair(unsigned d_tmem, unsigned long long a_desc,
                                   unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ inline void mma_ts_pair(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                   unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ inline void tmem_ld32(unsigned taddr, float (&r)[32]) {
  unsigned u[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"  // same statement: no use of the registers can move above it
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]),
        "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]),
        "=r"(u[14]), "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]),
        "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]),
        "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
// All 128 columns of a row: four 32-column loads in flight and one wait, in a single asm
// statement so that no use of the registers can be scheduled above the wait.
__device__ inline void tmem_ld128(unsigned taddr, float (&r)[128]) {
  unsigned u[128];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%128];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%129];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95}, [%130];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%131];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
        "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
        "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31]),
        "=r"(u[32]), "=r"(u[33]), "=r"(u[34]), "=r"(u[35]), "=r"(u[36]), "=r"(u[37]), "=r"(u[38]), "=r"(u[39]),
        "=r"(u[40]), "=r"(u[41]), "=r"(u[42]), "=r"(u[43]), "=r"(u[44]), "=r"(u[45]), "=r"(u[46]), "=r"(u[47]),
        "=r"(u[48]), "=r"(u[49]), "=r"(u[50]), "=r"(u[51]), "=r"(u[52]), "=r"(u[53]), "=r"(u[54]), "=r"(u[55]),
        "=r"(u[56]), "=r"(u[57]), "=r"(u[58]), "=r"(u[59]), "=r"(u[60]), "=r"(u[61]), "=r"(u[62]), "=r"(u[63]),
        "=r"(u[64]), "=r"(u[65]), "=r"(u[66]), "=r"(u[67]), "=r"(u[68]), "=r"(u[69]), "=r"(u[70]), "=r"(u[71]),
        "=r"(u[72]), "=r"(u[73]), "=r"(u[74]), "=r"(u[75]), "=r"(u[76]), "=r"(u[77]), "=r"(u[78]), "=r"(u[79]),
        "=r"(u[80]), "=r"(u[81]), "=r"(u[82]), "=r"(u[83]), "=r"(u[84]), "=r"(u[85]), "=r"(u[86]), "=r"(u[87]),
        "=r"(u[88]), "=r"(u[89]), "=r"(u[90]), "=r"(u[91]), "=r"(u[92]), "=r"(u[93]), "=r"(u[94]), "=r"(u[95]),
        "=r"(u[96]), "=r"(u[97]), "=r"(u[98]), "=r"(u[99]), "=r"(u[100]), "=r"(u[101]), "=r"(u[102]), "=r"(u[103]),
        "=r"(u[104]), "=r"(u[105]), "=r"(u[106]), "=r"(u[107]), "=r"(u[108]), "=r"(u[109]), "=r"(u[110]), "=r"(u[111]),
        "=r"(u[112]), "=r"(u[113]), "=r"(u[114]), "=r"(u[115]), "=r"(u[116]), "=r"(u[117]), "=r"(u[118]), "=r"(u[119]),
        "=r"(u[120]), "=r"(u[121]), "=r"(u[122]), "=r"(u[123]), "=r"(u[124]), "=r"(u[125]), "=r"(u[126]), "=r"(u[127])
      : "r"(taddr), "r"(taddr + 32), "r"(taddr + 64), "r"(taddr + 96)
      : "memory");
#pragma unroll
  for (int i = 0; i < 128; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ inline void tmem_st32(unsigned taddr, const float (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])),
      "r"(__float_as_uint(r[3])), "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])),
      "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])), "r"(__float_as_uint(r[8])),
      "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
      "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])),
      "r"(__float_as_uint(r[15])), "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])),
      "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])), "r"(__float_as_uint(r[20])),
      "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
      "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])),
      "r"(__float_as_uint(r[27])), "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])),
      "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
      : "memory");
}
__device__ inline void tmem_st16(unsigned taddr, const unsigned (&u)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
      "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15])
      : "memory");
}
// 32 packed columns from an array slice
__device__ inline void tmem_st32u(unsigned taddr, const unsigned* u) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
      "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]),
      "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]),
      "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]),
      "r"(u[29]), "r"(u[30]), "r"(u[31])
      : "memory");
}
__device__ inline float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// packed fp32x2 arithmetic: one instruction for two lanes of a float2
__device__ inline float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)),
        "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}
__device__ inline float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)),
        "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return d;
}
__device__ inline void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ inline float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory matrix descriptors for 128B-swizzled tiles (8-row groups 1024 B apart).
// K-major operand (rows = M or N index, 64 contiguous 16-bit elements of the contraction
// dimension per 128-byte row); the leading byte offset is unused for swizzled K-major.
__device__ inline unsigned long long desc_kmajor(unsigned saddr) {
  const unsigned lo = ((saddr & 0x3FFFFu) >> 4) | (1u << 16);
  const unsigned hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version 1, SWIZZLE_128B
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}
// MN-major operand (rows = contraction index, 64 contiguous elements of N per 128-byte row):
// leading byte offset = distance between 64-element N blocks (one 128-row box, 16 KiB),
// stride = between 8-row groups (1 KiB); one MMA (16 rows) advances the start by 2 KiB.
__device__ inline unsigned long long desc_mnmajor(unsigned saddr, unsigned lbo_bytes,
                                               unsigned sbo_bytes) {
  const unsigned lo = ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
  const unsigned hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}

// MN-major operand of 32-bit elements (TF32): the 128B swizzle that moves 32-byte pieces (TMA's
// SWIZZLE_128B_ATOM_32B), four rows of the contraction index per swizzle atom. Leading byte
// offset = distance between 32-element N blocks, stride = between 4-row groups (512 B).
__device__ inline unsigned long long desc_mnmajor_32b(unsigned saddr, unsigned lbo_bytes,
                                                      unsigned sbo_bytes) {
  const unsigned lo = ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
  const unsigned hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (1u << 29);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}

// Instruction descriptor, kind::f16: fp32 accumulate, A/B format (0 fp16, 1 bf16), A K-major,
// B K-major (b_mn = 0) or MN-major (1), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr unsigned make_idesc(unsigned fmt, unsigned b_mn, unsigned n,
                                                  unsigned m) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

struct TileRange {
  int lo, hi;  // key tiles [lo, hi) of a segment that some row of the block can see
};

// Visible key-tile range of key segment `sk` for a query block whose rows span positions
// [qmin, qmax] (both ends are positions of real rows).
template <int kTileKeys>
__device__ inline TileRange tile_range(const PosMap& kmap, int sk, int stride, bool causal,
                                       long long doc_len, int qmin, int qmax) {
  const int L = kmap.seg_len;
  const long long kb = kmap.base[sk];
  long long j_lo = 0, j_hi = L - 1;  // visible local key indices, inclusive
  if (causal) {
    const long long d = static_cast<long long>(qmax) - kb;
    if (d < 0) return {0, 0};
    j_hi = min(j_hi, d / stride);
  }
  if (doc_len > 0) {
    const long long p_lo = (static_cast<long long>(qmin) / doc_len) * doc_len;
    const long long p_hi = (static_cast<long long>(qmax) / doc_len + 1) * doc_len - 1;
    if (p_hi < kb) return {0, 0};
    j_hi = min(j_hi, (p_hi - kb) / stride);
    if (p_lo > kb) j_lo = (p_lo - kb + stride - 1) / stride;
  }
  if (j_hi < j_lo) return {0, 0};
  return {static_cast<int>(j_lo / kTileKeys), static_cast<int>(j_hi / kTileKeys) + 1};
}

struct TcArgs {
  float* out;
  float* m;
  float* l;
  int H, kvH, Sq;
  int n_qblocks_per_seg;
  PosMap qmap, kmap;
  int kseg_head[RA_MAX_SEG];  // key segment -> head-coordinate offset and first row in K / V
  int kseg_row[RA_MAX_SEG];
  int stride;
  unsigned flags;
  long long doc_len;
  int* status;
  unsigned long long wait_ns;  // limit of every device-side wait
  int stall_after;             // test hook: the producer stops after this many ring items (< 0: off)
  int kv_per_wave;             // block order: waves of this many KV heads (0: heads fastest)
};

// ---- host side ----------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// (D, rows, heads) tensor of 16-bit (RA_F16 / RA_BF16) or 32-bit (RA_F32) elements, box = one
// 128-byte row piece (64 or 32 elements) x box_rows rows x 1, 128B swizzle. With a box wider than
// the tensor (head_dim 32 in 16 bits) the upper elements of every row are out of bounds and
// arrive as zeros, which is exactly a head_dim 64 tile whose upper half is zero.
inline int make_map(CUtensorMap* map, int dtype, const void* base, int D, long long rows,
                    long long heads, long long head_stride_elems, int box_rows = 128,
                    bool swizzle_32b_atoms = false) {
  EncodeTiledFn fn = encode_fn();
  RAB_REQUIRE(fn != nullptr, RA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t es = dtype == RA_F32 ? 4 : 2;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(heads)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * es,
                                 static_cast<cuuint64_t>(head_stride_elems) * es};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType type = dtype == RA_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == RA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(map, type, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_32b_atoms ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RAB_REQUIRE(r == CUDA_SUCCESS, RA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d",
              static_cast<int>(r));
  return RA_OK;
}

// Limits set through the test hooks (step_tc.cu owns them).
unsigned long long tc_wait_limit_ns();
int tc_stall_after();

}  // namespace tcgen
}  // namespace rab
