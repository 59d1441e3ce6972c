// Thin inline-PTX wrappers for the sm_100a primitives the GEMM kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, no multicast anywhere), tcgen05 (TMEM
// allocation, MMA kind::i8, commit, ld) and the proxy / thread-sync fences.
//
// Every wait in this file is bounded: a spin that runs past WAIT_LIMIT_NS
// raises the CTA-wide abort flag, records a code in the host-visible status
// word and returns false, so a mistake upstream ends the kernel instead of
// hanging the GPU.
#pragma once

#include <cstdint>
#include <cuda.h>

namespace b200 {

// B200_TEST_WAIT_LIMIT_NS and B200_TEST_DROP_ACC_FULL_SIGNAL exist for ONE purpose: a test-only build of the
// library (never the shipped one) in which the MMA warp of the per-channel kernels does not signal "accumulator
// full", so that the epilogue's bounded wait runs out after a few milliseconds and the test can check that the
// kernel returns, reports STATUS_WAIT_TIMEOUT with the wait site, and leaves the context usable.
#ifdef B200_TEST_WAIT_LIMIT_NS
constexpr unsigned long long WAIT_LIMIT_NS = B200_TEST_WAIT_LIMIT_NS;
#else
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s
#endif
constexpr unsigned long long ABORT_DRAIN_NS = 200000ull;     // 0.2 ms, after a wait ran out only

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Error codes written to status[0] (status[1] = blockIdx.x, status[2] = site).
enum : int {
  STATUS_OK = 0,
  STATUS_WAIT_TIMEOUT = 1,
  STATUS_BAD_ARGUMENT = 2,
  STATUS_TASK_OVERFLOW = 3,  // grouped forward: the device-built task list did not fit; status[1] = tasks kept
  STATUS_TASK_ALIGNMENT = 4, // grouped forward, transposed lhs: a task starts on a row that is not a multiple of 16
                             // (status[1] = the task); the task was skipped
};

struct AbortCtx {
  volatile int* cta_flag;  // shared memory, one per CTA
  volatile int* status;    // host-mapped int[4], may be nullptr
};

// Bounded wait.  Returns false when the wait was abandoned (either this wait ran
// out of time or another role in the CTA already raised the abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtx& ctx,
                                          int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3FFu) == 0u) {
      if (*ctx.cta_flag) return false;
      if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
        *ctx.cta_flag = 1;
        if (ctx.status != nullptr && ctx.status[0] == STATUS_OK) {
          ctx.status[1] = static_cast<int>(blockIdx.x);
          ctx.status[2] = site;
          ctx.status[0] = STATUS_WAIT_TIMEOUT;
        }
        return false;
      }
    }
  }
}

// Bounded wait for a counter in global memory that other CTAs of the same (co-resident, persistent) grid raise.
// Same contract as mbar_wait: false when the wait was abandoned.
__device__ __forceinline__ bool flag_wait(const int* flag, int want, const AbortCtx& ctx, int site) {
  auto peek = [&]() -> int {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    return v;
  };
  if (peek() >= want) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (peek() >= want) return true;
    if ((++spins & 0xFFu) == 0u) {
      if (*ctx.cta_flag) return false;
      if (global_timer_ns() - t0 > WAIT_LIMIT_NS) {
        *ctx.cta_flag = 1;
        if (ctx.status != nullptr && ctx.status[0] == STATUS_OK) {
          ctx.status[1] = static_cast<int>(blockIdx.x);
          ctx.status[2] = site;
          ctx.status[0] = STATUS_WAIT_TIMEOUT;
        }
        return false;
      }
    }
  }
}

// One lane of a converged warp (the same lane every time within a call site is not guaranteed).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// CTA pairs (thread-block clusters of two)
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrive (count 1) on an mbarrier of any CTA of the cluster.  Default semantics (release at CTA scope), as
// for the waits: the data these barriers guard travels through the async proxy (TMA writes, tensor-core
// reads, tcgen05.commit), which orders itself against the barrier.  The explicitly cluster-scoped forms
// (arrive.release.cluster / try_wait.acquire.cluster) were measured: they made the pair kernels 2.4 times
// slower, one remote arrive then taking about a microsecond.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// fences
// ----------------------------------------------------------------------------
// Generic-proxy smem writes -> visible to the async proxy (TMA / tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA (2-D tiled loads; completion on an mbarrier of this CTA; no multicast)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// x = innermost coordinate (its byte offset must be a multiple of 16), y = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(src_smem)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all earlier bulk groups of this thread have finished READING shared memory (it may be rewritten)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recent bulk group of this thread have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read_keep1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// all but the N most recent bulk groups of this thread have finished reading shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read_keep() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// all earlier bulk groups of this thread are complete (their global writes are done)
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ----------------------------------------------------------------------------
// TMEM + tcgen05
// ----------------------------------------------------------------------------
// Whole-warp, converged.  Writes the TMEM base address to *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], s8 x s8 -> s32, issued by ONE thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive (count 1) on an mbarrier once every tcgen05.mma issued so far by this
// thread has completed.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// CTA-pair forms.  Allocation, release and deallocation are executed by the same warp of BOTH CTAs;
// the MMA and its commits by one thread of the leader CTA (rank 0) only.  The MMA reads A (128 rows)
// and B (N/2 columns) from each CTA's shared memory at the descriptor's offsets and writes rows
// 0..127 of the 256-row result to the leader's TMEM, rows 128..255 to the peer's.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand read from TMEM instead of shared memory: [a_tmem] addresses lanes = rows of this
// CTA's 128 rows of A and 8 columns per K = 32 step (four int8 values of consecutive k per 32-bit column).
__device__ __forceinline__ void umma_i8_pair_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (count 1) on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once every
// MMA issued so far by this thread has completed.  (A barrier signal, not a data load.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(static_cast<uint16_t>(3))
      : "memory");
}

// Each thread of the warp reads 32 consecutive 32-bit columns of its own TMEM
// lane (lane = 32 * (warp_id % 4) + lane_id, encoded in taddr bits [16,32)).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Each thread of the warp writes the same 32-bit value to 16 consecutive columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st_fill_32x32b_x16(uint32_t taddr, uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
      ::"r"(taddr), "r"(v)
      : "memory");
}
// Each thread of the warp writes 32 registers to 32 consecutive columns of its own TMEM lane.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// tcgen05.st is asynchronous too: its writes are in TMEM only after tcgen05.wait::st.
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_fence16(uint32_t (&r)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 8)
    asm volatile("" : "+r"(r[i]), "+r"(r[i + 1]), "+r"(r[i + 2]), "+r"(r[i + 3]), "+r"(r[i + 4]), "+r"(r[i + 5]),
                      "+r"(r[i + 6]), "+r"(r[i + 7])::"memory");
}
// tcgen05.ld is asynchronous: its destination registers are valid only after tcgen05.wait::ld.  When
// other work is placed between the load and the wait, this empty statement (after the wait) ties the
// registers to the wait so that the compiler cannot schedule a use of them before it.
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[32]) {
#pragma unroll
  for (int i = 0; i < 32; i += 8)
    asm volatile("" : "+r"(r[i]), "+r"(r[i + 1]), "+r"(r[i + 2]), "+r"(r[i + 3]), "+r"(r[i + 4]), "+r"(r[i + 5]),
                      "+r"(r[i + 6]), "+r"(r[i + 7])::"memory");
}

// Register re-balance between warpgroups (all four warps of the warpgroup must execute it).
template <int kRegs>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// UMMA descriptors
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version field = 1.
//   bits [0,14)  start address >> 4
//   bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4
//   bits [46,48) version (1)
//   bits [61,64) layout type (2 = SWIZZLE_128B)
// K-major operand  : rows of 128 bytes along K, 8-row groups SBO apart; LBO unused (1).
// MN-major operand : rows of 128 bytes along M/N, consecutive K rows 128 B apart, groups
//                    of 8 K rows SBO apart, 128-byte M/N blocks LBO apart.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::i8: s8 x s8 -> s32, dense, no saturation.
//   bits [4,6)=2 (S32 accumulator), [7,10)=1 (A signed 8-bit), [10,13)=1 (B signed 8-bit),
//   bit 15 = A is MN-major, bit 16 = B is MN-major, [17,23) = N>>3, [24,29) = M>>4.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int m, int n, bool a_mn_major,
                                                     bool b_mn_major) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace b200
