// PTX wrappers shared by the tensor-core kernels of this library (sm_100a): bounded mbarrier
// waits, cp.async / bulk copies that signal mbarriers, tensor-memory allocation and loads,
// tcgen05.mma issue and commit, and the shared-memory operand tile layout with its descriptors.
// Everything is in an unnamed namespace: each translation unit gets its own copy.
#pragma once
#include "wcn_common.cuh"

namespace {

constexpr long long kWaitCycles = 4000000000ll;        // about two seconds
constexpr unsigned kSuspendNs = 20000;                  // per-attempt parking limit of a barrier wait
constexpr long long kStatusPollCycles = 2000000ll;     // about a millisecond between looks at the status word


// ------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
// One wait attempt.  The hardware may park the thread until the phase completes or
// `kSuspendNs` elapse, so a waiting warp does not compete for issue slots with the
// warps that are doing work.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(kSuspendNs)
      : "memory");
  return done != 0;
}
// Bounded wait.  Returns false when the deadline passed or another thread's wait already ran
// out.  The status word lives in global memory and is looked at about once per millisecond of
// waiting.  An expired wait overrides whatever the word held (a skipped out-of-range index is
// reported with a compare-and-swap that never overrides anything, see wcn_report_bounds).
// The slow path is a function of its own (not inlined): the waits sit in the hot loops of single-thread
// roles, whose instruction footprint should stay small.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int32_t* dev_status, long long limit) {
  const long long poll = limit < kStatusPollCycles ? limit : kStatusPollCycles;
  const long long t0 = clock64();
  long long next_check = t0 + poll;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    const long long now = clock64();
    if (now > next_check) {
      if (*(volatile int32_t*)dev_status == (int)WCN_ERR_WAIT_EXPIRED) return false;
      if (now - t0 > limit) {
        atomicExch(dev_status, (int)WCN_ERR_WAIT_EXPIRED);
        return false;
      }
      next_check = now + poll;
    }
  }
}
// The wait of the kernels whose roles are long single-thread or single-slot loops: the limit is about two
// seconds, the slow path is a call.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t* dev_status) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, dev_status, kWaitCycles);
}
// The same wait entirely inline, for roles in which many threads block often while holding many live
// registers (the weight-gradient kernel's producers): a call there spills around every blocked wait.
__device__ __forceinline__ bool mbar_wait_inline(uint32_t bar, uint32_t parity, int32_t* dev_status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  long long next_check = t0 + kStatusPollCycles;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    const long long now = clock64();
    if (now > next_check) {
      if (*(volatile int32_t*)dev_status == (int)WCN_ERR_WAIT_EXPIRED) return false;
      if (now - t0 > kWaitCycles) {
        atomicExch(dev_status, (int)WCN_ERR_WAIT_EXPIRED);
        return false;
      }
      next_check = now + kStatusPollCycles;
    }
  }
}
// The same wait with a caller-chosen limit (the self test of the expiry path).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, int32_t* dev_status, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, dev_status, limit_cycles);
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  // no "memory" clobber: the data is only observed after an mbarrier wait, which has one
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
// Arrive on `bar` once all cp.async copies issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_drain() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// Row tiles are written by cp.async whose completion is signalled through the tile's mbarrier
// (cp.async.mbarrier.arrive); the MMA issuer waits on that barrier and then issues tcgen05.mma on
// the tile.  No fence.proxy.async sits between the two: it is the sequence NVIDIA's CUTLASS uses
// in its sm_100 cp.async + UMMA main loop (producer_commit with cpasync_barrier_arrive,
// consumer_wait, then the MMAs), and a per-slot proxy fence in the single issuing thread
// measured 4-8 % of the layer time here.
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory: rows of RB = BK*2 bytes, 8-row atoms of
// 8*RB bytes stacked along M/N, 16-byte chunks XOR-swizzled inside an atom.
//   RB = 128: SWIZZLE_128B (layout code 2), chunk ^= row & 7
//   RB =  64: SWIZZLE_64B  (layout code 4), chunk ^= (row & 7) >> 1
template <int RB> __device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  const int r8 = row & 7;
  const int x = (RB == 128) ? r8 : (r8 >> 1);
  return (uint32_t)((row >> 3) * (8 * RB) + r8 * RB + ((chunk ^ x) << 4));
}
template <int RB> __device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);         // start address, 16-byte units
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)((8 * RB) >> 4) << 32;            // stride byte offset between 8-row atoms
  d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
  d |= (uint64_t)(RB == 128 ? 2 : 4) << 61;        // swizzle mode
  return d;
}


// The same tile read as an MN-major operand: MN (channels) runs along the tile row — RB bytes =
// RB/2 contiguous elements per MN chunk — and K (tile rows) down the rows, eight rows per
// swizzle atom.  `chunk_bytes` is the distance between consecutive MN chunks (tiles holding
// the next RB/2 channels); an instruction's K = 16 covers two 8-row atoms.
template <int RB> __device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t chunk_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);         // start address, 16-byte units
  d |= (uint64_t)((chunk_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset: next MN chunk
  d |= (uint64_t)((8 * RB) >> 4) << 32;            // stride byte offset: next 8 rows of K
  d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
  d |= (uint64_t)(RB == 128 ? 2 : 4) << 61;        // swizzle mode
  return d;
}

// Multiprocessors of the current device (cached per device).
inline int num_sms() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace
