// Shared device / host helpers for the sm_100a kernels: PTX wrappers (mbarrier, TMA, tcgen05 / tensor memory),
// number-format conversions with the exact rounding the FlashIM reference prescribes, bounded waits and the status
// word they report to.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fim {

// ---- return codes of the C entry points (0 ok; positive cudaError_t values pass through) -----------------------
constexpr int kOk = 0;
constexpr int kBadLayout = -1;    // pointer alignment / shape the kernel cannot address
constexpr int kBadArgument = -2;  // null pointer, negative size, unknown mode
constexpr int kNoDriver = -3;     // cuTensorMapEncodeTiled could not be resolved / failed
constexpr int kUnsupported = 99;  // a tile or geometry outside what is compiled in

// ---- device status word: written once by the first CTA whose bounded wait ran out --------------------------------
constexpr int kStatusWaitFull = 0x101;       // producer -> MMA barrier never completed
constexpr int kStatusWaitEmpty = 0x102;      // MMA -> producer barrier never completed
constexpr int kStatusWaitTmemFull = 0x103;   // MMA -> epilogue barrier never completed
constexpr int kStatusWaitTmemEmpty = 0x104;  // epilogue -> MMA barrier never completed
constexpr int kStatusWaitRows = 0x105;       // depthwise row ring barrier never completed

__host__ __device__ constexpr int ceil_div(int a, int b) { return (a + b - 1) / b; }

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// A value the compiler must keep in a register: kernel parameters read inside the single-thread issue loops are otherwise
// re-read from the constant bank every iteration, and each such load is tens of cycles in a chain one thread walks alone.
__device__ __forceinline__ uint32_t in_register(uint32_t v) {
  uint32_t r;
  asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Longest time any wait inside a kernel may take before the CTA gives up (a healthy pipeline completes a phase in
// microseconds). Two seconds keeps a broken launch from hanging the device while never tripping on a busy GPU.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait on an mbarrier phase. Returns false when the CTA must abandon its work: either this wait exceeded
// kWaitLimitNs (the status word then receives `code`, first writer wins) or another thread of the CTA already
// raised `*abort_flag` (a word in shared memory).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if ((++spins & 31u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - start > kWaitLimitNs) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// Variants on a precomputed shared-memory address (the issue loops of the conv kernel keep them in registers).
__device__ __forceinline__ bool mbar_try_addr(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// `heed_abort` = false: only this wait's own time limit ends it. Warps that meet at a named barrier afterwards use it, so
// that all of them take the same decision (either the phase completes for all or it times out for all).
// `backoff_ns` > 0 sleeps that long between polls: a warp that expects to wait for microseconds (an epilogue warp during
// the main loop of its tile) then leaves the issue slots and the power budget to the warps that are working.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                            bool heed_abort, uint32_t backoff_ns) {
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_addr(bar, parity)) return true;
    if (backoff_ns != 0) __nanosleep(backoff_ns);
    if ((++spins & 31u) == 0u) {
      if (heed_abort && *abort_flag) return false;
      if (global_timer_ns() - start > kWaitLimitNs) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                               bool heed_abort = true, uint32_t backoff_ns = 0) {
  if (mbar_try_addr(bar, parity)) return true;
  if (mbar_try_addr(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code, heed_abort, backoff_ns);
}
// The wait as a whole warp takes it: every lane polls, and the warp agrees on the outcome, so the code after it stays
// warp-uniform (addresses and descriptors computed there can live in uniform registers).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                               bool heed_abort = true, uint32_t backoff_ns = 0) {
  const bool ok = mbar_wait_addr(bar, parity, abort_flag, status, code, heed_abort, backoff_ns);
  return __all_sync(0xffffffffu, ok) != 0;
}
// The same wait with its polling loop inlined: for kernels whose warps change their register allowance (setmaxnreg),
// where a function shared by regions with different allowances cannot be allocated.
__device__ __forceinline__ bool mbar_wait_inline(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                                 uint32_t backoff_ns = 0) {
  if (mbar_try_addr(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_addr(bar, parity)) return true;
    if (backoff_ns != 0) __nanosleep(backoff_ns);
    if ((++spins & 31u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - start > kWaitLimitNs) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_addr(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Barrier among `threads` threads of the CTA (a multiple of 32) on hardware barrier `id` (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- TMA ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_addr(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_addr(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_load_addr(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}
// ---- CTA pairs (a cluster of two CTAs driving one cta_group::2 tensor-core instruction stream) ------------------------
// Shared-memory addresses of the odd CTA of a pair carry this bit in the cluster's shared address space; clearing it
// names the same location in the even (leader) CTA, setting it the one in the odd CTA.
constexpr uint32_t kPeerBit = 1u << 24;
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tiled loads of a CTA pair: the bytes land in this CTA's shared memory and are counted on the barrier `bar`, which may
// live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// One arrival on a barrier anywhere in the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Tiled store shared -> global (clipped at the tensor bounds), tracked by the thread's bulk async-group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's committed store groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---- tensor memory + tcgen05 ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
// The same for a CTA pair: one warp (the same warp index) of each CTA of the pair executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// All tcgen05 operations this thread issued so far arrive on `bar` when they complete.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Pair form, issued by the leader CTA: arrives on the barrier at cluster address `bar` (either CTA of the pair) when the
// pair's tcgen05 operations issued so far complete.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 tensor-memory columns, replicated into the four 32-lane quarters.
__device__ __forceinline__ void tc_copy_scales(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
// Pair forms (issued by the leader): each CTA copies from its own shared memory into its own tensor memory; the MMA has
// M = 256 (128 rows per CTA), reads A and its half of B from each CTA's shared memory at the same offsets.
__device__ __forceinline__ void tc_copy_scales_pair(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// This thread's lane of tensor memory, 32 consecutive 32-bit columns starting at `addr`.
__device__ __forceinline__ void tmem_load_32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile whose rows are `row_bytes` (32, 64 or 128) long and
// swizzled with the matching TMA mode: 8-row groups are `8 * row_bytes` apart (stride byte offset), the leading
// offset is unused because one swizzle span covers the whole K extent of the tile.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t smem_addr, uint32_t row_bytes) {
  const uint64_t layout = row_bytes == 128 ? 2ull : (row_bytes == 64 ? 4ull : 6ull);
  uint64_t d = (smem_addr & 0x3FFFFu) >> 4;
  d |= static_cast<uint64_t>((8u * row_bytes) >> 4) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= layout << 61;
  return d;
}
// Descriptor of one 512-byte scale tile (32 rows x 16 bytes, no swizzle): 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t scale_desc(uint32_t smem_addr) {
  uint64_t d = (smem_addr & 0x3FFFFu) >> 4;
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= 1ull << 46;
  return d;
}

// ---- number formats ------------------------------------------------------------------------------------------------

// Unbiased E8M0 exponent of a block with maximum magnitude `amax` (>= 0): the reference's fp32 expression
// clamp(ceil(log2(amax / 448)), -127, 127), -127 for amax == 0, evaluated without floating point. With
// amax = m * 2**E (1 <= m < 2) the value is E - 8 when m <= 1.75 and E - 7 above, except that the fp32 logarithm of a
// ratio a few ulp above one rounds back to the integer E - 8: the reference keeps E - 8 for mantissas up to `slack` ulp
// above 1.75, where slack (0, 2, 4, 9, 20, 39) only depends on the binade of |E - 8|, i.e. on the ulp of the fp32 number
// E - 8 + epsilon. The thresholds were read off the reference expression for every exponent and the rule reproduces it
// on all boundary cases (tests compare the bytes).
__device__ __forceinline__ int e8m0_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  if (bits == 0u) return -127;
  const int E = static_cast<int>(bits >> 23) - 127;
  if (E == 128) return 127;  // inf / nan
  const int k = E - 8;
  const int m = k >= 0 ? k : -k - 1;
  const int binade = min(5, max(0, 30 - __clz(m)));
  const uint32_t slack = static_cast<uint32_t>(0x271409040200ull >> (8 * binade)) & 0xFFu;
  const uint32_t threshold = 0x600000u + slack + (E == -119 ? 1u : 0u);
  const int e = (bits & 0x7FFFFFu) > threshold ? k + 1 : k;
  return min(127, max(-127, e));
}

// The same value on the bits of a non-negative amax, arranged for issue slots: away from the narrow mantissa window where
// the reference's logarithm rounds back (40 ulp above 1.75) the answer is E - 8 + (mantissa > 1.75), clamped; inside
// the window (and for inf / nan) the full rule decides. The branch is taken about once in 200000 blocks.
__device__ __forceinline__ int e8m0_exponent_bits(uint32_t bits) {
  const uint32_t mantissa = bits & 0x7FFFFFu;
  const int biased = static_cast<int>(bits >> 23);
  int e = biased - 135 + (mantissa > 0x600000u ? 1 : 0);
  if ((mantissa - 0x600001u) < 40u || biased == 255) e = e8m0_exponent(__uint_as_float(bits));
  return min(127, max(-127, e));
}

// max over the lanes named in `mask` (every one of which executes this with the same mask)
__device__ __forceinline__ uint32_t redux_max(uint32_t value, uint32_t mask) {
  uint32_t r;
  asm volatile("redux.sync.max.u32 %0, %1, %2;" : "=r"(r) : "r"(value), "r"(mask));
  return r;
}

// 2**e for e in [-127, 127], exact (2**-127 is a subnormal).
__device__ __forceinline__ float exp2_int(int e) {
  return __uint_as_float(e == -127 ? 0x00400000u : static_cast<uint32_t>(e + 127) << 23);
}

// Two fp32 -> two E4M3 bytes (round to nearest even, saturating to +-448); `lo` lands in the low byte.
__device__ __forceinline__ uint16_t e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(e4m3x2(a, b)) | (static_cast<uint32_t>(e4m3x2(c, d)) << 16);
}

// round_half_even(value / scale) saturated to [-127, 127]: a true IEEE division, as the reference's quantiser.
__device__ __forceinline__ int int8_code(float value, float scale) {
  const float q = rintf(__fdiv_rn(value, scale));
  return static_cast<int>(fminf(fmaxf(q, -127.0f), 127.0f));
}

// The same code for many values under one scale, without a division instruction. With inv = RN(1 / scale), the product
// q0 = value * inv is within two ulp of the quotient, and each step q <- RN(q + (value - q * scale) * inv), whose residual
// the fma forms exactly, sharpens it: after the first step q is faithful (within one ulp), and a faithful q refined once
// more with a correctly rounded reciprocal IS the correctly rounded quotient (Markstein's division theorem; its one
// exception, a divisor whose significand is all ones, takes the IEEE division, as do scales whose reciprocal leaves the
// normal range). Values whose quotient is huge, infinite or NaN keep q0, which saturates the same way.
// Rounding to the nearest-even integer is then the fp32 addition of 1.5 * 2**23 (the sum has an ulp of one) after a clamp
// to +-127.25 (anything beyond rounds or saturates to +-127; NaN becomes -127 like the saturating division path): the low
// mantissa byte of the sum is the code in two's complement, so no round or convert instruction is needed either.
struct Int8Quantizer {
  float scale, inv;
  bool exact_only;
};
__device__ __forceinline__ Int8Quantizer make_int8_quantizer(float s) {
  Int8Quantizer q;
  q.scale = s;
  q.inv = __frcp_rn(s);
  q.exact_only = !(fabsf(s) >= 1e-25f && fabsf(s) <= 1e30f) || (__float_as_uint(s) & 0x7FFFFFu) == 0x7FFFFFu;
  return q;
}
__device__ __forceinline__ int int8_exact(float scale, float value) {
  return static_cast<int>(fminf(fmaxf(rintf(__fdiv_rn(value, scale)), -127.0f), 127.0f));
}
// bits whose low byte is the code
__device__ __forceinline__ uint32_t int8_bits(const Int8Quantizer& z, float value) {
  constexpr float kMagic = 12582912.0f;  // 0x4B400000
  const float q0 = value * z.inv;
  float q = fmaf(fmaf(-q0, z.scale, value), z.inv, q0);
  q = fmaf(fmaf(-q, z.scale, value), z.inv, q);
  q = fabsf(q0) < 1e6f ? q : q0;
  return __float_as_uint(fminf(fmaxf(q, -127.25f), 127.25f) + kMagic);
}
__device__ __forceinline__ int int8_code(const Int8Quantizer& z, float value) {
  if (z.exact_only) return int8_exact(z.scale, value);
  return static_cast<int>(static_cast<int8_t>(int8_bits(z, value) & 0xFFu));
}
// Two / four codes in the low bytes of a word (value 0 first).
__device__ __forceinline__ uint32_t int8_pack2(const Int8Quantizer& z, float v0, float v1) {
  if (z.exact_only) return (static_cast<uint32_t>(int8_exact(z.scale, v0)) & 0xFFu) | ((static_cast<uint32_t>(int8_exact(z.scale, v1)) & 0xFFu) << 8);
  return __byte_perm(int8_bits(z, v0), int8_bits(z, v1), 0x4440) & 0xFFFFu;
}
__device__ __forceinline__ uint32_t int8_pack4(const Int8Quantizer& z, float v0, float v1, float v2, float v3) {
  if (z.exact_only) {
    return (static_cast<uint32_t>(int8_exact(z.scale, v0)) & 0xFFu) | ((static_cast<uint32_t>(int8_exact(z.scale, v1)) & 0xFFu) << 8) |
           ((static_cast<uint32_t>(int8_exact(z.scale, v2)) & 0xFFu) << 16) | ((static_cast<uint32_t>(int8_exact(z.scale, v3)) & 0xFFu) << 24);
  }
  return __byte_perm(__byte_perm(int8_bits(z, v0), int8_bits(z, v1), 0x4440), __byte_perm(int8_bits(z, v2), int8_bits(z, v3), 0x4440), 0x5410);
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// GELU, erf form, in the operation order of torch's CPU kernel: x * 0.5 * (1 + erf(x * sqrt(1/2))).
__device__ __forceinline__ float gelu_erf(float x) { return x * 0.5f * (1.0f + erff(x * 0.70710678118654752440f)); }

// ---- packed fp32 pairs (one issue slot for two lanes' worth of fp32 work) -------------------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// bf16x2 word -> its two values as a packed fp32 pair (low half first)
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t w) { return pack2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u)); }

// ---- bf16x2 words (two bf16 values in one register; one instruction for both) ---------------------------------------
__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// magnitude max(|a|, |b|) per half; the sign bit of each half is the xor of the operands' signs (mask it off)
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// GELU through the complementary error function in the rational-exponential form of Abramowitz & Stegun 7.1.26
// (|error of erf| <= 1.5e-7): gelu(x) = x/2 * (2 - c) for x >= 0 and x/2 * c for x < 0 with c = erfc(|x|/sqrt 2).
// No branch, two MUFU operations. For every bf16 input with |x| < 3 the bf16-rounded result equals that of the erf form
// above; beyond x < -4.5 (|gelu| < 2e-5) both forms are dominated by their own rounding.
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// On a packed pair, arranged for issue slots (11 packed operations, 2 MUFU per element): with q = 1/2 - c/2 and
// c = erfc(|x| / sqrt 2) the value is x/2 + |x| q, which needs no sign select; the polynomial carries the factor -1/2, so
// q is one fma on the exponential, and the MUFU operations take their operands straight from the halves of the pair.
__device__ __forceinline__ uint64_t gelu_fast2(uint64_t x2) {
  float x0, x1;
  unpack2(x2, x0, x1);
  const uint64_t ax = pack2(fabsf(x0), fabsf(x1));
  float d0, d1;
  unpack2(fma2(pack2(0.23164190f, 0.23164190f), ax, pack2(1.0f, 1.0f)), d0, d1);  // 1 + 0.3275911 |x| / sqrt 2
  const uint64_t t = pack2(rcp_approx(d0), rcp_approx(d1));
  uint64_t poly = fma2(pack2(-0.5307027145f, -0.5307027145f), t, pack2(0.7265760135f, 0.7265760135f));  // -1/2 of A&S
  poly = fma2(poly, t, pack2(-0.7107068705f, -0.7107068705f));
  poly = fma2(poly, t, pack2(0.142248368f, 0.142248368f));
  poly = fma2(poly, t, pack2(-0.127414796f, -0.127414796f));
  float a0, a1;
  unpack2(mul2(mul2(x2, x2), pack2(-0.72134752044448170f, -0.72134752044448170f)), a0, a1);  // -x^2 / 2 * log2(e)
  const uint64_t q = fma2(mul2(poly, t), pack2(ex2_approx(a0), ex2_approx(a1)), pack2(0.5f, 0.5f));
  return fma2(ax, q, mul2(x2, pack2(0.5f, 0.5f)));
}

__device__ __forceinline__ float gelu_fast(float x) {
  float lo, hi;
  unpack2(gelu_fast2(pack2(x, x)), lo, hi);
  return lo;
}

constexpr int kActNone = 0, kActRelu = 1, kActGelu = 2, kActReluEarly = 3;
__device__ __forceinline__ float activate(float x, int act) {
  if (act == kActRelu) return fmaxf(x, 0.0f);
  if (act == kActGelu) return gelu_erf(x);
  return x;
}

// Byte offset of element (row, group) in the 128-row x 4-group swizzled scale layout with `group_tiles` tiles per row tile.
__device__ __forceinline__ size_t swizzled_scale_offset(size_t row, int group, int group_tiles) {
  return ((row >> 7) * group_tiles + (group >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (group & 3);
}

#endif  // __CUDACC__

// ---- host: per-device facts ------------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
inline int current_device() {
  int device = -1;
  return cudaGetDevice(&device) == cudaSuccess ? device : -1;
}
// SMs of the current device (148 on a B200), asked once per device; persistent grids are sized from it.
inline int sm_count() {
  static int cached[kMaxDevices] = {};
  const int device = current_device();
  if (device < 0 || device >= kMaxDevices) return 148;
  if (cached[device] == 0) {
    int n = 0;
    cached[device] = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && n > 0 ? n : 148;
  }
  return cached[device];
}

// ---- host: tensor maps without linking libcuda ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

inline CUtensorMapSwizzle swizzle_for_bytes(int inner_bytes) {
  if (inner_bytes == 128) return CU_TENSOR_MAP_SWIZZLE_128B;
  if (inner_bytes == 64) return CU_TENSOR_MAP_SWIZZLE_64B;
  if (inner_bytes == 32) return CU_TENSOR_MAP_SWIZZLE_32B;
  return CU_TENSOR_MAP_SWIZZLE_NONE;
}

// Tiled tensor map over `rank` dimensions (innermost first). `strides_bytes` has rank-1 entries (dimension 0 is dense).
inline int make_tensor_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                           CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           const uint32_t* element_strides = nullptr) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return kNoDriver;
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = element_strides != nullptr ? element_strides[i] : 1;
    if (i + 1 < rank) s[i] = strides_bytes[i];
  }
  const CUresult r = fn(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kNoDriver;
}

}  // namespace fim
