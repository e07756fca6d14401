// Inline-PTX wrappers for sm_100a: mbarrier, TMA (tiled and tile::gather4),
// tcgen05 (TMEM allocation, MMA, commit, ld/st, fences).
//
// Every wait in this file is bounded: a wait that runs out of its time budget
// returns false instead of spinning forever, so a logic error can never wedge a
// shared GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace chord {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(v));
  return v;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------- programmatic dependent launch --

// Blocks until every kernel this launch depends on has completed and its writes are
// visible.  Returns at once in a kernel launched without the programmatic
// stream-serialization attribute.  Everything before it may only touch what no earlier
// kernel in the stream writes (shared and tensor memory, the weights).
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Lets the next kernel in the stream (if it was launched with the attribute) become
// resident as SMs free up, instead of after this grid has drained.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier --

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrival by lane 0 of a converged warp, as one predicated instruction: written as
// `if (lane == 0) mbar_arrive(bar)` it costs a divergent branch with its convergence
// barrier around a single instruction, several times per pipeline step.
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, uint32_t lane) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.eq.u32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
      "}\n" ::"r"(bar), "r"(lane)
      : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// One try: returns at once if the phase has completed, otherwise the hardware parks the
// warp until it completes or an implementation-defined limit (measured: ~4 us) runs out.
// Parked warps take no issue slots, which matters here: most warps of a CTA wait on
// barriers much of the time, and a hot spin would crowd out the ones that work.
// Two forms.  With a suspend-time hint the compiler emits try, nanosleep, try: the
// general kernel, whose waiters are mostly lone threads, measured 3-7 % faster with it.
// Without a hint it is a single instruction: the decode kernel, whose 24 warps all
// wait warp-wide, measured 2.5 % faster with that.
constexpr uint32_t kSuspendHintNs = 200000;

template <bool kHint = true>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  if (kHint) {
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return done != 0;
}

// Bounded wait.  `abort_flag` is a shared-memory word any role may set when it
// gives up; once set, every other waiter leaves too.  Returns false on
// timeout (about two seconds of SM clock) or abort.  The common case - the phase
// has already completed - costs one try and one branch; everything else is kept
// out of line so that the hot loops stay short.
constexpr long long kWaitTimeoutCycles = 4000000000ll;

static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity,
                                            volatile uint32_t* abort_flag) {
  // A few immediate retries for waits that are about to end, then sleep between
  // tries: some twenty warps per CTA wait most of the time, and a polling loop that
  // never yields would take the issue slots the working warps need.
  for (uint32_t spin = 0; spin < 4; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const long long start = clock64();
  uint32_t sleep_ns = 32;
  for (uint32_t spin = 1;; ++spin) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return true;
    if (sleep_ns < 256) sleep_ns <<= 1;
    if ((spin & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > kWaitTimeoutCycles) return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag);
}

// Warp-uniform form: every lane waits (each needs the acquire).  A warp executes the
// try as one instruction on one address, so its first outcome is the same in every
// lane; only the slow path can end differently per lane, and there the warp votes so
// that a timeout never splits it.
template <bool kHint = true>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile uint32_t* abort_flag) {
  if (mbar_try_wait<kHint>(bar, parity)) return true;
  const bool ok = mbar_wait_slow(bar, parity, abort_flag);
  return __all_sync(__activemask(), ok);
}

// Bounded wait built on the single-instruction try_wait (a failed try has already
// parked the warp until the phase completed or an implementation-defined time passed,
// so the loop needs no sleep), with a sticky failure word instead of a result to
// branch on: `bad` stays 0 while every wait so far was satisfied and becomes 1 when one
// gives up.  A wait gives up when 4e9 cycles of SM clock (kWaitTimeoutCycles) have passed since its
// first failed try, when the CTA's abort flag is seen non-zero, or when `bad` was
// already set on entry and the first two tries fail; it then also raises the abort
// flag.  The loop lives in one asm statement, so that the satisfied case is the try and
// one branch, with no compiler-visible control flow around it; the caller tests `bad`
// where it is cheap (once per stage), not after every wait.
__device__ __forceinline__ void mbar_wait_sticky(uint32_t bar, uint32_t parity, uint32_t abort_addr,
                                                 uint32_t& bad) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 f;\n\t"
      ".reg .u64 c0, c1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra WAIT_DONE;\n\t"
      "mov.u64 c0, %%clock64;\n\t"
      "WAIT_RETRY:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra WAIT_DONE;\n\t"
      "ld.volatile.shared::cta.u32 f, [%3];\n\t"
      "or.b32 f, f, %0;\n\t"
      "setp.ne.u32 q, f, 0;\n\t"
      "@q bra WAIT_FAIL;\n\t"
      "mov.u64 c1, %%clock64;\n\t"
      "sub.u64 c1, c1, c0;\n\t"
      "setp.lt.u64 q, c1, 4000000000;\n\t"
      "@q bra WAIT_RETRY;\n\t"
      "WAIT_FAIL:\n\t"
      "mov.u32 %0, 1;\n\t"
      "st.volatile.shared::cta.u32 [%3], %0;\n\t"
      "WAIT_DONE:\n\t"
      "}\n"
      : "+r"(bad)
      : "r"(bar), "r"(parity), "r"(abort_addr)
      : "memory");
}

// --------------------------------------------------------------------- TMA --

__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, uint32_t bar,
                                                 int32_t c0, int32_t c1, uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "l"(hint)
      : "memory");
}

// Four rows (r0..r3) of a 2-D tensor, columns [c0, c0 + box width), land as
// four consecutive box rows at dst.  Rows outside the tensor read as zero.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* tmap, uint32_t bar,
                                            int32_t c0, int32_t r0, int32_t r1, int32_t r2,
                                            int32_t r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(r0), "r"(r1),
        "r"(r2), "r"(r3)
      : "memory");
}

// L2 eviction-priority descriptors for the .L2::cache_hint TMA forms.
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

// 8-byte shared-memory load from a 32-bit shared address plus a compile-time offset
// (the offset folds into the instruction, so unrolled loads share one address register).
template <int kOffset>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(kOffset) : "memory");
  return v;
}

// ------------------------------------------------------------ cp.async (LSU) --

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;  // 0 source bytes zero-fills the 16-byte slot
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}

// Deferred arrival: counts toward the barrier's expected arrivals (no pending-count
// increment) and fires when all cp.async issued so far by this thread have completed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// Returns once at most kPending of this thread's committed groups are still in flight.
template <int kPending>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// ----------------------------------------------------------------- tcgen05 --

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

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc], kind::f16 (BF16 inputs, FP32 accumulate).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The four K16 MMAs of one 64-wide K half in one statement: A columns a, a + 8, a + 16,
// a + 24 of tensor memory, B descriptor advanced by 32 bytes (two 16-byte units) per K16.
// Only the first one may start a new accumulation.  Written as one block so that the
// operand arithmetic stays next to the instructions and, with warp-uniform inputs, in
// uniform registers: a lone issuing thread that forms every operand with separate
// dependent instructions was measured at ~190 cycles per MMA on a busy SM, against 64
// cycles of tensor-pipe time for a 128 x 128 x 16 MMA.
__device__ __forceinline__ void mma_ts_k64(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, t;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      ".reg .b64 b1, b2, b3;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "add.u32 a2, %1, 16;\n\t"
      "add.u32 a3, %1, 24;\n\t"
      "add.u64 b1, %2, 2;\n\t"
      "add.u64 b2, %2, 4;\n\t"
      "add.u64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, t;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc].
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives (count 1) on `bar` once every tcgen05.mma issued so far by this
// thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 16 columns: thread i of the warp reads lane (base + i), register j
// is column (base + j).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"
      " {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32"
      " {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}

// 16 lanes x 32 columns.  Thread t of the warp supplies, for column group u
// (columns 4u .. 4u+3): r[2u] -> (lane t/4, column 4u + t%4) and
// r[2u+1] -> (lane t/4 + 8, column 4u + t%4).
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32"
      " [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// The 16x128b.x8 store with the final multiplication folded in: register 4j+{0,2} of the
// operand is d[4j+{0,2}] times the low BF16 of the scale word and 4j+{1,3} times its high
// BF16 (scale word s0 for j < 2, s1 for j >= 2).  Products and store live in one asm
// statement so that the products are formed in the sixteen consecutive registers the
// store reads, with no copies in between; the scale halves are broadcast with mov.b32
// unpack/pack, which the assembler folds into the multiplies' operand selectors (a
// byte-permute per broadcast, done outside, measured 2.5 % slower).
__device__ __forceinline__ void tmem_st_16x128b_x8_scaled(uint32_t taddr, const uint32_t (&d)[16],
                                                           uint32_t s0, uint32_t s1) {
  asm volatile(
      "{\n\t"
      ".reg .b32 t<16>;\n\t"
      ".reg .b16 a, b, c, e;\n\t"
      ".reg .b32 s0l, s0h, s1l, s1h;\n\t"
      "mov.b32 {a, b}, %17;\n\t"
      "mov.b32 {c, e}, %18;\n\t"
      "mov.b32 s0l, {a, a};\n\t"
      "mov.b32 s0h, {b, b};\n\t"
      "mov.b32 s1l, {c, c};\n\t"
      "mov.b32 s1h, {e, e};\n\t"
      "mul.rn.bf16x2 t0, %1, s0l;\n\t"
      "mul.rn.bf16x2 t1, %2, s0h;\n\t"
      "mul.rn.bf16x2 t2, %3, s0l;\n\t"
      "mul.rn.bf16x2 t3, %4, s0h;\n\t"
      "mul.rn.bf16x2 t4, %5, s0l;\n\t"
      "mul.rn.bf16x2 t5, %6, s0h;\n\t"
      "mul.rn.bf16x2 t6, %7, s0l;\n\t"
      "mul.rn.bf16x2 t7, %8, s0h;\n\t"
      "mul.rn.bf16x2 t8, %9, s1l;\n\t"
      "mul.rn.bf16x2 t9, %10, s1h;\n\t"
      "mul.rn.bf16x2 t10, %11, s1l;\n\t"
      "mul.rn.bf16x2 t11, %12, s1h;\n\t"
      "mul.rn.bf16x2 t12, %13, s1l;\n\t"
      "mul.rn.bf16x2 t13, %14, s1h;\n\t"
      "mul.rn.bf16x2 t14, %15, s1l;\n\t"
      "mul.rn.bf16x2 t15, %16, s1h;\n\t"
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "
      "{t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15};\n\t"
      "}\n"
      :
      : "r"(taddr), "r"(d[0]), "r"(d[1]), "r"(d[2]), "r"(d[3]), "r"(d[4]), "r"(d[5]), "r"(d[6]),
        "r"(d[7]), "r"(d[8]), "r"(d[9]), "r"(d[10]), "r"(d[11]), "r"(d[12]), "r"(d[13]), "r"(d[14]),
        "r"(d[15]), "r"(s0), "r"(s1)
      : "memory");
}

// 32 lanes x 8 columns: thread i writes lane (base + i), register j to column j.
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32"
      " [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7])
      : "memory");
}

// ------------------------------------------------------------- descriptors --

// K-major, 128-byte-swizzled operand tile in shared memory: rows of 64 BF16
// (128 bytes), eight-row groups 1024 bytes apart.  `addr` may point at a
// 32-byte K16 slice inside the 128-byte row.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                 // leading byte offset (unused; 16 B)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset: 8 rows
  d |= static_cast<uint64_t>(1) << 46;                 // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                 // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: BF16 x BF16 -> FP32, both operands K-major.
__device__ __forceinline__ uint32_t idesc_bf16_f32(uint32_t m, uint32_t n) {
  uint32_t d = 0;
  d |= 1u << 4;         // D format F32
  d |= 1u << 7;         // A format BF16
  d |= 1u << 10;        // B format BF16
  d |= (n >> 3) << 17;  // N
  d |= (m >> 4) << 24;  // M
  return d;
}

// ------------------------------------------------------- CTA pairs (cta_group::2) --
//
// Two CTAs of a cluster of two (ranks 0 and 1) on the two SMs of one TPC.  One thread of
// rank 0 issues tcgen05.mma.cta_group::2: A rows 0-127 come from rank 0's tensor memory
// and rows 128-255 from rank 1's (same address in both), B rows 0..N/2-1 from rank 0's
// shared memory and N/2..N-1 from rank 1's (same offset in both), and each CTA receives
// its 128 rows x N columns of D in its own tensor memory.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// All threads of both CTAs; orders shared-memory and barrier initialisation before the
// peer's first access.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The shared::cluster address of the same shared-memory location in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Arrival on a barrier of either CTA of the cluster (address from map_to_cta).
// Default semantics (as for a local arrival): a cluster-scope release was measured to
// double the dequant warps' time per stage; what the barrier orders here is tensor memory
// and TMA-written shared memory, which the tcgen05 fences and the transaction count cover.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// Tiled load into this CTA's shared memory whose bytes are counted on a barrier that may
// live in the peer CTA (address from map_to_cta).  No multicast: each CTA fetches its own
// rows.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t cluster_bar,
                                                 int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}

// Tensor-memory allocation for a CTA pair: the same warp index executes it in both CTAs
// with the same shared-memory destination; both receive the same column range.
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

// mma_ts_k64 for a CTA pair (M = 256 in the instruction descriptor).
__device__ __forceinline__ void mma_ts_k64_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, t;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      ".reg .b64 b1, b2, b3;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\t"
      "add.u32 a2, %1, 16;\n\t"
      "add.u32 a3, %1, 24;\n\t"
      "add.u64 b1, %2, 2;\n\t"
      "add.u64 b2, %2, 4;\n\t"
      "add.u64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a1], b1, %3, t;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a2], b2, %3, t;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [a3], b3, %3, t;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives (count 1) on the barrier at this shared-memory offset in both CTAs of the pair
// once every pair MMA issued so far by this thread has completed.  (A barrier arrival
// sent to two CTAs; no data is loaded.)
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t"
      "}\n" ::"r"(bar)
      : "memory");
}

// --------------------------------------------------------- global-memory sync --

__device__ __forceinline__ void red_release_add(int* addr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Shared-memory counter increment that orders the caller's earlier writes before it
// and later reads after it (CTA scope); returns the previous value.
__device__ __forceinline__ uint32_t atom_add_acq_rel_shared(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace ptx
}  // namespace chord
