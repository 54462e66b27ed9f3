// Thin inline-PTX layer for sm_100a: mbarriers with bounded waits, bulk/tensor
// async copies (TMA), tensor memory (TMEM) management and tcgen05 MMA issue.
// Everything here is a direct wrapper of one PTX instruction or a small
// descriptor builder; the kernels compose them.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace cfx {
namespace umma {

// Debug builds (-DCFX_CHECK): every wrapper verifies the alignment rules of its operands,
// reports a violation with printf and SKIPS the operation (the kernel's bounded waits then
// end it with a status code instead of a fault).
#ifdef CFX_CHECK
#define CFX_CHK(cond, what, a, b)                                                          \
    if (!(cond)) {                                                                         \
        printf("CFX_CHECK %s: block %d thread %d a=%llx b=%llx\n", what, (int)blockIdx.x,  \
               (int)threadIdx.x, (unsigned long long)(a), (unsigned long long)(b));        \
        return;                                                                            \
    }
#define CFX_CHK_BOOL(cond, what, a, b)                                                     \
    if (!(cond)) {                                                                         \
        printf("CFX_CHECK %s: block %d thread %d a=%llx b=%llx\n", what, (int)blockIdx.x,  \
               (int)threadIdx.x, (unsigned long long)(a), (unsigned long long)(b));        \
        return false;                                                                      \
    }
#else
#define CFX_CHK(cond, what, a, b)
#define CFX_CHK_BOOL(cond, what, a, b)
#endif

// ------------------------------------------------------------------ addresses
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    CFX_CHK((bar & 7) == 0 && bar < 233472, "mbar_init", bar, count)
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    CFX_CHK((bar & 7) == 0 && bar < 233472, "mbar_arrive", bar, 0)
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    CFX_CHK((bar & 7) == 0 && bar < 233472, "mbar_expect_tx", bar, bytes)
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    CFX_CHK_BOOL((bar & 7) == 0 && bar < 233472, "mbar_try_wait", bar, parity)
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of a phase.  In isolation on B200 a probe of a completed phase costs ~2
// cycles against ~67 for try_wait; inside the fused kernel, however, putting a test_wait in
// front of every worker wait made the kernel 6 % slower, so only the MMA warp polls with it.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    CFX_CHK_BOOL((bar & 7) == 0 && bar < 233472, "mbar_test_wait", bar, parity)
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// 32-byte global store (sm_100: 256-bit stores); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(float* p, const float (&v)[8]) {
    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]),
                 "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
}

// Deferred probe.  mbar_test_wait reads its predicate right away, so the caller stalls for the
// probe's shared-memory round trip (150-200 cycles inside the fused kernel, also when the phase
// is long complete).  Here the predicate stays in a named register that is read later, and
// whatever is issued in between overlaps the round trip.  A name is declared once per kernel,
// at the top of the kernel body (CFX_PROBE_DECL), and cleared before its first read.
#define CFX_PROBE_DECL(name) asm volatile(".reg .pred " #name ";\n\tsetp.ne.u32 " #name ", 0, 0;")
#define CFX_PROBE(name, bar, parity)                                                   \
    asm volatile("mbarrier.test_wait.parity.shared::cta.b64 " #name ", [%0], %1;" ::   \
                     "r"(bar), "r"(parity) : "memory")
#define CFX_PROBE_CLEAR(name) asm volatile("setp.ne.u32 " #name ", 0, 0;")
#define CFX_PROBE_READ(name, out) asm volatile("selp.u32 %0, 1, 0, " #name ";" : "=r"(out) : : "memory")

// Bounded wait: spins on try_wait; after kWaitLimitNs without completion (or as soon as
// another thread of the CTA has given up) it records `code` in *abort_flag (shared
// memory) and returns false.  Callers then skip their work and fall through to the
// common exit, so a lost signal ends the kernel with an error status instead of a hang.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

template <bool kBackoff = true>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, uint32_t code,
                                          uint64_t limit_ns = kWaitLimitNs) {
    // One loop and nothing in front of it: peeling the first probe out of the loop (try_wait
    // or test_wait) made the fused kernel 10 % slower on B200.
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        // back off between probes: 1 % faster kernel than polling flat out when whole warps wait;
        // a single copy-issuing thread polls without it (its wake-up time is on the ring's path)
        if (kBackoff) __nanosleep(100);
        // the timer and the abort flag are looked at only every 4096 failed polls: reading
        // %globaltimer costs a few hundred ns and must stay off the normal path
        if ((++spins & 4095u) == 0) {
            if (*abort_flag != 0) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                atomicCAS((uint32_t*)abort_flag, 0u, code);
                return false;
            }
        }
    }
}

// Same contract, but polls with test_wait only (never suspends): for the MMA-issuing thread,
// whose wake-up latency is on the critical path of every tile.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity,
                                               volatile uint32_t* abort_flag, uint32_t code) {
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((++spins & 16383u) == 0) {
            if (*abort_flag != 0) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > kWaitLimitNs) {
                atomicCAS((uint32_t*)abort_flag, 0u, code);
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ TMA
// 1-D bulk copy global -> shared, completion on an mbarrier (complete_tx bytes).
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
    CFX_CHK((dst_smem & 15) == 0 && ((uintptr_t)src & 15) == 0 && (bytes & 15) == 0 && (bar & 7) == 0, "bulk_g2s", dst_smem, (uintptr_t)src)
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// 1-D bulk copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                 "r"(src_smem), "r"(bytes)
                 : "memory");
}
// 2-D tiled tensor copy global -> shared.  x = innermost coordinate (x * elemsize must be
// a multiple of 16 bytes), y = outer coordinate.
__device__ __forceinline__ void tensor_g2s_2d(uint32_t dst_smem, const CUtensorMap* map, int x,
                                              int y, uint32_t bar) {
    CFX_CHK((dst_smem & 127) == 0 && ((uintptr_t)map & 63) == 0 && (bar & 7) == 0, "tensor_g2s", dst_smem, (uintptr_t)map)
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// The same copy issued by a CTA of a pair (cta_group::2): the data lands in the issuing CTA's
// shared memory, the completion (complete_tx) may be counted on an mbarrier of EITHER CTA of
// the pair; `cluster_bar` is a shared::cluster address (mapa).  No multicast.
__device__ __forceinline__ void tensor_g2s_2d_pair(uint32_t dst_smem, const CUtensorMap* map, int x,
                                                   int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
// 2-D tiled tensor copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void tensor_s2g_2d(const CUtensorMap* map, uint32_t src_smem, int x,
                                              int y) {
    CFX_CHK((src_smem & 127) == 0 && ((uintptr_t)map & 63) == 0, "tensor_s2g", src_smem, (uintptr_t)map)
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src_smem), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's bulk groups still READ their shared source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Asks the memory system to bring [src, src + bytes) into L2 (no completion tracking);
// src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ TMEM
// Allocation by one full warp; the base address is written to shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    CFX_CHK((dst_smem & 3) == 0, "tmem_alloc", dst_smem, ncols)
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

// ---- CTA pairs (cluster of two CTAs driving one 256-row MMA, cta_group::2) ----
// Allocation and release are collective: the same warp of BOTH CTAs issues them with the same
// arguments.
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
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs: arrive (release) and wait (acquire) on the cluster barrier.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Arrive on an mbarrier of any CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    // default semantics (release at CTA scope), as for a local arrive: a cluster-scope
    // release here measured ~1,000-1,400 cycles per arrive
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// 32 lanes x 32 bit, N consecutive columns per thread: thread t of the warp reads lane
// (lane_base + t), columns [col, col + N).  taddr = (lane << 16) | col.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ MMA
// Shared-memory operand descriptor for a K-major tile stored in the 128-byte-swizzled
// canonical layout: rows of 128 bytes (64 two-byte or 32 four-byte K elements), groups of
// 8 rows = one 1024-byte swizzle atom, 16-byte chunks XORed with (row & 7).  The tile base
// must be 1024-byte aligned; stepping K inside the 128-byte row adds the byte offset to
// the start address.  Fields: start>>4 [0,14), LBO>>4 [16,30) (unused for swizzled
// K-major, set to 1), SBO>>4 [32,46) = 1024 B between 8-row groups, version 1 at [46,48),
// layout type SWIZZLE_128B = 2 at [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor of tcgen05.mma kind::f16 / kind::tf32 with fp32 accumulation,
// both operands K-major: c_format F32 = 1 at [4,6); a/b format at [7,10)/[10,13)
// (0 = f16, 1 = bf16, 2 = tf32); N>>3 at [17,23); M>>4 at [24,29).
constexpr uint32_t kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2;
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, int M, int N) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Pair MMA: D (+)= A * B over the 256 rows of both CTAs (128 TMEM lanes each).  A comes from
// each CTA's own tensor memory, B from shared memory: each CTA holds N/2 rows of the B tile at
// the descriptor's address.  Issued by one thread of the even CTA only.
__device__ __forceinline__ void mma_f16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Pair commit: arrives on the mbarrier at this shared-memory offset in BOTH CTAs once all
// MMAs this thread issued so far are complete.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\t"
        "mov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}" ::"r"(bar)
        : "memory");
}
// Makes the mbarrier track completion of all MMAs this thread issued so far
// (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    CFX_CHK((bar & 7) == 0 && bar < 233472, "mma_commit", bar, 0)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

}  // namespace umma
}  // namespace cfx
