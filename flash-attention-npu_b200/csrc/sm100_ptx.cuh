// Blackwell (sm_100a) building blocks as inline PTX: mbarriers with bounded waits, TMA tile
// loads, tensor-memory allocation, tcgen05 MMA / commit / ld / st, UMMA descriptors.
#pragma once
#include <type_traits>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {
namespace sm100 {

// Every wait gives up after this many clock cycles (about two seconds), records an error code
// and lets the kernel tear down cleanly instead of hanging the device.
constexpr long long kWaitCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival that orders nothing but itself: for hand-offs of TENSOR-memory data, whose completion the thread has
// already awaited (tcgen05.wait) and fenced (tcgen05.fence::before_thread_sync).  The default arrival is a release
// and first waits until the thread's earlier global stores have been performed, which puts the latency of
// unrelated stores on the hand-off.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  `abort_flag` (shared memory) is raised by whoever times out first so that every
// other waiter of the CTA leaves too; `err` (global) keeps the code for the host.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
    return true;
}

// The same for waits that are long and not latency-critical (a producer waiting for its buffer): the warp sleeps
// between polls so that it does not take issue slots from the warps doing arithmetic on the same scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(40);
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
    return true;
}

// ---- thread-block cluster: peer shared memory and barriers -------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of this CTA's shared-memory location `saddr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t d;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(d) : "r"(saddr), "r"(rank));
    return d;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// arrive on a barrier of another CTA; this thread's earlier stores to that CTA are visible to whoever waits on it
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// the same without ordering this thread's earlier memory operations (for "I have finished reading" signals)
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait on a barrier that threads of the peer CTA arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicCAS(err, 0, code);
                return false;
            }
        }
    }
    return true;
}
// Asynchronous bulk copy from this CTA's shared memory into a peer CTA's shared memory; `bytes` (a multiple of 16)
// are counted on the PEER's barrier `peer_bar` when they have landed.  `peer_dst` and `peer_bar` are cluster addresses.
// A copy that completes on an mbarrier belongs to no bulk async-group, so nothing on the issuing side tells when
// the source has been read: reuse the source only after the receiver has acknowledged the data.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t peer_dst, uint32_t src, uint32_t bytes, uint32_t peer_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(peer_dst), "r"(src), "r"(bytes), "r"(peer_bar) : "memory");
}
// all threads of all CTAs of the cluster
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- work stealing for persistent CTAs: a running CTA asks the hardware for the next not yet started CTA of its
// grid and runs that CTA's work itself (the asked-for CTA is then never launched) -----------------------------------
// The 16-byte answer arrives in shared memory at `slot` and completes 16 bytes on `bar`.
__device__ __forceinline__ void next_cta_request(uint32_t slot, uint32_t bar) {
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 ::"r"(slot), "r"(bar) : "memory");
}
// Decode an answer read back from `slot`: returns false when no CTA was left to take over.
__device__ __forceinline__ bool next_cta_decode(uint32_t slot, int& x, int& y, int& z) {
    uint32_t ok, cx, cy, cz;
    asm volatile(
        "{\n\t.reg .b128 resp;\n\t.reg .pred p;\n\t.reg .b32 dummy;\n\t"
        "ld.shared.b128 resp, [%4];\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, resp;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "mov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
        "@p clusterlaunchcontrol.query_cancel.get_first_ctaid.v4.b32.b128 {%1, %2, %3, dummy}, resp;\n\t}"
        : "=r"(ok), "=r"(cx), "=r"(cy), "=r"(cz) : "r"(slot) : "memory");
    x = (int)cx; y = (int)cy; z = (int)cz;
    return ok != 0;
}

// ---- fences -----------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA (every copy goes to one CTA only) ----------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// Plain (untiled) bulk copy of `bytes` contiguous bytes from global to this CTA's shared memory; both addresses
// 16-byte aligned, `bytes` a multiple of 16; completes on `bar` like a tile load.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- UMMA -------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version field = 1.
// K-major operand ([rows][64 elements] tiles, 128 B per row): SBO = 1024 B between 8-row groups.
// MN-major operand ([k][64 elements] tiles): LBO = distance between 64-element column groups,
// SBO = 1024 B between 8-row (k) groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;     // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;     // SWIZZLE_128B
    return d;
}
// Shared-memory matrix descriptor WITHOUT swizzle for an MN-major operand stored as [chunk of 8 MN elements][k][16 bytes]:
// eight consecutive k rows of one chunk are a contiguous 128-byte core matrix; `k_group_bytes` = distance between
// 8-row groups along K (leading offset), `mn_chunk_bytes` = distance between neighbouring 8-element chunks along MN
// (stride offset).
__device__ __forceinline__ uint64_t umma_desc_mn_noswizzle(uint32_t saddr, uint32_t k_group_bytes, uint32_t mn_chunk_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((k_group_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((mn_chunk_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;     // descriptor version (sm_100)
    return d;
}
// Descriptor of the same tile `byte_off` further on (the start-address field counts 16-byte units and
// never carries out of its 14 bits for shared-memory addresses).
__device__ __forceinline__ uint64_t umma_desc_at(uint64_t base, uint32_t byte_off) { return base + (byte_off >> 4); }

// Instruction descriptor for kind::f16 with fp32 accumulation.
// fmt: 0 = f16, 1 = bf16.  *_mn = 1 when the operand is MN-major (transposed).
__host__ __device__ constexpr uint32_t umma_idesc(int fmt, int m, int n, int a_mn, int b_mn) {
    return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
           (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same with the accumulate flag as a template constant: nothing data-dependent in front of the MMA.
template <int ACC>
__device__ __forceinline__ void umma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC) : "memory");
}
template <int ACC>
__device__ __forceinline__ void umma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(ACC) : "memory");
}
// Whole-warp variants: every lane executes the surrounding (convergent) code, so descriptor arithmetic can
// stay in uniform registers; one elected lane issues.  elect.sync picks the same lane for the same mask, so
// the MMAs and the commit that tracks them come from one thread.
template <int ACC>
__device__ __forceinline__ void umma_ss_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC) : "memory");
}
template <int ACC>
__device__ __forceinline__ void umma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(ACC) : "memory");
}
// The same with the descriptors formed inside the statement from a base and a compile-time byte offset, so that
// the compiler keeps one base in registers instead of one descriptor per K step.
template <int ACC, uint32_t A_OFF, uint32_t B_OFF>
__device__ __forceinline__ void umma_ss_wo(uint32_t d_tmem, uint64_t a_base, uint64_t b_base, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "add.u64 da, %1, %5;\n\t"
        "add.u64 db, %2, %6;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_base), "l"(b_base), "r"(idesc), "n"(ACC), "n"(A_OFF >> 4), "n"(B_OFF >> 4) : "memory");
}
template <int ACC, uint32_t A_COL, uint32_t B_OFF>
__device__ __forceinline__ void umma_ts_wo(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_base, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t.reg .b32 ta;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "add.u32 ta, %1, %5;\n\t"
        "add.u64 db, %2, %6;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_base), "r"(idesc), "n"(ACC), "n"(A_COL), "n"(B_OFF >> 4) : "memory");
}
// Four MMAs issued under ONE elect, descriptors advanced by adding to their low words (the start-address field;
// offsets in 16-byte units, compile-time).  The issuing warp runs beside the arithmetic warps of its scheduler and
// every instruction it spends between "operand ready" and "MMA issued" is on the critical path of the tile: against
// one elect and two 64-bit additions per MMA this form measured 3.6 % on the whole forward.
// `acc0` is the accumulate flag of the first MMA, the other three accumulate.
#define FA_UMMA_SS_STEP(AOP, BOP, P) \
    "add.u32 x, %1, " AOP ";\n\tadd.u32 y, %3, " BOP ";\n\tmov.b64 da, {x, %2};\n\tmov.b64 db, {y, %4};\n\t" \
    "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, " P ";\n\t"
template <uint32_t A0, uint32_t A1, uint32_t A2, uint32_t A3, uint32_t B0, uint32_t B1, uint32_t B2, uint32_t B3>
__device__ __forceinline__ void umma_ss_group4(uint32_t d_tmem, uint64_t a_base, uint64_t b_base, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n\t.reg .pred q, p0, p1;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p0, %6, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        FA_UMMA_SS_STEP("%7", "%11", "p0") FA_UMMA_SS_STEP("%8", "%12", "p1") FA_UMMA_SS_STEP("%9", "%13", "p1") FA_UMMA_SS_STEP("%10", "%14", "p1")
        "}"
        ::"r"(d_tmem), "r"(static_cast<uint32_t>(a_base)), "r"(static_cast<uint32_t>(a_base >> 32)),
          "r"(static_cast<uint32_t>(b_base)), "r"(static_cast<uint32_t>(b_base >> 32)), "r"(idesc), "r"(acc0),
          "n"(A0), "n"(A1), "n"(A2), "n"(A3), "n"(B0), "n"(B1), "n"(B2), "n"(B3) : "memory");
}
#undef FA_UMMA_SS_STEP
// The same with A in tensor memory: A column C0 + i * CSTEP, B offset B0 + i * BSTEP for step i.
#define FA_UMMA_TS_STEP(COP, BOP, P) \
    "add.u32 ta, %1, " COP ";\n\tadd.u32 y, %2, " BOP ";\n\tmov.b64 db, {y, %3};\n\t" \
    "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, " P ";\n\t"
template <uint32_t C0, uint32_t CSTEP, uint32_t B0, uint32_t BSTEP>
__device__ __forceinline__ void umma_ts_group4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_base, uint32_t idesc, uint32_t acc0) {
    asm volatile(
        "{\n\t.reg .pred q, p0, p1;\n\t.reg .b64 db;\n\t.reg .b32 ta, y;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p0, %5, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        FA_UMMA_TS_STEP("%6", "%10", "p0") FA_UMMA_TS_STEP("%7", "%11", "p1") FA_UMMA_TS_STEP("%8", "%12", "p1") FA_UMMA_TS_STEP("%9", "%13", "p1")
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(static_cast<uint32_t>(b_base)), "r"(static_cast<uint32_t>(b_base >> 32)), "r"(idesc), "r"(acc0),
          "n"(C0), "n"(C0 + CSTEP), "n"(C0 + 2 * CSTEP), "n"(C0 + 3 * CSTEP),
          "n"(B0), "n"(B0 + BSTEP), "n"(B0 + 2 * BSTEP), "n"(B0 + 3 * BSTEP) : "memory");
}
#undef FA_UMMA_TS_STEP
// [128 x N] scores = A x B^T over KSTEPS * 16 head dims, both operands K-major tiles of 64-dim sub-tiles SUB bytes apart
template <int KSTEPS, uint32_t SUB>
__device__ __forceinline__ void umma_ss_scores(uint32_t d_tmem, uint64_t a_base, uint64_t b_base, uint32_t idesc) {
    static_assert(KSTEPS == 4 || KSTEPS == 8, "head dim 64 or 128");
    constexpr uint32_t S = SUB >> 4;
    umma_ss_group4<0, 2, 4, 6, 0, 2, 4, 6>(d_tmem, a_base, b_base, idesc, 0);
    if constexpr (KSTEPS == 8) umma_ss_group4<S, S + 2, S + 4, S + 6, S, S + 2, S + 4, S + 6>(d_tmem, a_base, b_base, idesc, 1);
}
__device__ __forceinline__ void umma_commit_w(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar) : "memory");
}
// Arrive on `bar` once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- TMEM <-> registers: each thread of a warp owns one lane (row), 32 consecutive 32-bit columns ----------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Compile-time loop: f(std::integral_constant<int, I>) for I in [B, E).
template <int B, int E, class F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (B < E) {
        f(std::integral_constant<int, B>{});
        static_for<B + 1, E>(f);
    }
}

// Warp-group register reallocation (all four warps of an aligned group execute it together).
template <int N> __device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs (sm_100): one instruction, two lanes of the FMA pipe.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// 2^x for two values on the FMA pipe instead of the special-function unit: x is split into its nearest integer n
// (adding 1.5*2^23 leaves n in the low mantissa bits) and f = x - n in [-0.5, 0.5]; a degree-4 polynomial gives 2^f
// to 2.7e-6 relative, and n is added to the exponent field.  Inputs below -125 return about 2^-125.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    const float2 big = make_float2(12582912.f, 12582912.f);
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 r = add2(x, big);
    const float2 n = add2(r, make_float2(-12582912.f, -12582912.f));
    const float2 fr = fma2(n, make_float2(-1.f, -1.f), x);
    float2 q = fma2(fr, make_float2(0.00957401655614376f, 0.00957401655614376f), make_float2(0.055918190628290176f, 0.055918190628290176f));
    q = fma2(q, fr, make_float2(0.2402464896440506f, 0.2402464896440506f));
    q = fma2(q, fr, make_float2(0.6931217312812805f, 0.6931217312812805f));
    q = fma2(q, fr, make_float2(0.9999992847442627f, 0.9999992847442627f));
    return make_float2(__uint_as_float(__float_as_uint(q.x) + (__float_as_uint(r.x) << 23)),
                       __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(r.y) << 23)));
}

}  // namespace sm100

// (dim, head, row, batch) view with a [64 x box_heads x box_rows x 1] box and 128-byte swizzle (fwd_sm100.cu); the box
// lands in shared memory as box_rows x box_heads rows of 128 bytes, heads fastest
int make_tile_map(CUtensorMap* map, int dtype, const void* ptr, int d, int heads, int64_t rows, int batch,
                  int64_t stride_h, int64_t stride_s, int64_t stride_b, int box_rows, int box_heads = 1);
bool tensor_map_encoder_available();
// (batch entry, head) pairs of one chunk of a tcgen05 kernel's grid (fwd_sm100.cu)
int grid_chunk(int64_t pairs, int64_t bytes_per_pair);
// code left by a timed-out wait in the backward kernels (bwd_sm100.cu); synchronises
int bwd_sm100_error_flag(bool clear);

}  // namespace fa
