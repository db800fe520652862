// Forward attention on Blackwell tensor cores (tcgen05 + TMEM + TMA), sm_100a: one CTA owns 256 query rows of one
// head (two 128-row tiles) and walks 128-key tiles; a TMA warp, an MMA-issuing warp and two softmax warp groups
// (thread = query row).  Math as the reference's forward (mha_fwd_kvcache.cpp:632-969, online_softmax.hpp:623-875,
// rescale_o.hpp:318-531).
//
// Every mbarrier wait is bounded; a timeout records a code in g_fwd_sm100_error and the CTA
// frees its tensor memory and returns.
#include "fa_utils.cuh"
#include "fa_internal.h"
#include "sm100_ptx.cuh"

namespace fa {

using namespace sm100;

__device__ int g_fwd_sm100_error = 0;

struct alignas(64) Sm100FwdArgs {
    CUtensorMap tq, tk, tv;
    void* o;
    float* lse;
    int64_t o_sb, o_ss, o_sh;
    int64_t lse_sb, lse_sh, lse_ss;
    const int32_t* cu_q;
    const int32_t* cu_k;
    // KV-cache calls: device-resident lengths, page table, cache row of a batch entry
    const int32_t* seqused_k;
    const int32_t* block_table;
    const int32_t* cache_batch_idx;
    int64_t bt_stride;
    int page_size, s_new;
    int b, sq, sk, hq, hkv;
    int d;                               // the call's head dim (a multiple of 8): the kernels run the next of 64 / 128 / 192 / 256, the tile copies
                                         // zero-fill the columns past d and the epilogue stores d columns
    float scale_log2;
    int causal, wl, wr;
    // score transforms of the BIAS instantiation: softcap (0 = off) and alibi slopes ((hq) or (b,hq), null = off)
    float softcap, cap_in;               // cap_in = scale / softcap
    const float* alibi;
    int64_t alibi_sb;
    int kv_box;                          // rows of one K/V copy: 128, or 64 when pages are an odd multiple of 64 tokens
    int gq;                              // two-tile kernel: 1, or the query group size when a KV head's heads are stacked into the tile rows
    // split-KV (two-tile kernel, cache calls): split s of a sequence takes keys [s * keys_per_split, (s + 1) * ...) and
    // leaves a normalised fp32 partial output and its LSE for the combine kernel (nsplit = 1: final output directly)
    int nsplit, keys_per_split;          // keys_per_split is a multiple of 128
    float* o_part;                       // (nsplit, rows_all, D), rows_all = batch * sq * hq, row = (b * sq + qpos) * hq + head
    float* lse_part;                     // (nsplit, rows_all)
    int64_t rows_all;
    int chunk, nheads_grid;              // grid order, see the kernels: (batch entry, head) pairs a chunk; heads of the grid
};

// =================================================================================================
// Two query tiles per CTA (256 rows), P kept in tensor memory.
//   warps 0-3 / 4-7   softmax of query tile A / B (thread = row, TMEM lane = warp % 4 * 32 + lane)
//   warp 8            TMA producer and TMEM allocation
//   warp 9            MMA issuer
// Tensor memory: S_A | S_B | O_A | O_B, 128 columns each.  P (16-bit pairs) overwrites the first 64
// columns of its score buffer and feeds the second MMA as the A operand straight from TMEM.
// The two tiles ping-pong: while tile A is in softmax the tensor core runs P_B V and Q_B K^T, and
// vice versa.  The running max used as exponent base is only moved when the true max has grown by
// more than 2^8 (the accumulator is rescaled then), so rescaling O is rare and stays in the
// softmax warps.
// =================================================================================================
template <int D>
struct FwdSm100Smem2 {
    static constexpr int kSub = 128 * 128;
    static constexpr int kQ = (D / 64) * kSub;              // one query tile
    static constexpr int kKV = (D / 64) * kSub;
    static constexpr int oQ = 0;                            // 2 tiles
    static constexpr int oK = oQ + 2 * kQ;                  // 2 stages
    static constexpr int oV = oK + 2 * kKV;                 // 2 stages
    static constexpr int oBar = oV + 2 * kKV;
    static constexpr int kBytes = oBar + 320;        // barriers and flags
};

#ifndef FA_FWD_POLY
#define FA_FWD_POLY 2      // pairs of every 8 whose exponential runs on the FMA pipe
#endif
enum { C_Q = 0, C_KF0, C_KF1, C_KE0, C_KE1, C_VF0, C_VF1, C_VE0, C_VE1, C_SA, C_SB, C_PA, C_PB, C_PA2, C_PB2, C_OA, C_OB, C_DRAIN, C_COUNT };

template <typename T, int D, bool BIAS>
__global__ void __launch_bounds__(384, 1) fwd_sm100_kernel2(const __grid_constant__ Sm100FwdArgs a) {
    using L = FwdSm100Smem2<D>;
    constexpr int NSUB = D / 64;
    constexpr int KSTEPS = D / 16;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int FMT = Elem<T>::kDtype == FA_BF16 ? 1 : 0;
    constexpr uint32_t IDESC_QK = umma_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_PV = umma_idesc(FMT, 128, D, 0, 1);
    constexpr float kRescaleThreshold = 8.f;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t sQ = sbase + L::oQ, sK = sbase + L::oK, sV = sbase + L::oV;
    const uint32_t bars = sbase + L::oBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::oBar + 8 * C_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + L::oBar + 8 * C_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Grid order.  CTAs are dispatched in the order of their linear index, and under a causal mask the last query block
    // of a head has the most key tiles.  The grid is (pair in chunk, query block x split, chunk) over chunks of `chunk`
    // (batch entry, head) pairs: inside a chunk the heaviest blocks of ALL its pairs start before any lighter one
    // (longest job first; with one head after the other the last head's heavy blocks would start when the launch is
    // almost over: 7 % of a forward of 2048 CTAs by list-scheduling arithmetic), and a chunk is small enough for the K
    // and V of its pairs to stay in L2 while its query blocks run (a launch in longest-first order over everything
    // lost 20 % at 128 pairs of 2 MiB).  Pairs past the end of the last chunk leave.
    const int pair = blockIdx.z * a.chunk + blockIdx.x;
    if (pair >= a.b * a.nheads_grid) return;
    const uint3 bi = make_uint3(blockIdx.y, pair % a.nheads_grid, pair / a.nheads_grid);   // (query block x split, head, batch entry)
    const int nbx = gridDim.y;
    const int b = bi.z;
    // Tile rows.  gq = 1: 128 consecutive query positions of one head.  gq = G (short queries under a query
    // group of G, a power of two up to 128): the G heads of one KV head are stacked, row t of a tile is query
    // position t / G of head t % G — the tile copy delivers exactly that order from a (dims, G heads, 128 / G rows)
    // box — so that a short chunk fills the 128-row tiles instead of one tile per head with few rows in it.
    const int gq = a.gq;
    const int qpt = 128 / gq;                                // query positions of one 128-row tile
    const int hk = gq > 1 ? (int)bi.y : (int)bi.y / (a.hq / a.hkv);
    const int h0 = gq > 1 ? hk * gq : (int)bi.y;             // head of tile row 0
    const int split = bi.x % a.nsplit;
    const int mblk = nbx / a.nsplit - 1 - bi.x / a.nsplit;
    int q_off = 0, k_off = 0, sq = a.sq, sk = a.sk;
    if (a.cu_q) { q_off = a.cu_q[b]; sq = a.cu_q[b + 1] - q_off; k_off = a.cu_k[b]; sk = a.cu_k[b + 1] - k_off; }
    if (a.seqused_k) {                                       // cache call: the length lives on the device
        sk = (int)max(0LL, min((long long)a.seqused_k[b] + a.s_new, (long long)a.sk));   // an oversized entry is truncated to the capacity
    }
    const int m0 = mblk * 2 * qpt;                           // first query position of the CTA
    if (m0 >= sq) return;
    if (g_fwd_sm100_error) return;
    const int wl = a.wl, wr = a.causal ? 0 : a.wr;
    const int rows_cta = min(256, (sq - m0) * gq);           // tile rows in use
    const bool has_b = rows_cta > 128;

    int lo_first, hi_first, lo_last, hi_last;
    window_bounds(m0, sq, sk, wl, wr, lo_first, hi_first);
    window_bounds(m0 + (rows_cta - 1) / gq, sq, sk, wl, wr, lo_last, hi_last);
    int t_lo = lo_first / 128, t_hi = hi_last < 0 ? 0 : hi_last / 128 + 1;
    if (sk <= 0 || lo_first >= sk) { t_lo = 0; t_hi = 0; }
    if (a.nsplit > 1) {                                      // this split's share of the key tiles
        t_lo = max(t_lo, split * (a.keys_per_split / 128));
        t_hi = min(t_hi, (split + 1) * (a.keys_per_split / 128));
    }
    const int ntiles = max(0, t_hi - t_lo);
    // The first 128 rows of the block may end before the last key tile of the block (under a causal mask they end one
    // tile earlier): they skip the tiles in which every one of their entries is masked.
    int nt0 = ntiles;
    if (has_b) {
        int lo_a, hi_a;
        window_bounds(m0 + qpt - 1, sq, sk, wl, wr, lo_a, hi_a);
        const int n = min(ntiles, (hi_a < 0 ? 0 : hi_a / 128 + 1) - t_lo);
        if (n >= 1) nt0 = n;
    }

    // output row and LSE slot of tile row t (0..255) of this CTA
    auto out_row = [&](int t) -> T* {
        return reinterpret_cast<T*>(a.o) + (a.cu_q ? 0 : (int64_t)b * a.o_sb) + (int64_t)(q_off + m0 + t / gq) * a.o_ss + (int64_t)(h0 + t % gq) * a.o_sh;
    };
    auto lse_slot = [&](int t) -> float* {
        return a.lse + (a.cu_q ? 0 : (int64_t)b * a.lse_sb) + (int64_t)(h0 + t % gq) * a.lse_sh + (int64_t)(q_off + m0 + t / gq) * a.lse_ss;
    };
    // split-KV: row of tile row t in the partial buffers
    auto part_row = [&](int t) -> int64_t {
        return (int64_t)split * a.rows_all + ((int64_t)b * a.sq + m0 + t / gq) * a.hq + h0 + t % gq;
    };

    if (ntiles == 0 && a.nsplit > 1) {                       // an empty split: weight zero in the combine, O never read
        if (tid < rows_cta) a.lse_part[part_row(tid)] = -INFINITY;
        return;
    }
    if (ntiles == 0) {
        if (tid < rows_cta) {
            uint4 z = make_uint4(0, 0, 0, 0);
            T* orow = out_row(tid);
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                if (c * 8 < a.d) reinterpret_cast<uint4*>(orow)[c] = z;
            if (a.lse) *lse_slot(tid) = INFINITY;
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < C_COUNT; ++i) mbar_init(bar(i), (i >= C_PA && i <= C_PB2) ? 128u : 1u);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_fwd_sm100_error;
    const int qrow0 = (a.cu_q ? q_off : 0) + m0;
    const int qb = a.cu_q ? 0 : b;

    // Register file split by warp group: the copy/MMA group (warps 8-11, of which 10 and 11 only
    // exist to complete the group) keeps 56 registers a thread, the two softmax groups take 224.  The sum
    // 128*48 + 256*224 must stay within what the CTA was launched with (384 threads * 168 registers): an
    // increase beyond the CTA's pool would block forever.
    static_assert(128 * 56 + 256 * 224 <= 384 * 168, "register split exceeds the CTA's allocation");
    if (warp >= 8) {
    reg_dealloc<56>();
    if (warp == 8) {
        if (lane == 0) {
            tma_prefetch_desc(&a.tq); tma_prefetch_desc(&a.tk); tma_prefetch_desc(&a.tv);
            mbar_expect_tx(bar(C_Q), has_b ? 2 * L::kQ : L::kQ);
#pragma unroll
            for (int s = 0; s < NSUB; ++s) tma_load_4d(sQ + s * L::kSub, &a.tq, bar(C_Q), s * 64, h0, qrow0, qb);
            if (has_b) {
#pragma unroll
                for (int s = 0; s < NSUB; ++s) tma_load_4d(sQ + L::kQ + s * L::kSub, &a.tq, bar(C_Q), s * 64, h0, qrow0 + qpt, qb);
            }
            // where key tile j lives: (row, outermost coordinate) of the K / V maps.  Dense and packed operands: row
            // in the batch entry; cache: row in the cache entry of this batch; paged cache: row inside the page
            // that the page table names (a tile never straddles pages when the page size is a multiple of 128; pages of
            // an odd multiple of 64 tokens are copied in two boxes of 64 rows, each from its own page)
            const int32_t* btab = a.block_table ? a.block_table + (int64_t)b * a.bt_stride : nullptr;
            const int kbatch = a.cu_q ? 0 : (a.cache_batch_idx ? a.cache_batch_idx[b] : b);
            bool ok = true;
            for (int j = 0; j < ntiles && ok; ++j) {
                const int st = j & 1, use = j >> 1;
                int krow = (a.cu_q ? k_off : 0) + (t_lo + j) * 128, kouter = kbatch;
                int krow2 = 0, kouter2 = 0;                       // second half of the tile when it is copied in two boxes of 64 rows
                if (btab) {
                    const int pos = (t_lo + j) * 128;
                    kouter = btab[pos / a.page_size];
                    krow = pos % a.page_size;
                    if (a.kv_box == 64) {
                        // the tile may end in the next page; a half past the table's end is never attended (its
                        // columns are masked by the length), it is read from the first half's page
                        const bool in_table = (pos + 64) / a.page_size < a.bt_stride;
                        kouter2 = in_table ? btab[(pos + 64) / a.page_size] : kouter;
                        krow2 = in_table ? (pos + 64) % a.page_size : krow;
                    }
                }
                if (use > 0) ok = mbar_wait(bar(C_KE0 + st), (use - 1) & 1, abort_flag, err, 1);
                if (!ok) break;
                mbar_expect_tx(bar(C_KF0 + st), L::kKV);
#pragma unroll
                for (int s = 0; s < NSUB; ++s) {
                    tma_load_4d(sK + st * L::kKV + s * L::kSub, &a.tk, bar(C_KF0 + st), s * 64, hk, krow, kouter);
                    if (a.kv_box == 64) tma_load_4d(sK + st * L::kKV + s * L::kSub + 64 * 128, &a.tk, bar(C_KF0 + st), s * 64, hk, krow2, kouter2);
                }
                if (use > 0) ok = mbar_wait(bar(C_VE0 + st), (use - 1) & 1, abort_flag, err, 2);
                if (!ok) break;
                mbar_expect_tx(bar(C_VF0 + st), L::kKV);
#pragma unroll
                for (int s = 0; s < NSUB; ++s) {
                    tma_load_4d(sV + st * L::kKV + s * L::kSub, &a.tv, bar(C_VF0 + st), s * 64, hk, krow, kouter);
                    if (a.kv_box == 64) tma_load_4d(sV + st * L::kKV + s * L::kSub + 64 * 128, &a.tv, bar(C_VF0 + st), s * 64, hk, krow2, kouter2);
                }
            }
        }
    } else if (warp == 9) {
        {   // whole warp, one elected lane issues (see umma_ss_w)
            // descriptors of the tile origins, built once; the grouped issue adds compile-time offsets
            const uint64_t dQ0 = umma_desc(sQ, 16, 1024), dK0 = umma_desc(sK, 16, 1024), dV0 = umma_desc(sV, L::kSub, 1024);
            auto issue_qk = [&](int x, int st) {
                umma_ss_scores<KSTEPS, L::kSub>(tmem + x * 128, umma_desc_at(dQ0, x * L::kQ), umma_desc_at(dK0, st * L::kKV), IDESC_QK);
                umma_commit_w(bar(C_SA + x));
            };
            // P·V of tile x in two halves of 64 keys (16 keys = 8 columns of P, 2048 bytes of V a step): the second
            // half waits for its own barrier
            auto issue_pv = [&](int x, int st, int j) -> bool {
                const uint64_t bv = umma_desc_at(dV0, st * L::kKV);
                const uint32_t d_o = tmem + 256 + x * 128, a_p = tmem + x * 128;
                umma_ts_group4<0, 8, 0, 128>(d_o, a_p, bv, IDESC_PV, j > 0);
                if (!mbar_wait(bar(C_PA2 + x), j & 1, abort_flag, err, 11)) return false;
                tc_fence_after();
                umma_ts_group4<32, 8, 512, 128>(d_o, a_p, bv, IDESC_PV, 1);
                return true;
            };
            bool ok = mbar_wait(bar(C_Q), 0, abort_flag, err, 3);
            if (ok) ok = mbar_wait(bar(C_KF0), 0, abort_flag, err, 4);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
                if (has_b) issue_qk(1, 0);
                umma_commit_w(bar(C_KE0));
            }
            for (int j = 0; j < ntiles && ok; ++j) {
                const int st = j & 1, use = j >> 1;
                const bool more = j + 1 < ntiles;
                const int st1 = (j + 1) & 1, use1 = (j + 1) >> 1;
                const bool a_on = j < nt0, a_more = j + 1 < nt0;          // the first 128 rows take part in tile j / j+1
                // The copies of V(j) and K(j+1) were started a whole tile ago: their barriers are passed first, so that
                // nothing but the MMAs themselves stands between "P is ready" and the tensor core (this warp's
                // instructions are on the critical path of both query tiles).
                ok = mbar_wait(bar(C_VF0 + st), use & 1, abort_flag, err, 6);
                if (ok && more) ok = mbar_wait(bar(C_KF0 + st1), use1 & 1, abort_flag, err, 7);
                if (!ok) break;
                if (a.seqused_k && (t_lo + j) * 128 + 128 > sk) {
                    // Rows of a cache past the sequence hold whatever was there before (possibly NaN patterns): their
                    // probabilities are exact zeros, but 0 x NaN is NaN, so the V rows are cleared before the MMA.
                    // A row is 128 bytes in every 64-column sub-tile whatever the swizzle.
                    // Only rows the tile copy fetched need it: rows past the capacity of a dense cache were zero-filled
                    // by the copy itself.
                    const int first = max(0, sk - (t_lo + j) * 128);
                    const int last = a.block_table ? 128 : min(128, a.sk - (t_lo + j) * 128);
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub)
                        for (int idx = first * 8 + lane; idx < last * 8; idx += 32)     // 16-byte chunks of rows first .. last - 1
                            *reinterpret_cast<uint4*>(sgen + L::oV + st * L::kKV + sub * L::kSub + idx * 16) = make_uint4(0, 0, 0, 0);
                    fence_proxy_async_smem();
                    __syncwarp();
                }
                if (a_on) {
                    ok = mbar_wait(bar(C_PA), j & 1, abort_flag, err, 5);
                    if (!ok) break;
                    tc_fence_after();
                    ok = issue_pv(0, st, j);
                    if (!ok) break;
                    if (!a_more) umma_commit_w(bar(C_OA));
                    else issue_qk(0, st1);
                }
                if (has_b) {
                    ok = mbar_wait(bar(C_PB), j & 1, abort_flag, err, 8);
                    if (!ok) break;
                    tc_fence_after();
                    ok = issue_pv(1, st, j);
                    if (!ok) break;
                }
                umma_commit_w(bar(C_VE0 + st));
                if (more) {
                    if (has_b) issue_qk(1, st1);
                    umma_commit_w(bar(C_KE0 + st1));
                } else if (has_b) {
                    umma_commit_w(bar(C_OB));
                }
            }
            // The release of the last K/V stage has no waiter, and with one query tile in use it is issued after the
            // commit the epilogue waits for.  An arrive that the tensor core performs after the CTA has left would land
            // in shared memory the CTA no longer owns.  Commits complete in issue order, so the warp waits for a last
            // one of its own before it leaves.
            if (ok) {
                umma_commit_w(bar(C_DRAIN));
                ok = mbar_wait(bar(C_DRAIN), 0, abort_flag, err, 13);
            }
        }
    }
    } else {
    reg_alloc<224>();
    if (warp < 4 || has_b) {
        // ---------------------------------------------------------------- softmax of tile x
        const int x = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem + lane_base + x * 128;
        const uint32_t t_o = tmem + lane_base + 256 + x * 128;
        const int rows = min(128, rows_cta - x * 128);
        const int qi = m0 + (x * 128 + r) / gq;                  // query position of this thread's row
        int klo = 1, khi = 0;
        if (r < rows) window_bounds(qi, sq, sk, wl, wr, klo, khi);
        int lo_l, hi_f, tmp;
        window_bounds(m0 + x * qpt, sq, sk, wl, wr, tmp, hi_f);
        window_bounds(m0 + (x * 128 + rows - 1) / gq, sq, sk, wl, wr, lo_l, tmp);
        float m_used = -INFINITY, l_run = 0.f;
        // BIAS instantiation: the scores are turned into their final log2-domain values in registers (softcap, then
        // alibi, as the general kernel and the golden do), and the softmax below runs with a unit scale
        const float sc = BIAS ? 1.f : a.scale_log2;
        const float cap_out = a.softcap * kLog2e;
        const float slope = (BIAS && a.alibi) ? a.alibi[(int64_t)b * a.alibi_sb + h0 + (x * 128 + r) % gq] * kLog2e : 0.f;
        const float rel = (float)(qi + sk - sq);                 // alibi distance of key j is |rel - j|
        bool ok = true;
        const int nt_x = x == 0 ? nt0 : ntiles;
        for (int j = 0; j < nt_x && ok; ++j) {
            const int n0 = (t_lo + j) * 128;
            ok = mbar_wait(bar(C_SA + x), j & 1, abort_flag, err, 9);
            if (!ok) break;
            tc_fence_after();
            uint32_t sreg[4][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tmem_ld32(t_s + c * 32, sreg[c]);
            tmem_wait_ld();
            // the second half of the row is in flight while the first half is reduced
#pragma unroll
            for (int c = 2; c < 4; ++c) tmem_ld32(t_s + c * 32, sreg[c]);
            const bool full = n0 >= lo_l && n0 + 127 <= hi_f;
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                if (hh == 1) tmem_wait_ld();
                if constexpr (BIAS) {
#pragma unroll
                    for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float xv = __uint_as_float(sreg[c][i]);
                            if (a.softcap > 0.f) {
                                // tanh(y) = 1 - 2 / (1 + e^(2y)): two special-function operations, absolute error ~1e-7
                                const float e2y = ex2_approx(xv * (a.cap_in * 2.f * kLog2e));
                                xv = cap_out * (1.f - __fdividef(2.f, 1.f + e2y));
                            } else {
                                xv *= a.scale_log2;
                            }
                            xv -= slope * fabsf(rel - (float)(n0 + c * 32 + i));
                            sreg[c][i] = __float_as_uint(xv);
                        }
                    }
                }
                if (!full) {
#pragma unroll
                    for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = n0 + c * 32 + i;
                            if (col < klo || col > khi) sreg[c][i] = 0xff800000u;     // -inf
                        }
                    }
                }
                // four independent chains of three-input maxima
#pragma unroll
                for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        mx0 = fmaxf(fmaxf(mx0, __uint_as_float(sreg[c][i])), __uint_as_float(sreg[c][i + 1]));
                        mx1 = fmaxf(fmaxf(mx1, __uint_as_float(sreg[c][i + 2])), __uint_as_float(sreg[c][i + 3]));
                        mx2 = fmaxf(fmaxf(mx2, __uint_as_float(sreg[c][i + 4])), __uint_as_float(sreg[c][i + 5]));
                        mx3 = fmaxf(fmaxf(mx3, __uint_as_float(sreg[c][i + 6])), __uint_as_float(sreg[c][i + 7]));
                    }
                }
            }
            const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc;       // log2 domain
            if (m_used == -INFINITY) m_used = m_new;
            if (j > 0 && __any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
                const float m_next = fmaxf(m_used, m_new);
                const float alpha = m_used == -INFINITY ? 1.f : ex2_approx(m_used - m_next);
                m_used = m_next;
                l_run *= alpha;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t oreg[32];
                    tmem_ld32(t_o + c * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st32(t_o + c * 32, oreg);
                }
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(neg_m, neg_m);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
            // NPOLY of every 8 pairs take the polynomial 2^x, spread evenly between the special-function ones
            auto exp_phase = [&](auto npoly_c) {
                constexpr int NPOLY = decltype(npoly_c)::value;
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    uint32_t preg[32];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint32_t* src = &sreg[2 * hlf + (g >> 1)][(g & 1) * 16];
                        static_for<0, 8>([&](auto pi) {
                            constexpr bool poly = (pi.value * NPOLY) % 8 < NPOLY;
                            const float2 xv = fma2(make_float2(__uint_as_float(src[2 * pi.value]), __uint_as_float(src[2 * pi.value + 1])), sc2, nm2);
                            float2 pv;
                            if constexpr (poly) pv = ex2_poly2(xv);
                            else pv = make_float2(ex2_approx(xv.x), ex2_approx(xv.y));
                            if constexpr (pi.value & 1) sum_b = add2(sum_b, pv); else sum_a = add2(sum_a, pv);
                            preg[g * 8 + pi.value] = Elem<T>::pack(pv.x, pv.y);
                        });
                    }
                    tmem_st32(t_s + hlf * 32, preg);
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar((hlf ? C_PA2 : C_PA) + x));
                }
            };
            // masked tiles keep the special-function path: it maps -inf to an exact zero
            if (full) exp_phase(std::integral_constant<int, FA_FWD_POLY>{});
            else exp_phase(std::integral_constant<int, 0>{});
            const float s0 = sum_a.x + sum_b.x, s1 = sum_a.y + sum_b.y;
            l_run += s0 + s1;
        }
        if (ok) ok = mbar_wait(bar(C_OA + x), 0, abort_flag, err, 10);
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            T* orow = out_row(x * 128 + r);
            float* prow = a.nsplit > 1 ? a.o_part + part_row(x * 128 + r) * a.d : nullptr;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t oreg[32];
                tmem_ld32(t_o + c * 32, oreg);
                tmem_wait_ld();
                if (r < rows && prow) {
#pragma unroll
                    for (int v = 0; v < 8; ++v)
                        if (c * 32 + v * 4 < a.d)
                            reinterpret_cast<float4*>(prow + c * 32)[v] = make_float4(__uint_as_float(oreg[4 * v]) * inv, __uint_as_float(oreg[4 * v + 1]) * inv,
                                                                                     __uint_as_float(oreg[4 * v + 2]) * inv, __uint_as_float(oreg[4 * v + 3]) * inv);
                } else if (r < rows) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 pk;
                        pk.x = Elem<T>::pack(__uint_as_float(oreg[8 * v + 0]) * inv, __uint_as_float(oreg[8 * v + 1]) * inv);
                        pk.y = Elem<T>::pack(__uint_as_float(oreg[8 * v + 2]) * inv, __uint_as_float(oreg[8 * v + 3]) * inv);
                        pk.z = Elem<T>::pack(__uint_as_float(oreg[8 * v + 4]) * inv, __uint_as_float(oreg[8 * v + 5]) * inv);
                        pk.w = Elem<T>::pack(__uint_as_float(oreg[8 * v + 6]) * inv, __uint_as_float(oreg[8 * v + 7]) * inv);
                        if (c * 32 + v * 8 < a.d) reinterpret_cast<uint4*>(orow + c * 32)[v] = pk;
                    }
                }
            }
            if (r < rows && prow) a.lse_part[part_row(x * 128 + r)] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : -INFINITY;
            else if (r < rows && a.lse) *lse_slot(x * 128 + r) = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : INFINITY;
        }
    }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// =================================================================================================
// Head dims 192 and 256: one 128-row query tile per CTA.  The output accumulator alone takes up to 256 tensor-memory
// columns, so instead of a second query tile the CTA keeps TWO score buffers of the same tile (columns 0-127 and
// 128-255): Q K^T of key tile j + 1 is issued before P V of tile j and runs while tile j is in its softmax.  K and V
// have one shared-memory buffer each (Q + K + V = 192 KiB at D = 256): K(j + 1) is requested as soon as the scores of
// tile j are done, V(j + 1) as soon as P V of tile j is done.  One softmax warp group (warps 0-3, thread = row);
// warp 8 TMA producer, warp 9 MMA issue.  Same arithmetic as the two-tile kernel.
// =================================================================================================
template <int D>
struct FwdSm100SmemWide {
    static constexpr int kSub = 128 * 128;
    static constexpr int kTile = (D / 64) * kSub;           // Q, K or V tile
    static constexpr int oQ = 0, oK = kTile, oV = 2 * kTile;
    static constexpr int oBar = 3 * kTile;
    static constexpr int kBytes = oBar + 320;
};
enum { W_Q = 0, W_KF, W_KE, W_VF, W_VE, W_S0, W_S1, W_P0, W_P1, W_P0B, W_P1B, W_O, W_COUNT };

template <typename T, int D, bool BIAS>
__global__ void __launch_bounds__(384, 1) fwd_sm100_kernel_wide(const __grid_constant__ Sm100FwdArgs a) {
    using L = FwdSm100SmemWide<D>;
    constexpr int NSUB = D / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_O = 256;
    constexpr int FMT = Elem<T>::kDtype == FA_BF16 ? 1 : 0;
    constexpr uint32_t IDESC_QK = umma_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_PV = umma_idesc(FMT, 128, D, 0, 1);
    constexpr float kRescaleThreshold = 8.f;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t sQ = sbase + L::oQ, sK = sbase + L::oK, sV = sbase + L::oV;
    const uint32_t bars = sbase + L::oBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::oBar + 8 * W_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + L::oBar + 8 * W_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = blockIdx.z * a.chunk + blockIdx.x;      // grid order as in the two-tile kernel
    if (pair >= a.b * a.nheads_grid) return;
    const int b = pair / a.nheads_grid, h = pair % a.nheads_grid;
    const int mblk = gridDim.y - 1 - blockIdx.y;
    int q_off = 0, k_off = 0, sq = a.sq, sk = a.sk;
    if (a.cu_q) { q_off = a.cu_q[b]; sq = a.cu_q[b + 1] - q_off; k_off = a.cu_k[b]; sk = a.cu_k[b + 1] - k_off; }
    if (a.seqused_k) sk = (int)max(0LL, min((long long)a.seqused_k[b] + a.s_new, (long long)a.sk));
    const int m0 = mblk * 128;
    if (m0 >= sq) return;
    if (g_fwd_sm100_error) return;
    const int hk = h / (a.hq / a.hkv);
    const int wl = a.wl, wr = a.causal ? 0 : a.wr;
    const int rows = min(128, sq - m0);

    int lo_first, hi_first, lo_last, hi_last;
    window_bounds(m0, sq, sk, wl, wr, lo_first, hi_first);
    window_bounds(m0 + rows - 1, sq, sk, wl, wr, lo_last, hi_last);
    int t_lo = lo_first / 128, t_hi = hi_last < 0 ? 0 : hi_last / 128 + 1;
    if (sk <= 0 || lo_first >= sk) { t_lo = 0; t_hi = 0; }
    const int ntiles = max(0, t_hi - t_lo);

    T* obase = reinterpret_cast<T*>(a.o) + (a.cu_q ? 0 : (int64_t)b * a.o_sb) + (int64_t)(q_off + m0) * a.o_ss + (int64_t)h * a.o_sh;
    float* lbase = a.lse ? a.lse + (a.cu_q ? 0 : (int64_t)b * a.lse_sb) + (int64_t)h * a.lse_sh + (int64_t)(q_off + m0) * a.lse_ss : nullptr;

    if (ntiles == 0) {
        if (tid < rows) {
            uint4 z = make_uint4(0, 0, 0, 0);
            T* orow = obase + (int64_t)tid * a.o_ss;
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                if (c * 8 < a.d) reinterpret_cast<uint4*>(orow)[c] = z;
            if (lbase) lbase[(int64_t)tid * a.lse_ss] = INFINITY;
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < W_COUNT; ++i) mbar_init(bar(i), (i >= W_P0 && i <= W_P1B) ? 128u : 1u);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_fwd_sm100_error;
    const int qrow0 = (a.cu_q ? q_off : 0) + m0;
    const int qb = a.cu_q ? 0 : b;

    static_assert(128 * 56 + 256 * 224 <= 384 * 168, "register split exceeds the CTA's allocation");
    if (warp >= 8) {
    reg_dealloc<56>();
    if (warp == 8) {
        if (lane == 0) {
            tma_prefetch_desc(&a.tq); tma_prefetch_desc(&a.tk); tma_prefetch_desc(&a.tv);
            mbar_expect_tx(bar(W_Q), L::kTile);
#pragma unroll
            for (int s = 0; s < NSUB; ++s) tma_load_4d(sQ + s * L::kSub, &a.tq, bar(W_Q), s * 64, h, qrow0, qb);
            const int32_t* btab = a.block_table ? a.block_table + (int64_t)b * a.bt_stride : nullptr;
            const int kbatch = a.cu_q ? 0 : (a.cache_batch_idx ? a.cache_batch_idx[b] : b);
            // where key tile j lives: (row, outermost coordinate), second half of the tile when it is copied in two boxes
            auto place = [&](int j, int& krow, int& kouter, int& krow2, int& kouter2) {
                krow = (a.cu_q ? k_off : 0) + (t_lo + j) * 128; kouter = kbatch; krow2 = 0; kouter2 = 0;
                if (btab) {
                    const int pos = (t_lo + j) * 128;
                    kouter = btab[pos / a.page_size];
                    krow = pos % a.page_size;
                    if (a.kv_box == 64) {
                        const bool in_table = (pos + 64) / a.page_size < a.bt_stride;
                        kouter2 = in_table ? btab[(pos + 64) / a.page_size] : kouter;
                        krow2 = in_table ? (pos + 64) % a.page_size : krow;
                    }
                }
            };
            auto load = [&](const CUtensorMap* map, uint32_t dst, int full_bar, int j) {
                int krow, kouter, krow2, kouter2;
                place(j, krow, kouter, krow2, kouter2);
                mbar_expect_tx(bar(full_bar), L::kTile);
#pragma unroll
                for (int s = 0; s < NSUB; ++s) {
                    tma_load_4d(dst + s * L::kSub, map, bar(full_bar), s * 64, hk, krow, kouter);
                    if (a.kv_box == 64) tma_load_4d(dst + s * L::kSub + 64 * 128, map, bar(full_bar), s * 64, hk, krow2, kouter2);
                }
            };
            // order of the requests: K(0) V(0) K(1) | K(2) V(1) | K(3) V(2) ...: K(j) follows the scores of tile j - 1,
            // V(j - 1) follows P V of tile j - 2
            bool ok = true;
            for (int j = 0; j <= ntiles && ok; ++j) {
                if (j < ntiles) {
                    if (j > 0) ok = mbar_wait(bar(W_KE), (j - 1) & 1, abort_flag, err, 1);
                    if (!ok) break;
                    load(&a.tk, sK, W_KF, j);
                }
                const int jv = j == 0 ? 0 : j - 1;           // V(0) right after K(0); afterwards V lags one tile
                if (j == 0 || j >= 2) {
                    if (jv >= 1) ok = mbar_wait(bar(W_VE), (jv - 1) & 1, abort_flag, err, 2);
                    if (!ok) break;
                    if (jv < ntiles) load(&a.tv, sV, W_VF, jv);
                }
            }
        }
    } else if (warp == 9) {
        const uint64_t dQ = umma_desc(sQ, 16, 1024), dK = umma_desc(sK, 16, 1024), dV = umma_desc(sV, L::kSub, 1024);
        auto issue_qk = [&](int j) {
            const uint32_t d_s = tmem + (j & 1) * 128;
            static_for<0, NSUB>([&](auto sub) {
                constexpr uint32_t o = sub.value * (L::kSub >> 4);
                umma_ss_group4<o, o + 2, o + 4, o + 6, o, o + 2, o + 4, o + 6>(d_s, dQ, dK, IDESC_QK, sub.value > 0);
            });
            umma_commit_w(bar(W_S0 + (j & 1)));
            umma_commit_w(bar(W_KE));
        };
        bool ok = mbar_wait(bar(W_Q), 0, abort_flag, err, 3);
        if (ok) ok = mbar_wait(bar(W_KF), 0, abort_flag, err, 4);
        if (ok) { tc_fence_after(); issue_qk(0); }
        for (int j = 0; j < ntiles && ok; ++j) {
            if (j + 1 < ntiles) {
                ok = mbar_wait(bar(W_KF), (j + 1) & 1, abort_flag, err, 7);
                if (!ok) break;
                tc_fence_after();
                issue_qk(j + 1);
            }
            ok = mbar_wait(bar(W_VF), j & 1, abort_flag, err, 6);
            if (!ok) break;
            if (a.seqused_k && (t_lo + j) * 128 + 128 > sk) {
                // stale cache rows past the sequence may hold NaN patterns: 0 x NaN is NaN, so the V rows are cleared
                const int first = max(0, sk - (t_lo + j) * 128);
                const int last = a.block_table ? 128 : min(128, a.sk - (t_lo + j) * 128);     // rows the copy fetched
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
                    for (int idx = first * 8 + lane; idx < last * 8; idx += 32)
                        *reinterpret_cast<uint4*>(sgen + L::oV + sub * L::kSub + idx * 16) = make_uint4(0, 0, 0, 0);
                fence_proxy_async_smem();
                __syncwarp();
            }
            const int buf = j & 1;
            ok = mbar_wait(bar(W_P0 + buf), (j >> 1) & 1, abort_flag, err, 5);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_o = tmem + COL_O, a_p = tmem + buf * 128;
            umma_ts_group4<0, 8, 0, 128>(d_o, a_p, dV, IDESC_PV, j > 0);
            ok = mbar_wait(bar(W_P0B + buf), (j >> 1) & 1, abort_flag, err, 11);
            if (!ok) break;
            tc_fence_after();
            umma_ts_group4<32, 8, 512, 128>(d_o, a_p, dV, IDESC_PV, 1);
            umma_commit_w(bar(W_VE));
            if (j + 1 == ntiles) umma_commit_w(bar(W_O));
        }
    }
    } else {
    reg_alloc<224>();
    if (warp < 4) {
        const int r = tid & 127;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t t_o = tmem + lane_base + COL_O;
        const int qi = m0 + r;
        int klo = 1, khi = 0;
        if (r < rows) window_bounds(qi, sq, sk, wl, wr, klo, khi);
        int lo_l, hi_f, tmp;
        window_bounds(m0, sq, sk, wl, wr, tmp, hi_f);
        window_bounds(m0 + rows - 1, sq, sk, wl, wr, lo_l, tmp);
        float m_used = -INFINITY, l_run = 0.f;
        const float sc = BIAS ? 1.f : a.scale_log2;
        const float cap_out = a.softcap * kLog2e;
        const float slope = (BIAS && a.alibi) ? a.alibi[(int64_t)b * a.alibi_sb + h] * kLog2e : 0.f;
        const float rel = (float)(qi + sk - sq);
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int n0 = (t_lo + j) * 128, buf = j & 1;
            const uint32_t t_s = tmem + lane_base + buf * 128;
            ok = mbar_wait(bar(W_S0 + buf), (j >> 1) & 1, abort_flag, err, 9);
            if (!ok) break;
            tc_fence_after();
            uint32_t sreg[4][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tmem_ld32(t_s + c * 32, sreg[c]);
            tmem_wait_ld();
#pragma unroll
            for (int c = 2; c < 4; ++c) tmem_ld32(t_s + c * 32, sreg[c]);
            const bool full = n0 >= lo_l && n0 + 127 <= hi_f;
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                if (hh == 1) tmem_wait_ld();
                if constexpr (BIAS) {
#pragma unroll
                    for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float xv = __uint_as_float(sreg[c][i]);
                            if (a.softcap > 0.f) {
                                const float e2y = ex2_approx(xv * (a.cap_in * 2.f * kLog2e));
                                xv = cap_out * (1.f - __fdividef(2.f, 1.f + e2y));
                            } else {
                                xv *= a.scale_log2;
                            }
                            xv -= slope * fabsf(rel - (float)(n0 + c * 32 + i));
                            sreg[c][i] = __float_as_uint(xv);
                        }
                    }
                }
                if (!full) {
#pragma unroll
                    for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = n0 + c * 32 + i;
                            if (col < klo || col > khi) sreg[c][i] = 0xff800000u;     // -inf
                        }
                    }
                }
#pragma unroll
                for (int c = 2 * hh; c < 2 * hh + 2; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        mx0 = fmaxf(fmaxf(mx0, __uint_as_float(sreg[c][i])), __uint_as_float(sreg[c][i + 1]));
                        mx1 = fmaxf(fmaxf(mx1, __uint_as_float(sreg[c][i + 2])), __uint_as_float(sreg[c][i + 3]));
                        mx2 = fmaxf(fmaxf(mx2, __uint_as_float(sreg[c][i + 4])), __uint_as_float(sreg[c][i + 5]));
                        mx3 = fmaxf(fmaxf(mx3, __uint_as_float(sreg[c][i + 6])), __uint_as_float(sreg[c][i + 7]));
                    }
                }
            }
            const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc;       // log2 domain
            if (m_used == -INFINITY) m_used = m_new;
            if (j > 0 && __any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
                // P V of tile j - 1 was issued AFTER the scores of this tile: wait for it before touching O
                ok = mbar_wait(bar(W_VE), (j - 1) & 1, abort_flag, err, 12);
                if (!ok) break;
                tc_fence_after();
                const float m_next = fmaxf(m_used, m_new);
                const float alpha = m_used == -INFINITY ? 1.f : ex2_approx(m_used - m_next);
                m_used = m_next;
                l_run *= alpha;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t oreg[32];
                    tmem_ld32(t_o + c * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st32(t_o + c * 32, oreg);
                }
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(neg_m, neg_m);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
            auto exp_phase = [&](auto npoly_c) {
                constexpr int NPOLY = decltype(npoly_c)::value;
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    uint32_t preg[32];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint32_t* src = &sreg[2 * hlf + (g >> 1)][(g & 1) * 16];
                        static_for<0, 8>([&](auto pi) {
                            constexpr bool poly = (pi.value * NPOLY) % 8 < NPOLY;
                            const float2 xv = fma2(make_float2(__uint_as_float(src[2 * pi.value]), __uint_as_float(src[2 * pi.value + 1])), sc2, nm2);
                            float2 pv;
                            if constexpr (poly) pv = ex2_poly2(xv);
                            else pv = make_float2(ex2_approx(xv.x), ex2_approx(xv.y));
                            if constexpr (pi.value & 1) sum_b = add2(sum_b, pv); else sum_a = add2(sum_a, pv);
                            preg[g * 8 + pi.value] = Elem<T>::pack(pv.x, pv.y);
                        });
                    }
                    tmem_st32(t_s + hlf * 32, preg);
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar((hlf ? W_P0B : W_P0) + buf));
                }
            };
            if (full) exp_phase(std::integral_constant<int, FA_FWD_POLY>{});
            else exp_phase(std::integral_constant<int, 0>{});
            l_run += (sum_a.x + sum_b.x) + (sum_a.y + sum_b.y);
        }
        if (ok) ok = mbar_wait(bar(W_O), 0, abort_flag, err, 10);
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            T* orow = obase + (int64_t)r * a.o_ss;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t oreg[32];
                tmem_ld32(t_o + c * 32, oreg);
                tmem_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 pk;
                        pk.x = Elem<T>::pack(__uint_as_float(oreg[8 * v + 0]) * inv, __uint_as_float(oreg[8 * v + 1]) * inv);
                        pk.y = Elem<T>::pack(__uint_as_float(oreg[8 * v + 2]) * inv, __uint_as_float(oreg[8 * v + 3]) * inv);
                        pk.z = Elem<T>::pack(__uint_as_float(oreg[8 * v + 4]) * inv, __uint_as_float(oreg[8 * v + 5]) * inv);
                        pk.w = Elem<T>::pack(__uint_as_float(oreg[8 * v + 6]) * inv, __uint_as_float(oreg[8 * v + 7]) * inv);
                        if (c * 32 + v * 8 < a.d) reinterpret_cast<uint4*>(orow + c * 32)[v] = pk;
                    }
                }
            }
            if (r < rows && lbase) lbase[(int64_t)r * a.lse_ss] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : INFINITY;
        }
    }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

bool tensor_map_encoder_available() { return encode_fn() != nullptr; }

// (dim, head, row, batch) view with a [64 x 1 x 128 x 1] box and 128-byte swizzle
int make_tile_map(CUtensorMap* map, int dtype, const void* ptr, int d, int heads, int64_t rows, int batch,
                  int64_t stride_h, int64_t stride_s, int64_t stride_b, int box_rows, int box_heads) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    // The encoder is a driver call and wants a current context.  A thread that has made no runtime call yet (an
    // autograd worker whose allocations all came from the framework's cache) has none: bind the device's primary
    // context once per thread.
    static thread_local bool context_bound = false;
    if (!context_bound) {
        cudaFree(nullptr);
        context_bound = true;
    }
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_s * 2, (cuuint64_t)stride_b * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, dtype == FA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                    const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {            // the thread's device was switched since: bind again, once
        cudaFree(nullptr);
        r = fn(map, dtype == FA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
               const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return FA_OK;
}

bool fwd_sm100_supported(const fa_fwd_params& p) {
    if (p.d != p.dv || p.d % 8 != 0 || p.d <= 0 || p.d > 256) return false;      // any head dim: the kernels pad it to 64 / 128 / 192 / 256
    if ((p.sq + 127) / 128 > 8192) return false;                                 // query blocks x splits stay inside a grid dimension
    const bool cache = p.block_table || p.seqused_k || p.cache_batch_idx;
    if (cache) {
        // KV-cache calls (prefill against a cache): lengths and pages are read on the device
        if (p.cu_seqlens_q || p.cu_seqlens_k || !p.seqused_k) return false;
        if (p.block_table && (p.page_size <= 0 || p.page_size % 64)) return false;
        // The tile maps of a cache must end with the cache (a copy touches the addresses of clipped box elements that lie
        // inside the declared tensor): without the number of pages / cache entries the call stays on kernels with plain,
        // guarded loads.
        if (p.kv_entries <= 0) return false;
        // Cache calls take this kernel at its own head dims only (64, 128, 192, 256); padded head dims stay on the
        // split-KV decode and general kernels.  (A box that reaches past a row's columns touches the following row, which
        // for the last row of a cache is only harmless when the tile map ends with the cache: see kv_entries above.  The
        // restriction was put in before that was understood and has not been measured without it since.)
        if (p.d != 64 && p.d != 128 && p.d != 192 && p.d != 256) return false;
        // Short queries (fewer than 64 a head).  Up to 16 stacked rows a KV head belong to the split-KV decode kernel.
        // Above that the two-tile kernel takes the call with the query group stacked into the tile rows and the keys
        // split over CTAs (partials + combine): a CTA streams its share of a KV head's cache once for all the rows.
        // A group that cannot be stacked (not a power of two) would read the cache once per head: such calls stay
        // with the decode kernel up to 64 stacked rows and come here above that, where the alternative is mma.sync.
        if (p.sq < 64) {
            const int G = p.hq / p.hkv;
            if (p.sq * G <= 16) return false;
            const bool stack = p.d <= 128 && G > 1 && G <= 128 && (G & (G - 1)) == 0;
            if (!stack && (p.sq * G <= 64 || p.d > 128)) return false;
        }
    }
    if ((p.cu_seqlens_q != nullptr) != (p.cu_seqlens_k != nullptr)) return false;
    if (p.kv_begin != 0 || p.kv_end > 0 || p.partials_only) return false;
    if (p.sq <= 0 || p.sk <= 0 || !(p.scale > 0.f)) return false;
    if (p.cu_seqlens_q && (p.total_q <= 0 || p.total_k <= 0)) return false;
    const fa_tensor* ts[3] = {&p.q, &p.k, &p.v};
    for (const fa_tensor* t : ts) {
        if (t->stride_h <= 0 || t->stride_s <= 0) return false;
        if (!p.cu_seqlens_q && p.b > 1 && t->stride_b <= 0) return false;
    }
    return encode_fn() != nullptr;
}

// (batch entry, head) pairs of one chunk of the grid: the largest power of two whose streamed operands (bytes_per_pair
// each) stay within 16 MiB, the whole launch if it is smaller than that
int grid_chunk(int64_t pairs, int64_t bytes_per_pair) {
    int64_t c = 1;
    const int64_t cap = 16ll << 20;          // measured 4-192 MiB at configuration 2 and at an eighth of it: flat up to 48, worse above
    while (c * 2 <= pairs && c * 2 * bytes_per_pair <= cap && c * 2 <= 1024) c *= 2;
    if (pairs * bytes_per_pair <= cap && pairs <= 1024) c = pairs;
    return (int)(c < 1 ? 1 : c);
}

template <typename T, int D, bool BIAS>
static int launch_sm100_b(const fa_fwd_params& p, Sm100FwdArgs& a) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    auto kern = fwd_sm100_kernel2<T, D, BIAS>;
    const int smem = FwdSm100Smem2<D>::kBytes + 1024;
    if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute")) return e;
    const int qpc = 256 / a.gq;                              // query positions of a CTA
    const unsigned nbx = (unsigned)(((p.sq + qpc - 1) / qpc) * a.nsplit);
    a.nheads_grid = a.gq > 1 ? p.hkv : p.hq;
    a.chunk = grid_chunk((int64_t)p.b * a.nheads_grid, (int64_t)p.sk * p.d * 4);
    dim3 grid(a.chunk, nbx, (unsigned)(((int64_t)p.b * a.nheads_grid + a.chunk - 1) / a.chunk));
    kern<<<grid, 384, smem, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "fwd_sm100 launch");
}
template <typename T, int D>
static int launch_sm100_t(const fa_fwd_params& p, Sm100FwdArgs& a) {
    return (p.softcap > 0.f || p.alibi_slopes) ? launch_sm100_b<T, D, true>(p, a) : launch_sm100_b<T, D, false>(p, a);
}
template <typename T, int D, bool BIAS>
static int launch_sm100_wide_b(const fa_fwd_params& p, Sm100FwdArgs& a) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    auto kern = fwd_sm100_kernel_wide<T, D, BIAS>;
    const int smem = FwdSm100SmemWide<D>::kBytes + 1024;
    if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute")) return e;
    a.nheads_grid = p.hq;
    a.chunk = grid_chunk((int64_t)p.b * p.hq, (int64_t)p.sk * p.d * 4);
    dim3 grid(a.chunk, (p.sq + 127) / 128, (unsigned)(((int64_t)p.b * p.hq + a.chunk - 1) / a.chunk));
    kern<<<grid, 384, smem, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "fwd_sm100 launch");
}
template <typename T, int D>
static int launch_sm100_wide_t(const fa_fwd_params& p, Sm100FwdArgs& a) {
    return (p.softcap > 0.f || p.alibi_slopes) ? launch_sm100_wide_b<T, D, true>(p, a) : launch_sm100_wide_b<T, D, false>(p, a);
}

// query group stacked into the tile rows of the two-tile kernel (dense q shorter than 128, power-of-two group)
static int sm100_stack_factor(const fa_fwd_params& p) {
    const int G = p.hq / p.hkv;
    return (!p.cu_seqlens_q && p.d <= 128 && p.sq < 128 && G > 1 && G <= 128 && (G & (G - 1)) == 0) ? G : 1;
}
// CTAs of one split of a dense / cache call
long fwd_sm100_ctas(const fa_fwd_params& p) {
    const int gq = sm100_stack_factor(p);
    const int rows_cta = p.d > 128 ? 128 : 256;
    return (long)(p.b > 0 ? p.b : 1) * (gq > 1 ? p.hkv : p.hq) * (((long)p.sq * gq + rows_cta - 1) / rows_cta);
}

int launch_fwd_sm100(const fa_fwd_params& p, int nsplit, int keys_per_split, float* o_part, float* lse_part) {
    Sm100FwdArgs a;
    a.kv_box = 128;
    a.nsplit = nsplit > 1 ? nsplit : 1; a.keys_per_split = keys_per_split; a.o_part = o_part; a.lse_part = lse_part;
    a.rows_all = (int64_t)p.b * p.sq * p.hq;
    const bool packed = p.cu_seqlens_q != nullptr;
    const int64_t q_rows = packed ? p.total_q : p.sq;
    const int64_t k_rows = packed ? p.total_k : p.sk;
    const int nb = packed ? 1 : p.b;
    auto bstride = [&](const fa_tensor& t, int64_t rows) { return packed || p.b == 1 ? rows * t.stride_s : t.stride_b; };
    // Short dense queries under a query group: the group's heads are stacked into the tile rows (two-tile kernel)
    a.gq = sm100_stack_factor(p);
    if (int e = make_tile_map(&a.tq, p.dtype, p.q.ptr, p.d, p.hq, q_rows, nb, p.q.stride_h, p.q.stride_s, bstride(p.q, q_rows), 128 / a.gq, a.gq)) return e;
    const bool cache = p.block_table || p.seqused_k || p.cache_batch_idx;
    if (cache) {
        // rows of one page / cache entry; the outermost extent is the number of pages or cache entries (the page table
        // and cache_batch_idx are valid by contract)
        const int64_t rows = p.block_table ? p.page_size : p.sk;
        const int outer = (int)(p.kv_entries < (1 << 24) ? p.kv_entries : 1 << 24);      // > 0: checked by the support predicate
        if (p.block_table && p.page_size % 128) a.kv_box = 64;
        if (int e = make_tile_map(&a.tk, p.dtype, p.k.ptr, p.d, p.hkv, rows, outer, p.k.stride_h, p.k.stride_s, p.k.stride_b, a.kv_box)) return e;
        if (int e = make_tile_map(&a.tv, p.dtype, p.v.ptr, p.d, p.hkv, rows, outer, p.v.stride_h, p.v.stride_s, p.v.stride_b, a.kv_box)) return e;
    } else {
        if (int e = make_tile_map(&a.tk, p.dtype, p.k.ptr, p.d, p.hkv, k_rows, nb, p.k.stride_h, p.k.stride_s, bstride(p.k, k_rows), 128)) return e;
        if (int e = make_tile_map(&a.tv, p.dtype, p.v.ptr, p.d, p.hkv, k_rows, nb, p.v.stride_h, p.v.stride_s, bstride(p.v, k_rows), 128)) return e;
    }
    a.seqused_k = p.seqused_k; a.block_table = p.block_table; a.cache_batch_idx = p.cache_batch_idx;
    a.bt_stride = p.block_table_stride; a.page_size = p.page_size; a.s_new = p.s_new;
    a.o = p.o.ptr; a.lse = p.lse;
    a.o_sb = p.o.stride_b; a.o_ss = p.o.stride_s; a.o_sh = p.o.stride_h;
    a.lse_sb = p.lse_stride_b; a.lse_sh = p.lse_stride_h; a.lse_ss = p.lse_stride_s;
    a.cu_q = p.cu_seqlens_q; a.cu_k = p.cu_seqlens_k;
    a.b = p.b; a.sq = p.sq; a.sk = p.sk; a.hq = p.hq; a.hkv = p.hkv;
    a.scale_log2 = p.scale * kLog2e;
    a.softcap = p.softcap; a.cap_in = p.softcap > 0.f ? p.scale / p.softcap : 0.f;
    a.alibi = p.alibi_slopes; a.alibi_sb = p.alibi_stride_b;
    a.causal = p.causal; a.wl = p.window_left; a.wr = p.window_right;
    a.d = p.d;
    if (p.d > 128) {
        note_kernel("sm100_tcgen05_wide");
        if (p.dtype == FA_F16) return p.d <= 192 ? launch_sm100_wide_t<__half, 192>(p, a) : launch_sm100_wide_t<__half, 256>(p, a);
        return p.d <= 192 ? launch_sm100_wide_t<__nv_bfloat16, 192>(p, a) : launch_sm100_wide_t<__nv_bfloat16, 256>(p, a);
    }
    note_kernel("sm100_tcgen05_2q");
    if (p.dtype == FA_F16) return p.d <= 64 ? launch_sm100_t<__half, 64>(p, a) : launch_sm100_t<__half, 128>(p, a);
    return p.d <= 64 ? launch_sm100_t<__nv_bfloat16, 64>(p, a) : launch_sm100_t<__nv_bfloat16, 128>(p, a);
}

int sm100_error_flag(bool clear) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_fwd_sm100_error, sizeof(int));
    if (clear) { int z = 0; cudaMemcpyToSymbol(g_fwd_sm100_error, &z, sizeof(int)); }
    const int w = bwd_sm100_error_flag(clear);
    const int m = mla_pair_error_flag(clear);
    return v ? v : (w ? w : m);
}

}  // namespace fa
