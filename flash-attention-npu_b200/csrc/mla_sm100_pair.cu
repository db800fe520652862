// int8 latent (MLA) paged decode on the tcgen05 tensor cores, one CTA PAIR (thread-block cluster of 2) per
// (KV split, sequence, tile of 128 heads).  No counterpart in the reference.
//
// The 576 score dimensions are split over the pair: CTA 0 holds latent dims [0,256) and the 64 rope dims, CTA 1
// latent dims [256,512).  Each CTA keeps its latent part of Q in tensor memory (128 columns: the A operand of the
// score MMAs, so that only K is read from shared memory), stages its part of every dequantised 64-token tile (40 KB,
// three buffers), computes PARTIAL scores S_r = Q_r K_r^T in tensor memory, and the softmax warps exchange
// the partials through distributed shared memory: each warp bulk-copies its 32 x 64 fp32 partial into the peer
// warp's receive buffer, both add own + peer (the same fp32 sum in both CTAs) and run the same online softmax.  P V then uses the
// CTA's own 256 latent columns as V, so each CTA owns one half of the output and nothing is computed twice.
//
//   warps 0-3   softmax + exchange: thread = head row; epilogue
//   warps 4-11  producers: int8 rows -> registers -> * scale -> bf16 -> swizzled shared memory (UMMA layout)
//   warp 12     issues the MMAs, owns the tensor memory (warps 13-15 only complete the last warp group)
// Tensor memory: O half (256 columns) + two 64-column score buffers + Q (128 columns).
#include "fa_utils.cuh"
#include "fa_internal.h"
#include "sm100_ptx.cuh"
#include "mla_dequant.cuh"

namespace fa {

using namespace sm100;

__device__ int g_mla_pair_error = 0;

int mla_pair_error_flag(bool clear) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_mla_pair_error, sizeof(int));
    if (clear) { int z = 0; cudaMemcpyToSymbol(g_mla_pair_error, &z, sizeof(int)); }
    return v;
}

namespace {

constexpr int kLat = 512, kRope = 64;
constexpr int kTile = 64;                       // tokens per tile
constexpr int kQSub = 128 * 128;                // bytes of one [128 heads x 64 dims] Q sub-tile
constexpr int kKSub = kTile * 128;              // bytes of one [64 tokens x 64 dims] K sub-tile
constexpr int kSubs = 5;                        // 4 latent sub-tiles + rope (CTA 0 only)
constexpr int kKBuf = kSubs * kKSub;            // one tile buffer
constexpr int kXchg = 32 * kTile * 4;            // partial scores of one softmax warp (32 rows x 64 tokens, fp32)
constexpr int kKBufs = 3;                        // tile buffers in flight
constexpr int kOffK = kQSub, kOffRecv = kOffK + kKBufs * kKBuf, kOffBar = kOffRecv + 4 * 2 * kXchg;      // per softmax warp: a send buffer and a receive buffer
constexpr int kSmemBytes = kOffBar + 256 + 1024;
constexpr int kThreads = 16 * 32;
static_assert(kSmemBytes <= 232448, "shared memory limit of a CTA");
// KF/KE: tile buffer full / free; QT: the latent part of Q is in tensor memory; S: partial scores complete; P: probabilities written; RF (one per softmax warp):
// the peer warp's partial has landed in my receive buffer; RC: the peer warp has read what I copied into its receive
// buffer; O: all MMAs done
enum { P_KF0 = 0, P_KF1, P_KF2, P_KE0, P_KE1, P_KE2, P_QT, P_S0, P_S1, P_P0, P_P1, P_RF0, P_RF1, P_RF2, P_RF3, P_RC0, P_RC1, P_RC2, P_RC3,
       P_O, P_COUNT };

struct MlaPairArgs {
    fa_mla_params p;
    int nsplit, tokens_per_split;
    float* o_part;
    float* lse_part;
    int final_direct;
    float scale_log2;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) mla_pair_kernel(const __grid_constant__ MlaPairArgs a) {
    using T = __nv_bfloat16;
    const fa_mla_params& p = a.p;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t IDESC_QK = umma_idesc(1, 128, kTile, 0, 0);
    constexpr uint32_t IDESC_PV = umma_idesc(1, 128, 256, 0, 1);
    constexpr float kRescaleThreshold = 8.f;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t sQ = sbase, sK = sbase + kOffK, bars = sbase + kOffBar;      // sQ: the rope part of Q only
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + kOffBar + 8 * P_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + kOffBar + 8 * P_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = (int)cluster_ctarank(), peer = rank ^ 1;             // rank = half of the dims and of the output
    const int split = blockIdx.y;
    const int head_tiles = (p.hq + 127) / 128;
    const int b = blockIdx.z / head_tiles, head0 = (blockIdx.z % head_tiles) * 128;
    // an oversized length is truncated to what the page-table row can address
    const int sk = (int)max(0LL, min((long long)p.cache_seqlens[b], (long long)p.block_table_stride * p.page_size));
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    const int t_begin = rb + split * a.tokens_per_split;
    const int t_end = min(re, t_begin + a.tokens_per_split);
    const int ntiles = t_end > t_begin ? (t_end - t_begin + kTile - 1) / kTile : 0;
    const int64_t rows_all = (int64_t)p.b * p.hq;

    if (ntiles == 0) {                           // nothing cached in this split's range: both CTAs of the pair leave
        const int h = head0 + tid;
        if (tid < 128 && h < p.hq) {
            const int64_t row = (int64_t)b * p.hq + h;
            if (a.final_direct) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + rank * 256);
                for (int i = 0; i < 32; ++i) dst[i] = make_uint4(0, 0, 0, 0);
                if (rank == 0 && p.lse) p.lse[row] = INFINITY;
            } else {
                if (a.nsplit == 1) {
                    float4* dst = reinterpret_cast<float4*>(a.o_part + row * kLat + rank * 256);
                    for (int i = 0; i < 64; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (rank == 0) a.lse_part[(int64_t)split * rows_all + row] = -INFINITY;
            }
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < kKBufs; ++i) { mbar_init(bar(P_KF0 + i), 8); mbar_init(bar(P_KE0 + i), 1); }
        mbar_init(bar(P_QT), 128);
        mbar_init(bar(P_S0), 1); mbar_init(bar(P_S1), 1);
        mbar_init(bar(P_P0), 128); mbar_init(bar(P_P1), 128);
        for (int w = 0; w < 4; ++w) { mbar_init(bar(P_RF0 + w), 1); mbar_init(bar(P_RC0 + w), 1); }
        mbar_init(bar(P_O), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 12) {
        tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    // ---- Q: the rope part (rank 0) goes to shared memory as one K-major [128 x 64] sub-tile with 128-byte swizzle;
    // the latent part goes to tensor memory (below, by the softmax warps)
    if (rank == 0) {
        const T* qr = reinterpret_cast<const T*>(p.q_rope) + (int64_t)b * p.q_rope_stride_b;
        for (int idx = tid; idx < 128 * 8; idx += kThreads) {
            const int r = idx >> 3, ch = idx & 7;
            const int h = head0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (h < p.hq) v = __ldg(reinterpret_cast<const uint4*>(qr + (int64_t)h * p.q_rope_stride_h + ch * 8));
            *reinterpret_cast<uint4*>(sgen + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_sync_all();                           // the peer's barriers exist before anyone arrives on them
    const uint32_t tmem = *tmem_slot;
    int* err = &g_mla_pair_error;
    const bool dead = g_mla_pair_error != 0;      // an earlier launch timed out: skip the work, keep the cluster protocol

    // Register file split by warp group (the CTA starts with 128 a thread).
    static_assert(128 * 96 + 256 * 96 + 128 * 224 <= 512 * 128, "register split exceeds the CTA's allocation");
    if (warp >= 12) {
        reg_dealloc<96>();
        if (warp == 12 && !dead) {
            // -------------------------------------------------------------- MMA issue (whole warp, one elected lane)
            // latent part of the scores: A = Q from tensor memory (columns 384..511, two elements a column), B = the tile
            // buffer; rope part (rank 0): both operands from shared memory
            const uint64_t dQr = umma_desc(sQ, 16, 1024);
            bool ok = mbar_wait(bar(P_QT), 0, abort_flag, err, 30);
            auto qk = [&](int j) -> bool {
                const int s = j & 1, kb = j % kKBufs;
                if (!mbar_wait(bar(P_KF0 + kb), (j / kKBufs) & 1, abort_flag, err, 31)) return false;
                tc_fence_after();
                const uint32_t d_s = tmem + 256 + s * 64;
                const uint64_t dK = umma_desc(sK + kb * kKBuf, 16, 1024);
                // 16 dims = 8 columns of Q and 32 bytes of the tile a step; the four 64-dim sub-tiles lie kKSub apart
                constexpr uint32_t KS = kKSub >> 4;
                umma_ts_group4<0, 8, 0, 2>(d_s, tmem + 384, dK, IDESC_QK, 0);
                umma_ts_group4<32, 8, KS, 2>(d_s, tmem + 384, dK, IDESC_QK, 1);
                umma_ts_group4<64, 8, 2 * KS, 2>(d_s, tmem + 384, dK, IDESC_QK, 1);
                umma_ts_group4<96, 8, 3 * KS, 2>(d_s, tmem + 384, dK, IDESC_QK, 1);
                if (rank == 0) umma_ss_group4<0, 2, 4, 6, 0, 2, 4, 6>(d_s, dQr, umma_desc_at(dK, 4 * kKSub), IDESC_QK, 1);
                umma_commit_w(bar(P_S0 + s));
                return true;
            };
            auto pv = [&](int j) -> bool {
                const int s = j & 1, kb = j % kKBufs;
                if (!mbar_wait(bar(P_P0 + s), (j >> 1) & 1, abort_flag, err, 32)) return false;
                tc_fence_after();
                const uint32_t a_p = tmem + 256 + s * 64;
                const uint64_t dV = umma_desc(sK + kb * kKBuf, kKSub, 1024);  // MN-major: four 64-column groups kKSub apart
                umma_ts_group4<0, 8, 0, 128>(tmem, a_p, dV, IDESC_PV, j > 0);
                umma_commit_w(bar(P_KE0 + kb));
                return true;
            };
            if (ok) ok = qk(0);
            for (int j = 1; j < ntiles && ok; ++j) {
                ok = qk(j);                       // the scores of tile j run while the softmax of tile j - 1 is busy
                if (ok) ok = pv(j - 1);
            }
            if (ok) ok = pv(ntiles - 1);
            if (ok) umma_commit_w(bar(P_O));
        }
    } else if (warp >= 4) {
        reg_dealloc<96>();
        if (!dead) {
        // ------------------------------------------------------------------ producers: dequantise into shared memory
        const int pw = warp - 4;
        const int cl = lane & 15;                                         // 16-byte chunk of this CTA's 256 latent values
        const int krow = pw * 2 + (lane >> 4);                            // + 16 * pass = token row of the tile
        const int sub_l = cl >> 2, cp = cl & 3;
        const int32_t* btab = p.block_table + (int64_t)b * p.block_table_stride;
        const int rrow = (tid - 128) >> 2, rch = (tid - 128) & 3;         // rope: 64 rows x 8 chunks, two per thread
        // two tiles of operands live in registers: a tile's loads are issued two iterations before they are stored, so
        // that HBM latency (longer than one tile's work) stays off the critical path
        uint4 regN[2][4], regR[2][2];
        float sc[2][4];
        auto tile_row = [&](int j) -> int64_t {                           // first cache row of tile j (inside one page)
            const int t0 = t_begin + j * kTile;
            const int jj = t0 < t_end ? t0 : t_begin;
            return (int64_t)__ldg(btab + jj / p.page_size) * p.page_size + jj % p.page_size;
        };
        auto load_tile = [&](auto par, int j, int64_t slot0) {
            constexpr int P = decltype(par)::value;
            const int t0 = t_begin + j * kTile;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = r * 16 + krow;
                const bool live = t0 + row < t_end;
                regN[P][r] = make_uint4(0, 0, 0, 0);                   // rows past the end become zero keys and values
                if (live) regN[P][r] = __ldg(reinterpret_cast<const uint4*>(p.latent + (slot0 + row) * kLat + rank * 256 + cl * 16));
                sc[P][r] = live ? __ldg(p.scales + slot0 + row) : 0.f;
            }
            if (rank == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    regR[P][i] = make_uint4(0, 0, 0, 0);
                    if (t0 + rrow < t_end)
                        regR[P][i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.rope) + (slot0 + rrow) * kRope + (rch * 2 + i) * 8));
                }
            }
        };
        int64_t row_next = tile_row(2);                                    // page-table entries are fetched one tile earlier still
        bool ok = true;
        auto body = [&](auto par, int j) {
            constexpr int P = decltype(par)::value;                        // = j & 1: register set
            const int kb = j % kKBufs;                                     // tile buffer
            if (j >= kKBufs) ok = mbar_wait_relaxed(bar(P_KE0 + kb), (j / kKBufs - 1) & 1, abort_flag, err, 33);
            if (!ok) return;
            unsigned char* kbuf = sgen + kOffK + kb * kKBuf;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = r * 16 + krow;
                uint4 lo, hi;
                dequant16(regN[P][r], sc[P][r], lo, hi);
                unsigned char* base = kbuf + sub_l * kKSub + row * 128;
                const int c0 = (2 * cp) ^ (row & 7), c1 = (2 * cp + 1) ^ (row & 7);
                // the two sub-tiles a quarter warp touches store their even / odd chunks in opposite order
                if (sub_l & 1) {
                    *reinterpret_cast<uint4*>(base + (c1 << 4)) = hi;
                    *reinterpret_cast<uint4*>(base + (c0 << 4)) = lo;
                } else {
                    *reinterpret_cast<uint4*>(base + (c0 << 4)) = lo;
                    *reinterpret_cast<uint4*>(base + (c1 << 4)) = hi;
                }
            }
            if (rank == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int ch = rch * 2 + i;
                    *reinterpret_cast<uint4*>(kbuf + 4 * kKSub + rrow * 128 + ((ch ^ (rrow & 7)) << 4)) = regR[P][i];
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_KF0 + kb));
            if (j + 2 < ntiles) {
                const int64_t slot0 = row_next;
                row_next = tile_row(j + 3);
                load_tile(par, j + 2, slot0);
            }
        };
        load_tile(std::integral_constant<int, 0>{}, 0, tile_row(0));
        if (ntiles > 1) load_tile(std::integral_constant<int, 1>{}, 1, tile_row(1));
        for (int j = 0; j < ntiles && ok; j += 2) {
            body(std::integral_constant<int, 0>{}, j);
            if (ok && j + 1 < ntiles) body(std::integral_constant<int, 1>{}, j + 1);
        }
        }
    } else {
        reg_alloc<224>();
        if (!dead) {
        // ------------------------------------------------------------------ softmax + exchange: thread = head row
        const int r = tid;                                                 // 0..127
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t t_o = tmem + lane_base;
        float m_used = -INFINITY, l_run = 0.f;
        const float scl = a.scale_log2;
        bool ok = true;
        {   // this head's 256 latent query values -> tensor-memory columns 384..511 (the raw pairs of bf16 values)
            const int h = head0 + r;
            const T* qn = reinterpret_cast<const T*>(p.q_nope) + (int64_t)b * p.q_nope_stride_b + (int64_t)h * p.q_nope_stride_h + rank * 256;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t w[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (h < p.hq) v = __ldg(reinterpret_cast<const uint4*>(qn + c * 64 + i * 8));
                    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
                }
                tmem_st32(tmem + lane_base + 384 + c * 32, w);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(P_QT));
        }
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            const uint32_t t_s = tmem + lane_base + 256 + s * 64;
            ok = mbar_wait(bar(P_S0 + s), (j >> 1) & 1, abort_flag, err, 34);
            if (!ok) break;
            tc_fence_after();
            uint32_t sreg[2][32];
            tmem_ld32(t_s, sreg[0]);
            tmem_ld32(t_s + 32, sreg[1]);
            tmem_wait_ld();
            // Exchange, warp by warp: my 32 x 64 partial goes to my send buffer ([16-byte chunk][lane], so that the
            // warp writes 512 contiguous bytes), one bulk copy moves it into the peer warp's receive buffer and counts
            // its bytes on the peer's barrier; the peer's partial arrives the same way and is added to mine.
            {
                unsigned char* send = sgen + kOffRecv + warp * 2 * kXchg;
                const unsigned char* recv = send + kXchg;
                if (lane == 0) {
                    mbar_expect_tx(bar(P_RF0 + warp), kXchg);            // the peer's copy of this tile
                    // The peer warp has read what I sent for the previous tile: that copy had landed there, so it has
                    // also finished reading my send buffer, which may now be overwritten.
                    if (j >= 1) ok = mbar_wait_cluster(bar(P_RC0 + warp), (j - 1) & 1, abort_flag, err, 35);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    reinterpret_cast<uint4*>(send)[c * 32 + lane] =
                        make_uint4(sreg[c >> 3][(c & 7) * 4], sreg[c >> 3][(c & 7) * 4 + 1], sreg[c >> 3][(c & 7) * 4 + 2], sreg[c >> 3][(c & 7) * 4 + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0)
                    bulk_copy_to_peer(map_to_cta(smem_addr(recv), peer), smem_addr(send), kXchg, map_to_cta(bar(P_RF0 + warp), peer));
                ok = mbar_wait_cluster(bar(P_RF0 + warp), j & 1, abort_flag, err, 36);
                if (!ok) break;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float4 v = reinterpret_cast<const float4*>(recv)[c * 32 + lane];
                    uint32_t* d = &sreg[c >> 3][(c & 7) * 4];
                    d[0] = __float_as_uint(__uint_as_float(d[0]) + v.x);
                    d[1] = __float_as_uint(__uint_as_float(d[1]) + v.y);
                    d[2] = __float_as_uint(__uint_as_float(d[2]) + v.z);
                    d[3] = __float_as_uint(__uint_as_float(d[3]) + v.w);
                }
                __syncwarp();
                // the values read above have been used, so the peer may overwrite my receive buffer: no release needed
                if (lane == 0) mbar_arrive_remote_relaxed(map_to_cta(bar(P_RC0 + warp), peer));
            }
            const int valid = t_end - (t_begin + j * kTile);               // tokens of this tile that exist
            if (valid < kTile) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i >= valid) sreg[c][i] = 0xff800000u;   // -inf
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    mx0 = fmaxf(fmaxf(mx0, __uint_as_float(sreg[c][i])), __uint_as_float(sreg[c][i + 1]));
                    mx1 = fmaxf(fmaxf(mx1, __uint_as_float(sreg[c][i + 2])), __uint_as_float(sreg[c][i + 3]));
                    mx2 = fmaxf(fmaxf(mx2, __uint_as_float(sreg[c][i + 4])), __uint_as_float(sreg[c][i + 5]));
                    mx3 = fmaxf(fmaxf(mx3, __uint_as_float(sreg[c][i + 6])), __uint_as_float(sreg[c][i + 7]));
                }
            }
            const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scl;   // log2 domain
            if (m_used == -INFINITY) m_used = m_new;
            // The exponent base moves only when the row maximum outgrows it by 2^8.  P V of tile j - 1 was issued
            // after the scores of tile j, so its completion is awaited before the accumulator is rescaled.
            if (j > 0 && __any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
                ok = mbar_wait(bar(P_KE0 + (j - 1) % kKBufs), ((j - 1) / kKBufs) & 1, abort_flag, err, 37);
                if (!ok) break;
                tc_fence_after();
                const float m_next = fmaxf(m_used, m_new);
                const float alpha = m_used == -INFINITY ? 1.f : ex2_approx(m_used - m_next);
                m_used = m_next;
                l_run *= alpha;
#pragma unroll 1
                for (int c = 0; c < 8; ++c) {
                    uint32_t oreg[32];
                    tmem_ld32(t_o + c * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st32(t_o + c * 32, oreg);
                }
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            const float2 sc2 = make_float2(scl, scl), nm2 = make_float2(neg_m, neg_m);
            float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
            uint32_t preg[32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float2 xa = fma2(make_float2(__uint_as_float(sreg[c][i]), __uint_as_float(sreg[c][i + 1])), sc2, nm2);
                    const float2 xb = fma2(make_float2(__uint_as_float(sreg[c][i + 2]), __uint_as_float(sreg[c][i + 3])), sc2, nm2);
                    const float2 pa = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
                    const float2 pb = make_float2(ex2_approx(xb.x), ex2_approx(xb.y));
                    sum_a = add2(sum_a, pa);
                    sum_b = add2(sum_b, pb);
                    preg[c * 16 + i / 2] = Elem<T>::pack(pa.x, pa.y);
                    preg[c * 16 + i / 2 + 1] = Elem<T>::pack(pb.x, pb.y);
                }
            }
            tmem_st32(t_s, preg);                                          // P over the first half of S's columns
            l_run += (sum_a.x + sum_b.x) + (sum_a.y + sum_b.y);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(P_P0 + s));
        }
        if (ok) ok = mbar_wait(bar(P_O), 0, abort_flag, err, 38);
        if (ok) {
            tc_fence_after();
            const int h = head0 + r;
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const int64_t row = (int64_t)b * p.hq + h;
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
                uint32_t oreg[32];
                tmem_ld32(t_o + c * 32, oreg);
                tmem_wait_ld();
                if (h < p.hq) {
                    if (a.final_direct) {
                        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + rank * 256 + c * 32);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 pk;
                            pk.x = Elem<T>::pack(__uint_as_float(oreg[8 * v]) * inv, __uint_as_float(oreg[8 * v + 1]) * inv);
                            pk.y = Elem<T>::pack(__uint_as_float(oreg[8 * v + 2]) * inv, __uint_as_float(oreg[8 * v + 3]) * inv);
                            pk.z = Elem<T>::pack(__uint_as_float(oreg[8 * v + 4]) * inv, __uint_as_float(oreg[8 * v + 5]) * inv);
                            pk.w = Elem<T>::pack(__uint_as_float(oreg[8 * v + 6]) * inv, __uint_as_float(oreg[8 * v + 7]) * inv);
                            dst[v] = pk;
                        }
                    } else {
                        float4* dst = reinterpret_cast<float4*>(a.o_part + ((int64_t)split * rows_all + row) * kLat + rank * 256 + c * 32);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_float4(__uint_as_float(oreg[4 * v]) * inv, __uint_as_float(oreg[4 * v + 1]) * inv,
                                                 __uint_as_float(oreg[4 * v + 2]) * inv, __uint_as_float(oreg[4 * v + 3]) * inv);
                    }
                }
            }
            if (h < p.hq && rank == 0) {
                if (a.final_direct) { if (p.lse) p.lse[row] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : INFINITY; }
                else a.lse_part[(int64_t)split * rows_all + row] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : -INFINITY;
            }
        }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    cluster_sync_all();                           // no CTA leaves while its peer may still write into it
}

}  // namespace

bool mla_pair_supported(const fa_mla_params& p) {
    // a tile of 64 tokens must lie inside one page
    return p.page_size % kTile == 0 && (p.kv_begin <= 0 || p.kv_begin % kTile == 0);
}

int launch_mla_pair(const fa_mla_params& p, int nsplit, int tokens_per_split, float* o_part, float* lse_part,
                    int final_direct, cudaStream_t st) {
    if (tokens_per_split % kTile) return fail(FA_ERR_BAD_SHAPE, "tokens per split must be a multiple of %d", kTile);
    MlaPairArgs a;
    a.p = p;
    a.nsplit = nsplit;
    a.tokens_per_split = tokens_per_split;
    a.o_part = o_part;
    a.lse_part = lse_part;
    a.final_direct = final_direct;
    a.scale_log2 = p.scale * kLog2e;
    if (int e = cuda_ok(cudaFuncSetAttribute(mla_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes), "cudaFuncSetAttribute")) return e;
    const int head_tiles = (p.hq + 127) / 128;
    dim3 grid(2, nsplit, p.b * head_tiles);       // x = the two CTAs of a cluster
    note_kernel("mla_int8_tcgen05_pair");
    mla_pair_kernel<<<grid, kThreads, kSmemBytes, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "mla_pair launch");
}

}  // namespace fa
