// int8 latent (MLA) paged decode on the tcgen05 tensor cores.  No counterpart in the reference.
//
// Per cached token j:  K_j = [scale_j * latent_j (512, int8 -> bf16) | rope_j (64 bf16)],  V_j = the dequantised
// latent.  One shared KV head, seqlen_q = 1, up to 128 query heads per CTA (the M dimension of the MMAs).
//
// A 128 x 512 fp32 output accumulator fills the whole tensor memory of an SM, so a CTA owns one HALF of the
// output columns (256 TMEM columns) and both halves compute the scores; what is left holds two 64-column score
// buffers.  CTA = (KV split, output half, sequence x head tile).  16 warps:
//   warps 0-3   softmax: thread = head row; S from TMEM, P (bf16) back into the same columns, epilogue
//   warps 4-11  producers: int8 rows -> registers -> (x - 0) * scale -> bf16 -> swizzled shared memory in the
//               UMMA layout, one tile of 64 tokens at a time; the same bytes are the K operand of Q K^T and the
//               V operand of P V
//   warp 12     issues the MMAs, owns the tensor memory (warps 13-15 idle: register reallocation works on groups of 4)
// Shared memory holds Q (128 x 576 bf16 = 144 KB) and ONE dequantised tile (64 x 576 bf16 = 72 KB).  The tile is
// split into an "early" group (the 256 latent columns of the OTHER half + rope) that only Q K^T reads, and a
// "late" group (the CTA's own 256 columns) that P V reads too: the early group of tile j+1 is refilled and
// multiplied while the softmax and P V of tile j are still running.
#include "fa_utils.cuh"
#include "fa_internal.h"
#include "sm100_ptx.cuh"
#include "mla_dequant.cuh"

namespace fa {

using namespace sm100;

__device__ int g_mla_sm100_error = 0;

int mla_sm100_error_flag(bool clear) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_mla_sm100_error, sizeof(int));
    if (clear) { int z = 0; cudaMemcpyToSymbol(g_mla_sm100_error, &z, sizeof(int)); }
    return v;
}

namespace {

constexpr int kLat = 512, kRope = 64;
constexpr int kTile = 64;                       // tokens per tile
constexpr int kQSub = 128 * 128;                // bytes of one [128 heads x 64 dims] Q sub-tile
constexpr int kKSub = kTile * 128;              // bytes of one [64 tokens x 64 dims] K sub-tile
constexpr int kSmemQ = 9 * kQSub, kSmemK = 9 * kKSub;
constexpr int kSmemBar = kSmemQ + kSmemK;
constexpr int kSmemBytes = kSmemBar + 256 + 1024;
constexpr int kThreads = 16 * 32;               // warps 13-15 only complete the last warp group
enum { M_KF_E = 0, M_KF_L, M_KE_E, M_KE_L, M_S0, M_S1, M_P0, M_P1, M_O, M_COUNT };

struct MlaSm100Args {
    fa_mla_params p;
    int nsplit, tokens_per_split;
    float* o_part;
    float* lse_part;
    int final_direct;
    float scale_log2;
};

__global__ void __launch_bounds__(kThreads, 1) mla_sm100_kernel(const __grid_constant__ MlaSm100Args a) {
    using T = __nv_bfloat16;
    const fa_mla_params& p = a.p;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t IDESC_QK = umma_idesc(1, 128, kTile, 0, 0);
    constexpr uint32_t IDESC_PV = umma_idesc(1, 128, 256, 0, 1);
    constexpr float kRescaleThreshold = 8.f;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t sQ = sbase, sK = sbase + kSmemQ, bars = sbase + kSmemBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + kSmemBar + 8 * M_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + kSmemBar + 8 * M_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, half = blockIdx.y;
    const int head_tiles = (p.hq + 127) / 128;
    const int b = blockIdx.z / head_tiles, head0 = (blockIdx.z % head_tiles) * 128;
    // an oversized length is truncated to what the page-table row can address
    const int sk = (int)max(0LL, min((long long)p.cache_seqlens[b], (long long)p.block_table_stride * p.page_size));
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    const int t_begin = rb + split * a.tokens_per_split;
    const int t_end = min(re, t_begin + a.tokens_per_split);
    const int ntiles = t_end > t_begin ? (t_end - t_begin + kTile - 1) / kTile : 0;
    const int64_t rows_all = (int64_t)p.b * p.hq;
    if (g_mla_sm100_error) return;

    if (ntiles == 0) {                           // nothing cached in this split's range
        const int h = head0 + tid;
        if (tid < 128 && h < p.hq) {
            const int64_t row = (int64_t)b * p.hq + h;
            if (a.final_direct) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + half * 256);
                for (int i = 0; i < 32; ++i) dst[i] = make_uint4(0, 0, 0, 0);
                if (half == 0 && p.lse) p.lse[row] = INFINITY;
            } else {
                if (a.nsplit == 1) {
                    float4* dst = reinterpret_cast<float4*>(a.o_part + row * kLat + half * 256);
                    for (int i = 0; i < 64; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (half == 0) a.lse_part[(int64_t)split * rows_all + row] = -INFINITY;
            }
        }
        return;
    }

    if (tid == 0) {
        mbar_init(bar(M_KF_E), 8); mbar_init(bar(M_KF_L), 8);
        mbar_init(bar(M_KE_E), 1); mbar_init(bar(M_KE_L), 1);
        mbar_init(bar(M_S0), 1); mbar_init(bar(M_S1), 1);
        mbar_init(bar(M_P0), 128); mbar_init(bar(M_P1), 128);
        mbar_init(bar(M_O), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 12) {
        tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    // ---- Q: 128 heads x (512 | 64) as nine K-major [128 x 64] sub-tiles, 128-byte swizzle ---------------------
    {
        const T* qn = reinterpret_cast<const T*>(p.q_nope) + (int64_t)b * p.q_nope_stride_b;
        const T* qr = reinterpret_cast<const T*>(p.q_rope) + (int64_t)b * p.q_rope_stride_b;
        for (int idx = tid; idx < 128 * 72; idx += kThreads) {
            const int r = idx / 72, c = idx % 72;                         // head row, 16-byte chunk of the 576 dims
            const int h = head0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (h < p.hq)
                v = __ldg(reinterpret_cast<const uint4*>(c < 64 ? qn + (int64_t)h * p.q_nope_stride_h + c * 8
                                                                 : qr + (int64_t)h * p.q_rope_stride_h + (c - 64) * 8));
            const int sub = c >> 3, ch = c & 7;
            *reinterpret_cast<uint4*>(sgen + sub * kQSub + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_mla_sm100_error;
    const int own0 = half * 4, oth0 = (1 - half) * 4;                      // first sub-tile of the own / other half

    // Register file split by warp group (the CTA starts with 128 a thread): 96 for the MMA group and for the two
    // producer groups, 224 for the softmax group; 128*96 + 256*96 + 128*224 = 512*128.
    static_assert(128 * 96 + 256 * 96 + 128 * 224 <= 512 * 128, "register split exceeds the CTA's allocation");
    if (warp >= 12) {
        reg_dealloc<96>();
        if (warp == 12) {
        // ------------------------------------------------------------------ MMA issue (whole warp, one elected lane)
        const uint64_t dQ = umma_desc(sQ, 16, 1024), dK = umma_desc(sK, 16, 1024);
        const uint64_t dV = umma_desc(sK + own0 * kKSub, kKSub, 1024);     // MN-major: four 64-column groups kKSub apart
        // scores += Q[:, sub] K[:, sub]^T over the 64 dims of sub-tile `sub`
        auto qk_sub = [&](uint32_t d_s, int sub, bool first) {
            const uint64_t aq = umma_desc_at(dQ, sub * kQSub), bk = umma_desc_at(dK, sub * kKSub);
            if (first) umma_ss_wo<0, 0, 0>(d_s, aq, bk, IDESC_QK); else umma_ss_wo<1, 0, 0>(d_s, aq, bk, IDESC_QK);
            umma_ss_wo<1, 32, 32>(d_s, aq, bk, IDESC_QK);
            umma_ss_wo<1, 64, 64>(d_s, aq, bk, IDESC_QK);
            umma_ss_wo<1, 96, 96>(d_s, aq, bk, IDESC_QK);
        };
        auto qk_early = [&](int j) {
            const uint32_t d_s = tmem + 256 + (j & 1) * 64;
#pragma unroll
            for (int s = 0; s < 4; ++s) qk_sub(d_s, oth0 + s, s == 0);
            qk_sub(d_s, 8, false);
            umma_commit_w(bar(M_KE_E));
        };
        bool ok = mbar_wait(bar(M_KF_E), 0, abort_flag, err, 21);
        if (ok) { tc_fence_after(); qk_early(0); }
        for (int j = 0; j < ntiles && ok; ++j) {
            const uint32_t d_s = tmem + 256 + (j & 1) * 64;
            ok = mbar_wait(bar(M_KF_L), j & 1, abort_flag, err, 22);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < 4; ++s) qk_sub(d_s, own0 + s, false);
            umma_commit_w(bar(M_S0 + (j & 1)));
            if (j + 1 < ntiles) {
                ok = mbar_wait(bar(M_KF_E), (j + 1) & 1, abort_flag, err, 23);
                if (!ok) break;
                tc_fence_after();
                qk_early(j + 1);
            }
            ok = mbar_wait(bar(M_P0 + (j & 1)), (j >> 1) & 1, abort_flag, err, 24);
            if (!ok) break;
            tc_fence_after();
            // O[:, own half] += P (TMEM, 64 tokens) V (the own sub-tiles read token-major)
            if (j > 0) umma_ts_wo<1, 0, 0>(tmem, d_s, dV, IDESC_PV); else umma_ts_wo<0, 0, 0>(tmem, d_s, dV, IDESC_PV);
            umma_ts_wo<1, 8, 2048>(tmem, d_s, dV, IDESC_PV);
            umma_ts_wo<1, 16, 4096>(tmem, d_s, dV, IDESC_PV);
            umma_ts_wo<1, 24, 6144>(tmem, d_s, dV, IDESC_PV);
            umma_commit_w(bar(M_KE_L));
        }
        if (ok) umma_commit_w(bar(M_O));
        }
    } else if (warp >= 4) {
        reg_dealloc<96>();
        // ------------------------------------------------------------------ producers: dequantise into shared memory
        const int pw = warp - 4;
        const int cl = lane & 15;                                         // 16-byte chunk of a 256-value half row
        const int krow = pw * 2 + (lane >> 4);                            // + 16 * pass = token row of the tile
        const int sub_l = cl >> 2, cp = cl & 3;                           // sub-tile within the group, chunk pair
        const int32_t* btab = p.block_table + (int64_t)b * p.block_table_stride;
        const int rrow = (tid - 128) >> 2, rch = (tid - 128) & 3;           // rope: 64 rows x 8 chunks, two per thread
        uint4 regE[4], regL[4], regR[2];
        float sc[4], sc_next[4];
        // first cache row of a tile (tiles never straddle a page); the page-table entry of the tile after the next
        // one is fetched a whole iteration before it is needed
        auto tile_row = [&](int j) -> int64_t {
            const int t0 = t_begin + j * kTile;
            const int jj = t0 < t_end ? t0 : t_begin;
            return (int64_t)__ldg(btab + jj / p.page_size) * p.page_size + jj % p.page_size;
        };
        int64_t slot0 = tile_row(0), slot_next = tile_row(1);
        auto tile_slot = [&](int j) { return t_begin + j * kTile; };
        auto load_group = [&](int j, int col0, uint4 (&reg)[4], bool with_scale) {
            const int t0 = tile_slot(j);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = r * 16 + krow;
                const bool live = t0 + row < t_end;
                reg[r] = make_uint4(0, 0, 0, 0);                       // rows past the end become zero keys and values
                if (live) reg[r] = __ldg(reinterpret_cast<const uint4*>(p.latent + (slot0 + row) * kLat + col0 + cl * 16));
                if (with_scale) sc_next[r] = live ? __ldg(p.scales + slot0 + row) : 0.f;
            }
        };
        auto load_rope = [&](int j) {
            const int t0 = tile_slot(j);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = rrow, ch = rch * 2 + i;
                regR[i] = make_uint4(0, 0, 0, 0);
                if (t0 + row < t_end)
                    regR[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.rope) + (slot0 + row) * kRope + ch * 8));
            }
        };
        auto store_group = [&](int sub0, const uint4 (&reg)[4]) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = r * 16 + krow;
                uint4 lo, hi;
                dequant16(reg[r], sc[r], lo, hi);
                unsigned char* base = sgen + kSmemQ + (sub0 + sub_l) * kKSub + row * 128;
                const int c0 = (2 * cp) ^ (row & 7), c1 = (2 * cp + 1) ^ (row & 7);
                // the two sub-tiles a quarter warp touches store their even / odd chunks in opposite order: 8 banks groups
                if (sub_l & 1) {
                    *reinterpret_cast<uint4*>(base + (c1 << 4)) = hi;
                    *reinterpret_cast<uint4*>(base + (c0 << 4)) = lo;
                } else {
                    *reinterpret_cast<uint4*>(base + (c0 << 4)) = lo;
                    *reinterpret_cast<uint4*>(base + (c1 << 4)) = hi;
                }
            }
        };
        auto store_rope = [&]() {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = rrow, ch = rch * 2 + i;
                *reinterpret_cast<uint4*>(sgen + kSmemQ + 8 * kKSub + row * 128 + ((ch ^ (row & 7)) << 4)) = regR[i];
            }
        };
        auto publish = [&](int which) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(which));
        };
        load_group(0, oth0 * 64, regE, true);
        load_rope(0);
        load_group(0, own0 * 64, regL, false);
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
#pragma unroll
            for (int r = 0; r < 4; ++r) sc[r] = sc_next[r];
            if (j > 0) ok = mbar_wait_relaxed(bar(M_KE_E), (j - 1) & 1, abort_flag, err, 25);
            if (!ok) break;
            store_group(oth0, regE);
            store_rope();
            publish(M_KF_E);
            // the next tile's early group travels while this tile's late group waits for its P V
            slot0 = slot_next;                                            // rows of tile j + 1 from here on
            slot_next = tile_row(j + 2);
            if (j + 1 < ntiles) {
                load_group(j + 1, oth0 * 64, regE, true);
                load_rope(j + 1);
            }
            if (j > 0) ok = mbar_wait_relaxed(bar(M_KE_L), (j - 1) & 1, abort_flag, err, 26);
            if (!ok) break;
            store_group(own0, regL);
            publish(M_KF_L);
            if (j + 1 < ntiles) load_group(j + 1, own0 * 64, regL, false);
        }
    } else {
        reg_alloc<224>();
        // ------------------------------------------------------------------ softmax: thread = head row
        const int r = tid;                                                 // 0..127
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t t_o = tmem + lane_base;
        float m_used = -INFINITY, l_run = 0.f;
        const float scl = a.scale_log2;
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const uint32_t t_s = tmem + lane_base + 256 + (j & 1) * 64;
            ok = mbar_wait(bar(M_S0 + (j & 1)), (j >> 1) & 1, abort_flag, err, 27);
            if (!ok) break;
            tc_fence_after();
            uint32_t sreg[2][32];
            tmem_ld32(t_s, sreg[0]);
            tmem_ld32(t_s + 32, sreg[1]);
            tmem_wait_ld();
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
            // The exponent base moves only when the row maximum outgrows it by 2^8; S of tile j being complete
            // means every earlier P V has finished, so the accumulator may be rescaled here.
            if (j > 0 && __any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
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
            mbar_arrive(bar(M_P0 + (j & 1)));
        }
        if (ok) ok = mbar_wait(bar(M_O), 0, abort_flag, err, 28);
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
                        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + half * 256 + c * 32);
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
                        float4* dst = reinterpret_cast<float4*>(a.o_part + ((int64_t)split * rows_all + row) * kLat + half * 256 + c * 32);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_float4(__uint_as_float(oreg[4 * v]) * inv, __uint_as_float(oreg[4 * v + 1]) * inv,
                                                 __uint_as_float(oreg[4 * v + 2]) * inv, __uint_as_float(oreg[4 * v + 3]) * inv);
                    }
                }
            }
            if (h < p.hq && half == 0) {
                if (a.final_direct) { if (p.lse) p.lse[row] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : INFINITY; }
                else a.lse_part[(int64_t)split * rows_all + row] = l_run > 0.f ? (m_used + log2f(l_run)) * kLn2 : -INFINITY;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace

bool mla_sm100_supported(const fa_mla_params& p) {
    // a tile of 64 tokens must lie inside one page
    return p.page_size % kTile == 0 && (p.kv_begin <= 0 || p.kv_begin % kTile == 0);
}

int launch_mla_sm100(const fa_mla_params& p, int nsplit, int tokens_per_split, float* o_part, float* lse_part,
                     int final_direct, cudaStream_t st) {
    if (tokens_per_split % kTile) return fail(FA_ERR_BAD_SHAPE, "tokens per split must be a multiple of %d", kTile);
    MlaSm100Args a;
    a.p = p;
    a.nsplit = nsplit;
    a.tokens_per_split = tokens_per_split;
    a.o_part = o_part;
    a.lse_part = lse_part;
    a.final_direct = final_direct;
    a.scale_log2 = p.scale * kLog2e;
    if (int e = cuda_ok(cudaFuncSetAttribute(mla_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes), "cudaFuncSetAttribute")) return e;
    const int head_tiles = (p.hq + 127) / 128;
    dim3 grid(nsplit, 2, p.b * head_tiles);
    note_kernel("mla_int8_tcgen05");
    mla_sm100_kernel<<<grid, kThreads, kSmemBytes, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "mla_sm100 launch");
}

}  // namespace fa
