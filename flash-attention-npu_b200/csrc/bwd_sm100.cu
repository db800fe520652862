// Backward attention on Blackwell tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
// Two kernels after the delta pass (D = rowsum(dO o O)), no atomics, fixed accumulation order:
//
//  dK/dV kernel   one CTA per (128-key tile, KV head, batch) walks the 128-row query tiles of every
//                 head of the group.  Scores are computed transposed so that keys sit on the TMEM
//                 lanes:  S^T = K Q^T, dP^T = V dO^T.  One thread per key row turns them into
//                 P^T = exp(S^T - LSE) and dS^T = P^T o (dP^T - D) (rounded to the input type, written
//                 back over the score columns), which feed dV += P^T dO and dK += dS^T Q as the
//                 TMEM-resident A operand.  dK and dV stay in TMEM across all query tiles and heads.
//  dQ kernel      one CTA per (128-row query tile, head, batch) walks the key tiles:
//                 S = Q K^T, dP = dO V^T, dS = P o (dP - D), dQ += dS K.
//
// Math as the reference's backward (fag_kernel.cpp:400-465, fag_epilogue_op.hpp:1287-1322, :1394,
// :1447-1480, fag_epilogue_post.hpp:149-200): P and dS rounded before the second GEMMs, dQ and dK
// multiplied by the softmax scale at the end.
//
// Both kernels work on whole 128 x 128 score tiles (N = 128 score MMAs; 64-column halves cost ~50 cycles a K step
// instead of 32).  dK/dV: tensor memory holds S^T | dP^T | dK | dV (128 columns each), nothing is double-buffered,
// and the overlap comes from the order on the in-order tensor pipe: S^T(s) dP^T(s) | dV(s) S^T(s+1) | dK(s)
// dP^T(s+1) | ...  -- P^T lies over S^T and dS^T over dP^T, so the next scores simply follow the MMA that reads
// what they overwrite, and the exponentials of block s+1 run while dK(s) and dP^T(s+1) are multiplied.  dQ: S has
// two buffers, dP one, dQ accumulates; order dP(t) S(t+1) dQ(t); K has three shared-memory stages (S(t+1) is
// multiplied before dQ(t-1) has released its K), V two.  Warps 0-15 do the element-wise work (thread = TMEM lane,
// each group of four warps takes 32 of a tile's 128 score columns) in two phases, exponentials then dS; warp 16 is
// the TMA producer, warp 17 issues all MMAs.  All waits are bounded.
#include "fa_utils.cuh"
#include "fa_internal.h"
#include "sm100_ptx.cuh"
#include <atomic>

namespace fa {

using namespace sm100;

__device__ int g_bwd_sm100_error = 0;

int bwd_sm100_error_flag(bool clear) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_bwd_sm100_error, sizeof(int));
    if (clear) { int z = 0; cudaMemcpyToSymbol(g_bwd_sm100_error, &z, sizeof(int)); }
    return v;
}

struct alignas(64) Sm100BwdArgs {
    CUtensorMap tq, tdo, tk, tv;
    void *dq, *dk, *dv;
    int64_t dq_sb, dq_ss, dq_sh, dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
    const float* lse;
    int64_t lse_sb, lse_sh, lse_ss;
    const float* delta;                 // [token][head]
    const int32_t* cu_q;
    const int32_t* cu_k;
    int b, sq, sk, hq, hkv;
    int chunk_kv, chunk_q;              // grid order: (batch entry, KV head) pairs a chunk of the dK/dV grid, (batch entry, head) pairs of the dQ grids
    int d;                              // the call's head dim (a multiple of 8, at most the kernels' 64 / 128): tile copies zero-fill
                                        // the columns past it, the epilogues store d columns
    float scale, scale_log2;
    int causal, wl, wr;
    // dS^T tiles handed from the dK/dV kernel to the dQ kernel through global memory (dense calls within the
    // workspace limit): tile (batch, head, key block n, query block m) = 128 keys x 128 queries of the input type,
    // stored as [16 chunks of 8 queries][128 keys][8 queries]
    void* ds_tiles;
    int nkb, nqb;
    // score transforms of the BIAS instantiation of the dK/dV kernel: softcap (0 = off) and alibi slopes (null = off)
    float softcap, cap_in2, cap_out;     // cap_in2 = 2 log2(e) scale / softcap, cap_out = softcap log2(e)
    const float* alibi;
    int64_t alibi_sb;
};

template <int D>
struct BwdSm100Smem {
    static constexpr int kSub = 128 * 128;
    static constexpr int kTileB = (D / 64) * kSub;          // one [128][D] tile
    static constexpr int oFix0 = 0;                         // K (dkdv) or Q (dq)
    static constexpr int oFix1 = oFix0 + kTileB;            // V (dkdv) or dO (dq)
    static constexpr int oRing0 = oFix1 + kTileB;           // 2 stages: Q (dkdv) or K (dq)
    static constexpr int oRing1 = oRing0 + 2 * kTileB;      // 2 stages: dO (dkdv) or V (dq)
    static constexpr int oVec = oRing1 + 2 * kTileB;        // per warp: 2 stages x (32 lse2 + 32 delta) floats
    static constexpr int oBar = oVec + 16 * 128 * 4;
    static constexpr int kBytes = oBar + 256;
};

enum { E_FIX = 0, E_RF0, E_RF1, E_RE0, E_RE1, E_S0, E_S1, E_P0, E_P1, E_F0, E_F1, E_ACC, E_COUNT };
// barriers of the dQ kernel: KF/KE, VF/VE K and V stage full / free; S scores done; SA scores read; DP dP done; DS dS stored
enum { G_FIX = 0, G_KF0, G_KF1, G_KF2, G_KE0, G_KE1, G_KE2, G_VF0, G_VF1, G_VE0, G_VE1, G_S0, G_S1, G_SA0, G_SA1, G_DP, G_DS,
       G_ACC, G_COUNT };

// 32 accumulator columns -> the row, scaled and rounded; `left` = columns of the row that remain from dst on (the
// kernels run a head dim padded to 64 / 128, the row holds the call's own head dim)
template <typename T>
__device__ __forceinline__ void store_row_scaled(T* dst, const uint32_t (&r)[32], float s, int left) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        if (v * 8 >= left) break;
        uint4 pk;
        pk.x = Elem<T>::pack(__uint_as_float(r[8 * v + 0]) * s, __uint_as_float(r[8 * v + 1]) * s);
        pk.y = Elem<T>::pack(__uint_as_float(r[8 * v + 2]) * s, __uint_as_float(r[8 * v + 3]) * s);
        pk.z = Elem<T>::pack(__uint_as_float(r[8 * v + 4]) * s, __uint_as_float(r[8 * v + 5]) * s);
        pk.w = Elem<T>::pack(__uint_as_float(r[8 * v + 6]) * s, __uint_as_float(r[8 * v + 7]) * s);
        reinterpret_cast<uint4*>(dst)[v] = pk;
    }
}

// ------------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------------
template <typename T, int D, bool BIAS>
__global__ void __launch_bounds__(608, 1) bwd_dkdv_sm100_kernel(const __grid_constant__ Sm100BwdArgs a) {
    using L = BwdSm100Smem<D>;
    constexpr int NSUB = D / 64, KSTEPS = D / 16;
    constexpr uint32_t TMEM_COLS = 512, COL_ST = 0, COL_DPT = 128, COL_DK = 256, COL_DV = 384;   // ST/DPT: 2 x 64
    constexpr int FMT = Elem<T>::kDtype == FA_BF16 ? 1 : 0;
    constexpr uint32_t IDESC_ST = umma_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_ACC = umma_idesc(FMT, 128, D, 0, 1);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t sK = sbase + L::oFix0, sV = sbase + L::oFix1, sQ = sbase + L::oRing0, sdO = sbase + L::oRing1;
    float* sVec = reinterpret_cast<float*>(sgen + L::oVec);
    const uint32_t bars = sbase + L::oBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::oBar + 8 * E_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + L::oBar + 8 * E_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Grid order: (pair in chunk, key block, chunk) over chunks of (batch entry, KV head) pairs, as in the forward: inside
    // a chunk the key blocks with the most query blocks to walk (the first ones under a causal mask) of ALL its pairs
    // start before any lighter one, and a chunk's Q and dO stay in L2 while its key blocks run.
    const int pair = blockIdx.z * a.chunk_kv + blockIdx.x;
    if (pair >= a.b * a.hkv) return;
    const uint3 bi = make_uint3(blockIdx.y, pair % a.hkv, pair / a.hkv);     // (key block, KV head, batch entry)
    const int b = bi.z, hk = bi.y, n0 = bi.x * 128;
    int q_off = 0, k_off = 0, sq = a.sq, sk = a.sk;
    if (a.cu_q) { q_off = a.cu_q[b]; sq = a.cu_q[b + 1] - q_off; k_off = a.cu_k[b]; sk = a.cu_k[b + 1] - k_off; }
    if (n0 >= sk) return;
    if (g_bwd_sm100_error) return;
    const int G = a.hq / a.hkv;
    const int wl = a.wl, wr = a.causal ? 0 : a.wr;
    const int diff = sk - sq;
    const int krows = min(128, sk - n0);

    int i_lo = 0, i_hi = sq - 1;
    if (wr >= 0) i_lo = max(0, n0 - diff - wr);
    if (wl >= 0) i_hi = min(sq - 1, n0 + krows - 1 + wl - diff);
    const int mb_lo = i_lo / 128, mb_hi = i_hi >= i_lo ? i_hi / 128 + 1 : mb_lo;
    const int nmb = mb_hi - mb_lo;
    const int steps = nmb * G;

    T* dkb = reinterpret_cast<T*>(a.dk) + (a.cu_q ? 0 : (int64_t)b * a.dk_sb) + (int64_t)(k_off + n0) * a.dk_ss + (int64_t)hk * a.dk_sh;
    T* dvb = reinterpret_cast<T*>(a.dv) + (a.cu_q ? 0 : (int64_t)b * a.dv_sb) + (int64_t)(k_off + n0) * a.dv_ss + (int64_t)hk * a.dv_sh;

    if (steps == 0) {                                       // no query sees these keys
        if (tid < 256) {
            const int r = tid & 127;
            T* row = (tid < 128 ? dkb + (int64_t)r * a.dk_ss : dvb + (int64_t)r * a.dv_ss);
            if (r < krows) {
                const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < D / 8; ++c)
                if (c * 8 < a.d) reinterpret_cast<uint4*>(row)[c] = z;      // the call's head dim, not the kernel's padded one
            }
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < E_COUNT; ++i) mbar_init(bar(i), (i == E_P0 || i == E_P1) ? 512u : 1u);   // P0: P^T stored, P1: dS^T stored
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 16) { tmem_alloc(smem_addr(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_bwd_sm100_error;
    const int bb = a.cu_q ? 0 : b;

    if (warp == 16) {
        if (lane == 0) {
            tma_prefetch_desc(&a.tq); tma_prefetch_desc(&a.tdo); tma_prefetch_desc(&a.tk); tma_prefetch_desc(&a.tv);
            mbar_expect_tx(bar(E_FIX), 2 * L::kTileB);
            const int krow = (a.cu_q ? k_off : 0) + n0;
#pragma unroll
            for (int s = 0; s < NSUB; ++s) {
                tma_load_4d(sK + s * L::kSub, &a.tk, bar(E_FIX), s * 64, hk, krow, bb);
                tma_load_4d(sV + s * L::kSub, &a.tv, bar(E_FIX), s * 64, hk, krow, bb);
            }
            bool ok = true;
            for (int s = 0; s < steps && ok; ++s) {
                const int st = s & 1, use = s >> 1;
                const int h = hk * G + s / nmb;
                const int qrow = (a.cu_q ? q_off : 0) + (mb_lo + s % nmb) * 128;
                if (use > 0) ok = mbar_wait(bar(E_RE0 + st), (use - 1) & 1, abort_flag, err, 21);
                if (!ok) break;
                mbar_expect_tx(bar(E_RF0 + st), 2 * L::kTileB);
#pragma unroll
                for (int c = 0; c < NSUB; ++c) {
                    tma_load_4d(sQ + st * L::kTileB + c * L::kSub, &a.tq, bar(E_RF0 + st), c * 64, h, qrow, bb);
                    tma_load_4d(sdO + st * L::kTileB + c * L::kSub, &a.tdo, bar(E_RF0 + st), c * 64, h, qrow, bb);
                }
            }
        }
    } else if (warp == 17) {
        {
            // One unit = one 128-query block.  E_S0: S^T done, E_S1: dP^T done, E_P0: P^T stored, E_P1: dS^T stored.
            // Order on the in-order tensor pipe: S^T(s) dP^T(s) | dV(s) S^T(s+1) | dK(s) dP^T(s+1) | ...: P^T lies over
            // S^T and dS^T over dP^T, so the next scores follow the MMA that read what they overwrite; the exponentials
            // of block s + 1 run while dK(s) and dP^T(s + 1) are multiplied.
            const uint64_t dK0 = umma_desc(sK, 16, 1024), dV0 = umma_desc(sV, 16, 1024);
            const uint64_t dQk = umma_desc(sQ, 16, 1024), dOk = umma_desc(sdO, 16, 1024);           // K-major views
            const uint64_t dQm = umma_desc(sQ, L::kSub, 1024), dOm = umma_desc(sdO, L::kSub, 1024); // MN-major views
            auto issue_scores = [&](uint32_t d_t, uint64_t a0, uint64_t b0, int st) {
                umma_ss_scores<KSTEPS, L::kSub>(d_t, a0, umma_desc_at(b0, st * L::kTileB), IDESC_ST);
            };
            // acc += A (tensor memory: 16 queries in 8 columns at a stride of 16) x B (query-major tile of stage st)
            auto issue_acc = [&](uint32_t d_t, uint32_t a_t, uint64_t b0, int st, bool first) {
                const uint64_t bt = umma_desc_at(b0, st * L::kTileB);
                umma_ts_group4<0, 16, 0, 128>(d_t, a_t, bt, IDESC_ACC, !first);
                umma_ts_group4<64, 16, 512, 128>(d_t, a_t, bt, IDESC_ACC, 1);
            };
            bool ok = mbar_wait(bar(E_FIX), 0, abort_flag, err, 22);
            if (ok) ok = mbar_wait(bar(E_RF0), 0, abort_flag, err, 23);
            if (ok) {
                tc_fence_after();
                issue_scores(tmem + COL_ST, dK0, dQk, 0);
                umma_commit_w(bar(E_S0));
                issue_scores(tmem + COL_DPT, dV0, dOk, 0);
                umma_commit_w(bar(E_S1));
            }
            for (int s = 0; s < steps && ok; ++s) {
                const int st = s & 1, s1 = (s + 1) & 1;
                ok = mbar_wait(bar(E_P0), s & 1, abort_flag, err, 24);
                if (!ok) break;
                tc_fence_after();
                issue_acc(tmem + COL_DV, tmem + COL_ST, dOm, st, s == 0);
                if (s + 1 < steps) {
                    ok = mbar_wait(bar(E_RF0 + s1), ((s + 1) >> 1) & 1, abort_flag, err, 23);
                    if (!ok) break;
                    tc_fence_after();
                    issue_scores(tmem + COL_ST, dK0, dQk, s1);
                    umma_commit_w(bar(E_S0));
                }
                ok = mbar_wait(bar(E_P1), s & 1, abort_flag, err, 27);
                if (!ok) break;
                tc_fence_after();
                issue_acc(tmem + COL_DK, tmem + COL_DPT, dQm, st, s == 0);
                umma_commit_w(bar(E_RE0 + st));
                if (s + 1 < steps) {
                    issue_scores(tmem + COL_DPT, dV0, dOk, s1);
                    umma_commit_w(bar(E_S1));
                }
            }
            if (ok) umma_commit_w(bar(E_ACC));
        }
    } else if (warp == 18) {
        // spare warp of the last group
    } else {
        // ------------------------------------------------------------ element-wise: thread = (key row, 32 query columns)
        const int cg = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                // TMEM lane = key row of the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int n = n0 + r;
        // query rows that see key n: [qi_lo, qi_hi]
        int qi_lo = 0, qi_hi = sq - 1;
        if (wr >= 0) qi_lo = max(0, n - diff - wr);
        if (wl >= 0) qi_hi = min(sq - 1, n + wl - diff);
        if (n >= sk) { qi_lo = 1; qi_hi = 0; }
        bool ok = true;
        // -LSE (log2 domain) and -delta of the warp's 32 query columns, one per lane, fetched one step ahead
        auto fetch_vec = [&](int s, float& nl, float& nd) {
            const int h = hk * G + s / nmb;
            const int i = (mb_lo + s % nmb) * 128 + cg * 32 + lane;
            nl = -INFINITY; nd = 0.f;
            if (i < sq) {
                const int64_t tok = (int64_t)q_off + i;
                nl = -a.lse[(a.cu_q ? 0 : (int64_t)b * a.lse_sb) + (int64_t)h * a.lse_sh + tok * a.lse_ss] * kLog2e;
                nd = -a.delta[((a.cu_q ? tok : (int64_t)b * a.sq + i)) * a.hq + h];
            }
        };
        float st_l, st_d;
        fetch_vec(0, st_l, st_d);
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);
        for (int s = 0; s < steps && ok; ++s) {
            const int i0 = (mb_lo + s % nmb) * 128 + cg * 32;           // first query row of this thread's 32 columns
            float* vec = sVec + warp * 128 + (s & 1) * 64;              // [0,32) -lse2, [32,64) -delta
            vec[lane] = st_l;
            vec[32 + lane] = st_d;
            __syncwarp();
            if (s + 1 < steps) fetch_vec(s + 1, st_l, st_d);
            // phase A: P^T = exp2(S^T c - LSE) -> registers (fp32) and, rounded, over S^T's columns
            ok = mbar_wait(bar(E_S0), s & 1, abort_flag, err, 25);
            if (!ok) break;
            tc_fence_after();
            uint32_t pr[32], lo8[8], hi8[8];
            tmem_ld32(tmem + lane_base + COL_ST + cg * 32, pr);
            tmem_wait_ld();
            const bool inside = __all_sync(0xffffffffu, i0 >= qi_lo && i0 + 31 <= qi_hi);
            float slope = 0.f;
            if constexpr (BIAS) { if (a.alibi) slope = a.alibi[(int64_t)b * a.alibi_sb + hk * G + s / nmb] * kLog2e; }
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 nl = *reinterpret_cast<const float4*>(vec + i);
                float2 x01, x23;
                float fac[4] = {1.f, 1.f, 1.f, 1.f};                      // d(capped score) / d(scaled score)
                if constexpr (BIAS) {
                    // scores -> their final log2-domain values: softcap (tanh(y) = 1 - 2 / (1 + e^(2y))), then the alibi
                    // bias -slope |query position + sk - sq - key|, as the forward did
                    float xv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float v = __uint_as_float(pr[i + e]);
                        if (a.softcap > 0.f) {
                            const float th = 1.f - __fdividef(2.f, 1.f + ex2_approx(v * a.cap_in2));
                            v = a.cap_out * th;
                            fac[e] = 1.f - th * th;
                        } else {
                            v *= a.scale_log2;
                        }
                        xv[e] = v - slope * fabsf((float)(i0 + i + e + sk - sq - n));
                    }
                    x01 = make_float2(xv[0] + nl.x, xv[1] + nl.y);
                    x23 = make_float2(xv[2] + nl.z, xv[3] + nl.w);
                } else {
                    x01 = fma2(make_float2(__uint_as_float(pr[i]), __uint_as_float(pr[i + 1])), sc2, make_float2(nl.x, nl.y));
                    x23 = fma2(make_float2(__uint_as_float(pr[i + 2]), __uint_as_float(pr[i + 3])), sc2, make_float2(nl.z, nl.w));
                }
                float2 p01 = make_float2(ex2_approx(x01.x), ex2_approx(x01.y));
                float2 p23 = make_float2(ex2_approx(x23.x), ex2_approx(x23.y));
                if (!inside) {
                    const int qi = i0 + i;
                    p01.x = (qi >= qi_lo && qi <= qi_hi) ? p01.x : 0.f;
                    p01.y = (qi + 1 >= qi_lo && qi + 1 <= qi_hi) ? p01.y : 0.f;
                    p23.x = (qi + 2 >= qi_lo && qi + 2 <= qi_hi) ? p23.x : 0.f;
                    p23.y = (qi + 3 >= qi_lo && qi + 3 <= qi_hi) ? p23.y : 0.f;
                }
                // kept for phase B: P (times the softcap derivative, which then multiplies dS)
                pr[i] = __float_as_uint(p01.x * fac[0]); pr[i + 1] = __float_as_uint(p01.y * fac[1]);
                pr[i + 2] = __float_as_uint(p23.x * fac[2]); pr[i + 3] = __float_as_uint(p23.y * fac[3]);
                const uint32_t w0 = Elem<T>::pack(p01.x, p01.y), w1 = Elem<T>::pack(p23.x, p23.y);
                if (i < 16) { lo8[i / 2] = w0; lo8[i / 2 + 1] = w1; } else { hi8[(i - 16) / 2] = w0; hi8[(i - 16) / 2 + 1] = w1; }
            }
            // each group of 16 queries (one K step of the accumulating MMAs) sits in 8 columns at a stride of 16
            tmem_st8(tmem + lane_base + COL_ST + cg * 32, lo8);
            tmem_st8(tmem + lane_base + COL_ST + cg * 32 + 16, hi8);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_relaxed(bar(E_P0));
            // phase B: dS^T = P^T (dP^T - delta), rounded, over dP^T's columns
            ok = mbar_wait(bar(E_S1), s & 1, abort_flag, err, 28);
            if (!ok) break;
            tc_fence_after();
            uint32_t dr[32];
            tmem_ld32(tmem + lane_base + COL_DPT + cg * 32, dr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 nd = *reinterpret_cast<const float4*>(vec + 32 + i);
                const float2 d01 = mul2(make_float2(__uint_as_float(pr[i]), __uint_as_float(pr[i + 1])),
                                        add2(make_float2(__uint_as_float(dr[i]), __uint_as_float(dr[i + 1])), make_float2(nd.x, nd.y)));
                const float2 d23 = mul2(make_float2(__uint_as_float(pr[i + 2]), __uint_as_float(pr[i + 3])),
                                        add2(make_float2(__uint_as_float(dr[i + 2]), __uint_as_float(dr[i + 3])), make_float2(nd.z, nd.w)));
                const uint32_t w0 = Elem<T>::pack(d01.x, d01.y), w1 = Elem<T>::pack(d23.x, d23.y);
                if (i < 16) { lo8[i / 2] = w0; lo8[i / 2 + 1] = w1; } else { hi8[(i - 16) / 2] = w0; hi8[(i - 16) / 2 + 1] = w1; }
            }
            tmem_st8(tmem + lane_base + COL_DPT + cg * 32, lo8);
            tmem_st8(tmem + lane_base + COL_DPT + cg * 32 + 16, hi8);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_relaxed(bar(E_P1));
            if (a.ds_tiles) {
                // the same rounded dS^T goes to global memory for the dQ kernel, which then needs one GEMM a tile
                // instead of recomputing S and dP.  Issued after the hand-off so that the stores are off the chain.
                const int64_t tile = (((int64_t)b * a.hq + (hk * G + s / nmb)) * a.nkb + bi.x) * a.nqb + (mb_lo + s % nmb);
                // tile layout [16 chunks of 8 queries][128 keys][16 bytes]: a warp's 32 rows of one chunk are 512
                // contiguous bytes (one fully coalesced store instruction), and the tile is at the same time the
                // unswizzled operand layout the dQ kernel's MMA reads
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(a.ds_tiles) + tile * (128 * 128 * 2)) + (cg * 4) * 128 + r;
                dst[0] = make_uint4(lo8[0], lo8[1], lo8[2], lo8[3]);
                dst[128] = make_uint4(lo8[4], lo8[5], lo8[6], lo8[7]);
                dst[256] = make_uint4(hi8[0], hi8[1], hi8[2], hi8[3]);
                dst[384] = make_uint4(hi8[4], hi8[5], hi8[6], hi8[7]);
            }
        }
        if (ok) ok = mbar_wait(bar(E_ACC), 0, abort_flag, err, 26);
        if (ok) {
            tc_fence_after();
            // warp groups 0,1 write the two halves of dK (x scale), groups 2,3 the halves of dV
            const bool is_dk = cg < 2;
            T* row = is_dk ? dkb + (int64_t)r * a.dk_ss : dvb + (int64_t)r * a.dv_ss;
            const float sc = is_dk ? a.scale : 1.f;
            const uint32_t col = is_dk ? COL_DK : COL_DV;
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                const int cc = (cg & 1) * (D / 64) + c;
                uint32_t acc[32];
                tmem_ld32(tmem + lane_base + col + cc * 32, acc);
                tmem_wait_ld();
                if (r < krows) store_row_scaled<T>(row + cc * 32, acc, sc, a.d - cc * 32);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 16) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------------
template <typename T, int D, bool BIAS>
__global__ void __launch_bounds__(608, 1) bwd_dq_sm100_kernel(const __grid_constant__ Sm100BwdArgs a) {
    using L = BwdSm100Smem<D>;
    constexpr int NSUB = D / 64, KSTEPS = D / 16;
    // One unit = one 128-key tile.  S has two buffers (the scores of the next tile are multiplied while this tile is in
    // the element-wise stage), dP one (dS is written over it and read by the dQ MMA), dQ accumulates.
    constexpr uint32_t TMEM_COLS = 512, COL_S = 0, COL_DP = 256, COL_DQ = 384;
    constexpr int FMT = Elem<T>::kDtype == FA_BF16 ? 1 : 0;
    constexpr uint32_t IDESC_S = umma_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_ACC = umma_idesc(FMT, 128, D, 0, 1);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    // Q | dO | three K stages | two V stages: the scores of tile t + 1 are multiplied before dQ of tile t - 1 has
    // released its K, so K needs one stage more than V
    constexpr int oK = 2 * L::kTileB, oV = 5 * L::kTileB, oBarQ = 7 * L::kTileB;
    const uint32_t sQ = sbase, sdO = sbase + L::kTileB, sK = sbase + oK, sV = sbase + oV;
    const uint32_t bars = sbase + oBarQ;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + oBarQ + 8 * G_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + oBarQ + 8 * G_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = blockIdx.z * a.chunk_q + blockIdx.x;    // grid order as in the dK/dV kernel, over (batch entry, head) pairs
    if (pair >= a.b * a.hq) return;
    const int b = pair / a.hq, h = pair % a.hq;
    const int mblk = gridDim.y - 1 - blockIdx.y;
    int q_off = 0, k_off = 0, sq = a.sq, sk = a.sk;
    if (a.cu_q) { q_off = a.cu_q[b]; sq = a.cu_q[b + 1] - q_off; k_off = a.cu_k[b]; sk = a.cu_k[b + 1] - k_off; }
    const int m0 = mblk * 128;
    if (m0 >= sq) return;
    if (g_bwd_sm100_error) return;
    const int hk = h / (a.hq / a.hkv);
    const int wl = a.wl, wr = a.causal ? 0 : a.wr;
    const int rows = min(128, sq - m0);

    int lo_first, hi_first, lo_last, hi_last;
    window_bounds(m0, sq, sk, wl, wr, lo_first, hi_first);
    window_bounds(m0 + rows - 1, sq, sk, wl, wr, lo_last, hi_last);
    int t_lo = lo_first / 128, t_hi = hi_last < 0 ? 0 : hi_last / 128 + 1;
    if (sk <= 0 || lo_first >= sk) { t_lo = 0; t_hi = 0; }
    const int ntiles = max(0, t_hi - t_lo);

    T* dqb = reinterpret_cast<T*>(a.dq) + (a.cu_q ? 0 : (int64_t)b * a.dq_sb) + (int64_t)(q_off + m0) * a.dq_ss + (int64_t)h * a.dq_sh;
    if (ntiles == 0) {
        if (tid < rows) {
            const uint4 z = make_uint4(0, 0, 0, 0);
            T* row = dqb + (int64_t)tid * a.dq_ss;
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                if (c * 8 < a.d) reinterpret_cast<uint4*>(row)[c] = z;      // the call's head dim, not the kernel's padded one
        }
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < G_COUNT; ++i) mbar_init(bar(i), (i == G_SA0 || i == G_SA1 || i == G_DS) ? 512u : 1u);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 16) { tmem_alloc(smem_addr(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_bwd_sm100_error;
    const int bb = a.cu_q ? 0 : b;

    if (warp == 16) {
        if (lane == 0) {
            tma_prefetch_desc(&a.tq); tma_prefetch_desc(&a.tdo); tma_prefetch_desc(&a.tk); tma_prefetch_desc(&a.tv);
            mbar_expect_tx(bar(G_FIX), 2 * L::kTileB);
            const int qrow = (a.cu_q ? q_off : 0) + m0;
#pragma unroll
            for (int s = 0; s < NSUB; ++s) {
                tma_load_4d(sQ + s * L::kSub, &a.tq, bar(G_FIX), s * 64, h, qrow, bb);
                tma_load_4d(sdO + s * L::kSub, &a.tdo, bar(G_FIX), s * 64, h, qrow, bb);
            }
            bool ok = true;
            for (int j = 0; j < ntiles && ok; ++j) {
                const int ks = j % 3, vs = j & 1;
                const int krow = (a.cu_q ? k_off : 0) + (t_lo + j) * 128;
                if (j >= 3) ok = mbar_wait(bar(G_KE0 + ks), (j / 3 - 1) & 1, abort_flag, err, 31);
                if (!ok) break;
                mbar_expect_tx(bar(G_KF0 + ks), L::kTileB);
#pragma unroll
                for (int c = 0; c < NSUB; ++c) tma_load_4d(sK + ks * L::kTileB + c * L::kSub, &a.tk, bar(G_KF0 + ks), c * 64, hk, krow, bb);
                if (j >= 2) ok = mbar_wait(bar(G_VE0 + vs), ((j >> 1) - 1) & 1, abort_flag, err, 39);
                if (!ok) break;
                mbar_expect_tx(bar(G_VF0 + vs), L::kTileB);
#pragma unroll
                for (int c = 0; c < NSUB; ++c) tma_load_4d(sV + vs * L::kTileB + c * L::kSub, &a.tv, bar(G_VF0 + vs), c * 64, hk, krow, bb);
            }
        }
    } else if (warp == 17) {
        {
            const uint64_t dQ0 = umma_desc(sQ, 16, 1024), dO0 = umma_desc(sdO, 16, 1024);
            const uint64_t dKk = umma_desc(sK, 16, 1024), dVk = umma_desc(sV, 16, 1024);
            const uint64_t dKm = umma_desc(sK, L::kSub, 1024);
            // [128 queries x 128 keys] = A (Q or dO, K-major) x B (K or V tile of stage st, K-major)
            auto issue_scores = [&](uint32_t d_t, uint64_t a0, uint64_t b0, int stage) {
                umma_ss_scores<KSTEPS, L::kSub>(d_t, a0, umma_desc_at(b0, stage * L::kTileB), IDESC_S);
            };
            bool ok = mbar_wait(bar(G_FIX), 0, abort_flag, err, 32);
            if (ok) ok = mbar_wait(bar(G_KF0), 0, abort_flag, err, 33);
            if (ok) {
                tc_fence_after();
                issue_scores(tmem + COL_S, dQ0, dKk, 0);
                umma_commit_w(bar(G_S0));
            }
            // Order on the (in-order) tensor pipe: dP(t), S(t+1), dQ(t).  dP(t) follows dQ(t-1) in program order, so dS
            // of the previous tile has been consumed before dP overwrites its columns.
            for (int t = 0; t < ntiles && ok; ++t) {
                const int ks = t % 3, vs = t & 1;
                ok = mbar_wait(bar(G_VF0 + vs), (t >> 1) & 1, abort_flag, err, 40);
                if (!ok) break;
                tc_fence_after();
                issue_scores(tmem + COL_DP, dO0, dVk, vs);
                umma_commit_w(bar(G_DP));
                umma_commit_w(bar(G_VE0 + vs));              // V of this tile is not read again
                if (t + 1 < ntiles) {
                    const int s1 = (t + 1) & 1, k1 = (t + 1) % 3;
                    ok = mbar_wait(bar(G_KF0 + k1), ((t + 1) / 3) & 1, abort_flag, err, 33);
                    // the element-wise warps have read the scores that lived in this buffer two tiles ago
                    if (ok && t >= 1) ok = mbar_wait(bar(G_SA0 + s1), ((t - 1) >> 1) & 1, abort_flag, err, 37);
                    if (!ok) break;
                    tc_fence_after();
                    issue_scores(tmem + COL_S + s1 * 128, dQ0, dKk, k1);
                    umma_commit_w(bar(G_S0 + s1));
                }
                ok = mbar_wait(bar(G_DS), t & 1, abort_flag, err, 34);
                if (!ok) break;
                tc_fence_after();
                // dQ += dS (tensor memory, 16 keys in 8 columns at a stride of 16) x K tile read key-major
                const uint64_t bk = umma_desc_at(dKm, ks * L::kTileB);
                umma_ts_group4<0, 16, 0, 128>(tmem + COL_DQ, tmem + COL_DP, bk, IDESC_ACC, t > 0);
                umma_ts_group4<64, 16, 512, 128>(tmem + COL_DQ, tmem + COL_DP, bk, IDESC_ACC, 1);
                umma_commit_w(bar(G_KE0 + ks));
            }
            if (ok) umma_commit_w(bar(G_ACC));
        }
    } else if (warp == 18) {
        // spare warp of the last group
    } else {
        // element-wise warps: thread = (query row, 32 of the tile's 128 key columns)
        const int cg = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int qi = m0 + r;
        int klo = 1, khi = 0;
        float lse2 = INFINITY, dl = 0.f;
        if (r < rows) {
            window_bounds(qi, sq, sk, wl, wr, klo, khi);
            const int64_t tok = (int64_t)q_off + qi;
            lse2 = a.lse[(a.cu_q ? 0 : (int64_t)b * a.lse_sb) + (int64_t)h * a.lse_sh + tok * a.lse_ss] * kLog2e;
            dl = a.delta[((a.cu_q ? tok : (int64_t)b * a.sq + qi)) * a.hq + h];
        }
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dl, -dl);
        const float slope = (BIAS && a.alibi) ? a.alibi[(int64_t)b * a.alibi_sb + h] * kLog2e : 0.f;
        bool ok = true;
        uint32_t pr[32];                                     // P of the tile in flight (fp32 bits)
        // phase A: P = exp2(S * c - LSE) of tile t into registers
        auto phase_a = [&](int t) {
            const int sb = t & 1;
            const int c0 = (t_lo + t) * 128 + cg * 32;      // first key of this thread's 32 columns
            ok = mbar_wait(bar(G_S0 + sb), (t >> 1) & 1, abort_flag, err, 35);
            if (!ok) return;
            tc_fence_after();
            tmem_ld32(tmem + lane_base + COL_S + sb * 128 + cg * 32, pr);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(G_SA0 + sb));                    // the score buffer may be overwritten
            const bool inside = __all_sync(0xffffffffu, c0 >= klo && c0 + 31 <= khi);
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float2 x;
                float f0 = 1.f, f1 = 1.f;                     // d(capped score) / d(scaled score)
                if constexpr (BIAS) {
                    // scores -> their final log2-domain values as in the forward: softcap, then the alibi bias
                    float v0 = __uint_as_float(pr[i]), v1 = __uint_as_float(pr[i + 1]);
                    if (a.softcap > 0.f) {
                        const float t0 = 1.f - __fdividef(2.f, 1.f + ex2_approx(v0 * a.cap_in2));
                        const float t1 = 1.f - __fdividef(2.f, 1.f + ex2_approx(v1 * a.cap_in2));
                        v0 = a.cap_out * t0; v1 = a.cap_out * t1;
                        f0 = 1.f - t0 * t0; f1 = 1.f - t1 * t1;
                    } else {
                        v0 *= a.scale_log2; v1 *= a.scale_log2;
                    }
                    const float rel = (float)(qi + sk - sq - (c0 + i));
                    x = make_float2(v0 - slope * fabsf(rel) - lse2, v1 - slope * fabsf(rel - 1.f) - lse2);
                } else {
                    x = fma2(make_float2(__uint_as_float(pr[i]), __uint_as_float(pr[i + 1])), sc2, nl2);
                }
                float2 p = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                if (!inside) {
                    const int col = c0 + i;
                    p.x = (col >= klo && col <= khi) ? p.x : 0.f;
                    p.y = (col + 1 >= klo && col + 1 <= khi) ? p.y : 0.f;
                }
                pr[i] = __float_as_uint(p.x * f0);          // kept for phase B: P times the softcap derivative
                pr[i + 1] = __float_as_uint(p.y * f1);
            }
        };
        phase_a(0);
        for (int t = 0; t < ntiles && ok; ++t) {
            // phase B: dS = P * (dP - delta), rounded, over dP's own columns
            ok = mbar_wait(bar(G_DP), t & 1, abort_flag, err, 38);
            if (!ok) break;
            tc_fence_after();
            uint32_t dr[32], lo8[8], hi8[8];
            tmem_ld32(tmem + lane_base + COL_DP + cg * 32, dr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float2 ds = mul2(make_float2(__uint_as_float(pr[i]), __uint_as_float(pr[i + 1])),
                                       add2(make_float2(__uint_as_float(dr[i]), __uint_as_float(dr[i + 1])), nd2));
                const uint32_t w = Elem<T>::pack(ds.x, ds.y);
                if (i < 16) lo8[i / 2] = w; else hi8[(i - 16) / 2] = w;
            }
            // each group of 16 keys (one K step of the dQ MMA) sits in 8 columns at a stride of 16, inside the columns
            // this thread has just read
            tmem_st8(tmem + lane_base + COL_DP + cg * 32, lo8);
            tmem_st8(tmem + lane_base + COL_DP + cg * 32 + 16, hi8);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(G_DS));
            if (t + 1 < ntiles) phase_a(t + 1);
        }
        if (ok) ok = mbar_wait(bar(G_ACC), 0, abort_flag, err, 36);
        if (ok) {
            tc_fence_after();
            // each group of four warps writes 32 columns of its row (groups beyond D / 32 have nothing to write)
            T* row = dqb + (int64_t)r * a.dq_ss;
            if (cg < D / 32) {
                uint32_t acc[32];
                tmem_ld32(tmem + lane_base + COL_DQ + cg * 32, acc);
                tmem_wait_ld();
                if (r < rows) store_row_scaled<T>(row + cg * 32, acc, a.scale, a.d - cg * 32);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 16) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------------
// dQ from stored dS^T tiles: dQ = scale * sum over key blocks of dS K, one GEMM a tile.  The dK/dV kernel has
// written every (key block, query block) tile it visited; this kernel visits exactly the same pairs (it derives its
// key blocks from the dK/dV kernel's rule), streams dS^T and K tiles through a three-stage TMA ring and multiplies.
// No element-wise work, no exponentials: HBM-bound on reading the dS^T tiles once.
//   warp 0 TMA producer, warp 1 MMA issuer (also owns the tensor memory), warps 2-5 epilogue (thread = query row)
// ------------------------------------------------------------------------------------------------------
enum { H_KF0 = 0, H_KF1, H_KF2, H_KE0, H_KE1, H_KE2, H_ACC, H_COUNT };

template <typename T, int D>
__global__ void __launch_bounds__(192, 1) bwd_dq_from_ds_sm100_kernel(const __grid_constant__ Sm100BwdArgs a) {
    using L = BwdSm100Smem<D>;
    constexpr int NSUB = D / 64;
    constexpr int kStage = 2 * L::kSub + L::kTileB;          // dS^T tile (128 x 128) + K tile (128 x D)
    constexpr uint32_t TMEM_COLS = D <= 64 ? 64 : 128;
    constexpr int FMT = Elem<T>::kDtype == FA_BF16 ? 1 : 0;
    // M = 128 queries, N = D, K = keys; both operands are read "across" their tiles: A = dS^T tile [key][query]
    // (query-contiguous), B = K tile [key][dim] (dim-contiguous)
    constexpr uint32_t IDESC = umma_idesc(FMT, 128, D, 1, 1);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* sgen = smem_raw + (sbase - smem_addr(smem_raw));
    const uint32_t bars = sbase + 3 * kStage;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + 3 * kStage + 8 * H_COUNT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + 3 * kStage + 8 * H_COUNT + 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pair = blockIdx.z * a.chunk_q + blockIdx.x;    // grid order as in the dK/dV kernel, over (batch entry, head) pairs
    if (pair >= a.b * a.hq) return;
    const int b = pair / a.hq, h = pair % a.hq;
    const int mblk = gridDim.y - 1 - blockIdx.y;
    const int sq = a.sq, sk = a.sk;
    const int m0 = mblk * 128;
    if (m0 >= sq) return;
    if (g_bwd_sm100_error) return;
    const int hk = h / (a.hq / a.hkv);
    const int wl = a.wl, wr = a.causal ? 0 : a.wr;
    const int diff = sk - sq;
    const int rows = min(128, sq - m0);
    // key blocks whose dK/dV CTA walked this query block (the rule of bwd_dkdv_sm100_kernel); they form one range
    int t_lo = a.nkb, t_hi = 0;
    for (int n = 0; n < a.nkb; ++n) {
        const int n0 = n * 128, krows = min(128, sk - n0);
        int i_lo = 0, i_hi = sq - 1;
        if (wr >= 0) i_lo = max(0, n0 - diff - wr);
        if (wl >= 0) i_hi = min(sq - 1, n0 + krows - 1 + wl - diff);
        const int mb_lo = i_lo / 128, mb_hi = i_hi >= i_lo ? i_hi / 128 + 1 : mb_lo;
        if (mblk >= mb_lo && mblk < mb_hi) { t_lo = min(t_lo, n); t_hi = max(t_hi, n + 1); }
    }
    const int ntiles = max(0, t_hi - t_lo);
    T* dqb = reinterpret_cast<T*>(a.dq) + (int64_t)b * a.dq_sb + (int64_t)m0 * a.dq_ss + (int64_t)h * a.dq_sh;
    if (ntiles == 0) {
        if (tid < rows) {
            const uint4 z = make_uint4(0, 0, 0, 0);
            T* row = dqb + (int64_t)tid * a.dq_ss;
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                if (c * 8 < a.d) reinterpret_cast<uint4*>(row)[c] = z;      // the call's head dim, not the kernel's padded one
        }
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < H_COUNT; ++i) mbar_init(bar(i), 1u);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(smem_addr(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int* err = &g_bwd_sm100_error;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&a.tk);
            bool ok = true;
            for (int j = 0; j < ntiles && ok; ++j) {
                const int st = j % 3;
                if (j >= 3) ok = mbar_wait(bar(H_KE0 + st), (j / 3 - 1) & 1, abort_flag, err, 51);
                if (!ok) break;
                const int n = t_lo + j;
                const int64_t tile = (((int64_t)b * a.hq + h) * a.nkb + n) * a.nqb + mblk;
                mbar_expect_tx(bar(H_KF0 + st), kStage);
                const uint32_t s0 = sbase + st * kStage;
                bulk_load_1d(s0, reinterpret_cast<const unsigned char*>(a.ds_tiles) + tile * (128 * 128 * 2), 2 * L::kSub, bar(H_KF0 + st));
#pragma unroll
                for (int c = 0; c < NSUB; ++c) tma_load_4d(s0 + 2 * L::kSub + c * L::kSub, &a.tk, bar(H_KF0 + st), c * 64, hk, n * 128, b);
            }
        }
    } else if (warp == 1) {
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int st = j % 3;
            ok = mbar_wait(bar(H_KF0 + st), (j / 3) & 1, abort_flag, err, 52);
            if (!ok) break;
            tc_fence_after();
            const uint32_t s0 = sbase + st * kStage;
            // A: the dS^T tile as stored ([chunk][key][16 B], no swizzle): 8 keys of a chunk are 128 contiguous bytes,
            // chunks are 2048 bytes apart, a K step of 16 keys is 256 bytes further on; B: the K tile (128-byte swizzle)
            const uint64_t dA = umma_desc_mn_noswizzle(s0, 128, 2048), dB = umma_desc(s0 + 2 * L::kSub, L::kSub, 1024);
            umma_ss_group4<0, 16, 32, 48, 0, 128, 256, 384>(tmem, dA, dB, IDESC, j > 0);
            umma_ss_group4<64, 80, 96, 112, 512, 640, 768, 896>(tmem, dA, dB, IDESC, 1);
            umma_commit_w(bar(H_KE0 + st));
        }
        if (ok) umma_commit_w(bar(H_ACC));
    } else {
        // Rows of tiles past the last key hold zeros (their probabilities are zero), so nothing needs masking here.
        const int r = (warp & 3) * 32 + lane;               // warps 2..5 cover the four lane quarters 2,3,0,1
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        if (mbar_wait(bar(H_ACC), 0, abort_flag, err, 53)) {
            tc_fence_after();
            T* row = dqb + (int64_t)r * a.dq_ss;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t acc[32];
                tmem_ld32(tmem + lane_base + c * 32, acc);
                tmem_wait_ld();
                if (r < rows) store_row_scaled<T>(row + c * 32, acc, a.scale, a.d - c * 32);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------------
// delta[row] = sum_d O[row, d] * dO[row, d].  HBM-bound: D/8 lanes share a row with one 16-byte load each of O and
// dO.  One row per thread and pass (kU = 1) keeps the kernel at 32 registers, i.e. eight blocks an SM: measured
// 54 us for 268 MB against 91 us with four rows in flight per thread (80 registers, three blocks an SM).
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_delta_sm100_kernel(const fa_bwd_params p, float* delta) {
    constexpr int LPR = D / 8, RPW = 32 / LPR, kU = 1;
    const int lane = threadIdx.x & 31, sub = lane / LPR, c = (lane % LPR) * 8;
    const int64_t toks = p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq;
    const int64_t rows = toks * p.hq;
    const int64_t warp_g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t step = (int64_t)gridDim.x * (blockDim.x >> 5) * (kU * RPW);
    const T* o_base = reinterpret_cast<const T*>(p.o.ptr);
    const T* d_base = reinterpret_cast<const T*>(p.dout.ptr);
    const bool small = rows < (1ll << 31);
    for (int64_t base = warp_g * (kU * RPW); base < rows; base += step) {
        uint4 ov[kU], dv[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t row = base + u * RPW + sub;
            ov[u] = make_uint4(0, 0, 0, 0);
            dv[u] = make_uint4(0, 0, 0, 0);
            if (row < rows && c < p.d) {
                int64_t tok, bb = 0, i;
                int h;
                if (small) { const uint32_t r32 = (uint32_t)row; tok = r32 / (uint32_t)p.hq; h = (int)(r32 % (uint32_t)p.hq); }
                else { tok = row / p.hq; h = (int)(row % p.hq); }
                i = tok;
                if (!p.cu_seqlens_q) {
                    if (small) { bb = (uint32_t)tok / (uint32_t)p.sq; i = (uint32_t)tok % (uint32_t)p.sq; }
                    else { bb = tok / p.sq; i = tok % p.sq; }
                }
                const int64_t ooff = bb * p.o.stride_b + i * p.o.stride_s + (int64_t)h * p.o.stride_h;
                const int64_t doff = bb * p.dout.stride_b + i * p.dout.stride_s + (int64_t)h * p.dout.stride_h;
                ov[u] = __ldg(reinterpret_cast<const uint4*>(o_base + ooff + c));
                dv[u] = __ldg(reinterpret_cast<const uint4*>(d_base + doff + c));
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const T* oe = reinterpret_cast<const T*>(&ov[u]);
            const T* de = reinterpret_cast<const T*>(&dv[u]);
            float acc = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc += Elem<T>::to_float(oe[e]) * Elem<T>::to_float(de[e]);
#pragma unroll
            for (int sft = LPR / 2; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
            const int64_t row = base + u * RPW + sub;
            if (c == 0 && row < rows) delta[row] = acc;
        }
    }
}

// 1 (default): dense calls hand dS^T from the dK/dV kernel to a one-GEMM dQ kernel through the workspace;
// 0: the dQ kernel always recomputes S and dP (fa_debug_set key 7)
static std::atomic<int> g_ds_spill{1};
void bwd_sm100_set_ds_spill(int v) { g_ds_spill = v; }

static size_t ds_tiles_bytes(const fa_bwd_params& p);

bool bwd_sm100_supported(const fa_bwd_params& p) {
    if (p.d != p.dv_dim || p.d % 8 != 0 || p.d <= 0 || p.d > 128) return false;       // any head dim up to 128: padded to 64 / 128
    if ((p.sq + 127) / 128 > 65535 || (p.sk + 127) / 128 > 65535) return false;       // blocks stay inside a grid dimension
    if (!(p.scale > 0.f)) return false;

    if ((p.cu_seqlens_q != nullptr) != (p.cu_seqlens_k != nullptr)) return false;
    if (p.sq <= 0 || p.sk <= 0) return false;
    if (p.cu_seqlens_q && (p.total_q <= 0 || p.total_k <= 0)) return false;
    const fa_tensor* ts[4] = {&p.q, &p.k, &p.v, &p.dout};
    for (const fa_tensor* t : ts) {
        if (t->stride_h <= 0 || t->stride_s <= 0) return false;
        if (!p.cu_seqlens_q && p.b > 1 && t->stride_b <= 0) return false;
    }
    return tensor_map_encoder_available();
}

// The dK/dV kernel can hand its dS^T tiles to the dQ kernel through the workspace (then the backward executes the
// algorithm's five GEMMs a tile pair instead of seven): dense calls whose tiles fit into this many bytes.
constexpr size_t kDsTileBytes = 128 * 128 * 2;
constexpr size_t kDsWorkspaceLimit = (size_t)6 << 30;
static size_t ds_tiles_bytes(const fa_bwd_params& p) {
    if (p.cu_seqlens_q || p.cu_seqlens_k || p.b <= 0) return 0;
    const size_t tiles = (size_t)p.b * p.hq * ((p.sk + 127) / 128) * ((p.sq + 127) / 128);
    const size_t bytes = tiles * kDsTileBytes;
    return bytes <= kDsWorkspaceLimit ? bytes : 0;
}
static size_t delta_bytes(const fa_bwd_params& p) { return (bwd_generic_workspace(p) + 255) & ~(size_t)255; }

size_t bwd_sm100_workspace(const fa_bwd_params& p) { return delta_bytes(p) + ds_tiles_bytes(p); }

template <typename T, int D>
static int launch_bwd_sm100_t(const fa_bwd_params& p, Sm100BwdArgs& a, float* delta, cudaStream_t st) {
    const int64_t toks = p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq;
    const int64_t rows = toks * p.hq;
    {
        constexpr int kRowsPerBlock = 8 * 1 * (32 / (D / 8));      // warps x rows in flight x rows per warp pass
        const int64_t want = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
        const unsigned blocks = (unsigned)(want < 148 * 16 ? (want < 1 ? 1 : want) : 148 * 16);
        bwd_delta_sm100_kernel<T, D><<<blocks, 256, 0, st>>>(p, delta);
    }
    mark_kernel(st);
    const bool bias = p.softcap > 0.f || p.alibi_slopes;
    auto k1 = bias ? bwd_dkdv_sm100_kernel<T, D, true> : bwd_dkdv_sm100_kernel<T, D, false>;
    auto k2 = bias ? bwd_dq_sm100_kernel<T, D, true> : bwd_dq_sm100_kernel<T, D, false>;
    const int smem = BwdSm100Smem<D>::kBytes + 1024;
    if (int e = cuda_ok(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute")) return e;
    if (a.ds_tiles) {
        // five-GEMM path: the dQ kernel consumes the dS^T tiles the dK/dV kernel leaves, so it runs after it
        auto k3 = bwd_dq_from_ds_sm100_kernel<T, D>;
        const int smem3 = 3 * (2 * BwdSm100Smem<D>::kSub + BwdSm100Smem<D>::kTileB) + 256 + 1024;
        if (int e = cuda_ok(cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, smem3), "cudaFuncSetAttribute")) return e;
        const unsigned nk = (unsigned)((p.sk + 127) / 128), nq = (unsigned)((p.sq + 127) / 128);
        dim3 g1(a.chunk_kv, nk, (unsigned)(((int64_t)p.b * p.hkv + a.chunk_kv - 1) / a.chunk_kv));
        dim3 g3(a.chunk_q, nq, (unsigned)(((int64_t)p.b * p.hq + a.chunk_q - 1) / a.chunk_q));
        k1<<<g1, 608, smem, st>>>(a);
        mark_kernel(st);
        k3<<<g3, 192, smem3, st>>>(a);
        mark_kernel(st);
        return cuda_ok(cudaGetLastError(), "bwd_sm100 launch");
    }
    const int smem_dq = 7 * BwdSm100Smem<D>::kTileB + 256 + 1024;     // Q, dO, three K stages, two V stages, barriers
    if (int e = cuda_ok(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq), "cudaFuncSetAttribute")) return e;
    const unsigned nk = (unsigned)((p.sk + 127) / 128), nq = (unsigned)((p.sq + 127) / 128);
    dim3 g1(a.chunk_kv, nk, (unsigned)(((int64_t)p.b * p.hkv + a.chunk_kv - 1) / a.chunk_kv));
    dim3 g2(a.chunk_q, nq, (unsigned)(((int64_t)p.b * p.hq + a.chunk_q - 1) / a.chunk_q));
    // packed calls and calls beyond the workspace limit: the dQ kernel recomputes S and dP; both kernels on the
    // caller's stream, one after the other
    k1<<<g1, 608, smem, st>>>(a);
    mark_kernel(st);
    k2<<<g2, 608, smem_dq, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "bwd_sm100 launch");
}

int launch_bwd_sm100(const fa_bwd_params& p) {
    Sm100BwdArgs a;
    const bool packed = p.cu_seqlens_q != nullptr;
    const int64_t q_rows = packed ? p.total_q : p.sq, k_rows = packed ? p.total_k : p.sk;
    const int nb = packed ? 1 : p.b;
    auto bstride = [&](const fa_tensor& t, int64_t rows) { return packed || p.b == 1 ? rows * t.stride_s : t.stride_b; };
    if (int e = make_tile_map(&a.tq, p.dtype, p.q.ptr, p.d, p.hq, q_rows, nb, p.q.stride_h, p.q.stride_s, bstride(p.q, q_rows), 128)) return e;
    if (int e = make_tile_map(&a.tdo, p.dtype, p.dout.ptr, p.d, p.hq, q_rows, nb, p.dout.stride_h, p.dout.stride_s, bstride(p.dout, q_rows), 128)) return e;
    if (int e = make_tile_map(&a.tk, p.dtype, p.k.ptr, p.d, p.hkv, k_rows, nb, p.k.stride_h, p.k.stride_s, bstride(p.k, k_rows), 128)) return e;
    if (int e = make_tile_map(&a.tv, p.dtype, p.v.ptr, p.d, p.hkv, k_rows, nb, p.v.stride_h, p.v.stride_s, bstride(p.v, k_rows), 128)) return e;
    a.dq = p.dq.ptr; a.dk = p.dk.ptr; a.dv = p.dv.ptr;
    a.dq_sb = p.dq.stride_b; a.dq_ss = p.dq.stride_s; a.dq_sh = p.dq.stride_h;
    a.dk_sb = p.dk.stride_b; a.dk_ss = p.dk.stride_s; a.dk_sh = p.dk.stride_h;
    a.dv_sb = p.dv.stride_b; a.dv_ss = p.dv.stride_s; a.dv_sh = p.dv.stride_h;
    a.lse = p.lse; a.lse_sb = p.lse_stride_b; a.lse_sh = p.lse_stride_h; a.lse_ss = p.lse_stride_s;
    a.delta = reinterpret_cast<const float*>(p.workspace);
    a.ds_tiles = nullptr; a.nkb = (p.sk + 127) / 128; a.nqb = (p.sq + 127) / 128;
    if (g_ds_spill && ds_tiles_bytes(p) > 0 && p.workspace_bytes >= delta_bytes(p) + ds_tiles_bytes(p)) {
        a.ds_tiles = reinterpret_cast<unsigned char*>(p.workspace) + delta_bytes(p);
    }
    a.cu_q = p.cu_seqlens_q; a.cu_k = p.cu_seqlens_k;
    a.b = p.b; a.sq = p.sq; a.sk = p.sk; a.hq = p.hq; a.hkv = p.hkv; a.d = p.d;
    // a dK/dV chunk streams the Q and dO of its pairs' query groups, a dQ chunk the K (and V) of its pairs
    a.chunk_kv = grid_chunk((int64_t)p.b * p.hkv, (int64_t)(p.hq / p.hkv) * p.sq * p.d * 4);
    a.chunk_q = grid_chunk((int64_t)p.b * p.hq, (int64_t)p.sk * p.d * 4);
    a.scale = p.scale; a.scale_log2 = p.scale * kLog2e;
    a.softcap = p.softcap; a.cap_in2 = p.softcap > 0.f ? 2.f * kLog2e * p.scale / p.softcap : 0.f; a.cap_out = p.softcap * kLog2e;
    a.alibi = p.alibi_slopes; a.alibi_sb = p.alibi_stride_b;
    a.causal = p.causal; a.wl = p.window_left; a.wr = p.window_right;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    float* delta = reinterpret_cast<float*>(p.workspace);
    note_kernel(a.ds_tiles ? "sm100_tcgen05_bwd_5gemm" : "sm100_tcgen05_bwd");
    if (p.dtype == FA_F16) return p.d <= 64 ? launch_bwd_sm100_t<__half, 64>(p, a, delta, st) : launch_bwd_sm100_t<__half, 128>(p, a, delta, st);
    return p.d <= 64 ? launch_bwd_sm100_t<__nv_bfloat16, 64>(p, a, delta, st) : launch_bwd_sm100_t<__nv_bfloat16, 128>(p, a, delta, st);
}

}  // namespace fa
