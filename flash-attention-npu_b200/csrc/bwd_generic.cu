// General backward attention kernels (mma.sync tensor cores).
//
// Three launches, no atomics, fixed accumulation order (bitwise reproducible):
//   1. delta:  D[row] = sum_d dO*O                      (fag_epilogue_sfmg.hpp:284-286)
//   2. dK/dV:  one CTA per (KV block, KV head, batch) walks the query blocks of every head of
//              the group: S = QK^T, dP = dO V^T, P = exp(S - LSE), dS = P o (dP - D);
//              dV += P^T dO, dK += dS^T Q               (fag_kernel.cpp:400-465, fag_epilogue_op.hpp
//              :1287-1322, :1394, :1447-1480), GQA heads summed in registers
//              (tests/fa_small_op_golden.py:91-101).
//   3. dQ:     one CTA per (query block, head, batch) walks the KV blocks: recompute dS,
//              dQ += dS K.  dQ and dK are multiplied by the softmax scale at the end
//              (fag_epilogue_post.hpp:149, :177).
// P and dS are rounded to the input type before the second GEMMs, as the reference does.
#include "fa_utils.cuh"
#include "fa_internal.h"

namespace fa {

template <int PITCH>
__device__ __forceinline__ uint32_t swzp(int row, int chunk) {
    if constexpr (PITCH >= 128) return swz<PITCH>(row, chunk);
    else return static_cast<uint32_t>(row * PITCH + ((chunk ^ ((row >> 1) & 3)) << 4));
}

struct BwdSeq {
    int q_off, k_off, sq, sk;
};
__device__ __forceinline__ BwdSeq bwd_seq(const fa_bwd_params& p, int b) {
    BwdSeq s{0, 0, p.sq, p.sk};
    if (p.cu_seqlens_q) { s.q_off = p.cu_seqlens_q[b]; s.sq = p.cu_seqlens_q[b + 1] - s.q_off; }
    if (p.cu_seqlens_k) { s.k_off = p.cu_seqlens_k[b]; s.sk = p.cu_seqlens_k[b + 1] - s.k_off; }
    return s;
}

// ---- 1. delta ---------------------------------------------------------------------------------
template <typename T>
__global__ void bwd_delta_kernel(const fa_bwd_params p, float* delta) {
    // one warp per (token, head); delta laid out [token][head]
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t toks = p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq;
    if (row >= toks * p.hq) return;
    const int lane = threadIdx.x & 31;
    const int64_t tok = row / p.hq;
    const int h = (int)(row % p.hq);
    int64_t ooff, doff;
    if (p.cu_seqlens_q) {
        ooff = tok * p.o.stride_s + (int64_t)h * p.o.stride_h;
        doff = tok * p.dout.stride_s + (int64_t)h * p.dout.stride_h;
    } else {
        const int64_t bb = tok / p.sq, i = tok % p.sq;
        ooff = bb * p.o.stride_b + i * p.o.stride_s + (int64_t)h * p.o.stride_h;
        doff = bb * p.dout.stride_b + i * p.dout.stride_s + (int64_t)h * p.dout.stride_h;
    }
    const T* o = reinterpret_cast<const T*>(p.o.ptr) + ooff;
    const T* d = reinterpret_cast<const T*>(p.dout.ptr) + doff;
    float acc = 0.f;
    for (int c = lane; c < p.dv_dim; c += 32) acc += Elem<T>::to_float(o[c]) * Elem<T>::to_float(d[c]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) delta[row] = acc;
}

// shared helper: rows of a (rows x HD) tile from a strided tensor, zero-filled out of range
template <typename T, int HD, int ROWS>
__device__ __forceinline__ void load_tile(unsigned char* dst, const T* base, int64_t row_stride, int first_row, int limit,
                                          int cols, int tid) {
    constexpr int PITCH = HD * 2, CHUNKS = HD / 8;
    for (int idx = tid; idx < ROWS * CHUNKS; idx += 128) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        const bool ok = first_row + r < limit && c * 8 < cols;
        cp_async16(smem_u32(dst) + swz<PITCH>(r, c), ok ? base + (int64_t)(first_row + r) * row_stride + c * 8 : base, ok ? 16 : 0);
    }
}

// ---- 2. dK / dV --------------------------------------------------------------------------------
template <typename T, int HD, int BN, int DSPLIT>
__global__ void __launch_bounds__(128) bwd_dkdv_kernel(const fa_bwd_params p, const float* __restrict__ delta) {
    constexpr int BM = 64;
    constexpr int PITCH = HD * 2;
    constexpr int PP = BN * 2;                       // pitch of the P / dS tiles
    constexpr int NW = BN / 16;                      // warps along the key dimension in the N-phase
    constexpr int DW = HD / DSPLIT;                  // head-dim columns per warp in the N-phase
    static_assert(NW * DSPLIT == 4, "four warps");
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sK = smem;
    unsigned char* sV = sK + BN * PITCH;
    unsigned char* sQ = sV + BN * PITCH;             // 2 stages
    unsigned char* sdO = sQ + 2 * BM * PITCH;        // 2 stages
    unsigned char* sP = sdO + 2 * BM * PITCH;
    unsigned char* sdS = sP + BM * PP;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, hk = blockIdx.y, n0 = blockIdx.x * BN;
    const BwdSeq sq_ = bwd_seq(p, b);
    const int sq = sq_.sq, sk = sq_.sk;
    if (n0 >= sk) return;
    const int G = p.hq / p.hkv;
    const int wl = p.window_left, wr = p.causal ? 0 : p.window_right;
    const int diff = sk - sq;

    const T* kbase = reinterpret_cast<const T*>(p.k.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.k.stride_b) + (int64_t)sq_.k_off * p.k.stride_s + (int64_t)hk * p.k.stride_h;
    const T* vbase = reinterpret_cast<const T*>(p.v.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.v.stride_b) + (int64_t)sq_.k_off * p.v.stride_s + (int64_t)hk * p.v.stride_h;
    load_tile<T, HD, BN>(sK, kbase, p.k.stride_s, n0, sk, p.d, tid);
    load_tile<T, HD, BN>(sV, vbase, p.v.stride_s, n0, sk, p.dv_dim, tid);

    // query rows that can see this key block
    int i_lo = 0, i_hi = sq - 1;
    if (wr >= 0) i_lo = max(0, n0 - diff - wr);
    if (wl >= 0) i_hi = min(sq - 1, n0 + BN - 1 + wl - diff);
    const int mb_lo = i_lo / BM, mb_hi = i_hi >= i_lo ? i_hi / BM + 1 : mb_lo;
    const int nmb = mb_hi - mb_lo;
    const int steps = nmb * G;

    auto load_q = [&](int step, int stage) {
        const int gi = step / nmb, mb = mb_lo + step % nmb;
        const int h = hk * G + gi;
        const T* qb = reinterpret_cast<const T*>(p.q.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.q.stride_b) + (int64_t)sq_.q_off * p.q.stride_s + (int64_t)h * p.q.stride_h;
        const T* db = reinterpret_cast<const T*>(p.dout.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.dout.stride_b) + (int64_t)sq_.q_off * p.dout.stride_s + (int64_t)h * p.dout.stride_h;
        load_tile<T, HD, BM>(sQ + stage * BM * PITCH, qb, p.q.stride_s, mb * BM, sq, p.d, tid);
        load_tile<T, HD, BM>(sdO + stage * BM * PITCH, db, p.dout.stride_s, mb * BM, sq, p.dv_dim, tid);
    };

    constexpr int NT = DW / 8;                       // accumulator n-tiles per warp
    float dk_acc[NT][4], dv_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        dk_acc[i][0] = dk_acc[i][1] = dk_acc[i][2] = dk_acc[i][3] = 0.f;
        dv_acc[i][0] = dv_acc[i][1] = dv_acc[i][2] = dv_acc[i][3] = 0.f;
    }
    if (steps > 0) load_q(0, 0);
    cp_async_commit();

    const float scale_log2 = p.scale * kLog2e;
    const bool has_cap = p.softcap > 0.f;
    const float cap_in = has_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    const int ksteps = ceil_div(p.d, 16), vsteps = ceil_div(p.dv_dim, 16);
    const int nw = warp % NW, dw = warp / NW;

    for (int step = 0; step < steps; ++step) {
        const int stage = step & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (step + 1 < steps) load_q(step + 1, stage ^ 1);
        cp_async_commit();
        const int gi = step / nmb, mb = mb_lo + step % nmb;
        const int h = hk * G + gi;
        const float slope = p.alibi_slopes ? p.alibi_slopes[(int64_t)b * p.alibi_stride_b + h] * kLog2e : 0.f;
        const uint32_t sQs = smem_u32(sQ) + stage * BM * PITCH, sdOs = smem_u32(sdO) + stage * BM * PITCH;

        // ---- M-phase: this warp owns query rows [16 warp, +16) ------------------------------
        float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            if (kk < ksteps) {
                uint32_t aq[4];
                ldmatrix_x4(aq[0], aq[1], aq[2], aq[3], sQs + swz<PITCH>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int n2 = 0; n2 < BN / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(sK) + swz<PITCH>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816<T>(s[2 * n2], aq, b0, b1);
                    mma16816<T>(s[2 * n2 + 1], aq, b2, b3);
                }
            }
            if (kk < vsteps) {
                uint32_t ad[4];
                ldmatrix_x4(ad[0], ad[1], ad[2], ad[3], sdOs + swz<PITCH>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int n2 = 0; n2 < BN / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(sV) + swz<PITCH>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816<T>(dp[2 * n2], ad, b0, b1);
                    mma16816<T>(dp[2 * n2 + 1], ad, b2, b3);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int i = mb * BM + warp * 16 + g + r * 8;
            const bool ok = i < sq;
            int lo = 1, hi = 0;
            float lse2 = INFINITY, dl = 0.f;
            const float rel = (float)(i + sk - sq);      // alibi: distance of key j is |rel - j|
            if (ok) {
                window_bounds(i, sq, sk, wl, wr, lo, hi);
                const int64_t tok = (int64_t)sq_.q_off + i;
                lse2 = p.lse[(p.cu_seqlens_q ? 0 : (int64_t)b * p.lse_stride_b) + (int64_t)h * p.lse_stride_h + tok * p.lse_stride_s] * kLog2e;
                dl = delta[((p.cu_seqlens_q ? tok : (int64_t)b * p.sq + i)) * p.hq + h];
            }
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = n0 + nt * 8 + 2 * t + e;
                    float x = s[nt][2 * r + e], fac = 1.f;
                    if (has_cap) { const float th = tanhf(x * cap_in); x = cap_out * th; fac = 1.f - th * th; }
                    else x *= scale_log2;
                    if (p.alibi_slopes) x -= slope * fabsf(rel - (float)col);
                    const float pr = (col >= lo && col <= hi) ? exp2f(x - lse2) : 0.f;
                    s[nt][2 * r + e] = pr;
                    dp[nt][2 * r + e] = pr * (dp[nt][2 * r + e] - dl) * fac;
                }
                const int row = warp * 16 + g + r * 8;
                *reinterpret_cast<uint32_t*>(sP + swzp<PP>(row, nt) + t * 4) = Elem<T>::pack(s[nt][2 * r], s[nt][2 * r + 1]);
                *reinterpret_cast<uint32_t*>(sdS + swzp<PP>(row, nt) + t * 4) = Elem<T>::pack(dp[nt][2 * r], dp[nt][2 * r + 1]);
            }
        }
        __syncthreads();

        // ---- N-phase: this warp owns keys [16 nw, +16) and head-dim columns [DW dw, +DW) ------
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
            uint32_t ap[4], as_[4];
            const int mrow = kk * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int nch = nw * 2 + ((lane >> 3) & 1);
            ldmatrix_x4_trans(ap[0], ap[1], ap[2], ap[3], smem_u32(sP) + swzp<PP>(mrow, nch));
            ldmatrix_x4_trans(as_[0], as_[1], as_[2], as_[3], smem_u32(sdS) + swzp<PP>(mrow, nch));
            const int brow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
            for (int d2 = 0; d2 < DW / 16; ++d2) {
                const int ch = (dw * DW) / 8 + d2 * 2 + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                if (dw * DW + d2 * 16 < p.dv_dim) {
                    ldmatrix_x4_trans(b0, b1, b2, b3, sdOs + swz<PITCH>(brow, ch));
                    mma16816<T>(dv_acc[2 * d2], ap, b0, b1);
                    mma16816<T>(dv_acc[2 * d2 + 1], ap, b2, b3);
                }
                if (dw * DW + d2 * 16 < p.d) {
                    ldmatrix_x4_trans(b0, b1, b2, b3, sQs + swz<PITCH>(brow, ch));
                    mma16816<T>(dk_acc[2 * d2], as_, b0, b1);
                    mma16816<T>(dk_acc[2 * d2 + 1], as_, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- write dK (x scale) and dV -----------------------------------------------------------------
    T* dkb = reinterpret_cast<T*>(p.dk.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.dk.stride_b) + (int64_t)sq_.k_off * p.dk.stride_s + (int64_t)hk * p.dk.stride_h;
    T* dvb = reinterpret_cast<T*>(p.dv.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.dv.stride_b) + (int64_t)sq_.k_off * p.dv.stride_s + (int64_t)hk * p.dv.stride_h;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int n = n0 + nw * 16 + g + r * 8;
        if (n >= sk) continue;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int col = dw * DW + i * 8 + 2 * t;
            if (col < p.d) *reinterpret_cast<uint32_t*>(dkb + (int64_t)n * p.dk.stride_s + col) = Elem<T>::pack(dk_acc[i][2 * r] * p.scale, dk_acc[i][2 * r + 1] * p.scale);
            if (col < p.dv_dim) *reinterpret_cast<uint32_t*>(dvb + (int64_t)n * p.dv.stride_s + col) = Elem<T>::pack(dv_acc[i][2 * r], dv_acc[i][2 * r + 1]);
        }
    }
}

// ---- 3. dQ ----------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(128) bwd_dq_kernel(const fa_bwd_params p, const float* __restrict__ delta) {
    constexpr int BM = 64, BN = 64;
    constexpr int PITCH = HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sQ = smem;
    unsigned char* sdO = sQ + BM * PITCH;
    unsigned char* sK = sdO + BM * PITCH;            // 2 stages
    unsigned char* sV = sK + 2 * BN * PITCH;         // 2 stages

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, h = blockIdx.y, m0 = blockIdx.x * BM;
    const BwdSeq sq_ = bwd_seq(p, b);
    const int sq = sq_.sq, sk = sq_.sk;
    if (m0 >= sq) return;
    const int hk = h / (p.hq / p.hkv);
    const int wl = p.window_left, wr = p.causal ? 0 : p.window_right;

    const T* qb = reinterpret_cast<const T*>(p.q.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.q.stride_b) + (int64_t)sq_.q_off * p.q.stride_s + (int64_t)h * p.q.stride_h;
    const T* db = reinterpret_cast<const T*>(p.dout.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.dout.stride_b) + (int64_t)sq_.q_off * p.dout.stride_s + (int64_t)h * p.dout.stride_h;
    const T* kbase = reinterpret_cast<const T*>(p.k.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.k.stride_b) + (int64_t)sq_.k_off * p.k.stride_s + (int64_t)hk * p.k.stride_h;
    const T* vbase = reinterpret_cast<const T*>(p.v.ptr) + (p.cu_seqlens_k ? 0 : (int64_t)b * p.v.stride_b) + (int64_t)sq_.k_off * p.v.stride_s + (int64_t)hk * p.v.stride_h;
    load_tile<T, HD, BM>(sQ, qb, p.q.stride_s, m0, sq, p.d, tid);
    load_tile<T, HD, BM>(sdO, db, p.dout.stride_s, m0, sq, p.dv_dim, tid);

    int nb_lo = 0, nb_hi = ceil_div(sk, BN);
    {
        int lo, hi, lo2, hi2;
        window_bounds(m0, sq, sk, wl, wr, lo, hi);
        window_bounds(min(sq, m0 + BM) - 1, sq, sk, wl, wr, lo2, hi2);
        nb_lo = max(nb_lo, lo / BN);
        nb_hi = hi2 < 0 ? nb_lo : min(nb_hi, hi2 / BN + 1);
    }
    auto load_kv = [&](int nb, int stage) {
        load_tile<T, HD, BN>(sK + stage * BN * PITCH, kbase, p.k.stride_s, nb * BN, sk, p.d, tid);
        load_tile<T, HD, BN>(sV + stage * BN * PITCH, vbase, p.v.stride_s, nb * BN, sk, p.dv_dim, tid);
    };
    if (nb_lo < nb_hi) load_kv(nb_lo, 0);
    cp_async_commit();

    int lo[2], hi[2];
    float lse2[2], dl[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = m0 + warp * 16 + g + r * 8;
        lo[r] = 1; hi[r] = 0; lse2[r] = INFINITY; dl[r] = 0.f;
        if (i < sq) {
            window_bounds(i, sq, sk, wl, wr, lo[r], hi[r]);
            const int64_t tok = (int64_t)sq_.q_off + i;
            lse2[r] = p.lse[(p.cu_seqlens_q ? 0 : (int64_t)b * p.lse_stride_b) + (int64_t)h * p.lse_stride_h + tok * p.lse_stride_s] * kLog2e;
            dl[r] = delta[((p.cu_seqlens_q ? tok : (int64_t)b * p.sq + i)) * p.hq + h];
        }
    }
    float dq_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { dq_acc[i][0] = dq_acc[i][1] = dq_acc[i][2] = dq_acc[i][3] = 0.f; }

    const float scale_log2 = p.scale * kLog2e;
    const bool has_cap = p.softcap > 0.f;
    const float cap_in = has_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    const float slope = p.alibi_slopes ? p.alibi_slopes[(int64_t)b * p.alibi_stride_b + h] * kLog2e : 0.f;
    const int ksteps = ceil_div(p.d, 16), vsteps = ceil_div(p.dv_dim, 16);

    for (int nb = nb_lo; nb < nb_hi; ++nb) {
        const int stage = (nb - nb_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (nb + 1 < nb_hi) load_kv(nb + 1, stage ^ 1);
        cp_async_commit();
        const uint32_t sKs = smem_u32(sK) + stage * BN * PITCH, sVs = smem_u32(sV) + stage * BN * PITCH;
        float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            if (kk < ksteps) {
                uint32_t aq[4];
                ldmatrix_x4(aq[0], aq[1], aq[2], aq[3], smem_u32(sQ) + swz<PITCH>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int n2 = 0; n2 < BN / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, sKs + swz<PITCH>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816<T>(s[2 * n2], aq, b0, b1);
                    mma16816<T>(s[2 * n2 + 1], aq, b2, b3);
                }
            }
            if (kk < vsteps) {
                uint32_t ad[4];
                ldmatrix_x4(ad[0], ad[1], ad[2], ad[3], smem_u32(sdO) + swz<PITCH>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
                for (int n2 = 0; n2 < BN / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, sVs + swz<PITCH>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816<T>(dp[2 * n2], ad, b0, b1);
                    mma16816<T>(dp[2 * n2 + 1], ad, b2, b3);
                }
            }
        }
        const int n0 = nb * BN;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = n0 + nt * 8 + 2 * t + e;
                    float x = s[nt][2 * r + e], fac = 1.f;
                    if (has_cap) { const float th = tanhf(x * cap_in); x = cap_out * th; fac = 1.f - th * th; }
                    else x *= scale_log2;
                    if (p.alibi_slopes) x -= slope * fabsf((float)(m0 + warp * 16 + g + r * 8 + sk - sq - col));
                    const float pr = (col >= lo[r] && col <= hi[r]) ? exp2f(x - lse2[r]) : 0.f;
                    dp[nt][2 * r + e] = pr * (dp[nt][2 * r + e] - dl[r]) * fac;
                }
            }
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = Elem<T>::pack(dp[2 * kk][0], dp[2 * kk][1]);
            a[1] = Elem<T>::pack(dp[2 * kk][2], dp[2 * kk][3]);
            a[2] = Elem<T>::pack(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
            a[3] = Elem<T>::pack(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < HD / 16; ++d2) {
                if (d2 < ksteps) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sKs + swz<PITCH>(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), d2 * 2 + (lane >> 4)));
                    mma16816<T>(dq_acc[2 * d2], a, b0, b1);
                    mma16816<T>(dq_acc[2 * d2 + 1], a, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    T* dqb = reinterpret_cast<T*>(p.dq.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.dq.stride_b) + (int64_t)sq_.q_off * p.dq.stride_s + (int64_t)h * p.dq.stride_h;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = m0 + warp * 16 + g + r * 8;
        if (i >= sq) continue;
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
            const int col = c * 8 + 2 * t;
            if (col < p.d) *reinterpret_cast<uint32_t*>(dqb + (int64_t)i * p.dq.stride_s + col) = Elem<T>::pack(dq_acc[c][2 * r] * p.scale, dq_acc[c][2 * r + 1] * p.scale);
        }
    }
}

size_t bwd_generic_workspace(const fa_bwd_params& p) {
    const int64_t toks = p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq;
    return (size_t)(toks * p.hq) * sizeof(float) + 256;
}

template <typename T, int HD, int BN, int DSPLIT>
static int launch_bwd_t(const fa_bwd_params& p, float* delta, cudaStream_t st) {
    const int64_t toks = p.cu_seqlens_q ? p.total_q : (int64_t)p.b * p.sq;
    const int64_t rows = toks * p.hq;
    if (rows > 0) { bwd_delta_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(p, delta); mark_kernel(st); }
    const size_t smem1 = (size_t)(2 * BN + 4 * 64) * HD * 2 + 2 * 64 * BN * 2;
    const size_t smem2 = (size_t)(2 * 64 + 4 * 64) * HD * 2;
    auto k1 = bwd_dkdv_kernel<T, HD, BN, DSPLIT>;
    auto k2 = bwd_dq_kernel<T, HD>;
    if (int e = cuda_ok(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1), "cudaFuncSetAttribute")) return e;
    if (int e = cuda_ok(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2), "cudaFuncSetAttribute")) return e;
    dim3 g1(ceil_div(p.sk, BN), p.hkv, p.b), g2(ceil_div(p.sq, 64), p.hq, p.b);
    if (g1.x && g1.y && g1.z) { k1<<<g1, 128, smem1, st>>>(p, delta); mark_kernel(st); }
    if (g2.x && g2.y && g2.z) { k2<<<g2, 128, smem2, st>>>(p, delta); mark_kernel(st); }
    return cuda_ok(cudaGetLastError(), "bwd_generic launch");
}

int launch_bwd_generic(const fa_bwd_params& p) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    float* delta = reinterpret_cast<float*>(p.workspace);
    const int dmax = p.d > p.dv_dim ? p.d : p.dv_dim;
    note_kernel("generic_mma_bwd");
    if (p.dtype == FA_F16) {
        if (dmax <= 64) return launch_bwd_t<__half, 64, 64, 1>(p, delta, st);
        if (dmax <= 128) return launch_bwd_t<__half, 128, 64, 1>(p, delta, st);
        return launch_bwd_t<__half, 256, 32, 2>(p, delta, st);
    }
    if (dmax <= 64) return launch_bwd_t<__nv_bfloat16, 64, 64, 1>(p, delta, st);
    if (dmax <= 128) return launch_bwd_t<__nv_bfloat16, 128, 64, 1>(p, delta, st);
    return launch_bwd_t<__nv_bfloat16, 256, 32, 2>(p, delta, st);
}

}  // namespace fa
