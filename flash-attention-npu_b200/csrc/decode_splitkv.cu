// Split-KV decode kernel for the KV-cache forward: HBM-bound, built to keep bytes in flight.
//
// Used when all query rows of one KV head fit one 16-row MMA tile (seqlen_q x group <= 16).
// A CTA has four warps; warp w serves KV head 4 y + w over the same token range, so the CTA
// streams adjacent 256-byte rows of the cache ((blocks, page, Hkv, D) layout) at the same time.
// Every warp runs its own cp.async pipeline (32-token tiles, three stages, 16-byte vector loads
// addressed through the block table), its own online softmax and its own P.V: there is no
// CTA-wide barrier in the loop.  The query group of the KV head is stacked into the M dimension
// (row = q_pos * group + head_in_group) like the reference does for decode (GetQNBlockTile,
// kernel_common.hpp:85-92; mha_fwd_kvcache.cpp:541).  Each (sequence, KV head, split) leaves a
// normalised fp32 partial O and its LSE (rescale_o.hpp:498-563) unless there is a single split,
// in which case the output is written directly.
#include "fa_utils.cuh"
#include "fa_internal.h"
#include "sm100_ptx.cuh"
#include <atomic>

namespace fa {

struct DecodeArgs {
    fa_fwd_params p;
    int nsplit;
    int tokens_per_split;
    float* o_part;
    float* lse_part;
    const int32_t* meta;          // scheduler-metadata blob or null
};

// Keys per split for sequence b: the blob's per-sequence figure when the blob was built for this launch (same batch
// and split count) and for the length the kernel itself reads now; otherwise the host's uniform plan.  A blob of
// another call shape, or one that has gone stale because the lengths moved on, is therefore ignored, never trusted.
__device__ __forceinline__ int keys_per_split(const DecodeArgs& a, int b, int sk) {
    const int32_t* m = a.meta;
    if (!m || m[0] != kSchedMagic || m[1] != a.p.b || m[2] != a.nsplit) return a.tokens_per_split;
    const int32_t* s = m + kSchedHeaderInts + kSchedSeqInts * b;
    if (s[0] != sk || s[3] <= 0 || (long long)s[3] * a.nsplit < sk) return a.tokens_per_split;
    return s[3];
}

constexpr int kDecStages = 3;

template <typename T, int HD>
__global__ void __launch_bounds__(128) decode_splitkv_kernel(const DecodeArgs a) {
    constexpr int kDecTile = HD > 128 ? 16 : 32;                 // tokens per pipeline stage
    constexpr int PITCH = HD * 2;
    constexpr int CHUNKS = HD / 8;
    constexpr int TILE_BYTES = kDecTile * PITCH;                 // one K or V tile
    const fa_fwd_params& p = a.p;
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, b = blockIdx.z;
    const int hk = blockIdx.y * 4 + warp;
    if (hk >= p.hkv) return;
    unsigned char* wsm = smem + warp * (2 * kDecStages * TILE_BYTES);
    const uint32_t sKw = smem_u32(wsm), sVw = sKw + kDecStages * TILE_BYTES;

    const int G = p.hq / p.hkv;
    int q_off = 0, sq = p.sq, sk = p.sk;
    if (p.cu_seqlens_q) { q_off = p.cu_seqlens_q[b]; sq = p.cu_seqlens_q[b + 1] - q_off; }
    if (p.seqused_k) sk = cache_len(p, b);
    const int kb = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
    const int rows_total = sq * G;
    if (rows_total <= 0) return;
    const int wl = p.window_left, wr = p.causal ? 0 : p.window_right;
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    const int tps = keys_per_split(a, b, sk);

    // token range of this split, intersected with what any row can see
    int lo_any, hi_any, tmp;
    window_bounds(0, sq, sk, wl, wr, lo_any, tmp);
    window_bounds(sq - 1, sq, sk, wl, wr, tmp, hi_any);
    int t_begin = max(max(rb, lo_any), rb + split * tps);
    int t_end = min(min(re, hi_any + 1), rb + (split + 1) * tps);
    t_begin = t_begin / kDecTile * kDecTile;

    int vrow[2], qpos[2], head[2], klo[2], khi[2];
    float slope[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        vrow[r] = g + r * 8;
        const bool ok = vrow[r] < rows_total;
        qpos[r] = ok ? vrow[r] / G : 0;
        head[r] = hk * G + (ok ? vrow[r] % G : 0);
        klo[r] = 1; khi[r] = 0;
        if (ok) {
            window_bounds(qpos[r], sq, sk, wl, wr, klo[r], khi[r]);
            klo[r] = max(max(klo[r], rb), rb + split * tps);
            khi[r] = min(min(khi[r], re - 1), rb + (split + 1) * tps - 1);
        }
        slope[r] = p.alibi_slopes ? p.alibi_slopes[(int64_t)b * p.alibi_stride_b + head[r]] * kLog2e : 0.f;
    }

    // ---- Q fragments (A operand) straight from global memory: rows g / g+8, columns 16 kk + 2t (+8) ----
    const T* qbase = reinterpret_cast<const T*>(p.q.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.q.stride_b);
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int col = kk * 16 + hf * 8 + 2 * t;
                uint32_t v = 0;
                if (vrow[r] < rows_total && col < p.d)
                    v = *reinterpret_cast<const uint32_t*>(qbase + (int64_t)(q_off + qpos[r]) * p.q.stride_s + (int64_t)head[r] * p.q.stride_h + col);
                qf[kk][hf * 2 + r] = v;
            }
        }
    }

    const T* kbase = reinterpret_cast<const T*>(p.k.ptr);
    const T* vbase = reinterpret_cast<const T*>(p.v.ptr);
    const int32_t* btab = p.block_table ? p.block_table + (int64_t)b * p.block_table_stride : nullptr;
    const bool page32 = btab && (p.page_size % kDecTile) == 0;

    auto load_tile = [&](int tok0, int stage) {
        int64_t kpage = 0, vpage = 0;
        if (page32) {
            const int blk = btab[tok0 / p.page_size];
            kpage = (int64_t)blk * p.k.stride_b;
            vpage = (int64_t)blk * p.v.stride_b;
        }
#pragma unroll
        for (int i = 0; i < kDecTile * CHUNKS / 32; ++i) {
            const int idx = i * 32 + lane;
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            const int tok = tok0 + r;
            const bool ok = tok < sk;
            int64_t koff = 0, voff = 0;
            if (ok) {
                if (page32) {
                    const int rin = tok % p.page_size;
                    koff = kpage + (int64_t)rin * p.k.stride_s;
                    voff = vpage + (int64_t)rin * p.v.stride_s;
                } else if (btab) {
                    const int blk = btab[tok / p.page_size], rin = tok % p.page_size;
                    koff = (int64_t)blk * p.k.stride_b + (int64_t)rin * p.k.stride_s;
                    voff = (int64_t)blk * p.v.stride_b + (int64_t)rin * p.v.stride_s;
                } else {
                    koff = (int64_t)kb * p.k.stride_b + (int64_t)tok * p.k.stride_s;
                    voff = (int64_t)kb * p.v.stride_b + (int64_t)tok * p.v.stride_s;
                }
                koff += (int64_t)hk * p.k.stride_h + c * 8;
                voff += (int64_t)hk * p.v.stride_h + c * 8;
            }
            const bool okk = ok && c * 8 < p.d, okv = ok && c * 8 < p.dv;
            cp_async16(sKw + stage * TILE_BYTES + swz<PITCH>(r, c), okk ? kbase + koff : kbase, okk ? 16 : 0);
            cp_async16(sVw + stage * TILE_BYTES + swz<PITCH>(r, c), okv ? vbase + voff : vbase, okv ? 16 : 0);
        }
    };

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};

    const int ntiles = t_end > t_begin ? (t_end - t_begin + kDecTile - 1) / kDecTile : 0;
#pragma unroll
    for (int s = 0; s < kDecStages - 1; ++s) {
        if (s < ntiles) load_tile(t_begin + s * kDecTile, s);
        cp_async_commit();
    }
    const float scale_log2 = p.scale * kLog2e;
    const bool has_cap = p.softcap > 0.f;
    const float cap_in = has_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    const int ksteps = ceil_div(p.d, 16), vsteps = ceil_div(p.dv, 16);

    for (int it = 0; it < ntiles; ++it) {
        const int stage = it % kDecStages;
        cp_async_wait<kDecStages - 2>();
        __syncwarp();
        if (it + kDecStages - 1 < ntiles) load_tile(t_begin + (it + kDecStages - 1) * kDecTile, (it + kDecStages - 1) % kDecStages);
        cp_async_commit();
        const uint32_t sKs = sKw + stage * TILE_BYTES, sVs = sVw + stage * TILE_BYTES;
        const int n0 = t_begin + it * kDecTile;
        float s[kDecTile / 8][4];
#pragma unroll
        for (int i = 0; i < kDecTile / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            if (kk < ksteps) {
#pragma unroll
                for (int n2 = 0; n2 < kDecTile / 16; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, sKs + swz<PITCH>(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    mma16816<T>(s[2 * n2], qf[kk], b0, b1);
                    mma16816<T>(s[2 * n2 + 1], qf[kk], b2, b3);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < kDecTile / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = n0 + nt * 8 + 2 * t + e;
                    float x = s[nt][2 * r + e];
                    x = has_cap ? cap_out * tanhf(x * cap_in) : x * scale_log2;
                    if (p.alibi_slopes) x -= slope[r] * fabsf((float)(qpos[r] + sk - sq - col));
                    x = (col >= klo[r] && col <= khi[r]) ? x : -INFINITY;
                    s[nt][2 * r + e] = x;
                    mx = fmaxf(mx, x);
                }
            }
            mx = quad_max(mx);
            const float m_new = fmaxf(m_i[r], mx);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            const float corr = exp2f(m_i[r] - m_safe);
            m_i[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < kDecTile / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pv = exp2f(s[nt][2 * r + e] - m_safe);
                    s[nt][2 * r + e] = pv;
                    sum += pv;
                }
            }
            l_i[r] = l_i[r] * corr + sum;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o_acc[i][2 * r] *= corr; o_acc[i][2 * r + 1] *= corr; }
        }
#pragma unroll
        for (int kk = 0; kk < kDecTile / 16; ++kk) {
            uint32_t ap[4];
            ap[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
            ap[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
            ap[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            ap[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < HD / 16; ++d2) {
                if (d2 < vsteps) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sVs + swz<PITCH>(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), d2 * 2 + (lane >> 4)));
                    mma16816<T>(o_acc[2 * d2], ap, b0, b1);
                    mma16816<T>(o_acc[2 * d2 + 1], ap, b2, b3);
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // ---- epilogue ---------------------------------------------------------------------------------------
    const bool to_part = a.o_part != nullptr;
    const int64_t rows_all = (p.cu_seqlens_q ? (int64_t)p.total_q : (int64_t)p.b * p.sq) * p.hq;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float l = quad_sum(l_i[r]);
        if (vrow[r] >= rows_total) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t tok = p.cu_seqlens_q ? (int64_t)q_off + qpos[r] : (int64_t)b * p.sq + qpos[r];
        if (to_part) {
            const int64_t row = tok * p.hq + head[r];
            float* dst = a.o_part + ((int64_t)split * rows_all + row) * p.dv;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const int col = i * 8 + 2 * t;
                if (col < p.dv) *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            }
            if (t == 0) a.lse_part[(int64_t)split * rows_all + row] = l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : -INFINITY;
        } else {
            T* dst = reinterpret_cast<T*>(p.o.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.o.stride_b) +
                     (int64_t)(q_off + qpos[r]) * p.o.stride_s + (int64_t)head[r] * p.o.stride_h;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const int col = i * 8 + 2 * t;
                if (col < p.dv) *reinterpret_cast<uint32_t*>(dst + col) = Elem<T>::pack(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            }
            if (t == 0 && p.lse)
                p.lse[(p.cu_seqlens_q ? 0 : (int64_t)b * p.lse_stride_b) + (int64_t)head[r] * p.lse_stride_h + ((int64_t)q_off + qpos[r]) * p.lse_stride_s] =
                    l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : INFINITY;
        }
    }
}


// -------------------------------------------------------------------------------------------------------
// The same kernel with the cache tiles brought in by TMA (cp.async.bulk.tensor, each copy to one CTA).
// 16-byte cp.async copies are tracked by the SM's load/store unit, which caps the bytes a warp can keep in
// flight far below what HBM3e needs; a bulk tensor copy of a (32 tokens x 64 dims) box is one request.
// Lane 0 of each warp arms the stage's mbarrier and issues the boxes, addressed by
// (dim, KV head, row in page, block id) for a paged cache or (dim, KV head, token, batch) for a dense one.
// Requires head dim 64/128/256 with d == dv and, for paged caches, a page size that is a multiple of the
// tile (32 tokens; 16 for head dim 256).
// -------------------------------------------------------------------------------------------------------
__device__ int g_decode_error = 0;

struct alignas(64) DecodeTmaArgs {
    CUtensorMap tk, tv;
    DecodeArgs d;
};

// WIDE = false: each of the four warps streams the keys of its own KV head and owns a private ring (up to 16 stacked
// query rows per KV head).  WIDE = true (17-64 stacked rows: several new tokens per step, or large GQA groups): the
// four warps take 16 rows each of ONE KV head and share one ring, filled by a fifth warp; every tile is fetched
// once per CTA, a stage is refilled when all four warps have arrived on its "empty" barrier.
constexpr int kDecWideStages = 6;
template <typename T, int HD, bool WIDE>
__global__ void __launch_bounds__(WIDE ? 160 : 128) decode_tma_kernel(const __grid_constant__ DecodeTmaArgs ta) {
    using namespace sm100;
    constexpr int TILE = HD > 128 ? 16 : 32;
    constexpr int NSUB = HD / 64;
    constexpr int SUB_BYTES = TILE * 128;
    constexpr int TILE_BYTES = NSUB * SUB_BYTES;
    constexpr int STAGES = WIDE ? kDecWideStages : kDecStages;
    constexpr int WARP_BYTES = 2 * STAGES * TILE_BYTES;
    const DecodeArgs& a = ta.d;
    const fa_fwd_params& p = a.p;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t sbase = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, b = blockIdx.z;
    const int hk = WIDE ? blockIdx.y : blockIdx.y * 4 + warp;
    if (hk >= p.hkv) return;
    const int row_base = WIDE ? warp * 16 : 0;
    const uint32_t sKw = sbase + (WIDE ? 0 : warp * WARP_BYTES), sVw = sKw + STAGES * TILE_BYTES;
    const uint32_t bars = sbase + (WIDE ? WARP_BYTES : 4 * WARP_BYTES + warp * 64);     // full[STAGES], then (WIDE) empty[STAGES]
    unsigned char* gen_base = smem_raw + (sbase - smem_addr(smem_raw));

    const int G = p.hq / p.hkv;
    int q_off = 0, sq = p.sq, sk = p.sk;
    if (p.cu_seqlens_q) { q_off = p.cu_seqlens_q[b]; sq = p.cu_seqlens_q[b + 1] - q_off; }
    if (p.seqused_k) sk = cache_len(p, b);
    const int kb = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
    const int rows_total = sq * G;
    if (rows_total <= 0) return;
    const int wl = p.window_left, wr = p.causal ? 0 : p.window_right;
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    const int tps = keys_per_split(a, b, sk);
    int lo_any, hi_any, tmp;
    window_bounds(0, sq, sk, wl, wr, lo_any, tmp);
    window_bounds(sq - 1, sq, sk, wl, wr, tmp, hi_any);
    int t_begin = max(max(rb, lo_any), rb + split * tps);
    int t_end = min(min(re, hi_any + 1), rb + (split + 1) * tps);
    t_begin = t_begin / TILE * TILE;

    int vrow[2], qpos[2], head[2], klo[2], khi[2];
    float slope[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        vrow[r] = row_base + g + r * 8;
        const bool ok = vrow[r] < rows_total;
        qpos[r] = ok ? vrow[r] / G : 0;
        head[r] = hk * G + (ok ? vrow[r] % G : 0);
        klo[r] = 1; khi[r] = 0;
        if (ok) {
            window_bounds(qpos[r], sq, sk, wl, wr, klo[r], khi[r]);
            klo[r] = max(max(klo[r], rb), rb + split * tps);
            khi[r] = min(min(khi[r], re - 1), rb + (split + 1) * tps - 1);
        }
        slope[r] = p.alibi_slopes ? p.alibi_slopes[(int64_t)b * p.alibi_stride_b + head[r]] * kLog2e : 0.f;
    }
    const T* qbase = reinterpret_cast<const T*>(p.q.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.q.stride_b);
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int col = kk * 16 + hf * 8 + 2 * t;
                uint32_t v = 0;
                if (vrow[r] < rows_total)
                    v = *reinterpret_cast<const uint32_t*>(qbase + (int64_t)(q_off + qpos[r]) * p.q.stride_s + (int64_t)head[r] * p.q.stride_h + col);
                qf[kk][hf * 2 + r] = v;
            }
        }
    }
    const int32_t* btab = p.block_table ? p.block_table + (int64_t)b * p.block_table_stride : nullptr;
    if constexpr (WIDE) {
        if (threadIdx.x == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (STAGES + s), (rows_total + 15) / 16); }
            mbar_fence_init();
            tma_prefetch_desc(&ta.tk);
            tma_prefetch_desc(&ta.tv);
        }
        __syncthreads();
        if (warp < 4 && row_base >= rows_total) return;      // a warp without rows (17-48 rows): the stages are released by the others
    } else {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8 * s, 1);
            mbar_fence_init();
            tma_prefetch_desc(&ta.tk);
            tma_prefetch_desc(&ta.tv);
        }
        __syncwarp();
    }

    auto issue_tile = [&](int tok0, int stage) {       // lane 0 only
        int c2 = tok0, c3 = kb;
        if (btab) { c3 = btab[tok0 / p.page_size]; c2 = tok0 % p.page_size; }
        mbar_expect_tx(bars + 8 * stage, 2 * TILE_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
            tma_load_4d(sKw + stage * TILE_BYTES + s * SUB_BYTES, &ta.tk, bars + 8 * stage, s * 64, hk, c2, c3);
            tma_load_4d(sVw + stage * TILE_BYTES + s * SUB_BYTES, &ta.tv, bars + 8 * stage, s * 64, hk, c2, c3);
        }
    };
    auto sw = [&](int row, int chunk) -> uint32_t {
        return static_cast<uint32_t>((chunk >> 3) * SUB_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
    };

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    const int ntiles = t_end > t_begin ? (t_end - t_begin + TILE - 1) / TILE : 0;
    if constexpr (WIDE) {
        if (warp == 4) {                                      // producer: refills a stage once its four readers have left it
            if (lane == 0) {
                for (int it = 0; it < ntiles; ++it) {
                    const int stage = it % STAGES, use = it / STAGES;
                    if (use > 0) {
                        const uint32_t bar = bars + 8 * (STAGES + stage), parity = (use - 1) & 1;
                        if (!mbar_try_wait(bar, parity)) {
                            const long long t0 = clock64();
                            bool alive = true;
                            while (!mbar_try_wait(bar, parity)) {
                                if (clock64() - t0 > kWaitCycles) { alive = false; break; }
                            }
                            if (!alive) { atomicCAS(&g_decode_error, 0, 42); break; }     // the readers time out on their side
                        }
                    }
                    issue_tile(t_begin + it * TILE, stage);
                }
            }
            return;
        }
    } else {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES - 1; ++s)
                if (s < ntiles) issue_tile(t_begin + s * TILE, s);
        }
    }
    const float scale_log2 = p.scale * kLog2e;
    const bool has_cap = p.softcap > 0.f;
    const float cap_in = has_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    bool alive = true;

    for (int it = 0; it < ntiles && alive; ++it) {
        const int stage = it % STAGES;
        __syncwarp();                                         // everyone is done with the stage refilled next
        if constexpr (WIDE) {
            if (it > 0 && lane == 0) mbar_arrive(bars + 8 * (STAGES + (it - 1) % STAGES));
        } else {
            if (lane == 0 && it + STAGES - 1 < ntiles) issue_tile(t_begin + (it + STAGES - 1) * TILE, (it + STAGES - 1) % STAGES);
        }
        {   // bounded wait for this tile
            const uint32_t bar = bars + 8 * stage, parity = (it / STAGES) & 1;
            if (!mbar_try_wait(bar, parity)) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, parity)) {
                    if (clock64() - t0 > kWaitCycles) { alive = false; break; }
                }
            }
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) { if (lane == 0) atomicCAS(&g_decode_error, 0, 41); break; }
        }
        const uint32_t sKs = sKw + stage * TILE_BYTES, sVs = sVw + stage * TILE_BYTES;
        const int n0 = t_begin + it * TILE;
        if (n0 + TILE > sk) {                                 // rows past the sequence end hold stale cache bytes
            // (rows past the capacity of a dense cache were zero-filled by the copy itself)
            unsigned char* vgen = gen_base + (sVs - sbase);
            const int fetched = btab ? TILE : min(TILE, p.sk - n0);
            for (int idx = lane; idx < TILE * (HD / 8); idx += 32) {
                const int r = idx / (HD / 8), c = idx % (HD / 8);
                if (n0 + r >= sk && r < fetched) *reinterpret_cast<uint4*>(vgen + sw(r, c)) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }
        float s[TILE / 8][4];
#pragma unroll
        for (int i = 0; i < TILE / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < TILE / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, sKs + sw(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                mma16816<T>(s[2 * n2], qf[kk], b0, b1);
                mma16816<T>(s[2 * n2 + 1], qf[kk], b2, b3);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < TILE / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = n0 + nt * 8 + 2 * t + e;
                    float x = s[nt][2 * r + e];
                    x = has_cap ? cap_out * tanhf(x * cap_in) : x * scale_log2;
                    if (p.alibi_slopes) x -= slope[r] * fabsf((float)(qpos[r] + sk - sq - col));
                    x = (col >= klo[r] && col <= khi[r]) ? x : -INFINITY;
                    s[nt][2 * r + e] = x;
                    mx = fmaxf(mx, x);
                }
            }
            mx = quad_max(mx);
            const float m_new = fmaxf(m_i[r], mx);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            const float corr = exp2f(m_i[r] - m_safe);
            m_i[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < TILE / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pv = exp2f(s[nt][2 * r + e] - m_safe);
                    s[nt][2 * r + e] = pv;
                    sum += pv;
                }
            }
            l_i[r] = l_i[r] * corr + sum;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o_acc[i][2 * r] *= corr; o_acc[i][2 * r + 1] *= corr; }
        }
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
            uint32_t ap[4];
            ap[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
            ap[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
            ap[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            ap[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < HD / 16; ++d2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, sVs + sw(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), d2 * 2 + (lane >> 4)));
                mma16816<T>(o_acc[2 * d2], ap, b0, b1);
                mma16816<T>(o_acc[2 * d2 + 1], ap, b2, b3);
            }
        }
    }
    if (!alive) return;

    const bool to_part = a.o_part != nullptr;
    const int64_t rows_all = (p.cu_seqlens_q ? (int64_t)p.total_q : (int64_t)p.b * p.sq) * p.hq;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float l = quad_sum(l_i[r]);
        if (vrow[r] >= rows_total) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t tok = p.cu_seqlens_q ? (int64_t)q_off + qpos[r] : (int64_t)b * p.sq + qpos[r];
        if (to_part) {
            const int64_t row = tok * p.hq + head[r];
            float* dst = a.o_part + ((int64_t)split * rows_all + row) * p.dv;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = make_float2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            if (t == 0) a.lse_part[(int64_t)split * rows_all + row] = l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : -INFINITY;
        } else {
            T* dst = reinterpret_cast<T*>(p.o.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.o.stride_b) +
                     (int64_t)(q_off + qpos[r]) * p.o.stride_s + (int64_t)head[r] * p.o.stride_h;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = Elem<T>::pack(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            if (t == 0 && p.lse)
                p.lse[(p.cu_seqlens_q ? 0 : (int64_t)b * p.lse_stride_b) + (int64_t)head[r] * p.lse_stride_h + ((int64_t)q_off + qpos[r]) * p.lse_stride_s] =
                    l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : INFINITY;
        }
    }
}

static bool decode_tma_ok(const fa_fwd_params& p) {
    if (p.d != p.dv || (p.d != 64 && p.d != 128 && p.d != 256)) return false;
    if (p.kv_entries <= 0) return false;           // the tile maps need the cache's own outermost extent (see fa_fwd_params)
    const int tile = p.d > 128 ? 16 : 32;
    if (p.block_table && (p.page_size % tile) != 0) return false;
    if (p.k.stride_h <= 0 || p.k.stride_s <= 0 || p.k.stride_b <= 0 || p.v.stride_h <= 0 || p.v.stride_s <= 0 || p.v.stride_b <= 0) return false;
    return tensor_map_encoder_available();
}

template <typename T, int HD>
static int launch_decode_tma_t(const DecodeArgs& a, cudaStream_t st) {
    const fa_fwd_params& p = a.p;
    constexpr int TILE = HD > 128 ? 16 : 32;
    const bool wide = p.sq * (p.hq / p.hkv) > 16;
    DecodeTmaArgs ta;
    ta.d = a;
    // rows: tokens of a page (paged) or of the cache (dense); the outermost extent is the number of pages / cache
    // entries; every index the kernel uses comes from the block table / batch index
    const int64_t rows = p.block_table ? p.page_size : p.sk;
    const int outer = (int)(p.kv_entries < (1 << 24) ? p.kv_entries : 1 << 24);      // > 0: checked by the support predicate
    if (int e = make_tile_map(&ta.tk, p.dtype, p.k.ptr, p.d, p.hkv, rows, outer, p.k.stride_h, p.k.stride_s, p.k.stride_b, TILE)) return e;
    if (int e = make_tile_map(&ta.tv, p.dtype, p.v.ptr, p.dv, p.hkv, rows, outer, p.v.stride_h, p.v.stride_s, p.v.stride_b, TILE)) return e;
    if (wide) {
        const size_t smem = (size_t)2 * kDecWideStages * TILE * HD * 2 + 2 * kDecWideStages * 8 + 1024;
        auto kern = decode_tma_kernel<T, HD, true>;
        if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute")) return e;
        dim3 grid(a.nsplit, p.hkv, p.b);
        kern<<<grid, 160, smem, st>>>(ta);
    } else {
        const size_t smem = (size_t)4 * 2 * kDecStages * TILE * HD * 2 + 4 * 64 + 1024;
        auto kern = decode_tma_kernel<T, HD, false>;
        if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute")) return e;
        dim3 grid(a.nsplit, (p.hkv + 3) / 4, p.b);
        kern<<<grid, 128, smem, st>>>(ta);
    }
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "decode_tma launch");
}

int decode_error_flag(bool clear) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_decode_error, sizeof(int));
    if (clear) { int z = 0; cudaMemcpyToSymbol(g_decode_error, &z, sizeof(int)); }
    return v;
}

template <typename T, int HD>
static int launch_decode_t(const DecodeArgs& a, cudaStream_t st) {
    const fa_fwd_params& p = a.p;
    const size_t smem = (size_t)4 * 2 * kDecStages * (HD > 128 ? 16 : 32) * HD * 2;
    auto kern = decode_splitkv_kernel<T, HD>;
    if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute")) return e;
    dim3 grid(a.nsplit, (p.hkv + 3) / 4, p.b);
    kern<<<grid, 128, smem, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "decode_splitkv launch");
}

static std::atomic<int> g_decode_use_tma{1};
void decode_set_use_tma(int v) { g_decode_use_tma = v; }

bool fwd_decode_supported(const fa_fwd_params& p) {
    const int G = p.hq / p.hkv;
    if (!(p.seqused_k || p.block_table)) return false;       // KV-cache calls only
    if (p.cu_seqlens_k) return false;
    if (p.sq * G <= 16) return true;
    // 17-64 stacked rows: only the TMA kernel has the form in which four warps share a KV head's tiles
    return p.sq * G <= 64 && g_decode_use_tma && decode_tma_ok(p);
}

int launch_fwd_decode(const fa_fwd_params& p, const FwdPlan& plan, float* o_part, float* lse_part) {
    DecodeArgs a;
    a.p = p;
    a.nsplit = plan.nsplit;
    a.tokens_per_split = plan.blocks_per_split * kGenericBN;
    a.o_part = o_part;
    a.lse_part = lse_part;
    // the blob plans whole sequences; a call restricted to a key range keeps the host's uniform plan
    a.meta = (p.kv_begin <= 0 && p.kv_end <= 0) ? reinterpret_cast<const int32_t*>(p.sched_meta) : nullptr;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    const int dmax = p.d > p.dv ? p.d : p.dv;
    if (g_decode_use_tma && decode_tma_ok(p)) {
        note_kernel("decode_splitkv_tma");
        if (p.dtype == FA_F16) {
            if (p.d == 64) return launch_decode_tma_t<__half, 64>(a, st);
            if (p.d == 128) return launch_decode_tma_t<__half, 128>(a, st);
            return launch_decode_tma_t<__half, 256>(a, st);
        }
        if (p.d == 64) return launch_decode_tma_t<__nv_bfloat16, 64>(a, st);
        if (p.d == 128) return launch_decode_tma_t<__nv_bfloat16, 128>(a, st);
        return launch_decode_tma_t<__nv_bfloat16, 256>(a, st);
    }
    note_kernel("decode_splitkv");
    if (p.dtype == FA_F16) {
        if (dmax <= 64) return launch_decode_t<__half, 64>(a, st);
        if (dmax <= 128) return launch_decode_t<__half, 128>(a, st);
        return launch_decode_t<__half, 256>(a, st);
    }
    if (dmax <= 64) return launch_decode_t<__nv_bfloat16, 64>(a, st);
    if (dmax <= 128) return launch_decode_t<__nv_bfloat16, 128>(a, st);
    return launch_decode_t<__nv_bfloat16, 256>(a, st);
}

}  // namespace fa
