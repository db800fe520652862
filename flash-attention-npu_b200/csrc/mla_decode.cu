// int8 latent (MLA) paged decode.  No counterpart in the reference (it has no quantised path).
//
// Per cached token j:  K_j = [scale_j * latent_j (512, int8 -> bf16) | rope_j (64 bf16)],  V_j = the same
// dequantised latent.  One shared KV head, seqlen_q = 1, 128-ish query heads, softmax over all tokens.
// The int8 rows are loaded with 16-byte vector loads, multiplied by the token's fp32 scale and rounded
// to bf16 IN REGISTERS, then stored once into swizzled shared memory where the same bytes serve as the
// K operand of Q K^T (576-wide) and as the V operand of P V (first 512 columns).
//
// CTA = (KV split, half of the query heads (64), sequence); 8 warps: warp = (head group of 16, half of
// the 512 output columns).  Tiles of 64 tokens, register-prefetched one tile ahead.  mma.sync tensor
// cores; each (sequence, split) leaves fp32 partial (O, LSE) that the combine kernel merges.
#include "fa_utils.cuh"
#include "fa_internal.h"

namespace fa {

constexpr int kMlaLatent = 512, kMlaRope = 64, kMlaK = kMlaLatent + kMlaRope;
constexpr int kMlaTile = 64;
constexpr int kMlaPitch = kMlaK * 2;                 // 1152 bytes per row
constexpr int kMlaHeadsPerCta = 64;

struct MlaArgs {
    fa_mla_params p;
    int nsplit, tokens_per_split;
    float* o_part;
    float* lse_part;
    int final_direct;                                // single split: write bf16 output directly
};

__device__ __forceinline__ uint32_t mla_swz(int row, int chunk) {
    return static_cast<uint32_t>(row * kMlaPitch + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

__global__ void __launch_bounds__(256, 1) mla_decode_kernel(const MlaArgs a) {
    using T = __nv_bfloat16;
    const fa_mla_params& p = a.p;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sQ = smem;                                        // [64][576]
    unsigned char* sKV = smem + kMlaHeadsPerCta * kMlaPitch;         // 2 stages of [64][576]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hh = blockIdx.y, b = blockIdx.z;
    const int hg = warp & 3, dh = warp >> 2;
    const int head0 = hh * kMlaHeadsPerCta;
    if (head0 >= p.hq) return;
    // an oversized length is truncated to what the page-table row can address
    const int sk = (int)max(0LL, min((long long)p.cache_seqlens[b], (long long)p.block_table_stride * p.page_size));
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    const int t_begin = rb + split * a.tokens_per_split;
    const int t_end = min(re, t_begin + a.tokens_per_split);
    const int ntiles = t_end > t_begin ? (t_end - t_begin + kMlaTile - 1) / kMlaTile : 0;
    const int32_t* btab = p.block_table + (int64_t)b * p.block_table_stride;

    // ---- Q tile: 64 heads x (512 nope | 64 rope) ------------------------------------------------------
    {
        const T* qn = reinterpret_cast<const T*>(p.q_nope) + (int64_t)b * p.q_nope_stride_b;
        const T* qr = reinterpret_cast<const T*>(p.q_rope) + (int64_t)b * p.q_rope_stride_b;
        for (int idx = tid; idx < kMlaHeadsPerCta * (kMlaK / 8); idx += 256) {
            const int r = idx / (kMlaK / 8), c = idx % (kMlaK / 8);
            const int h = head0 + r;
            const bool ok = h < p.hq;
            const T* src = c < 64 ? qn + (int64_t)h * p.q_nope_stride_h + c * 8 : qr + (int64_t)h * p.q_rope_stride_h + (c - 64) * 8;
            cp_async16(smem_u32(sQ) + mla_swz(r, c), ok ? src : qn, ok ? 16 : 0);
        }
        cp_async_commit();
    }

    // ---- tile prefetch into registers: 8 latent chunks (16 int8) + 2 rope chunks per thread ----------------
    uint4 lat[8];
    float sc[8];
    uint4 rope[2];
    auto prefetch = [&](int tok0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = i * 256 + tid;                               // 64 tokens x 32 chunks
            const int r = idx >> 5, c = idx & 31;
            const int tok = tok0 + r;
            lat[i] = make_uint4(0, 0, 0, 0);
            sc[i] = 0.f;
            if (tok < t_end) {
                const int64_t slot = (int64_t)btab[tok / p.page_size] * p.page_size + tok % p.page_size;
                lat[i] = *reinterpret_cast<const uint4*>(p.latent + slot * kMlaLatent + c * 16);
                sc[i] = p.scales[slot];
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = i * 256 + tid;                               // 64 tokens x 8 chunks
            const int r = idx >> 3, c = idx & 7;
            const int tok = tok0 + r;
            rope[i] = make_uint4(0, 0, 0, 0);
            if (tok < t_end) {
                const int64_t slot = (int64_t)btab[tok / p.page_size] * p.page_size + tok % p.page_size;
                rope[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.rope) + slot * kMlaRope + c * 8);
            }
        }
    };
    auto deq2 = [](int lo, int hi, float s) -> uint32_t {
        return Elem<T>::pack(static_cast<float>(lo) * s, static_cast<float>(hi) * s);
    };
    auto commit_tile = [&](int stage) {                                   // registers -> bf16 in shared memory
        unsigned char* dst = sKV + stage * kMlaTile * kMlaPitch;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = i * 256 + tid;
            const int r = idx >> 5, c = idx & 31;                        // int8 chunk c = bf16 chunks 2c, 2c+1
            const uint32_t w[4] = {lat[i].x, lat[i].y, lat[i].z, lat[i].w};
            uint32_t o[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int b0 = (int)(int8_t)(w[k] & 0xff), b1 = (int)(int8_t)((w[k] >> 8) & 0xff);
                const int b2 = (int)(int8_t)((w[k] >> 16) & 0xff), b3 = (int)(int8_t)(w[k] >> 24);
                o[2 * k] = deq2(b0, b1, sc[i]);
                o[2 * k + 1] = deq2(b2, b3, sc[i]);
            }
            *reinterpret_cast<uint4*>(dst + mla_swz(r, 2 * c)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + mla_swz(r, 2 * c + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = i * 256 + tid;
            const int r = idx >> 3, c = idx & 7;
            *reinterpret_cast<uint4*>(dst + mla_swz(r, 64 + c)) = rope[i];
        }
    };

    float o_acc[32][4];                                                   // 16 heads x 256 output columns
#pragma unroll
    for (int i = 0; i < 32; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
    const float scale_log2 = p.scale * kLog2e;

    if (ntiles > 0) { prefetch(t_begin); commit_tile(0); }
    cp_async_wait<0>();
    __syncthreads();

    for (int it = 0; it < ntiles; ++it) {
        const int stage = it & 1;
        if (it + 1 < ntiles) prefetch(t_begin + (it + 1) * kMlaTile);     // global loads in flight during the math
        const uint32_t sT = smem_u32(sKV) + stage * kMlaTile * kMlaPitch;
        const int n0 = t_begin + it * kMlaTile;
        float s[kMlaTile / 8][4];
#pragma unroll
        for (int i = 0; i < kMlaTile / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll 4
        for (int kk = 0; kk < kMlaK / 16; ++kk) {
            uint32_t aq[4];
            ldmatrix_x4(aq[0], aq[1], aq[2], aq[3], smem_u32(sQ) + mla_swz(hg * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
            for (int n2 = 0; n2 < kMlaTile / 16; ++n2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, sT + mla_swz(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                mma16816<T>(s[2 * n2], aq, b0, b1);
                mma16816<T>(s[2 * n2 + 1], aq, b2, b3);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < kMlaTile / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = n0 + nt * 8 + 2 * t + e;
                    const float x = col < t_end ? s[nt][2 * r + e] * scale_log2 : -INFINITY;
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
            for (int nt = 0; nt < kMlaTile / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pv = exp2f(s[nt][2 * r + e] - m_safe);
                    s[nt][2 * r + e] = pv;
                    sum += pv;
                }
            }
            l_i[r] = l_i[r] * corr + sum;
#pragma unroll
            for (int i = 0; i < 32; ++i) { o_acc[i][2 * r] *= corr; o_acc[i][2 * r + 1] *= corr; }
        }
#pragma unroll
        for (int kk = 0; kk < kMlaTile / 16; ++kk) {
            uint32_t ap[4];
            ap[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
            ap[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
            ap[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            ap[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < 16; ++d2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, sT + mla_swz(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), dh * 32 + d2 * 2 + (lane >> 4)));
                mma16816<T>(o_acc[2 * d2], ap, b0, b1);
                mma16816<T>(o_acc[2 * d2 + 1], ap, b2, b3);
            }
        }
        if (it + 1 < ntiles) commit_tile(stage ^ 1);      // the other stage was last read one iteration ago
        __syncthreads();
    }

    // ---- epilogue: heads head0 + hg*16 + {g, g+8}, columns dh*256 .. +255 -----------------------------------
    const int64_t rows_all = (int64_t)p.b * p.hq;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float l = quad_sum(l_i[r]);
        const int h = head0 + hg * 16 + g + r * 8;
        if (h >= p.hq) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int64_t row = (int64_t)b * p.hq + h;
        if (a.final_direct) {
            T* dst = reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + dh * 256;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = Elem<T>::pack(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            if (t == 0 && dh == 0 && p.lse) p.lse[row] = l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : INFINITY;
        } else {
            float* dst = a.o_part + ((int64_t)split * rows_all + row) * kMlaLatent + dh * 256;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = make_float2(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
            if (t == 0 && dh == 0) a.lse_part[(int64_t)split * rows_all + row] = l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : -INFINITY;
        }
    }
}

static void plan_mla(const fa_mla_params& p, int& nsplit, int& tps, int max_len) {
    long n = 1;
    if (p.num_splits > 1) n = p.num_splits;
    else if (p.num_splits == 0) {
        // the tcgen05 kernel stages all of Q (144 KB) per CTA, so its splits are longer
        const long per_split = (kernel_policy() == 0 && mla_pair_supported(p)) ? 8192 : 2048;
        const long by_bal = (max_len + per_split - 1) / per_split;
        const long base = 2L * (p.b > 0 ? p.b : 1);
        const long by_occ = (2L * sm_count() + base - 1) / base;
        const long cap = (max_len + 255) / 256;
        n = by_bal > by_occ ? by_bal : by_occ;
        if (n > cap) n = cap;
    }
    if (n < 1) n = 1;
    if (n > 512) n = 512;
    tps = (int)(((max_len + n - 1) / n + kMlaTile - 1) / kMlaTile * kMlaTile);
    if (tps < kMlaTile) tps = kMlaTile;
    nsplit = (max_len + tps - 1) / tps;
    if (nsplit < 1) nsplit = 1;
}

// longest range any sequence can cover, known without reading device memory
static int mla_max_len(const fa_mla_params& p) {
    const int cap = (int)(p.block_table_stride * p.page_size);
    const int hi = p.kv_end > 0 && p.kv_end < cap ? p.kv_end : cap;
    const int lo = p.kv_begin > 0 ? p.kv_begin : 0;
    return hi > lo ? hi - lo : 0;
}

}  // namespace fa

using namespace fa;

extern "C" {

int fa_mla_num_splits(const fa_mla_params* p) {
    if (!p || p->page_size <= 0) return 1;
    int n, tps;
    plan_mla(*p, n, tps, mla_max_len(*p));
    return n;
}

size_t fa_mla_workspace_bytes(const fa_mla_params* p) {
    if (!p) return 0;
    const int n = fa_mla_num_splits(p);
    if (n <= 1) return 0;
    const size_t rows = (size_t)p->b * p->hq;
    return ((size_t)n * rows * (kMlaLatent + 1) * sizeof(float) + 511) & ~(size_t)255;
}

int fa_mla_decode(const fa_mla_params* pp) {
    if (!pp) return fail(FA_ERR_NULL, "params is null");
    const fa_mla_params& p = *pp;
    if (!p.q_nope || !p.q_rope || !p.latent || !p.scales || !p.rope || !p.block_table || !p.cache_seqlens)
        return fail(FA_ERR_NULL, "null pointer");
    if (p.partials_only ? (!p.o_partial || !p.lse_partial) : !p.o) return fail(FA_ERR_NULL, "output pointer is null");
    if (p.b <= 0 || p.hq <= 0 || p.page_size <= 0) return fail(FA_ERR_BAD_SHAPE, "bad sizes");
    if ((p.q_nope_stride_h % 8) || (p.q_rope_stride_h % 8) || (p.q_nope_stride_b % 8) || (p.q_rope_stride_b % 8) ||
        (p.o_stride_h % 8) || (p.o_stride_b % 8))
        return fail(FA_ERR_MISALIGNED, "strides must be multiples of 8 elements");
    MlaArgs a;
    a.p = p;
    plan_mla(p, a.nsplit, a.tokens_per_split, mla_max_len(p));
    const size_t rows = (size_t)p.b * p.hq;
    a.final_direct = (a.nsplit == 1 && !p.partials_only) ? 1 : 0;
    a.o_part = nullptr; a.lse_part = nullptr;
    if (!a.final_direct) {
        if (a.nsplit == 1) { a.o_part = p.o_partial; a.lse_part = p.lse_partial; }
        else {
            const size_t need = fa_mla_workspace_bytes(pp);
            if (!p.workspace || p.workspace_bytes < need)
                return fail(FA_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", need, p.workspace_bytes);
            a.o_part = reinterpret_cast<float*>(p.workspace);
            a.lse_part = a.o_part + (size_t)a.nsplit * rows * kMlaLatent;
        }
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    if (kernel_policy() == 0 && mla_pair_supported(p)) {
        if (int e = launch_mla_pair(p, a.nsplit, a.tokens_per_split, a.o_part, a.lse_part, a.final_direct, st)) return e;
    } else {
        const int smem = 3 * kMlaTile * kMlaPitch;
        if (int e = cuda_ok(cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute")) return e;
        dim3 grid(a.nsplit, (p.hq + kMlaHeadsPerCta - 1) / kMlaHeadsPerCta, p.b);
        note_kernel("mla_int8_decode");
        mla_decode_kernel<<<grid, 256, smem, st>>>(a);
        mark_kernel(st);
        if (int e = cuda_ok(cudaGetLastError(), "mla_decode launch")) return e;
    }
    if (a.nsplit > 1) {
        fa_combine_params c = {};
        c.o_partial = a.o_part; c.lse_partial = a.lse_part;
        c.o_split_stride = (int64_t)rows * kMlaLatent; c.o_row_stride = kMlaLatent; c.lse_split_stride = (int64_t)rows;
        c.nsplit = a.nsplit; c.rows = (int32_t)rows; c.dv = kMlaLatent; c.stream = p.stream;
        if (p.partials_only) {
            c.o = p.o_partial; c.o_stride = kMlaLatent; c.lse = p.lse_partial; c.out_dtype = 2;
            return combine_flat_keep(c);
        }
        if (p.o_stride_h != kMlaLatent || p.o_stride_b != (int64_t)p.hq * kMlaLatent)
            return fail(FA_ERR_UNSUPPORTED, "split MLA decode needs a contiguous (b, hq, 512) output");
        c.o = p.o; c.o_stride = kMlaLatent; c.lse = p.lse; c.out_dtype = FA_BF16;
        return combine_flat(c);
    }
    return FA_OK;
}

}  // extern "C"
