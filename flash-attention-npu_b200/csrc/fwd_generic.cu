// General forward attention kernel (mma.sync tensor cores, cp.async double buffering).
//
// Covers every feature of the forward API: dense / packed / paged KV, bottom-right causal
// and sliding windows, softcap, alibi, GQA with optional stacking of a KV head's query
// group into the M dimension, split-KV with fp32 partials, any head dim <= 256 that is a
// multiple of 8.  The tcgen05 kernel takes the shapes it supports; this one takes the rest.
//
// Math follows the reference's forward kernel (csrc/ascend910/flash_attn_npu/
// mha_fwd_kvcache.cpp:632-969, online_softmax.hpp:479-875, rescale_o.hpp:318-531):
// scores scaled, soft-capped, masked; online softmax in fp32; P rounded to the input type
// before P.V while the row sum uses the unrounded P; O = acc / l rounded once;
// LSE = m + ln l; rows without a visible key give O = 0, LSE = +inf.
#include "fa_utils.cuh"
#include "fa_internal.h"

namespace fa {

struct FwdArgs {
    fa_fwd_params p;
    int nsplit;
    int blocks_per_split;
    int pack;
    float* o_part;
    float* lse_part;
    int part_minus_inf;   // partial LSE of an empty range is -inf (else final +inf)
};

template <typename T, int HD>
__global__ void __launch_bounds__(128) fwd_generic_kernel(const FwdArgs a) {
    constexpr int BM = kGenericBM, BN = kGenericBN;
    constexpr int PITCH = HD * 2;
    constexpr int CHUNKS = HD / 8;
    const fa_fwd_params& p = a.p;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sQ = smem;
    unsigned char* sK = smem + BM * PITCH;                 // 2 stages
    unsigned char* sV = sK + 2 * BN * PITCH;               // 2 stages

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z / a.nsplit, split = blockIdx.z % a.nsplit;
    const int G = p.hq / p.hkv;

    int q_off = 0, sq = p.sq, k_off = 0, sk = p.sk;
    if (p.cu_seqlens_q) { q_off = p.cu_seqlens_q[b]; sq = p.cu_seqlens_q[b + 1] - q_off; }
    if (p.cu_seqlens_k) { k_off = p.cu_seqlens_k[b]; sk = p.cu_seqlens_k[b + 1] - k_off; }
    if (p.seqused_k) sk = cache_len(p, b);
    const int kb = p.cache_batch_idx ? p.cache_batch_idx[b] : b;

    const int rows_total = a.pack ? sq * G : sq;
    const int m0 = blockIdx.x * BM;
    if (m0 >= rows_total) return;
    const int hk = a.pack ? blockIdx.y : blockIdx.y / G;
    const int wl = p.window_left, wr = p.causal ? 0 : p.window_right;

    // key range of this call (cross-device shard) and of this CTA (window, split)
    const int rb = max(0, p.kv_begin), re = p.kv_end > 0 ? min(sk, p.kv_end) : sk;
    int nb_lo = rb / BN, nb_hi = ceil_div(max(re, 0), BN);
    {
        const int qlo = a.pack ? m0 / G : m0;
        const int qhi = a.pack ? (min(rows_total, m0 + BM) - 1) / G : min(rows_total, m0 + BM) - 1;
        int lo, hi, lo2, hi2;
        window_bounds(qlo, sq, sk, wl, wr, lo, hi);
        window_bounds(qhi, sq, sk, wl, wr, lo2, hi2);
        nb_lo = max(nb_lo, lo / BN);
        nb_hi = min(nb_hi, hi2 / BN + 1);
        if (hi2 < 0) nb_hi = nb_lo;
    }
    if (a.nsplit > 1) {
        const int s_lo = nb_lo + split * a.blocks_per_split;
        nb_hi = min(nb_hi, s_lo + a.blocks_per_split);
        nb_lo = s_lo;
    }

    // ---- per-thread row bookkeeping (two rows: g and g + 8 of the warp's 16) -----------
    int vrow[2], qpos[2], head[2], klo[2], khi[2];
    float slope[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        vrow[r] = m0 + warp * 16 + g + r * 8;
        const bool ok = vrow[r] < rows_total;
        qpos[r] = a.pack ? vrow[r] / G : vrow[r];
        head[r] = a.pack ? hk * G + vrow[r] % G : blockIdx.y;
        if (ok) {
            window_bounds(qpos[r], sq, sk, wl, wr, klo[r], khi[r]);
            klo[r] = max(klo[r], rb);
            khi[r] = min(khi[r], re - 1);
        } else {
            klo[r] = 1; khi[r] = 0; head[r] = hk * G;
        }
        slope[r] = p.alibi_slopes ? p.alibi_slopes[(int64_t)b * p.alibi_stride_b + head[r]] * kLog2e : 0.f;
    }

    const T* qbase = reinterpret_cast<const T*>(p.q.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.q.stride_b);
    const T* kbase = reinterpret_cast<const T*>(p.k.ptr);
    const T* vbase = reinterpret_cast<const T*>(p.v.ptr);
    const int32_t* btab = p.block_table ? p.block_table + (int64_t)b * p.block_table_stride : nullptr;

    // ---- Q tile ------------------------------------------------------------------------
    for (int idx = tid; idx < BM * CHUNKS; idx += 128) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        const int vr = m0 + r;
        const bool ok = vr < rows_total && c * 8 < p.d;
        const int qp = a.pack ? vr / G : vr;
        const int hh = a.pack ? hk * G + vr % G : blockIdx.y;
        const T* src = ok ? qbase + (int64_t)(q_off + qp) * p.q.stride_s + (int64_t)hh * p.q.stride_h + c * 8 : qbase;
        cp_async16(smem_u32(sQ) + swz<PITCH>(r, c), src, ok ? 16 : 0);
    }

    auto load_kv = [&](int nb, int stage) {
        const int n0 = nb * BN;
        for (int idx = tid; idx < BN * CHUNKS; idx += 128) {
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            const int tok = n0 + r;
            const bool ok = tok < sk;
            int64_t koff = 0, voff = 0;
            if (ok) {
                if (btab) {
                    const int blk = btab[tok / p.page_size];
                    const int rowin = tok % p.page_size;
                    koff = (int64_t)blk * p.k.stride_b + (int64_t)rowin * p.k.stride_s;
                    voff = (int64_t)blk * p.v.stride_b + (int64_t)rowin * p.v.stride_s;
                } else {
                    const int64_t bb = p.cu_seqlens_k ? 0 : kb;
                    koff = bb * p.k.stride_b + (int64_t)(k_off + tok) * p.k.stride_s;
                    voff = bb * p.v.stride_b + (int64_t)(k_off + tok) * p.v.stride_s;
                }
                koff += (int64_t)hk * p.k.stride_h + c * 8;
                voff += (int64_t)hk * p.v.stride_h + c * 8;
            }
            const bool okk = ok && c * 8 < p.d, okv = ok && c * 8 < p.dv;
            cp_async16(smem_u32(sK) + stage * BN * PITCH + swz<PITCH>(r, c), okk ? kbase + koff : kbase, okk ? 16 : 0);
            cp_async16(smem_u32(sV) + stage * BN * PITCH + swz<PITCH>(r, c), okv ? vbase + voff : vbase, okv ? 16 : 0);
        }
    };

    float o_acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
    float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};

    if (nb_lo < nb_hi) load_kv(nb_lo, 0);
    cp_async_commit();

    const float scale_log2 = p.scale * kLog2e;
    const bool has_cap = p.softcap > 0.f;
    const float cap_in = has_cap ? p.scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;
    const int ksteps = ceil_div(p.d, 16), vsteps = ceil_div(p.dv, 16);

    for (int nb = nb_lo; nb < nb_hi; ++nb) {
        const int stage = (nb - nb_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (nb + 1 < nb_hi) load_kv(nb + 1, stage ^ 1);
        cp_async_commit();

        const uint32_t sKs = smem_u32(sK) + stage * BN * PITCH;
        const uint32_t sVs = smem_u32(sV) + stage * BN * PITCH;
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
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
        }

        // ---- scale, softcap, alibi, mask, online softmax ---------------------------------
        const int n0 = nb * BN;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
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
            for (int nt = 0; nt < BN / 8; ++nt) {
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

        // ---- O += P V -----------------------------------------------------------------------
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
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
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- epilogue ---------------------------------------------------------------------------
    float inv[2], lse[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float l = quad_sum(l_i[r]);
        inv[r] = l > 0.f ? 1.f / l : 0.f;
        lse[r] = l > 0.f ? (m_i[r] + log2f(l)) * kLn2 : (a.part_minus_inf ? -INFINITY : INFINITY);
    }
    const bool to_part = a.o_part != nullptr;
    if (to_part) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (vrow[r] >= rows_total) continue;
            const int64_t tok = p.cu_seqlens_q ? (int64_t)q_off + qpos[r] : (int64_t)b * p.sq + qpos[r];
            const int64_t row = tok * p.hq + head[r];
            const int64_t rows_all = (p.cu_seqlens_q ? (int64_t)p.total_q : (int64_t)p.b * p.sq) * p.hq;
            float* dst = a.o_part + ((int64_t)split * rows_all + row) * p.dv;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const int col = i * 8 + 2 * t;
                if (col < p.dv) *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[i][2 * r] * inv[r], o_acc[i][2 * r + 1] * inv[r]);
            }
            if (t == 0) a.lse_part[(int64_t)split * rows_all + row] = lse[r];
        }
        return;
    }
    // stage the warp's 16 rows through its own slice of the Q tile, then 16-byte stores
    __syncwarp();
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = warp * 16 + g + r * 8;
            const uint32_t v = Elem<T>::pack(o_acc[i][2 * r] * inv[r], o_acc[i][2 * r + 1] * inv[r]);
            *reinterpret_cast<uint32_t*>(sQ + swz<PITCH>(row, i) + t * 4) = v;
        }
    }
    __syncwarp();
    T* obase = reinterpret_cast<T*>(p.o.ptr) + (p.cu_seqlens_q ? 0 : (int64_t)b * p.o.stride_b);
    for (int idx = lane; idx < 16 * CHUNKS; idx += 32) {
        const int r = warp * 16 + idx / CHUNKS, c = idx % CHUNKS;
        const int vr = m0 + r;
        if (vr < rows_total && c * 8 < p.dv) {
            const int qp = a.pack ? vr / G : vr;
            const int hh = a.pack ? hk * G + vr % G : blockIdx.y;
            const uint4 v = *reinterpret_cast<const uint4*>(sQ + swz<PITCH>(r, c));
            *reinterpret_cast<uint4*>(obase + (int64_t)(q_off + qp) * p.o.stride_s + (int64_t)hh * p.o.stride_h + c * 8) = v;
        }
    }
    if (t == 0 && p.lse) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (vrow[r] < rows_total) {
                const int64_t tok = (int64_t)q_off + qpos[r];
                p.lse[(p.cu_seqlens_q ? 0 : (int64_t)b * p.lse_stride_b) + (int64_t)head[r] * p.lse_stride_h + tok * p.lse_stride_s] = lse[r];
            }
        }
    }
}

template <typename T, int HD>
static int launch_one(const FwdArgs& a, cudaStream_t st) {
    const fa_fwd_params& p = a.p;
    const int G = p.hq / p.hkv;
    const size_t smem = (size_t)(kGenericBM + 4 * kGenericBN) * HD * 2;
    auto kern = fwd_generic_kernel<T, HD>;
    static bool configured[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !configured[dev]) {
        if (int e = cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute")) return e;
        configured[dev] = true;
    } else if (dev >= 16) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int rows = a.pack ? p.sq * G : p.sq;
    dim3 grid(ceil_div(rows, kGenericBM), a.pack ? p.hkv : p.hq, p.b * a.nsplit);
    if (grid.x == 0 || grid.y == 0 || grid.z == 0) return FA_OK;
    kern<<<grid, 128, smem, st>>>(a);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "fwd_generic launch");
}

int launch_fwd_generic(const fa_fwd_params& p, const FwdPlan& plan, float* o_part, float* lse_part) {
    FwdArgs a;
    a.p = p;
    a.nsplit = plan.nsplit;
    a.blocks_per_split = plan.blocks_per_split;
    a.pack = plan.pack_gqa;
    a.o_part = o_part;
    a.lse_part = lse_part;
    a.part_minus_inf = o_part != nullptr;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    const int dmax = p.d > p.dv ? p.d : p.dv;
    note_kernel("generic_mma");
    if (p.dtype == FA_F16) {
        if (dmax <= 64) return launch_one<__half, 64>(a, st);
        if (dmax <= 128) return launch_one<__half, 128>(a, st);
        return launch_one<__half, 256>(a, st);
    }
    if (dmax <= 64) return launch_one<__nv_bfloat16, 64>(a, st);
    if (dmax <= 128) return launch_one<__nv_bfloat16, 128>(a, st);
    return launch_one<__nv_bfloat16, 256>(a, st);
}

// ---------------------------------------------------------------------------------------------
// In-place KV append with rotary embedding, and rotation of q into a scratch buffer.
// Positions: new key i of sequence b sits at seqused_k[b] + i; query i at seqused_k[b] + i when
// the call is causal or windowed, else at seqused_k[b] (flash_attn_npu_interface.py:1469-1474).
// fp32 arithmetic with separately rounded products and one round-to-nearest-even, so the result
// is bit-identical to the CPU restatement.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T rotate_elem(const T* x, int e, int rd, int interleaved, const T* cosr, const T* sinr) {
    if (e >= rd) return x[e];
    int j, partner;
    bool first;
    if (interleaved) { j = e >> 1; first = (e & 1) == 0; partner = first ? e + 1 : e - 1; }
    else { first = e < rd / 2; j = first ? e : e - rd / 2; partner = first ? e + rd / 2 : e - rd / 2; }
    const float c = Elem<T>::to_float(cosr[j]), s = Elem<T>::to_float(sinr[j]);
    const float xe = Elem<T>::to_float(x[e]), xp = Elem<T>::to_float(x[partner]);
    const float r = first ? __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xp, s))
                          : __fadd_rn(__fmul_rn(xp, s), __fmul_rn(xe, c));
    return Elem<T>::from_float(r);
}

template <typename T>
__global__ void append_rotary_kernel(const fa_fwd_params p, T* q_rot, int rotate_q_by_pos) {
    const int b = blockIdx.z;
    const int L = p.seqused_k[b];
    const int rd = p.rotary_cos ? p.rotary_dim : 0;
    const T* cosb = reinterpret_cast<const T*>(p.rotary_cos);
    const T* sinb = reinterpret_cast<const T*>(p.rotary_sin);
    const int kv_rows = p.s_new * p.hkv;
    const int row = blockIdx.x;
    if (row < kv_rows) {
        if (!p.k_new.ptr) return;
        const int i = row / p.hkv, h = row % p.hkv;
        const int pos = L + i;
        // a length that points outside the cache (or past the page-table row) appends nothing
        if (pos < 0 || pos >= p.sk) return;
        int64_t koff, voff;
        if (p.block_table) {
            const int blk = p.block_table[(int64_t)b * p.block_table_stride + pos / p.page_size];
            const int rin = pos % p.page_size;
            koff = (int64_t)blk * p.k.stride_b + (int64_t)rin * p.k.stride_s + (int64_t)h * p.k.stride_h;
            voff = (int64_t)blk * p.v.stride_b + (int64_t)rin * p.v.stride_s + (int64_t)h * p.v.stride_h;
        } else {
            const int kb = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
            koff = (int64_t)kb * p.k.stride_b + (int64_t)pos * p.k.stride_s + (int64_t)h * p.k.stride_h;
            voff = (int64_t)kb * p.v.stride_b + (int64_t)pos * p.v.stride_s + (int64_t)h * p.v.stride_h;
        }
        const T* ksrc = reinterpret_cast<const T*>(p.k_new.ptr) + (int64_t)b * p.k_new.stride_b + (int64_t)i * p.k_new.stride_s + (int64_t)h * p.k_new.stride_h;
        const T* vsrc = reinterpret_cast<const T*>(p.v_new.ptr) + (int64_t)b * p.v_new.stride_b + (int64_t)i * p.v_new.stride_s + (int64_t)h * p.v_new.stride_h;
        T* kdst = reinterpret_cast<T*>(p.k.ptr) + koff;
        T* vdst = reinterpret_cast<T*>(p.v.ptr) + voff;
        const int cpos = max(0, min(pos, p.seqlen_ro - 1));
        for (int e = threadIdx.x; e < p.d; e += blockDim.x)
            kdst[e] = rd ? rotate_elem<T>(ksrc, e, rd, p.rotary_interleaved, cosb + (int64_t)cpos * (rd / 2), sinb + (int64_t)cpos * (rd / 2)) : ksrc[e];
        for (int e = threadIdx.x; e < p.dv; e += blockDim.x) vdst[e] = vsrc[e];
        return;
    }
    if (!q_rot) return;
    const int qr = row - kv_rows;              // (qpos, head)
    if (qr >= p.sq * p.hq) return;
    const int i = qr / p.hq, h = qr % p.hq;
    const int pos = max(0, min(L + (rotate_q_by_pos ? i : 0), p.seqlen_ro - 1));
    const T* src = reinterpret_cast<const T*>(p.q.ptr) + (int64_t)b * p.q.stride_b + (int64_t)i * p.q.stride_s + (int64_t)h * p.q.stride_h;
    T* dst = q_rot + (((int64_t)b * p.sq + i) * p.hq + h) * p.d;
    for (int e = threadIdx.x; e < p.d; e += blockDim.x)
        dst[e] = rotate_elem<T>(src, e, rd, p.rotary_interleaved, cosb + (int64_t)pos * (rd / 2), sinb + (int64_t)pos * (rd / 2));
}

int launch_append_rotary(const fa_fwd_params& p, void* q_rot, int rotate_q_by_pos) {
    const int rows = p.s_new * p.hkv + (q_rot ? p.sq * p.hq : 0);
    if (rows == 0 || p.b == 0) return FA_OK;
    dim3 grid(rows, 1, p.b);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    if (p.dtype == FA_F16) append_rotary_kernel<__half><<<grid, 64, 0, st>>>(p, reinterpret_cast<__half*>(q_rot), rotate_q_by_pos);
    else append_rotary_kernel<__nv_bfloat16><<<grid, 64, 0, st>>>(p, reinterpret_cast<__nv_bfloat16*>(q_rot), rotate_q_by_pos);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "append_rotary launch");
}

// ---------------------------------------------------------------------------------------------
// LSE-weighted combine of split partials (CombineScale.hpp:165-316): one warp per output row.
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void store_out(OutT* dst, float v);
template <> __device__ __forceinline__ void store_out<float>(float* d, float v) { *d = v; }
template <> __device__ __forceinline__ void store_out<__half>(__half* d, float v) { *d = __float2half_rn(v); }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* d, float v) { *d = __float2bfloat16_rn(v); }

// One warp per output row.  The weights exp(lse_s - lse) are computed once per row (lanes stride over the splits) and
// kept in shared memory; the partial outputs are then read with 16-byte loads, four splits in flight per lane.
constexpr int kCombineWarps = 4, kCombineMaxSplits = 512;

template <typename OutT>
__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(
    const float* __restrict__ o_part, const float* __restrict__ lse_part, int64_t o_split_stride, int64_t o_row_stride,
    int64_t lse_split_stride, OutT* o, float* lse, int nsplit, int64_t rows, int dv,
    // output addressing: row = tok * hq + head
    int hq, int sq_dense, int64_t o_sb, int64_t o_ss, int64_t o_sh, int64_t l_sb, int64_t l_sh, int64_t l_ss,
    int keep_minus_inf) {
    __shared__ float s_w[kCombineWarps][kCombineMaxSplits];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kCombineWarps + wid;
    if (row >= rows) return;
    float* w = s_w[wid];
    float m = -INFINITY;
    for (int s = lane; s < nsplit; s += 32) {
        const float ls = lse_part[s * lse_split_stride + row];
        w[s] = ls;
        m = fmaxf(m, ls);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float ms = m == -INFINITY ? 0.f : m;
    float tot = 0.f;
    for (int s = lane; s < nsplit; s += 32) tot += expf(w[s] - ms);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
    const float l = tot > 0.f ? ms + logf(tot) : -INFINITY;
    // a split that saw no key (lse = -inf) gets weight 0 and its O slot is never read (it may hold anything)
    for (int s = lane; s < nsplit; s += 32) w[s] = w[s] == -INFINITY ? 0.f : expf(w[s] - l);
    __syncwarp();
    const int64_t tok = row / hq;
    const int head = (int)(row % hq);
    int64_t ooff, loff;
    if (sq_dense > 0) {
        const int64_t bb = tok / sq_dense, qp = tok % sq_dense;
        ooff = bb * o_sb + qp * o_ss + head * o_sh;
        loff = bb * l_sb + head * l_sh + qp * l_ss;
    } else {
        ooff = tok * o_ss + head * o_sh;
        loff = head * l_sh + tok * l_ss;
    }
    const float* src = o_part + row * o_row_stride;
    const bool vec = (dv % 4 == 0) && (o_row_stride % 4 == 0) && (o_split_stride % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(o_part) & 15) == 0);
    if (vec) {
        for (int c = lane * 4; c < dv; c += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int s = 0;
            for (; s + 4 <= nsplit; s += 4) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    v[u] = w[s + u] != 0.f ? *reinterpret_cast<const float4*>(src + (s + u) * o_split_stride + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    acc.x += w[s + u] * v[u].x; acc.y += w[s + u] * v[u].y; acc.z += w[s + u] * v[u].z; acc.w += w[s + u] * v[u].w;
                }
            }
            for (; s < nsplit; ++s) {
                if (w[s] == 0.f) continue;
                const float4 v = *reinterpret_cast<const float4*>(src + s * o_split_stride + c);
                acc.x += w[s] * v.x; acc.y += w[s] * v.y; acc.z += w[s] * v.z; acc.w += w[s] * v.w;
            }
            store_out<OutT>(o + ooff + c, acc.x);
            store_out<OutT>(o + ooff + c + 1, acc.y);
            store_out<OutT>(o + ooff + c + 2, acc.z);
            store_out<OutT>(o + ooff + c + 3, acc.w);
        }
    } else {
        for (int c = lane; c < dv; c += 32) {
            float acc = 0.f;
            for (int s = 0; s < nsplit; ++s) {
                if (w[s] == 0.f) continue;
                acc += w[s] * src[s * o_split_stride + c];
            }
            store_out<OutT>(o + ooff + c, acc);
        }
    }
    if (lane == 0 && lse) lse[loff] = (tot > 0.f || keep_minus_inf) ? l : INFINITY;
}

int launch_fwd_combine(const fa_fwd_params& p, int nsplit, const float* o_part, const float* lse_part, int to_partial) {
    // rows are enumerated as (token, head)
    const int64_t toks = p.cu_seqlens_q ? (int64_t)p.total_q : (int64_t)p.b * p.sq;
    const int64_t rows = toks * p.hq;
    if (rows == 0) return FA_OK;
    if (nsplit > kCombineMaxSplits) return fail(FA_ERR_BAD_SHAPE, "at most %d splits can be combined", kCombineMaxSplits);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(p.stream);
    const int wpb = kCombineWarps;
    dim3 grid((unsigned)((rows + wpb - 1) / wpb));
    const int sq_dense = p.cu_seqlens_q ? 0 : p.sq;
    if (to_partial) {
        combine_kernel<float><<<grid, wpb * 32, 0, st>>>(o_part, lse_part, rows * p.dv, p.dv, rows, p.o_partial, p.lse_partial,
                                                        nsplit, rows, p.dv, p.hq, 0, 0, (int64_t)p.hq * p.dv, p.dv, 0, 1, p.hq, 1);
    } else if (p.dtype == FA_F16) {
        combine_kernel<__half><<<grid, wpb * 32, 0, st>>>(o_part, lse_part, rows * p.dv, p.dv, rows, reinterpret_cast<__half*>(p.o.ptr), p.lse,
                                                         nsplit, rows, p.dv, p.hq, sq_dense, p.o.stride_b, p.o.stride_s, p.o.stride_h,
                                                         p.lse_stride_b, p.lse_stride_h, p.lse_stride_s, 0);
    } else {
        combine_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, st>>>(o_part, lse_part, rows * p.dv, p.dv, rows, reinterpret_cast<__nv_bfloat16*>(p.o.ptr), p.lse,
                                                                nsplit, rows, p.dv, p.hq, sq_dense, p.o.stride_b, p.o.stride_s, p.o.stride_h,
                                                                p.lse_stride_b, p.lse_stride_h, p.lse_stride_s, 0);
    }
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "combine launch");
}

// public combine entry (flat rows)
template <typename OutT>
static void launch_flat_combine(const fa_combine_params& c, cudaStream_t st, int keep = 0) {
    const int wpb = kCombineWarps;
    dim3 grid((unsigned)((c.rows + wpb - 1) / wpb));
    combine_kernel<OutT><<<grid, wpb * 32, 0, st>>>(c.o_partial, c.lse_partial, c.o_split_stride, c.o_row_stride, c.lse_split_stride,
                                                   reinterpret_cast<OutT*>(c.o), c.lse, c.nsplit, c.rows, c.dv,
                                                   1, 0, 0, c.o_stride, 0, 0, 0, 1, keep);
}

// fp32 output, rows that saw no key keep LSE = -inf (partials that will be combined again)
int combine_flat_keep(const fa_combine_params& c) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(c.stream);
    if (c.rows == 0) return FA_OK;
    if (c.nsplit > kCombineMaxSplits) return fail(FA_ERR_BAD_SHAPE, "at most %d splits can be combined", kCombineMaxSplits);
    launch_flat_combine<float>(c, st, 1);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "combine launch");
}

int combine_flat(const fa_combine_params& c) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(c.stream);
    if (c.rows == 0) return FA_OK;
    if (c.nsplit > kCombineMaxSplits) return fail(FA_ERR_BAD_SHAPE, "at most %d splits can be combined", kCombineMaxSplits);
    if (c.out_dtype == FA_F16) launch_flat_combine<__half>(c, st);
    else if (c.out_dtype == FA_BF16) launch_flat_combine<__nv_bfloat16>(c, st);
    else launch_flat_combine<float>(c, st);
    mark_kernel(st);
    return cuda_ok(cudaGetLastError(), "combine launch");
}

}  // namespace fa
