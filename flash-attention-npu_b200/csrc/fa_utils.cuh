// Device primitives shared by the attention kernels: cp.async, ldmatrix, mma.sync,
// conversions, swizzled shared-memory addressing and the mask / window arithmetic.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/fa_b200.h"

namespace fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- element types -------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
    static constexpr int kDtype = FA_F16;
};
template <> struct Elem<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
    static constexpr int kDtype = FA_BF16;
};

// ---- async copies ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte global->shared copy; src_bytes (0 or 16) of it are read, the rest is zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---- tensor-core fragments (mma.sync m16n8k16) -----------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows are PITCH bytes
// (a multiple of 128): chunks are XOR-permuted inside each 128-byte group by the row.
template <int PITCH>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>(row * PITCH + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return v;
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// ---- per-sequence geometry -------------------------------------------------------------
struct SeqInfo {
    int q_off;      // first row of the sequence in a packed q tensor (0 for dense)
    int k_off;      // first row in a packed k tensor
    int sq, sk;     // lengths
    int kb;         // batch index into the KV tensors (cache_batch_idx applied)
};

// Length of sequence b of a KV-cache call, read on the device.  A stale or oversized entry is truncated to the
// capacity the host passed (`sk`: rows of a dense cache, page-table width x page size of a paged one), so that no
// kernel indexes past the table or the cache.
__device__ __forceinline__ int cache_len(const fa_fwd_params& p, int b) {
    const long long len = (long long)p.seqused_k[b] + p.s_new;
    return (int)max(0LL, min(len, (long long)p.sk));
}

// Visible key range of query position i (bottom-right aligned): [lo, hi] inclusive.
__device__ __forceinline__ void window_bounds(int i, int sq, int sk, int wl, int wr, int& lo, int& hi) {
    const int diag = i + sk - sq;
    lo = wl < 0 ? 0 : max(0, diag - wl);
    hi = wr < 0 ? sk - 1 : min(sk - 1, diag + wr);
}

}  // namespace fa
