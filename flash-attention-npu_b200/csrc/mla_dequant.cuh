// Dequantisation of int8 latent rows, shared by the tcgen05 latent-decode kernels.
#pragma once
#include "fa_utils.cuh"
#include "sm100_ptx.cuh"

namespace fa {

// 16 int8 values times `s`, rounded to bf16: bytes are biased to unsigned, dropped into the mantissa of 2^23 and
// the bias subtracted again, which is exact; the product is the one fp32 multiply the plain conversion makes.
__device__ __forceinline__ void dequant16(const uint4 w, float s, uint4& lo, uint4& hi) {
    const uint32_t in[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    uint32_t o[8];
    const float2 bias = make_float2(-8388736.f, -8388736.f), s2 = make_float2(s, s);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 a = make_float2(__uint_as_float(__byte_perm(in[k], 0x4B000000u, 0x7650)),
                                     __uint_as_float(__byte_perm(in[k], 0x4B000000u, 0x7651)));
        const float2 b = make_float2(__uint_as_float(__byte_perm(in[k], 0x4B000000u, 0x7652)),
                                     __uint_as_float(__byte_perm(in[k], 0x4B000000u, 0x7653)));
        const float2 ra = sm100::mul2(sm100::add2(a, bias), s2), rb = sm100::mul2(sm100::add2(b, bias), s2);
        o[2 * k] = Elem<__nv_bfloat16>::pack(ra.x, ra.y);
        o[2 * k + 1] = Elem<__nv_bfloat16>::pack(rb.x, rb.y);
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace fa
