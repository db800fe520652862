"""Helpers shared by the GPU parity tests: the tolerance rule and oracle wrappers.

Tolerance (stated with every check): max-abs error against the oracle run in fp32 must not
exceed 2 x max-abs(oracle in the low-precision dtype - oracle in fp32) on the same inputs,
with two floors: for LSE 1e-5 * max(1, max|LSE|) (the oracle's own LSE error is exactly 0
because it computes scores and the row sum in fp32 in both modes; 4 x that floor is allowed),
and for tensors half a unit in the last place of the output dtype at the tensor's largest
magnitude (one rounding of a correct result to bf16 / fp16 can be that far from fp32, and the
oracle's own maximum is a sample of the same rounding noise)."""
import math

import torch

from oracle import attention_oracle as orc


def half_ulp(dtype, magnitude):
    bits = {torch.bfloat16: 8, torch.float16: 11}.get(dtype)
    if bits is None or magnitude <= 0:
        return 0.0
    return 2.0 ** (math.floor(math.log2(magnitude)) - bits)


def assert_within(name, got, ref_lp, ref32, floor=orc.ABS_FLOOR, slack=1.0, roundings=1):
    """`roundings`: how many low-precision roundings sit between fp32 truth and the result that the
    oracle does not share: 1 for the forward (the output cast), 3 for the backward: the kernels, like
    the reference's device code (fag_epilogue_op.hpp:1394, :1480), round P and dS to the input dtype
    before the second GEMMs and read the forward's already rounded O for D = rowsum(dO o O), while the
    float64 golden does none of that; then the output cast."""
    fin = torch.isfinite(ref32)
    mag = ref32[fin].abs().max().item() if fin.any() else 0.0
    floor = max(floor, roundings * half_ulp(got.dtype, mag))
    tol = orc.tolerance(ref_lp, ref32, floor) * slack
    err = orc.max_abs_err(got.detach().cpu(), ref32)
    assert err <= tol, f"{name}: max-abs err {err:.3e} > tol {tol:.3e} (2 x oracle lp-vs-fp32 error)"
    return err, tol


def assert_lse(lse, ref_lse):
    floor = orc.lse_floor(ref_lse)
    err = orc.max_abs_err(lse.detach().cpu(), ref_lse)
    assert err <= floor * 4, f"lse: max-abs err {err:.3e} > {4 * floor:.3e}"
    return err


def fwd_refs(q, k, v, scale, causal, window, softcap, alibi=None):
    lp = orc.attention_fwd(q, k, v, scale, causal, window, softcap, alibi_slopes=alibi)
    f32 = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, window, softcap,
                            data_type=torch.float32, alibi_slopes=alibi)
    return lp, f32
