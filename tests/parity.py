"""Helpers shared by the GPU parity tests (and by the benchmark's per-rank checks): the tolerance rule and
oracle wrappers.

Tolerance (stated with every check): max-abs error against the oracle run in fp32 must not
exceed 2 x max-abs(oracle in the low-precision dtype - oracle in fp32) on the same inputs,
with two floors: for LSE 1e-5 * max(1, max|LSE|) (the oracle's own LSE error is exactly 0
because it computes scores and the row sum in fp32 in both modes; 4 x that floor is allowed),
and for tensors half a unit in the last place of the output dtype at the tensor's largest
magnitude (one rounding of a correct result to bf16 / fp16 can be that far from fp32, and the
oracle's own maximum is a sample of the same rounding noise).  Every result says which of the
two bounds, 2 x golden or the floor, was the binding one."""
import math

import torch

from oracle import attention_oracle as orc


def half_ulp(dtype, magnitude):
    bits = {torch.bfloat16: 8, torch.float16: 11}.get(dtype)
    if bits is None or magnitude <= 0:
        return 0.0
    return 2.0 ** (math.floor(math.log2(magnitude)) - bits)


def check_within(name, got, ref_lp, ref32, floor=orc.ABS_FLOOR, slack=1.0, roundings=1):
    """The tolerance rule as numbers: {name, err, two_x_golden, floor, tol, binding, ok}.
    `roundings`: how many low-precision roundings sit between fp32 truth and the result that the
    oracle does not share: 1 for the forward (the output cast), 3 for the backward: the kernels, like
    the reference's device code (fag_epilogue_op.hpp:1394, :1480), round P and dS to the input dtype
    before the second GEMMs and read the forward's already rounded O for D = rowsum(dO o O), while the
    float64 golden does none of that; then the output cast."""
    fin = torch.isfinite(ref32)
    mag = ref32[fin].abs().max().item() if fin.any() else 0.0
    floor = max(floor, roundings * half_ulp(got.dtype, mag))
    two_x = orc.tolerance(ref_lp, ref32, 0.0)
    tol = max(two_x, floor) * slack
    err = orc.max_abs_err(got.detach().cpu(), ref32)
    return {"name": name, "err": err, "two_x_golden": two_x, "floor": floor, "tol": tol,
            "binding": "2x golden" if two_x >= floor else "floor", "ok": bool(err <= tol)}


def describe(res):
    return (f"{res['name']}: max-abs err {res['err']:.3e} vs tol {res['tol']:.3e} "
            f"(2 x golden lp-vs-fp32 {res['two_x_golden']:.3e}, floor {res['floor']:.3e}, binding: {res['binding']})")


def assert_within(name, got, ref_lp, ref32, floor=orc.ABS_FLOOR, slack=1.0, roundings=1):
    res = check_within(name, got, ref_lp, ref32, floor, slack, roundings)
    assert res["ok"], describe(res)
    return res["err"], res["tol"]


def check_lse(lse, ref_lse):
    floor = orc.lse_floor(ref_lse)
    err = orc.max_abs_err(lse.detach().cpu(), ref_lse)
    return {"name": "lse", "err": err, "two_x_golden": 0.0, "floor": 4 * floor, "tol": 4 * floor, "binding": "floor",
            "ok": bool(err <= 4 * floor)}


def assert_lse(lse, ref_lse):
    res = check_lse(lse, ref_lse)
    assert res["ok"], describe(res)
    return res["err"]


def fwd_refs(q, k, v, scale, causal, window, softcap, alibi=None):
    lp = orc.attention_fwd(q, k, v, scale, causal, window, softcap, alibi_slopes=alibi)
    f32 = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, window, softcap,
                            data_type=torch.float32, alibi_slopes=alibi)
    return lp, f32
