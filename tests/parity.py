"""Helpers shared by the GPU parity tests: the tolerance rule and oracle wrappers.

Tolerance (stated with every check): max-abs error against the oracle run in fp32 must not
exceed 2 x max-abs(oracle in the low-precision dtype - oracle in fp32) on the same inputs,
with a floor of 1e-5 * max(1, max|LSE|) for LSE (the oracle's own LSE error is exactly 0
because it computes scores and the row sum in fp32 in both modes) and 1e-5 for tensors."""
import torch

from oracle import attention_oracle as orc


def assert_within(name, got, ref_lp, ref32, floor=orc.ABS_FLOOR, slack=1.0):
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
