"""Random ragged shapes: the tcgen05 kernels against the general mma.sync kernels of the same library (both were
checked against the oracle elsewhere; this sweep looks for shape-dependent slips: partial tiles, windows that cut
tiles, grouped heads, packed batches with empty sequences)."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(policy, fn):
    import fa_b200_capi as capi
    capi.lib.fa_set_kernel_policy(policy)
    try:
        res = fn()
        torch.cuda.synchronize()
        return res, capi.last_kernel()
    finally:
        capi.lib.fa_set_kernel_policy(0)


def _close(a, b, what):
    a, b = a.float(), b.float()
    scale = max(1.0, b.abs().max().item())
    err = (a - b).abs().max().item()
    assert err <= 4 * 2 ** -8 * scale, f"{what}: {err} vs magnitude {scale}"


@pytest.mark.parametrize("seed", range(12))
def test_dense_forward_backward_random(seed):
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    rnd = random.Random(seed)
    d = rnd.choice([64, 128])
    hkv = rnd.choice([1, 2, 3])
    h = hkv * rnd.choice([1, 2, 4])
    b = rnd.choice([1, 2, 3])
    sq, sk = rnd.randint(1, 700), rnd.randint(1, 900)
    mode = rnd.choice(["full", "causal", "window"])
    causal = mode == "causal"
    wl, wr = (rnd.randint(0, 300), rnd.randint(0, 300)) if mode == "window" else (-1, -1)
    dt = rnd.choice([torch.bfloat16, torch.float16])
    g = torch.Generator(device="cuda").manual_seed(1000 + seed)
    q = torch.randn(b, sq, h, d, device="cuda", generator=g).to(dt)
    k = torch.randn(b, sk, hkv, d, device="cuda", generator=g).to(dt)
    v = torch.randn(b, sk, hkv, d, device="cuda", generator=g).to(dt)
    do = torch.randn(b, sq, h, d, device="cuda", generator=g).to(dt)
    scale = d ** -0.5

    def call():
        out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, scale, causal, wl, wr, 0.0, False, None)
        fk = capi.last_kernel()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ext.bwd(do, q, k, v, out, lse, dq, dk, dv, None, 0.0, scale, causal, wl, wr, 0.0, False, None, None)
        return out, lse, dq, dk, dv, fk

    (o1, l1, dq1, dk1, dv1, f1), b1 = _run(0, call)
    (o2, l2, dq2, dk2, dv2, f2), b2 = _run(1, call)
    assert f1.startswith("sm100_tcgen05") and b1.startswith("sm100_tcgen05_bwd"), (f1, b1)
    assert f2 == "generic_mma" and b2 == "generic_mma_bwd", (f2, b2)
    assert capi.lib.fa_debug_get(2) == 0
    tag = f"seed {seed}: b{b} sq{sq} sk{sk} h{h}/{hkv} d{d} {mode} ({wl},{wr}) {dt}"
    _close(o1, o2, tag + " out")
    fin = torch.isfinite(l2)
    assert torch.equal(torch.isfinite(l1), fin), tag + " lse finiteness"
    assert (l1[fin] - l2[fin]).abs().max().item() <= 1e-4 * max(1.0, l2[fin].abs().max().item()) if fin.any() else True
    _close(dq1, dq2, tag + " dq")
    _close(dk1, dk2, tag + " dk")
    _close(dv1, dv2, tag + " dv")


@pytest.mark.parametrize("seed", range(6))
def test_packed_forward_backward_random(seed):
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    rnd = random.Random(100 + seed)
    d = rnd.choice([64, 128])
    hkv = rnd.choice([1, 2])
    h = hkv * rnd.choice([1, 4])
    n = rnd.randint(2, 6)
    lens = [rnd.choice([0, 1, rnd.randint(2, 500)]) for _ in range(n)]
    if sum(lens) == 0:
        lens[0] = 77
    causal = rnd.choice([True, False])
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    t = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(2000 + seed)
    q = torch.randn(t, h, d, device="cuda", generator=g).bfloat16()
    k = torch.randn(t, hkv, d, device="cuda", generator=g).bfloat16()
    v = torch.randn(t, hkv, d, device="cuda", generator=g).bfloat16()
    do = torch.randn(t, h, d, device="cuda", generator=g).bfloat16()
    scale = d ** -0.5

    def call():
        out, lse, _, _ = ext.varlen_fwd(q, k, v, None, cu, cu, None, None, None, None, max(lens), max(lens), 0.0, scale,
                                        False, causal, -1, -1, 0.0, False, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ext.varlen_bwd(do, q, k, v, out, lse, dq, dk, dv, cu, cu, None, max(lens), max(lens), 0.0, scale, False, causal,
                       -1, -1, 0.0, False, None, None)
        return out, dq, dk, dv

    (o1, dq1, dk1, dv1), b1 = _run(0, call)
    (o2, dq2, dk2, dv2), b2 = _run(1, call)
    assert b1.startswith("sm100_tcgen05_bwd") and b2 == "generic_mma_bwd", (b1, b2)
    assert capi.lib.fa_debug_get(2) == 0
    tag = f"seed {seed}: lens {lens} h{h}/{hkv} d{d} causal {causal}"
    _close(o1, o2, tag + " out")
    _close(dq1, dq2, tag + " dq")
    _close(dk1, dk2, tag + " dk")
    _close(dv1, dv2, tag + " dv")


@pytest.mark.parametrize("sq,sk,causal,wl,wr", [
    (512, 512, True, -1, -1),        # the first 128 rows of every block end one key tile before the last 128
    (512, 300, True, -1, -1),        # bottom-right aligned: rows 0..211 see no key, the first half of block 0 none at all
    (300, 1000, True, -1, -1),       # more keys than queries: both halves start late
    (384, 384, True, -1, -1),        # last block has one half only
    (640, 640, False, 200, 0),       # window with the causal edge
    (640, 900, False, 64, 100),      # window whose right edge lies between the two halves' last tiles
    (257, 129, False, -1, 0),        # one row in the second half
])
def test_forward_tile_ranges_of_the_two_query_halves(sq, sk, causal, wl, wr):
    """The tcgen05 forward gives the first 128 rows of a 256-row block their own last key tile; every boundary case of
    that against the general kernel (bit patterns of -inf rows included: zero output, +inf LSE)."""
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    g = torch.Generator(device="cuda").manual_seed(sq * 7 + sk)
    b, h, hkv, d = 2, 4, 2, 128
    q = torch.randn(b, sq, h, d, device="cuda", generator=g).bfloat16()
    k = torch.randn(b, sk, hkv, d, device="cuda", generator=g).bfloat16()
    v = torch.randn(b, sk, hkv, d, device="cuda", generator=g).bfloat16()

    def call():
        out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, d ** -0.5, causal, wl, wr, 0.0, False, None)
        return out, lse

    (o1, l1), k1 = _run(0, call)
    (o2, l2), k2 = _run(1, call)
    assert k1.startswith("sm100_tcgen05") and k2 == "generic_mma", (k1, k2)
    assert capi.lib.fa_debug_get(2) == 0
    assert not torch.isnan(o1.float()).any()
    _close(o1, o2, "out")
    fin = torch.isfinite(l2)
    assert torch.equal(torch.isfinite(l1), fin)
    assert torch.equal(l1[~fin], l2[~fin])
    if fin.any():
        assert (l1[fin] - l2[fin]).abs().max().item() <= 1e-4 * max(1.0, l2[fin].abs().max().item())
