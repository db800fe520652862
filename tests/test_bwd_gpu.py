"""Backward parity on the GPU: autograd through flash_attn_func / flash_attn_varlen_func against the
float64 oracle (restating tests/fa_small_op_golden.py) and the reference-generated fixtures."""
import os

import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_within

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _api(version):
    if version == 2:
        import flash_attn_npu as m
    else:
        import flash_attn_npu_3 as m
    return m


def gpu_grads(version, q, k, v, do, scale, causal, window, softcap, deterministic=False):
    m = _api(version)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    if version == 2:
        out, lse, _ = m.flash_attn_func(qc, kc, vc, softmax_scale=scale, causal=causal, window_size=window,
                                        softcap=softcap, deterministic=deterministic, return_attn_probs=True)
    else:
        out, lse = m.flash_attn_func(qc, kc, vc, softmax_scale=scale, causal=causal, window_size=window,
                                     softcap=softcap, deterministic=deterministic, return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    return out.detach().cpu(), lse.detach().cpu(), dq.cpu(), dk.cpu(), dv.cpu()


def oracle_grads(q, k, v, do, scale, causal, window, softcap):
    """(low-precision golden, fp32 golden): the same function fed the low-precision tensors (its score
    recompute then runs in that dtype) and fed fp32 copies; LSE from the fp32 forward oracle."""
    _, lse = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, window, softcap, data_type=torch.float32)
    lp = orc.attention_bwd(q, k, v, do, lse, scale, causal, window, softcap)
    f32 = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), lse, scale, causal, window, softcap)
    return lp, f32


@pytest.mark.parametrize("idx", range(4))
def test_reference_golden_fixtures(idx):
    fx = torch.load(os.path.join(GOLD, "bwd_cases.pt"), weights_only=False)[idx]
    _, _, dq, dk, dv = gpu_grads(2, fx["q"], fx["k"], fx["v"], fx["dout"], fx["scale"], fx["causal"], fx["window"], fx["softcap"])
    # the fixture is the reference golden's low-precision output; its own distance to fp32 is ~1e-2
    for name, got, ref in (("dq", dq, fx["dq"]), ("dk", dk, fx["dk"]), ("dv", dv, fx["dv"])):
        assert (got.float() - ref.float()).abs().max().item() <= 1e-2 + 1e-2 * ref.float().abs().max().item(), name


# (dtype, B, H, Hkv, Sq, Sk, D, causal, wl, wr, softcap): from tests/test_flash_attn_npu_v2_bwd.py:147-283
CASES = [
    (torch.bfloat16, 1, 2, 2, 256, 256, 128, True, -1, -1, 0.0),
    (torch.bfloat16, 2, 4, 4, 512, 512, 128, False, -1, -1, 0.0),
    (torch.float16, 2, 4, 2, 300, 420, 64, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 8, 2, 513, 513, 128, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 4, 1, 384, 384, 128, True, 128, 0, 0.0),
    (torch.float16, 1, 2, 2, 256, 320, 64, False, 64, 32, 0.0),
    (torch.bfloat16, 1, 2, 2, 200, 200, 192, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 2, 1, 160, 224, 256, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 2, 2, 128, 128, 72, True, -1, -1, 0.0),
    (torch.float16, 1, 2, 2, 256, 256, 128, True, -1, -1, 20.0),
    (torch.bfloat16, 1, 2, 2, 300, 100, 64, True, -1, -1, 0.0),
    (torch.bfloat16, 2, 4, 4, 1024, 1024, 128, True, -1, -1, 0.0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
@pytest.mark.parametrize("version", [2, 3])
def test_dense_backward_matrix(case, version):
    dt, b, h, hkv, sq, sk, d, causal, wl, wr, cap = case
    if version == 3 and (b, sq) != (1, 256) and sq not in (300, 513):
        pytest.skip("v3 shares the kernels; a subset suffices")
    q = (torch.rand(b, sq, h, d) * 2 - 1).to(dt)
    k = (torch.rand(b, sk, hkv, d) * 2 - 1).to(dt)
    v = (torch.rand(b, sk, hkv, d) * 2 - 1).to(dt)
    do = (torch.rand(b, sq, h, d) * 2 - 1).to(dt)
    scale = d ** -0.5
    lp, f32 = oracle_grads(q, k, v, do, scale, causal, (wl, wr), cap)
    _, _, dq, dk, dv = gpu_grads(version, q, k, v, do, scale, causal, (wl, wr), cap)
    for name, got, a, b_ in zip(("dq", "dk", "dv"), (dq, dk, dv), lp, f32):
        assert_within(name, got, a, b_, roundings=3)


def test_backward_is_bitwise_reproducible():
    torch.manual_seed(11)
    q, k, v, do = (torch.randn(1, 700, 4, 128).bfloat16() for _ in range(4))
    a = gpu_grads(2, q, k, v, do, 0.09, True, (-1, -1), 0.0, deterministic=True)
    b = gpu_grads(2, q, k, v, do, 0.09, True, (-1, -1), 0.0, deterministic=True)
    for x, y in zip(a[2:], b[2:]):
        assert torch.equal(x, y)


@pytest.mark.parametrize("version", [2, 3])
def test_varlen_backward(version):
    fx = torch.load(os.path.join(GOLD, "varlen_bwd_case.pt"), weights_only=False)
    m = _api(version)
    cu_q = torch.tensor([0] + torch.tensor(fx["lens_q"]).cumsum(0).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + torch.tensor(fx["lens_k"]).cumsum(0).tolist(), dtype=torch.int32)
    qc, kc, vc = (fx[n].cuda().requires_grad_(True) for n in ("q", "k", "v"))
    res = m.flash_attn_varlen_func(qc, kc, vc, cu_q.cuda(), cu_k.cuda(), max(fx["lens_q"]), max(fx["lens_k"]),
                                   softmax_scale=fx["scale"], causal=True, return_attn_probs=True)
    out = res[0]
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), fx["dout"].cuda())
    _, lse32 = orc.attention_varlen_fwd(fx["q"].float(), fx["k"].float(), fx["v"].float(), cu_q, cu_k, fx["scale"], True,
                                        data_type=torch.float32)
    f32 = orc.attention_varlen_bwd(fx["q"].float(), fx["k"].float(), fx["v"].float(), fx["dout"].float(), lse32, cu_q,
                                   cu_k, fx["scale"], True)
    lp = (fx["dq"], fx["dk"], fx["dv"])
    for name, got, a, b_ in zip(("dq", "dk", "dv"), (dq, dk, dv), lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)


def test_packed_backward_variants():
    import flash_attn_npu as m
    torch.manual_seed(12)
    b, s, h, d = 1, 200, 2, 64
    qkv = (torch.rand(b, s, 3, h, d) * 2 - 1).bfloat16()
    do = (torch.rand(b, s, h, d) * 2 - 1).bfloat16()
    lp, f32 = oracle_grads(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], do, d ** -0.5, True, (-1, -1), 0.0)
    x = qkv.cuda().requires_grad_(True)
    out = m.flash_attn_qkvpacked_func(x, causal=True)
    (g,) = torch.autograd.grad(out, (x,), do.cuda())
    for i, name in enumerate(("dq", "dk", "dv")):
        assert_within(name, g[:, :, i].cpu(), lp[i], f32[i], roundings=3)


def test_backward_uses_the_mask_of_the_forward_when_queries_outnumber_keys():
    """seqlen_q > seqlen_k with a right window in [seqlen_k, seqlen_q - 1): the forward host rule turns that side
    into "unbounded" and then, under a sliding window, into seqlen_k keys past the diagonal (flash_api.cpp:684-704),
    which changes the mask; the saved LSE belongs to that mask, so the backward must differentiate the same one (the
    reference's two host files disagree here; this library keeps the forward's mask in both directions)."""
    import flash_attn_npu as m
    torch.manual_seed(5)
    b, sq, sk, h, d, win = 1, 300, 128, 2, 128, (40, 200)
    q, do = (torch.rand(b, sq, h, d) * 2 - 1).bfloat16(), (torch.rand(b, sq, h, d) * 2 - 1).bfloat16()
    k, v = (torch.rand(b, sk, h, d) * 2 - 1).bfloat16(), (torch.rand(b, sk, h, d) * 2 - 1).bfloat16()
    eff = (40, sk)                                            # what the forward attends under
    scale = d ** -0.5
    lp_o, _ = orc.attention_fwd(q, k, v, scale, False, win)
    f_o, f_l = orc.attention_fwd(q.float(), k.float(), v.float(), scale, False, win, data_type=torch.float32)
    same_o, same_l = orc.attention_fwd(q.float(), k.float(), v.float(), scale, False, eff, data_type=torch.float32)
    assert torch.equal(f_o, same_o) and torch.equal(f_l, same_l)          # the oracle's forward applies the same rule
    lp = orc.attention_bwd(q, k, v, do, f_l, scale, False, eff)
    f32 = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), f_l, scale, False, eff)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = m.flash_attn_func(qc, kc, vc, softmax_scale=scale, window_size=win)
    grads = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    assert_within("out", out.detach().cpu(), lp_o, f_o)
    for name, got, a, b_ in zip(("dq", "dk", "dv"), grads, lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)


@pytest.mark.parametrize("per_batch", [False, True])
@pytest.mark.parametrize("causal,window,cap", [(True, (-1, -1), 0.0), (False, (48, 16), 0.0), (True, (-1, -1), 15.0)])
def test_alibi_backward(per_batch, causal, window, cap):
    """Alibi slopes in the backward (the reference's backward takes and ignores them): the bias of the forward is
    added to the recomputed scores, so the gradients belong to the forward that was run.  Dense and packed."""
    import flash_attn_npu as m
    torch.manual_seed(21)
    b, sq, sk, h, hkv, d = 2, 200, 264, 4, 2, 128
    q, do = (torch.rand(b, sq, h, d) * 2 - 1).bfloat16(), (torch.rand(b, sq, h, d) * 2 - 1).bfloat16()
    k, v = (torch.rand(b, sk, hkv, d) * 2 - 1).bfloat16(), (torch.rand(b, sk, hkv, d) * 2 - 1).bfloat16()
    slopes = torch.rand(b, h) * 0.3 if per_batch else torch.rand(h) * 0.3
    scale = d ** -0.5
    _, f_l = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, window, cap, data_type=torch.float32,
                               alibi_slopes=slopes)
    lp = orc.attention_bwd(q, k, v, do, f_l, scale, causal, window, cap, alibi_slopes=slopes)
    f32 = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), f_l, scale, causal, window, cap,
                            alibi_slopes=slopes)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, lse, _ = m.flash_attn_func(qc, kc, vc, softmax_scale=scale, causal=causal, window_size=window, softcap=cap,
                                    alibi_slopes=slopes.cuda(), return_attn_probs=True)
    grads = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    for name, got, a, b_ in zip(("dq", "dk", "dv"), grads, lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)
    # the same call straight through the extension module (autograd runs it on a worker thread, the kernel name is
    # kept per calling thread): the tcgen05 dK/dV kernel applies cap and bias itself, bit-identical results
    import fa_b200_capi as capi
    from flash_attn_npu import flash_attn_npu as ext
    dq, dk, dv = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
    ext.bwd(do.cuda(), qc.detach(), kc.detach(), vc.detach(), out.detach(), lse, dq, dk, dv, slopes.cuda(), 0.0, scale, causal,
            window[0], window[1], cap, False, None, None)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_bwd_5gemm"
    assert all(torch.equal(x, y) for x, y in zip((dq, dk, dv), grads))
    # without the slopes the gradients differ by far more than the tolerance: the bias is really applied
    plain = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), f_l, scale, causal, window, cap)
    assert (plain[0] - f32[0]).abs().max() > 0.05


@pytest.mark.parametrize("d", [8, 40, 72, 96, 112])
def test_any_head_dim_runs_on_the_tcgen05_kernels(d):
    """Head dims that are not 64 or 128 (the reference's lists hold 111 -> 112, 1 and 4 -> 8 after the interface's padding):
    the tcgen05 kernels run the next size up, the tile copies zero-fill the columns past the head dim and the epilogues
    store the head dim's columns only.  Forward and backward, GQA, causal with ragged tails; tensors with guard columns
    behind every row so that a store past the head dim would be seen."""
    import fa_b200_capi as capi
    from flash_attn_npu import flash_attn_npu as ext
    torch.manual_seed(140 + d)
    b, sq, sk, h, hkv, dt = 2, 333, 400, 4, 2, torch.bfloat16
    pad = 8                                                     # guard columns (row stride d + 8)
    def make(n, heads):
        full = torch.randn(b, n, heads, d + pad).to(dt)
        return full, full[..., :d]
    qf, q = make(sq, h); kf, k = make(sk, hkv); vf, v = make(sk, hkv); dof, do = make(sq, h)
    scale = d ** -0.5
    lp_o, _ = orc.attention_fwd(q, k, v, scale, True)
    f_o, f_l = orc.attention_fwd(q.float(), k.float(), v.float(), scale, True, data_type=torch.float32)
    lp = orc.attention_bwd(q, k, v, do, f_l, scale, True)
    f32 = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), f_l, scale, True)
    qg, kg, vg, dog = (t.cuda()[..., :d] for t in (qf, kf, vf, dof))
    sentinel = 7.0
    outf = torch.full((b, sq, h, d + pad), sentinel, dtype=dt, device="cuda")
    out, lse, _, _ = ext.fwd(qg, kg, vg, outf[..., :d], None, 0.0, scale, True, -1, -1, 0.0, False, None)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_2q"
    assert (outf[..., d:] == sentinel).all()
    assert_within("out", out.cpu(), lp_o, f_o)
    grads = [torch.full((b, n, heads, d + pad), sentinel, dtype=dt, device="cuda") for n, heads in ((sq, h), (sk, hkv), (sk, hkv))]
    ext.bwd(dog, qg, kg, vg, out, lse, grads[0][..., :d], grads[1][..., :d], grads[2][..., :d], None, 0.0, scale, True, -1, -1, 0.0,
            False, None, None)
    torch.cuda.synchronize()
    assert capi.last_kernel().startswith("sm100_tcgen05_bwd")
    assert capi.lib.fa_debug_get(2) == 0
    for name, g, a, b_ in zip(("dq", "dk", "dv"), grads, lp, f32):
        assert (g[..., d:] == sentinel).all(), name
        assert_within(name, g[..., :d].cpu(), a, b_, roundings=3)


def test_softcap_backward_of_packed_sequences_on_tcgen05():
    """Packed (varlen) backward with softcap: the dQ kernel that recomputes S and dP caps the scores itself, so packed
    calls stay on the tcgen05 kernels too.  Ragged sequences including an empty one, GQA, causal."""
    import fa_b200_capi as capi
    from flash_attn_npu import flash_attn_npu as ext
    torch.manual_seed(77)
    lq, lk, h, hkv, d, dt, cap = [300, 0, 129, 77], [300, 64, 400, 77], 4, 2, 128, torch.bfloat16, 3.0
    q, do = (torch.randn(sum(lq), h, d) * 2).to(dt), torch.randn(sum(lq), h, d).to(dt)
    k, v = torch.randn(sum(lk), hkv, d).to(dt), torch.randn(sum(lk), hkv, d).to(dt)
    cu_q = torch.tensor([0] + torch.tensor(lq).cumsum(0).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + torch.tensor(lk).cumsum(0).tolist(), dtype=torch.int32)
    scale = d ** -0.5
    _, lse32 = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cu_q, cu_k, scale, True, (-1, -1), cap, data_type=torch.float32)
    lp = orc.attention_varlen_bwd(q, k, v, do, lse32, cu_q, cu_k, scale, True, (-1, -1), cap)
    f32 = orc.attention_varlen_bwd(q.float(), k.float(), v.float(), do.float(), lse32, cu_q, cu_k, scale, True, (-1, -1), cap)
    qg, kg, vg, dog = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    out, lse, _, _ = ext.varlen_fwd(qg, kg, vg, None, cu_q.cuda(), cu_k.cuda(), None, None, None, None, max(lq), max(lk), 0.0, scale,
                                    False, True, -1, -1, cap, False, None)
    dq, dk, dv = torch.empty_like(qg), torch.empty_like(kg), torch.empty_like(vg)
    ext.varlen_bwd(dog, qg, kg, vg, out, lse, dq, dk, dv, cu_q.cuda(), cu_k.cuda(), None, max(lq), max(lk), 0.0, scale, False, True,
                   -1, -1, cap, False, None, None)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_bwd"
    assert capi.lib.fa_debug_get(2) == 0
    for name, got, a, b_ in zip(("dq", "dk", "dv"), (dq, dk, dv), lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)


def test_alibi_backward_without_the_ds_workspace():
    """The same dense alibi + softcap backward with the dS hand-off switched off: the recomputing dQ kernel applies cap
    and bias itself and gives the gradients of the five-GEMM path within rounding."""
    import fa_b200_capi as capi
    from flash_attn_npu import flash_attn_npu as ext
    torch.manual_seed(3)
    b, sq, sk, h, hkv, d, cap = 2, 200, 264, 4, 2, 128, 4.0
    q, do = torch.randn(b, sq, h, d).bfloat16().cuda(), torch.randn(b, sq, h, d).bfloat16().cuda()
    k, v = torch.randn(b, sk, hkv, d).bfloat16().cuda(), torch.randn(b, sk, hkv, d).bfloat16().cuda()
    slopes = (torch.rand(b, h) * 0.3).cuda()
    scale = d ** -0.5
    out, lse, _, _ = ext.fwd(q, k, v, None, slopes, 0.0, scale, True, -1, -1, cap, False, None)
    res = []
    for spill in (1, 0):
        capi.lib.fa_debug_set(7, spill)
        try:
            g = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
            ext.bwd(do, q, k, v, out, lse, g[0], g[1], g[2], slopes, 0.0, scale, True, -1, -1, cap, False, None, None)
            torch.cuda.synchronize()
            assert capi.last_kernel() == ("sm100_tcgen05_bwd_5gemm" if spill else "sm100_tcgen05_bwd")
            res.append(g)
        finally:
            capi.lib.fa_debug_set(7, 1)
    for name, x, y in zip(("dq", "dk", "dv"), res[0], res[1]):
        assert (x.float() - y.float()).abs().max().item() <= 2.0 ** -7 * max(1.0, x.float().abs().max().item()), name


@pytest.mark.parametrize("packed", [True, False])
def test_zero_fill_of_padded_head_dims_stays_inside_the_rows(packed):
    """Head dim 8 runs on the kernels for 64.  Blocks that no key (or no query) reaches are filled with zeros: the
    fill must write the call's 8 columns, not the kernel's 64 (it once ran 112 bytes past the last row, into whatever
    the allocator had put behind dq).  dq, dk and dv are views into buffers with sentinel rows on both sides; packed
    case: sequences without keys and without queries; dense case: causal with more queries than keys."""
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(336)
    h, hkv, d, dt = 6, 3, 8, torch.float16
    scale = d ** -0.5
    if packed:
        lq, lk = [1, 1, 1, 1, 444, 0], [1, 0, 281, 612, 0, 1]
        cq = [0] + torch.tensor(lq).cumsum(0).tolist()
        ck = [0] + torch.tensor(lk).cumsum(0).tolist()
        q = torch.randn(sum(lq), h, d, generator=g).to(dt)
        k = torch.randn(sum(lk), hkv, d, generator=g).to(dt)
        v = torch.randn(sum(lk), hkv, d, generator=g).to(dt)
    else:
        q = torch.randn(2, 300, h, d, generator=g).to(dt)
        k = torch.randn(2, 40, hkv, d, generator=g).to(dt)
        v = torch.randn(2, 40, hkv, d, generator=g).to(dt)
    do = torch.randn(q.shape, generator=g).to(dt)
    if packed:
        _, rl = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cq, ck, scale, True, data_type=torch.float32)
        ref = orc.attention_varlen_bwd(q.float(), k.float(), v.float(), do.float(), rl, cq, ck, scale, True)
    else:
        _, rl = orc.attention_fwd(q.float(), k.float(), v.float(), scale, True, data_type=torch.float32)
        ref = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), rl, scale, True)

    def guarded(t):          # a view of t's shape with four sentinel rows before and behind it
        flat = torch.full((t.numel() + 8 * t.shape[-1] * t.shape[-2],), 777.0, dtype=dt, device="cuda")
        off = 4 * t.shape[-1] * t.shape[-2]
        return flat, flat[off:off + t.numel()].view(t.shape)

    qg, kg, vg, dog = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    bufs = [guarded(t) for t in (q, k, v)]
    dq, dk, dv = (b[1] for b in bufs)
    if packed:
        cuq = torch.tensor(cq, dtype=torch.int32, device="cuda")
        cuk = torch.tensor(ck, dtype=torch.int32, device="cuda")
        out, lse, _, _ = ext.varlen_fwd(qg, kg, vg, None, cuq, cuk, None, None, None, None, max(lq), max(lk), 0.0, scale, False,
                                        True, -1, -1, 0.0, False, None)
        ext.varlen_bwd(dog, qg, kg, vg, out, lse, dq, dk, dv, cuq, cuk, None, max(lq), max(lk), 0.0, scale, False, True,
                       -1, -1, 0.0, False, None, None)
    else:
        out, lse, _, _ = ext.fwd(qg, kg, vg, None, None, 0.0, scale, True, -1, -1, 0.0, False, None)
        ext.bwd(dog, qg, kg, vg, out, lse, dq, dk, dv, None, 0.0, scale, True, -1, -1, 0.0, False, None, None)
    torch.cuda.synchronize()
    assert capi.last_kernel().startswith("sm100_tcgen05_bwd")
    for name, (flat, view), r in zip(("dq", "dk", "dv"), bufs, ref):
        off = (flat.numel() - view.numel()) // 2
        assert (flat[:off] == 777.0).all() and (flat[off + view.numel():] == 777.0).all(), name + ": sentinel rows overwritten"
        err = (view.cpu().float() - r.float()).abs().max().item()
        assert err <= 2e-3 * max(1.0, r.abs().max().item()), (name, err)
