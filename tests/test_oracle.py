"""The CPU oracle against fixtures produced by the reference's own Python goldens
(tests/golden/make_golden.py). No GPU."""
import os

import pytest
import torch

from oracle import attention_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return torch.load(os.path.join(GOLD, name), weights_only=False)


def test_config1_forward_matches_reference_golden():
    fx = load("config1_fwd.pt")
    torch.manual_seed(fx["seed"])
    q = torch.randn(*fx["shape"])
    k = torch.randn(*fx["shape"])
    v = torch.randn(*fx["shape"])
    assert abs(q.double().sum().item() - fx["q_sum"]) < 1e-9, "seeded inputs differ from the fixture's"
    out, lse = orc.attention_fwd(q, k, v, fx["scale"], causal=fx["causal"], data_type=torch.float32)
    assert (lse - fx["lse"]).abs().max().item() < 2e-6
    assert (out[0, ::37] - fx["out_fp32_sample"]).abs().max().item() < 2e-6
    assert (out - fx["out"].float()).abs().max().item() < 2e-3   # fixture stored as fp16


@pytest.mark.parametrize("idx", range(10))
def test_forward_cases_match_reference_golden(idx):
    fx = load("fwd_cases.pt")[idx]
    q, k, v = fx["q"], fx["k"], fx["v"]
    out, lse = orc.attention_fwd(q, k, v, fx["scale"], causal=fx["causal"], window=fx["window"],
                                 softcap=fx["softcap"])
    fin = torch.isfinite(fx["lse"])
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - fx["lse"][fin]).abs().max().item() < 1e-5
    # identical up to one rounding of the output type
    ulp = 2 ** -7 if q.dtype == torch.bfloat16 else 2 ** -10
    assert (out.float() - fx["out"].float()).abs().max().item() <= ulp * max(1.0, fx["out"].float().abs().max().item())


def test_paged_gather_matches_reference_golden():
    fx = load("paged_case.pt")
    out, lse = orc.kvcache_fwd(fx["q"], fx["k_cache"], fx["v_cache"], fx["cache_seqlens"], fx["scale"],
                               block_table=fx["block_table"], causal=fx["causal"])
    assert (lse - fx["lse"]).abs().max().item() < 1e-5
    assert (out.float() - fx["out"].float()).abs().max().item() <= 2 ** -7 * 5
    k0 = orc.gather_paged(fx["k_cache"], fx["block_table"][0], 100)
    page = fx["k_cache"].shape[1]
    for j in (0, 15, 16, 99):
        assert torch.equal(k0[j], fx["k_cache"][int(fx["block_table"][0][j // page]), j % page])


@pytest.mark.parametrize("idx", range(5))
def test_backward_cases_match_reference_golden(idx):
    fx = load("bwd_cases.pt")[idx]
    dq, dk, dv = orc.attention_bwd(fx["q"], fx["k"], fx["v"], fx["dout"], fx["lse"], fx["scale"],
                                   causal=fx["causal"], window=fx["window"], softcap=fx["softcap"])
    for got, ref in ((dq, fx["dq"]), (dk, fx["dk"]), (dv, fx["dv"])):
        ulp = {torch.bfloat16: 2 ** -7, torch.float16: 2 ** -10, torch.float32: 1e-6}[ref.dtype]
        assert (got.float() - ref.float()).abs().max().item() <= ulp * max(1.0, ref.float().abs().max().item())


def test_varlen_backward_matches_reference_golden():
    fx = load("varlen_bwd_case.pt")
    cu_q = [0] + torch.tensor(fx["lens_q"]).cumsum(0).tolist()
    cu_k = [0] + torch.tensor(fx["lens_k"]).cumsum(0).tolist()
    out, lse = orc.attention_varlen_fwd(fx["q"], fx["k"], fx["v"], cu_q, cu_k, fx["scale"], causal=True)
    assert (lse - fx["lse"]).abs().max().item() < 1e-5
    assert (out.float() - fx["out"].float()).abs().max().item() <= 2 ** -7 * 5
    dq, dk, dv = orc.attention_varlen_bwd(fx["q"], fx["k"], fx["v"], fx["dout"], fx["lse"], cu_q, cu_k,
                                          fx["scale"], causal=True)
    for got, ref in ((dq, fx["dq"]), (dk, fx["dk"]), (dv, fx["dv"])):
        assert (got.float() - ref.float()).abs().max().item() <= 2 ** -7 * max(1.0, ref.float().abs().max().item())


def test_combine_equals_unsplit():
    torch.manual_seed(1)
    q = torch.randn(1, 1, 4, 64).bfloat16()
    k = torch.randn(1, 300, 2, 64).bfloat16()
    v = torch.randn(1, 300, 2, 64).bfloat16()
    full, lse = orc.attention_fwd(q, k, v, 0.125, data_type=torch.float32)
    parts, lses = [], []
    for lo, hi in ((0, 128), (128, 300)):
        o, l = orc.attention_fwd(q, k[:, lo:hi], v[:, lo:hi], 0.125, data_type=torch.float32)
        parts.append(o.reshape(4, 64))
        lses.append(l.reshape(4))
    parts.append(torch.zeros(4, 64))
    lses.append(torch.full((4,), float("-inf")))
    o, l = orc.combine_partials(torch.stack(parts), torch.stack(lses), torch.float32)
    assert (o - full.reshape(4, 64)).abs().max().item() < 1e-5
    assert (l - lse.reshape(4)).abs().max().item() < 1e-5


def test_rotary_and_append_invariants():
    torch.manual_seed(2)
    cos, sin = orc.rotary_tables(64, 32)
    x = torch.randn(5, 2, 48).bfloat16()
    pos = torch.tensor([3, 4, 5, 6, 7])
    for inter in (False, True):
        y = orc.apply_rotary(x, cos, sin, pos, inter)
        assert torch.equal(y[..., 32:], x[..., 32:])          # tail passes through bit-exact
        y0 = orc.apply_rotary(x, cos, sin, torch.zeros(5, dtype=torch.long), inter)
        assert torch.equal(y0, x)                              # angle 0 is the identity
    kc = torch.randn(2, 32, 2, 48).bfloat16()
    vc = torch.randn(2, 32, 2, 48).bfloat16()
    k0, v0 = kc.clone(), vc.clone()
    kn, vn = torch.randn(2, 1, 2, 48).bfloat16(), torch.randn(2, 1, 2, 48).bfloat16()
    q = torch.randn(2, 1, 4, 48).bfloat16()
    orc.kvcache_fwd(q, kc, vc, [7, 20], 0.1, k_new=kn, v_new=vn, causal=True)
    assert torch.equal(vc[0, 7], vn[0, 0]) and torch.equal(kc[1, 20], kn[1, 0])
    kc[0, 7], kc[1, 20], vc[0, 7], vc[1, 20] = k0[0, 7], k0[1, 20], v0[0, 7], v0[1, 20]
    assert torch.equal(kc, k0) and torch.equal(vc, v0)         # nothing else was touched


def test_mla_split_equals_unsplit():
    torch.manual_seed(3)
    blocks, page, h = 6, 16, 8
    lat, sc = orc.quantize_latent(torch.randn(blocks, page, 512))
    rope = torch.randn(blocks, page, 64).bfloat16()
    table = torch.randperm(blocks).int().reshape(1, blocks)
    qn, qr = torch.randn(1, 1, h, 512).bfloat16(), torch.randn(1, 1, h, 64).bfloat16()
    full, lse = orc.mla_decode(qn, qr, lat, sc, rope, table, [90], 576 ** -0.5)
    po, pl = [], []
    for rng in ((0, 48), (48, 96)):
        o, l = orc.mla_decode(qn, qr, lat, sc, rope, table, [90], 576 ** -0.5, kv_range=rng)
        po.append(o.reshape(h, 512))
        pl.append(l.reshape(h))
    o, l = orc.combine_partials(torch.stack(po), torch.stack(pl))
    assert (o.float() - full.reshape(h, 512).float()).abs().max().item() < 2e-2
    assert (l - lse.reshape(h)).abs().max().item() < 1e-5


def test_alibi_backward_of_the_oracle_is_the_derivative_of_its_forward():
    """The reference holds no golden for alibi in the backward (its backward ignores the slopes), so the restatement
    is pinned against autograd through the plain formula softmax(scale q k^T - slope |i + sk - sq - j| + mask) v in
    float64, with the same bottom-right causal mask."""
    torch.manual_seed(2)
    b, sq, sk, h, hkv, d = 1, 24, 40, 4, 2, 16
    q, do = torch.randn(b, sq, h, d, dtype=torch.float64), torch.randn(b, sq, h, d, dtype=torch.float64)
    k, v = torch.randn(b, sk, hkv, d, dtype=torch.float64), torch.randn(b, sk, hkv, d, dtype=torch.float64)
    slopes = torch.rand(h) * 0.5
    scale = 0.3
    _, lse = orc.attention_fwd(q, k, v, scale, True, data_type=torch.float64, alibi_slopes=slopes)
    dq, dk, dv = orc.attention_bwd(q, k, v, do, lse, scale, True, alibi_slopes=slopes)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    kk = ka.repeat_interleave(h // hkv, dim=2)
    vv = va.repeat_interleave(h // hkv, dim=2)
    s = torch.einsum("bihd,bjhd->bhij", qa, kk) * scale
    i, j = torch.arange(sq).view(-1, 1), torch.arange(sk).view(1, -1)
    s = s - slopes.double().view(1, h, 1, 1) * (i + sk - sq - j).abs().double()
    s = s.masked_fill(j > i + sk - sq, float("-inf"))
    out = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), vv)
    gq, gk, gv = torch.autograd.grad(out, (qa, ka, va), do)
    for got, ref in ((dq, gq), (dk, gk), (dv, gv)):
        assert (got - ref).abs().max().item() < 1e-5          # the saved LSE is fp32
