"""The five benchmark configurations at their full sizes.  The oracle cannot run them whole in seconds, so
each test checks (a) sampled (sequence, head) slices against the oracle with the usual tolerance rule and
(b) size-independent properties: a packed sequence equals the same sequence run alone, split equals unsplit,
appended cache rows are bit-exact and every other cache byte is untouched."""
import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_lse, assert_within

pytestmark = pytest.mark.gpu


def test_config2_dense_fwd_bwd_full_size():
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(2)
    b, s, h, d = 4, 4096, 32, 128
    q, k, v, do = (torch.randn(b, s, h, d, generator=g).bfloat16() for _ in range(4))
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, lse, _ = fa.flash_attn_func(qc, kc, vc, causal=True, return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    scale = d ** -0.5
    for bi, hs in ((0, slice(0, 2)), (3, slice(30, 32))):
        qs, ks, vs, dos = (t[bi:bi + 1, :, hs] for t in (q, k, v, do))
        lp_o, _ = orc.attention_fwd(qs, ks, vs, scale, True)
        f_o, f_l = orc.attention_fwd(qs.float(), ks.float(), vs.float(), scale, True, data_type=torch.float32)
        assert_within("out", out[bi:bi + 1, :, hs].detach().cpu(), lp_o, f_o)
        assert_lse(lse[bi:bi + 1, hs].cpu(), f_l)
        lp = orc.attention_bwd(qs, ks, vs, dos, f_l, scale, True, head_chunk=1)
        f32 = orc.attention_bwd(qs.float(), ks.float(), vs.float(), dos.float(), f_l, scale, True, head_chunk=1)
        for name, got, a, b_ in zip(("dq", "dk", "dv"), (dq, dk, dv), lp, f32):
            assert_within(name, got[bi:bi + 1, :, hs].cpu(), a, b_, roundings=3)
    # property: rows of exp(S - LSE) sum to one (checked in fp32 on the device for one head)
    sc = (qc[1, :, 5].float() @ kc[1, :, 5].float().T) * scale
    sc = sc.masked_fill(torch.ones(s, s, device="cuda").triu(1).bool(), float("-inf"))
    assert (torch.exp(sc - lse[1, 5].unsqueeze(-1)).sum(-1) - 1).abs().max().item() < 1e-3


def test_config3_varlen_gqa_full_size():
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(256, 8193, (16,), generator=g).tolist()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    t, h, hkv, d = sum(lens), 32, 8, 128
    q = torch.randn(t, h, d, generator=g).bfloat16()
    k = torch.randn(t, hkv, d, generator=g).bfloat16()
    v = torch.randn(t, hkv, d, generator=g).bfloat16()
    out, lse, _ = fa.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
                                            causal=True, return_attn_probs=True)
    scale = d ** -0.5
    order = sorted(range(16), key=lambda i: lens[i])
    for i in (order[0], order[1], order[-1]):
        a, e = int(cu[i]), int(cu[i + 1])
        # property: the packed sequence equals the same sequence through the dense API
        o1, l1, _ = fa.flash_attn_func(q[a:e].unsqueeze(0).cuda(), k[a:e].unsqueeze(0).cuda(), v[a:e].unsqueeze(0).cuda(),
                                       causal=True, return_attn_probs=True)
        assert torch.equal(o1[0], out[a:e]) and torch.equal(l1[0], lse[:, a:e])
    for i in order[:2]:                      # oracle on the two shortest sequences, 4 query heads of one KV head
        a, e = int(cu[i]), int(cu[i + 1])
        qs, ks, vs = q[a:e, 8:12].unsqueeze(0), k[a:e, 2:3].unsqueeze(0), v[a:e, 2:3].unsqueeze(0)
        lp_o, _ = orc.attention_fwd(qs, ks, vs, scale, True)
        f_o, f_l = orc.attention_fwd(qs.float(), ks.float(), vs.float(), scale, True, data_type=torch.float32)
        assert_within("out", out[a:e, 8:12].cpu().unsqueeze(0), lp_o, f_o)
        assert_lse(lse[8:12, a:e].cpu().unsqueeze(0), f_l)


def test_config4_paged_decode_full_size():
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(4)
    b, hq, hkv, d, page = 128, 32, 8, 128, 256
    lens = torch.randint(1024, 32769, (b,), generator=g, dtype=torch.int32)
    nblk = (lens + 1 + page - 1) // page
    pool = int(nblk.sum())
    perm = torch.randperm(pool, generator=g).int()
    table = torch.zeros(b, int(nblk.max()), dtype=torch.int32)
    off = 0
    for i in range(b):
        n = int(nblk[i])
        table[i, :n] = perm[off:off + n]
        off += n
    gd = torch.Generator(device="cuda").manual_seed(44)
    kc = torch.randn(pool, page, hkv, d, device="cuda", generator=gd).bfloat16()
    vc = torch.randn(pool, page, hkv, d, device="cuda", generator=gd).bfloat16()
    k0, v0 = kc.clone(), vc.clone()
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16()
    kn = torch.randn(b, 1, hkv, d, generator=g).bfloat16()
    vn = torch.randn(b, 1, hkv, d, generator=g).bfloat16()
    cos, sin = orc.rotary_tables(32800, d)
    out, lse = fa.flash_attn_with_kvcache(q.cuda(), kc, vc, kn.cuda(), vn.cuda(), rotary_cos=cos.cuda(), rotary_sin=sin.cuda(),
                                          cache_seqlens=lens.cuda(), block_table=table.cuda(), causal=True,
                                          rotary_interleaved=False, return_softmax_lse=True)
    # appended rows bit-exact, nothing else touched
    kn_rot = torch.stack([orc.apply_rotary(kn[i], cos, sin, torch.tensor([int(lens[i])]), False) for i in range(b)])
    blk = table[torch.arange(b), (lens // page).long()].long().cuda()
    row = (lens % page).long().cuda()
    assert torch.equal(kc[blk, row].cpu().view(torch.int16), kn_rot[:, 0].view(torch.int16))
    assert torch.equal(vc[blk, row].cpu().view(torch.int16), vn[:, 0].view(torch.int16))
    kc[blk, row], vc[blk, row] = k0[blk, row], v0[blk, row]
    assert torch.equal(kc, k0) and torch.equal(vc, v0)
    kc[blk, row], vc[blk, row] = kn_rot[:, 0].cuda(), vn[:, 0].cuda()
    del k0, v0
    # oracle on three sequences (shortest, median, longest)
    order = torch.argsort(lens).tolist()
    for i in (order[0], order[b // 2], order[-1]):
        L = int(lens[i]) + 1
        ki = orc.gather_paged(kc, table[i].cuda(), L).cpu().unsqueeze(0)
        vi = orc.gather_paged(vc, table[i].cuda(), L).cpu().unsqueeze(0)
        qi = orc.apply_rotary(q[i], cos, sin, torch.tensor([L - 1]), False).unsqueeze(0)
        lp_o, _ = orc.attention_fwd(qi, ki, vi, d ** -0.5, True)
        f_o, f_l = orc.attention_fwd(qi.float(), ki.float(), vi.float(), d ** -0.5, True, data_type=torch.float32)
        assert_within("out", out[i:i + 1].cpu(), lp_o, f_o)
        assert_lse(lse[i:i + 1].cpu(), f_l)
    # property: split equals unsplit
    q_rot = torch.stack([orc.apply_rotary(q[i], cos, sin, torch.tensor([int(lens[i])]), False) for i in range(b)])
    many = fa.flash_attn_with_kvcache(q_rot.cuda(), kc, vc, cache_seqlens=(lens + 1).cuda(), block_table=table.cuda(),
                                      causal=True, num_splits=0)
    one = fa.flash_attn_with_kvcache(q_rot.cuda(), kc, vc, cache_seqlens=(lens + 1).cuda(), block_table=table.cuda(),
                                     causal=True, num_splits=1)
    assert (one.float() - many.float()).abs().max().item() <= 2 ** -7
    assert (out.float() - many.float()).abs().max().item() <= 2 ** -7


def test_config5_mla_int8_decode_full_size():
    import flash_attn_npu_3 as fa3
    g = torch.Generator().manual_seed(5)
    b, h, page = 64, 128, 256
    lens = torch.randint(4096, 131073, (b,), generator=g, dtype=torch.int32)
    nblk = (lens + page - 1) // page
    pool = int(nblk.sum())
    perm = torch.randperm(pool, generator=g).int()
    table = torch.zeros(b, int(nblk.max()), dtype=torch.int32)
    off = 0
    for i in range(b):
        n = int(nblk[i])
        table[i, :n] = perm[off:off + n]
        off += n
    gd = torch.Generator(device="cuda").manual_seed(55)
    x = torch.randn(pool, page, 512, device="cuda", generator=gd)
    sc = x.abs().amax(dim=-1).clamp_min(1e-12) / 127.0
    lat = torch.round(x / sc.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
    del x
    rope = torch.randn(pool, page, 64, device="cuda", generator=gd).bfloat16()
    qn = torch.randn(b, 1, h, 512, generator=g).bfloat16()
    qr = torch.randn(b, 1, h, 64, generator=g).bfloat16()
    args = (qn.cuda(), qr.cuda(), lat, sc.float(), rope, lens.cuda(), table.cuda())
    out, lse = fa3.flash_attn_mla_with_kvcache(*args, return_softmax_lse=True)
    order = torch.argsort(lens).tolist()
    for i in order[:2]:
        L = int(lens[i])
        j = torch.arange(L, device="cuda")
        blk = table[i].cuda().long()[j // page]
        li, si, ri = lat[blk, j % page].cpu(), sc[blk, j % page].cpu().float(), rope[blk, j % page].cpu()
        t1 = torch.arange((L + page - 1) // page, dtype=torch.int32).unsqueeze(0)
        pad = t1.numel() * page - L
        li = torch.cat((li, torch.zeros(pad, 512, dtype=torch.int8))).reshape(-1, page, 512)
        si = torch.cat((si, torch.ones(pad))).reshape(-1, page)
        ri = torch.cat((ri, torch.zeros(pad, 64, dtype=torch.bfloat16))).reshape(-1, page, 64)
        r_o, r_l = orc.mla_decode(qn[i:i + 1], qr[i:i + 1], li, si, ri, t1, [L], 576 ** -0.5)
        assert (out[i:i + 1].cpu().float() - r_o.float()).abs().max().item() <= 2 ** -7
        assert_lse(lse[i:i + 1].cpu(), r_l)
    one = fa3.flash_attn_mla_with_kvcache(*args, num_splits=1)
    assert (one.float() - out.float()).abs().max().item() <= 2 ** -7
