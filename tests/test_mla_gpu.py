"""int8 latent (MLA) paged decode against the CPU restatement (parity unpinned: the reference has no
quantised path; the oracle restates K = [scale*int8 | rope], V = scale*int8 and reuses the forward golden)."""
import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_lse, assert_within

pytestmark = pytest.mark.gpu


def make_case(gen, b, h, lens, page=64):
    nblk = [(l + page - 1) // page for l in lens]
    pool = sum(nblk)
    perm = torch.randperm(pool, generator=gen).int()
    table = torch.zeros(b, max(nblk), dtype=torch.int32)
    off = 0
    for i, n in enumerate(nblk):
        table[i, :n] = perm[off:off + n]
        off += n
    lat, sc = orc.quantize_latent(torch.randn(pool, page, 512, generator=gen))
    rope = torch.randn(pool, page, 64, generator=gen).bfloat16()
    qn = torch.randn(b, 1, h, 512, generator=gen).bfloat16()
    qr = torch.randn(b, 1, h, 64, generator=gen).bfloat16()
    return qn, qr, lat, sc, rope, table


def oracle_fp32(qn, qr, lat, sc, rope, table, lens, scale):
    """The same math with fp32 P and output: the target of the tolerance rule."""
    outs, lses = [], []
    for i, L in enumerate(lens):
        j = torch.arange(L)
        page = lat.shape[1]
        blk = table[i].long()[j // page]
        latf = (lat[blk, j % page].float() * sc[blk, j % page].unsqueeze(-1)).to(torch.bfloat16).float()
        kk = torch.cat((latf, rope[blk, j % page].float()), dim=-1).unsqueeze(1)
        qq = torch.cat((qn[i], qr[i]), dim=-1).float()
        o, l = orc.fwd_one_sequence(qq, kk, latf.unsqueeze(1), scale, None, torch.float32)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


@pytest.mark.parametrize("b,h,lens,splits", [
    (2, 128, [300, 1000], 0),
    (3, 128, [64, 65, 2049], 1),
    (2, 128, [5000, 777], 0),
    (1, 16, [1500], 3),
    (2, 80, [129, 4000], 5),
])
@pytest.mark.parametrize("page,family", [(64, "mla_int8_tcgen05_pair"), (256, "mla_int8_tcgen05_pair"),
                                         (48, "mla_int8_decode"), (64, "forced:mla_int8_decode")])
def test_mla_decode_matches_oracle(b, h, lens, splits, page, family):
    """Both kernel families: the tcgen05 kernel (a CTA pair that splits the score dims) takes pages that hold whole
    64-token tiles, the mma.sync kernel everything else (and everything when the generic policy is forced)."""
    import flash_attn_npu_3 as m3
    import fa_b200_capi as capi
    gen = torch.Generator().manual_seed(50 + b + h)
    qn, qr, lat, sc, rope, table = make_case(gen, b, h, lens, page=page)
    scale = 576 ** -0.5
    lp_o, lp_l = orc.mla_decode(qn, qr, lat, sc, rope, table, lens, scale)
    f_o, f_l = oracle_fp32(qn, qr, lat, sc, rope, table, lens, scale)
    forced = family.startswith("forced:")
    capi.lib.fa_set_kernel_policy(1 if forced else 0)
    try:
        out, lse = m3.flash_attn_mla_with_kvcache(qn.cuda(), qr.cuda(), lat.cuda(), sc.cuda(), rope.cuda(),
                                                  torch.tensor(lens, dtype=torch.int32).cuda(), table.cuda(),
                                                  num_splits=splits, return_softmax_lse=True)
        torch.cuda.synchronize()
    finally:
        capi.lib.fa_set_kernel_policy(0)
    assert capi.last_kernel() == family.split(":")[-1]
    assert capi.lib.fa_debug_get(2) == 0
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse.cpu(), f_l)


def test_mla_key_range_partials_recombine():
    """Sequences sharded over the key range (the cross-device mode): partial (O, LSE) per range, combined,
    equal the unsharded call."""
    import flash_attn_npu_3 as m3
    from flash_attn_npu_3 import flash_attn_npu_3 as ext
    gen = torch.Generator().manual_seed(77)
    b, h, lens = 2, 128, [3000, 900]
    qn, qr, lat, sc, rope, table = make_case(gen, b, h, lens)
    args = [t.cuda() for t in (qn, qr, lat, sc, rope, table)] + [torch.tensor(lens, dtype=torch.int32).cuda()]
    full, full_lse = ext.mla_decode(*args, 576 ** -0.5)
    shards, per = 4, 768
    po = torch.empty(shards, b * h, 512, device="cuda")
    pl = torch.empty(shards, b * h, device="cuda")
    for s in range(shards):
        ext.mla_decode(*args, 576 ** -0.5, 0, kv_range=(s * per, (s + 1) * per), partials=(po[s], pl[s]))
    out, lse = m3.flash_attn_combine(po, pl, out_dtype=torch.bfloat16)
    assert (out.reshape(b, 1, h, 512).float() - full.float()).abs().max().item() <= 2 ** -7
    assert (lse.reshape(b, h, 1) - full_lse).abs().max().item() < 1e-4
