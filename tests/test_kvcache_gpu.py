"""flash_attn_with_kvcache on the GPU: paged gathers, in-place append and rotary (bit-exact),
split-KV and combine, GQA stacking, the v3 packed-q path and the scheduler metadata."""
import os

import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_lse, assert_within

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def paged_setup(gen, b, lens, hkv, d, page, dt, extra=1, scale=1.0):
    nblk = [(l + extra + page - 1) // page for l in lens]
    pool = sum(nblk)
    perm = torch.randperm(pool, generator=gen).int()
    table = torch.zeros(b, max(nblk), dtype=torch.int32)
    off = 0
    for i, n in enumerate(nblk):
        table[i, :n] = perm[off:off + n]
        off += n
    kc = (torch.randn(pool, page, hkv, d, generator=gen) * scale).to(dt)
    vc = (torch.randn(pool, page, hkv, d, generator=gen) * scale).to(dt)
    return kc, vc, table


def test_paged_fixture_from_reference_golden():
    import flash_attn_npu as m
    fx = torch.load(os.path.join(GOLD, "paged_case.pt"), weights_only=False)
    lens = torch.tensor(fx["cache_seqlens"], dtype=torch.int32)
    for ns in (0, 1, 3):
        out, lse = m.flash_attn_with_kvcache(fx["q"].cuda(), fx["k_cache"].cuda(), fx["v_cache"].cuda(),
                                             cache_seqlens=lens.cuda(), block_table=fx["block_table"].cuda(),
                                             softmax_scale=fx["scale"], causal=True, num_splits=ns,
                                             return_softmax_lse=True)
        assert (out.cpu().float() - fx["out"].float()).abs().max().item() <= 2 ** -6
        assert_lse(lse, fx["lse"])


# (dtype, B, H, Hkv, Sq, Sk, D, paged, causal, wl, wr, softcap) -- tests/test_flash_attn_npu_v2.py:145-286
CASES = [
    (torch.bfloat16, 1, 1, 1, 1, 1024, 128, 1, True, -1, -1, 0.0),
    (torch.bfloat16, 2, 4, 4, 1024, 1024, 128, 1, True, -1, -1, 0.0),
    (torch.float16, 3, 1, 1, 512, 512, 128, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 1, 1, 1, 4096, 128, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 6, 2, 2, 1024, 128, 1, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 1, 1, 1024, 1024, 128, 1, True, 512, 256, 0.0),
    (torch.float16, 1, 128, 1, 1, 1024, 128, 0, True, 542, 647, 0.0),
    (torch.bfloat16, 4, 32, 8, 1, 2048, 128, 0, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 64, 8, 1, 4096, 128, 0, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 128, 8, 1, 4096, 128, 0, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 32, 4, 16, 1024, 256, 0, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 32, 4, 1, 2048, 128, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 128, 4, 1, 2048, 128, 1, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 32, 8, 1, 2048, 256, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 16, 2, 5, 4096, 128, 1, True, -1, -1, 0.0),
    (torch.bfloat16, 1, 32, 8, 13, 2048, 256, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 32, 8, 65, 2048, 128, 0, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 10, 2, 15, 2048, 128, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 3, 1, 128, 2048, 1, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 2, 256, 16, 8, 640, 1, 1, False, -1, -1, 0.0),
    (torch.bfloat16, 1, 32, 4, 4, 2048, 128, 1, False, -1, -1, 30.0),
    (torch.bfloat16, 1, 64, 4, 8, 2048, 128, 1, True, -1, -1, 30.0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
def test_kvcache_matrix(case):
    import flash_attn_npu as m
    dt, b, h, hkv, sq, sk, d, paged, causal, wl, wr, cap = case
    page = 128
    q = (torch.rand(b, sq, h, d) * 10 - 5).to(dt)
    if paged:
        nb = (sk + page - 1) // page
        kc = (torch.rand(max(64, nb * b), page, hkv, d) * 10 - 5).to(dt)
        vc = (torch.rand(max(64, nb * b), page, hkv, d) * 10 - 5).to(dt)
        table = torch.arange(nb * b, dtype=torch.int32).reshape(b, nb)
    else:
        kc = (torch.rand(b, sk, hkv, d) * 10 - 5).to(dt)
        vc = (torch.rand(b, sk, hkv, d) * 10 - 5).to(dt)
        table = None
    lens = torch.full((b,), sk, dtype=torch.int32)
    scale = d ** -0.5
    lp_o, _ = orc.kvcache_fwd(q, kc.clone(), vc.clone(), lens, scale, block_table=table, causal=causal, window=(wl, wr), softcap=cap)
    f_o, f_l = orc.kvcache_fwd(q.float(), kc.float(), vc.float(), lens, scale, block_table=table, causal=causal,
                               window=(wl, wr), softcap=cap)
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens.cuda(),
                                         block_table=None if table is None else table.cuda(), softmax_scale=scale,
                                         causal=causal, window_size=(wl, wr), softcap=cap, return_softmax_lse=True)
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


# (dtype, B, H, Hkv, Sq, D, paged, causal, window, softcap): 17 to 64 stacked rows (Sq x group) a KV head
WIDE_CASES = [
    (torch.bfloat16, 3, 32, 4, 4, 128, True, True, (-1, -1), 0.0),       # 32 rows: four new tokens a step, group of 8
    (torch.bfloat16, 2, 32, 1, 1, 128, False, False, (-1, -1), 0.0),     # 32 rows: one token, group of 32 (multi-query)
    (torch.float16, 2, 16, 2, 5, 64, True, True, (-1, -1), 0.0),         # 40 rows: the last warp is half empty
    (torch.bfloat16, 2, 16, 2, 8, 128, True, True, (300, 0), 0.0),       # 64 rows, sliding window
    (torch.bfloat16, 1, 48, 3, 3, 256, False, True, (-1, -1), 0.0),      # 48 rows, head dim 256 (16-token tiles)
    (torch.bfloat16, 2, 24, 8, 6, 128, True, False, (-1, -1), 25.0),     # 18 rows, softcap
]


@pytest.mark.parametrize("case", WIDE_CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
@pytest.mark.parametrize("num_splits", [0, 1, 5])
def test_decode_with_17_to_64_stacked_rows(case, num_splits):
    """Several new tokens a step and large query groups stack more than 16 rows on a KV head.  A power-of-two group at
    head dim <= 128 runs on the tcgen05 forward with the group stacked into the tile rows and the keys split over CTAs
    (partials + combine; one split, the planner's count and a forced count of 5); other groups and head dim 256 run on
    the decode kernel's form in which four warps share a head's tiles.  Ragged device-resident lengths (one shorter
    than a tile), NaN past the lengths."""
    import flash_attn_npu as m
    import fa_b200_capi as capi
    dt, b, h, hkv, sq, d, paged, causal, win, cap = case
    gen = torch.Generator().manual_seed(5 + h + sq)
    lens = [1500, 9, 777][:b]
    page, capacity = 64, 2048
    q = torch.randn(b, sq, h, d, generator=gen).to(dt)
    if paged:
        kc, vc, table = paged_setup(gen, b, [capacity - 1] * b, hkv, d, page, dt)
        for i, L in enumerate(lens):
            for j in range(table.shape[1]):
                lo = max(0, L - j * page)
                if lo < page:
                    kc[table[i, j], lo:] = float("nan")
                    vc[table[i, j], lo:] = float("nan")
    else:
        kc, vc, table = torch.randn(b, capacity, hkv, d, generator=gen).to(dt), torch.randn(b, capacity, hkv, d, generator=gen).to(dt), None
        for i, L in enumerate(lens):
            kc[i, L:] = float("nan")
            vc[i, L:] = float("nan")
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    rk, rv = torch.nan_to_num(kc.clone()), torch.nan_to_num(vc.clone())
    lp_o, _ = orc.kvcache_fwd(q, rk.clone(), rv.clone(), lens_t, scale, block_table=table, causal=causal, window=win, softcap=cap)
    f_o, f_l = orc.kvcache_fwd(q.float(), rk.float(), rv.float(), lens_t, scale, block_table=table, causal=causal, window=win,
                               softcap=cap)
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens_t.cuda(),
                                         block_table=None if table is None else table.cuda(), softmax_scale=scale,
                                         causal=causal, window_size=win, softcap=cap, num_splits=num_splits,
                                         return_softmax_lse=True)
    torch.cuda.synchronize()
    g_ = h // hkv
    stacked = d <= 128 and g_ & (g_ - 1) == 0
    assert capi.last_kernel() == ("sm100_tcgen05_2q" if stacked else "decode_splitkv_tma")
    assert capi.lib.fa_debug_get(2) == 0
    assert torch.isfinite(out).all()
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("paged", [True, False])
@pytest.mark.parametrize("s_new,sq,causal", [(1, 1, True), (3, 3, True), (2, 5, False)])
def test_append_and_rotary_bit_exact(interleaved, paged, s_new, sq, causal):
    """KV append and block_table gathers are bit-exact: every appended row equals the oracle's bits (rotary in
    fp32 with separately rounded products), and no other cache byte changes."""
    import flash_attn_npu as m
    gen = torch.Generator().manual_seed(21 + s_new)
    b, h, hkv, d, page, rd = 3, 8, 2, 128, 64, 64
    lens = [70, 127, 200]
    dt = torch.bfloat16
    if paged:
        kc, vc, table = paged_setup(gen, b, lens, hkv, d, page, dt, extra=s_new)
    else:
        kc = torch.randn(b, 256, hkv, d, generator=gen).to(dt)
        vc = torch.randn(b, 256, hkv, d, generator=gen).to(dt)
        table = None
    q = torch.randn(b, sq, h, d, generator=gen).to(dt)
    kn = torch.randn(b, s_new, hkv, d, generator=gen).to(dt)
    vn = torch.randn(b, s_new, hkv, d, generator=gen).to(dt)
    cos, sin = orc.rotary_tables(512, rd, dtype=dt)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref_o, ref_l = orc.kvcache_fwd(q, kc_ref, vc_ref, lens, d ** -0.5, k_new=kn, v_new=vn, rotary_cos=cos, rotary_sin=sin,
                                   rotary_interleaved=interleaved, block_table=table, causal=causal)
    kc32, vc32 = kc.clone(), vc.clone()
    f_o, f_l = orc.kvcache_fwd(q, kc32, vc32, lens, d ** -0.5, k_new=kn, v_new=vn, rotary_cos=cos, rotary_sin=sin,
                               rotary_interleaved=interleaved, block_table=table, causal=causal)
    kg, vg = kc.cuda(), vc.cuda()
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kg, vg, kn.cuda(), vn.cuda(), rotary_cos=cos.cuda(), rotary_sin=sin.cuda(),
                                         cache_seqlens=lens_t.cuda(), block_table=None if table is None else table.cuda(),
                                         causal=causal, rotary_interleaved=interleaved, return_softmax_lse=True)
    assert torch.equal(kg.cpu().view(torch.int16), kc_ref.view(torch.int16)), "K cache differs from the oracle's bits"
    assert torch.equal(vg.cpu().view(torch.int16), vc_ref.view(torch.int16)), "V cache differs from the oracle's bits"
    assert not torch.equal(kc_ref, kc)
    assert (out.cpu().float() - ref_o.float()).abs().max().item() <= 2 ** -6
    assert_lse(lse, ref_l)


def test_config4_shape_small_with_splits():
    """Configuration 4 scaled down: GQA 32/8, D128, page 256, permuted table, append + rotary, varied lengths."""
    import flash_attn_npu as m
    gen = torch.Generator().manual_seed(4)
    b, h, hkv, d, page = 6, 32, 8, 128, 256
    lens = torch.randint(100, 5000, (b,), generator=gen).tolist()
    dt = torch.bfloat16
    kc, vc, table = paged_setup(gen, b, lens, hkv, d, page, dt)
    q = torch.randn(b, 1, h, d, generator=gen).to(dt)
    kn = torch.randn(b, 1, hkv, d, generator=gen).to(dt)
    vn = torch.randn(b, 1, hkv, d, generator=gen).to(dt)
    cos, sin = orc.rotary_tables(8192, 128, dtype=dt)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    kr, vr = kc.clone(), vc.clone()
    ref_o, ref_l = orc.kvcache_fwd(q, kr, vr, lens, d ** -0.5, k_new=kn, v_new=vn, rotary_cos=cos, rotary_sin=sin,
                                   rotary_interleaved=False, block_table=table, causal=True)
    kf, vf = kc.float(), vc.float()
    cosf, sinf = cos, sin
    for ns in (0, 1, 5):
        kg, vg = kc.cuda(), vc.cuda()
        out, lse = m.flash_attn_with_kvcache(q.cuda(), kg, vg, kn.cuda(), vn.cuda(), rotary_cos=cos.cuda(),
                                             rotary_sin=sin.cuda(), cache_seqlens=lens_t.cuda(), block_table=table.cuda(),
                                             causal=True, rotary_interleaved=False, num_splits=ns, return_softmax_lse=True)
        assert torch.equal(kg.cpu().view(torch.int16), kr.view(torch.int16))
        assert torch.equal(vg.cpu().view(torch.int16), vr.view(torch.int16))
        assert (out.cpu().float() - ref_o.float()).abs().max().item() <= 2 ** -6
        assert_lse(lse, ref_l)


def test_cache_batch_idx_and_int_seqlens():
    import flash_attn_npu as m
    torch.manual_seed(8)
    kc, vc = torch.randn(5, 300, 2, 64).bfloat16(), torch.randn(5, 300, 2, 64).bfloat16()
    q = torch.randn(2, 1, 4, 64).bfloat16()
    idx = torch.tensor([3, 1], dtype=torch.int32)
    ref_o, ref_l = orc.kvcache_fwd(q, kc, vc, [222, 222], 0.125, cache_batch_idx=idx)
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=222, cache_batch_idx=idx.cuda(),
                                         return_softmax_lse=True)
    assert (out.cpu().float() - ref_o.float()).abs().max().item() <= 2 ** -6
    assert_lse(lse, ref_l)


@pytest.mark.parametrize("num_splits", [0, 2])
def test_v3_packed_q_paged_varied_lengths(num_splits):
    """v3 kvcache with packed q (cu_seqlens_q), paged cache and per-sequence lengths
    (tests/test_flash_attn_npu_v3.py:305-331)."""
    import flash_attn_npu_3 as m3
    gen = torch.Generator().manual_seed(1234)
    b, h, hkv, d, page = 4, 8, 2, 128, 128
    lq = torch.randint(1, 17, (b,), generator=gen).tolist()
    lk = [int(torch.randint(q_, 1500, (1,), generator=gen)) for q_ in lq]
    dt = torch.bfloat16
    kc, vc, table = paged_setup(gen, b, lk, hkv, d, page, dt, extra=0, scale=2.0)
    q = (torch.randn(sum(lq), h, d, generator=gen) * 2).to(dt)
    cu_q = torch.tensor([0] + torch.tensor(lq).cumsum(0).tolist(), dtype=torch.int32)
    out, lse, *_ = m3.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=torch.tensor(lk, dtype=torch.int32).cuda(),
                                              page_table=table.cuda(), cu_seqlens_q=cu_q.cuda(), max_seqlen_q=max(lq), causal=True,
                                              num_splits=num_splits, return_softmax_lse=True)
    o = 0
    for i in range(b):
        ki = orc.gather_paged(kc, table[i], lk[i])
        vi = orc.gather_paged(vc, table[i], lk[i])
        qi = q[o:o + lq[i]].unsqueeze(0)
        r_o, r_l = orc.attention_fwd(qi, ki.unsqueeze(0), vi.unsqueeze(0), d ** -0.5, True)
        assert (out[o:o + lq[i]].cpu().float() - r_o[0].float()).abs().max().item() <= 2 ** -5
        assert_lse(lse[:, o:o + lq[i]], r_l[0])
        o += lq[i]


def test_combine_entry_point_matches_oracle():
    import flash_attn_npu_3 as m3
    torch.manual_seed(9)
    op = torch.randn(5, 3, 7, 64)
    lp = torch.randn(5, 3, 7) * 3
    lp[2] = float("-inf")
    lp[:, 1, 3] = float("-inf")
    out, lse = m3.flash_attn_combine(op.cuda(), lp.cuda(), out_dtype=torch.float32)
    r_o, r_l = orc.combine_partials(op.reshape(5, 21, 64), lp.reshape(5, 21), torch.float32)
    assert (out.cpu().reshape(21, 64) - r_o).abs().max().item() < 1e-5
    assert orc.max_abs_err(lse.cpu().reshape(21), r_l) < 1e-5


def test_kv_range_partials_recombine_to_the_full_result():
    """The cross-device mode: every shard attends to a key range and leaves fp32 (O, LSE); combining the shards'
    partials equals the unsharded call."""
    import flash_attn_npu as m
    import flash_attn_npu_3 as m3
    from flash_attn_npu import flash_attn_npu as ext
    gen = torch.Generator().manual_seed(10)
    b, h, hkv, d, page = 3, 8, 2, 128, 64
    lens = [900, 130, 2000]
    kc, vc, table = paged_setup(gen, b, lens, hkv, d, page, torch.bfloat16, extra=0)
    q = torch.randn(b, 1, h, d, generator=gen).bfloat16()
    lens_t = torch.tensor(lens, dtype=torch.int32).cuda()
    full, full_lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens_t, block_table=table.cuda(),
                                               return_softmax_lse=True)
    shards = 4
    per = (max(lens) + shards * page - 1) // (shards * page) * page
    po = torch.empty(shards, b * h, d, device="cuda")
    pl = torch.empty(shards, b * h, device="cuda")
    for s in range(shards):
        ext.kvcache_forward(q.cuda(), kc.cuda(), vc.cuda(), None, None, lens_t, None, None, None, table.cuda(), None, None,
                            d ** -0.5, False, -1, -1, 0.0, False, 0, kv_range=(s * per, (s + 1) * per), partials=(po[s], pl[s]))
    out, lse = m3.flash_attn_combine(po, pl, out_dtype=torch.bfloat16)
    assert (out.reshape(b, 1, h, d).float() - full.float()).abs().max().item() <= 2 ** -7
    assert (lse.reshape(b, h, 1) - full_lse).abs().max().item() < 1e-4


def test_scheduler_metadata_blob_layout():
    """The device-built blob against the same plan worked out on the host from the lengths (layout: sched_meta.cu)."""
    import flash_attn_npu_3 as m3
    lens = torch.tensor([1000, 64, 65, 7000, 1], dtype=torch.int32)
    meta = m3.get_scheduler_metadata(5, 1, 8192, 32, 8, 128, lens.cuda(), page_size=256, causal=True).view(torch.int32).cpu()
    assert meta.numel() == 8 + 8 * 5
    assert meta[0].item() == 0x46413130 and meta[1].item() == 5
    nsplit, bps = meta[2].item(), meta[3].item()
    assert meta[4].item() == 7000
    nb = [(l + 63) // 64 for l in lens.tolist()]
    assert meta[5].item() == sum(nb)
    run = 0
    for i, l in enumerate(lens.tolist()):
        act = min(nsplit, (nb[i] + bps - 1) // bps)
        per = ((l + act - 1) // act + 63) // 64 * 64
        assert meta[8 + 8 * i: 13 + 8 * i].tolist() == [l, nb[i], act, per, run]
        assert act * per >= l
        run += act
    assert meta[6].item() == run


def test_scheduler_metadata_is_consumed_by_the_decode():
    """Configuration 4's length spread, scaled down: with the blob every sequence spreads its keys evenly over the
    splits it needs, so fewer (sequence, split) pairs are active than the grid has and no active split is nearly
    empty; the result matches the oracle exactly as the call without the blob does.  A blob built for other
    lengths is ignored (the call still gives the right answer)."""
    import flash_attn_npu_3 as m3
    import fa_b200_capi as capi
    gen = torch.Generator().manual_seed(14)
    b, h, hkv, d, page = 16, 32, 8, 128, 256
    lens = torch.randint(1024, 32769, (b,), generator=gen, dtype=torch.int32)
    kc, vc, table = paged_setup(gen, b, lens.tolist(), hkv, d, page, torch.bfloat16, extra=0)
    q = torch.randn(b, 1, h, d, generator=gen).bfloat16()
    cap = table.shape[1] * page
    meta = m3.get_scheduler_metadata(b, 1, cap, h, hkv, d, lens.cuda(), page_size=page, causal=True)
    hdr = meta.view(torch.int32).cpu()
    nsplit, active = hdr[2].item(), hdr[6].item()
    assert nsplit > 1 and active < b * nsplit                       # a grid of b x nsplit, only `active` pairs do work
    kg, vg, tg, lg, qg = kc.cuda(), vc.cuda(), table.cuda(), lens.cuda(), q.cuda()
    with_blob, lse_a, *_ = m3.flash_attn_with_kvcache(qg, kg, vg, cache_seqlens=lg, page_table=tg, causal=True,
                                                      scheduler_metadata=meta, return_softmax_lse=True)
    assert capi.last_kernel() == "decode_splitkv_tma"
    without, lse_b, *_ = m3.flash_attn_with_kvcache(qg, kg, vg, cache_seqlens=lg, page_table=tg, causal=True, return_softmax_lse=True)
    # What the kernel did with the blob, seen through the partial LSEs it left in the workspace of a call made
    # straight through the C-ABI: a split without keys leaves -inf.  With the blob exactly the planned number of
    # splits per sequence carry keys and every one of them carries its even share.
    from fa_b200_capi import FwdParams, tensor4
    out_c, lse_c = torch.empty_like(qg), torch.empty(b, h, 1, device="cuda")
    p = FwdParams()
    p.q, p.k, p.v, p.o = tensor4(qg), tensor4(kg), tensor4(vg), tensor4(out_c)
    p.kv_entries = kg.shape[0]
    p.lse, p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = lse_c.data_ptr(), lse_c.stride(0), lse_c.stride(1), lse_c.stride(2)
    p.block_table, p.block_table_stride, p.page_size, p.seqused_k = tg.data_ptr(), tg.stride(0), page, lg.data_ptr()
    p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv = b, 1, cap, h, hkv, d, d
    p.scale, p.causal, p.window_left, p.window_right, p.dtype = d ** -0.5, 1, -1, -1, 1
    p.stream = torch.cuda.current_stream().cuda_stream
    assert capi.lib.fa_fwd_num_splits(p) == nsplit
    ws = torch.zeros(capi.lib.fa_fwd_workspace_bytes(p), dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    rows = b * h
    o_bytes = (nsplit * rows * d * 4 + 255) // 256 * 256
    plan = hdr[8:].reshape(b, 8)
    for blob in (None, meta):
        p.sched_meta = None if blob is None else blob.data_ptr()
        assert capi.lib.fa_fwd_kvcache(p) == 0, capi.lib.fa_last_error()
        torch.cuda.synchronize()
        part = ws[o_bytes: o_bytes + nsplit * rows * 4].view(torch.float32).view(nsplit, b, h)
        used = torch.isfinite(part[:, :, 0]).sum(0).cpu()                # splits with keys, per sequence
        if blob is None:
            uniform_used = used
        else:
            assert used.tolist() == plan[:, 2].tolist()                   # the blob's active splits, no more, no fewer
            assert (used <= uniform_used).all() and used.sum().item() == active
        assert torch.equal(out_c, with_blob if blob is not None else without)
    for i in torch.argsort(lens).tolist()[:3]:
        L = int(lens[i])
        ki, vi = orc.gather_paged(kc, table[i], L).unsqueeze(0), orc.gather_paged(vc, table[i], L).unsqueeze(0)
        lp_o, _ = orc.attention_fwd(q[i:i + 1], ki, vi, d ** -0.5, True)
        f_o, f_l = orc.attention_fwd(q[i:i + 1].float(), ki.float(), vi.float(), d ** -0.5, True, data_type=torch.float32)
        for out, lse in ((with_blob, lse_a), (without, lse_b)):
            assert_within("out", out[i:i + 1].cpu(), lp_o, f_o)
            assert_lse(lse[i:i + 1], f_l)
    assert (with_blob.float() - without.float()).abs().max().item() <= 2 ** -7
    stale = m3.get_scheduler_metadata(b, 1, cap, h, hkv, d, (lens // 2).cuda(), page_size=page, causal=True)
    again = m3.flash_attn_with_kvcache(qg, kg, vg, cache_seqlens=lg, page_table=tg, causal=True, scheduler_metadata=stale)
    assert torch.equal(again, without)                              # ignored: the host's uniform plan ran
    other = m3.get_scheduler_metadata(b + 1, 1, cap, h, hkv, d, torch.cat((lens, lens[:1])).cuda(), page_size=page, causal=True)
    again = m3.flash_attn_with_kvcache(qg, kg, vg, cache_seqlens=lg, page_table=tg, causal=True, scheduler_metadata=other)
    assert torch.equal(again, without)
    with pytest.raises(RuntimeError):
        m3.flash_attn_with_kvcache(qg, kg, vg, cache_seqlens=lg, page_table=tg, causal=True, scheduler_metadata=meta[:16])


@pytest.mark.parametrize("paged,page", [(True, 128), (True, 256), (True, 64), (True, 192), (False, 0)])
@pytest.mark.parametrize("append", [False, True])
def test_prefill_against_cache_uses_tcgen05(paged, page, append):
    """A chunk of queries against a KV cache (chunked prefill): ragged device-resident lengths, GQA, optional
    in-place append of the chunk's own keys, cache rows past the lengths filled with NaN (they must not leak
    into the output); the tcgen05 kernel serves the call.  Pages of 64 and 192 tokens make key tiles that span two
    pages (copied as two boxes of 64 rows)."""
    import flash_attn_npu as m
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(321)
    dt, b, h, hkv, sq, d = torch.bfloat16, 3, 8, 2, 200, 128
    lens = [700, 1, 1337]
    cap = 2048
    q = torch.randn(b, sq, h, d, generator=g).to(dt)
    kn = torch.randn(b, sq, hkv, d, generator=g).to(dt) if append else None
    vn = torch.randn(b, sq, hkv, d, generator=g).to(dt) if append else None
    if paged:
        nb = cap // page
        kc = torch.randn(nb * b + 3, page, hkv, d, generator=g).to(dt)
        vc = torch.randn(nb * b + 3, page, hkv, d, generator=g).to(dt)
        table = torch.randperm(nb * b + 3, generator=g)[: nb * b].int().reshape(b, nb)
        for i, L in enumerate(lens):                         # poison everything past the (appended) length
            end = L + (sq if append else 0)
            for j in range(nb):
                lo = max(0, end - j * page)
                if lo < page:
                    kc[table[i, j], lo:] = float("nan")
                    vc[table[i, j], lo:] = float("nan")
    else:
        kc = torch.randn(b, cap, hkv, d, generator=g).to(dt)
        vc = torch.randn(b, cap, hkv, d, generator=g).to(dt)
        table = None
        for i, L in enumerate(lens):
            end = L + (sq if append else 0)
            kc[i, end:] = float("nan")
            vc[i, end:] = float("nan")
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    # a dense cache read without append also goes through cache_batch_idx (entry i of the batch uses cache row idx[i])
    idx = None
    if not paged and not append:
        idx = torch.tensor([2, 0, 1], dtype=torch.int32)
        inv = torch.argsort(idx.long())
        kc, vc = kc[inv].contiguous(), vc[inv].contiguous()     # row idx[i] of the cache now holds entry i
    ref_k, ref_v = torch.nan_to_num(kc.clone()), torch.nan_to_num(vc.clone())
    lp_o, _ = orc.kvcache_fwd(q, ref_k.clone(), ref_v.clone(), lens_t, scale, k_new=kn, v_new=vn, block_table=table,
                              cache_batch_idx=idx, causal=True)
    f_o, f_l = orc.kvcache_fwd(q.float(), ref_k.float(), ref_v.float(), lens_t, scale, k_new=None if kn is None else kn.float(),
                               v_new=None if vn is None else vn.float(), block_table=table, cache_batch_idx=idx, causal=True)
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), None if kn is None else kn.cuda(),
                                         None if vn is None else vn.cuda(), cache_seqlens=lens_t.cuda(),
                                         cache_batch_idx=None if idx is None else idx.cuda(),
                                         block_table=None if table is None else table.cuda(), softmax_scale=scale,
                                         causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_2q"
    assert capi.lib.fa_debug_get(2) == 0
    assert torch.isfinite(out).all()
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


def test_short_chunk_with_many_stacked_rows_runs_on_tcgen05():
    """32 new tokens a sequence under a query group of 8 are 256 stacked rows a KV head: too many for the split-KV
    decode kernel, fewer than 64 rows a head; the tcgen05 forward takes the call with the group stacked into its tile
    rows (rows past the chunk are zero-filled by the tile copy).  Append + causal, ragged lengths."""
    import flash_attn_npu as m
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(7)
    dt, b, h, hkv, sq, d, page = torch.bfloat16, 4, 32, 4, 32, 128, 128
    lens = [900, 17, 2000, 1024]
    q = torch.randn(b, sq, h, d, generator=g).to(dt)
    kn, vn = torch.randn(b, sq, hkv, d, generator=g).to(dt), torch.randn(b, sq, hkv, d, generator=g).to(dt)
    kc, vc, table = paged_setup(g, b, [2200] * b, hkv, d, page, dt)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    lp_o, _ = orc.kvcache_fwd(q, kc.clone(), vc.clone(), lens_t, scale, k_new=kn, v_new=vn, block_table=table, causal=True)
    f_o, f_l = orc.kvcache_fwd(q.float(), kc.float(), vc.float(), lens_t, scale, k_new=kn.float(), v_new=vn.float(),
                               block_table=table, causal=True)
    kg, vg = kc.cuda(), vc.cuda()
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kg, vg, kn.cuda(), vn.cuda(), cache_seqlens=lens_t.cuda(),
                                         block_table=table.cuda(), softmax_scale=scale, causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_2q"
    assert capi.lib.fa_debug_get(2) == 0
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)
    # a single sequence does not fill the GPU with (sequence, KV head) CTAs: the same kernel then splits the keys over
    # CTAs and the partials are combined (the cache now holds the appended chunk)
    out1 = m.flash_attn_with_kvcache(q[:1].cuda(), kg, vg, cache_seqlens=lens_t[:1].cuda() + sq,
                                     block_table=table[:1].cuda(), softmax_scale=scale, causal=True)
    assert capi.last_kernel() == "sm100_tcgen05_2q"
    assert_within("single sequence", out1.cpu(), lp_o[:1], f_o[:1])


@pytest.mark.parametrize("page", [64, 256])
def test_prefill_against_cache_with_head_dim_256(page):
    """Chunked prefill at head dim 256 (the one-tile tcgen05 kernel): paged cache, in-place append of the chunk, GQA,
    ragged lengths, NaN past the appended length."""
    import flash_attn_npu as m
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(99)
    dt, b, h, hkv, sq, d = torch.bfloat16, 2, 4, 2, 150, 256
    lens, cap = [500, 1111], 2048
    q = torch.randn(b, sq, h, d, generator=g).to(dt)
    kn, vn = torch.randn(b, sq, hkv, d, generator=g).to(dt), torch.randn(b, sq, hkv, d, generator=g).to(dt)
    nb = cap // page
    kc = torch.randn(nb * b + 2, page, hkv, d, generator=g).to(dt)
    vc = torch.randn(nb * b + 2, page, hkv, d, generator=g).to(dt)
    table = torch.randperm(nb * b + 2, generator=g)[: nb * b].int().reshape(b, nb)
    for i, L in enumerate(lens):
        for j in range(nb):
            lo = max(0, L + sq - j * page)
            if lo < page:
                kc[table[i, j], lo:] = float("nan")
                vc[table[i, j], lo:] = float("nan")
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    rk, rv = torch.nan_to_num(kc.clone()), torch.nan_to_num(vc.clone())
    lp_o, _ = orc.kvcache_fwd(q, rk.clone(), rv.clone(), lens_t, scale, k_new=kn, v_new=vn, block_table=table, causal=True)
    f_o, f_l = orc.kvcache_fwd(q.float(), rk.float(), rv.float(), lens_t, scale, k_new=kn.float(), v_new=vn.float(),
                               block_table=table, causal=True)
    out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), kn.cuda(), vn.cuda(), cache_seqlens=lens_t.cuda(),
                                         block_table=table.cuda(), softmax_scale=scale, causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    assert capi.last_kernel() == "sm100_tcgen05_wide"
    assert capi.lib.fa_debug_get(2) == 0
    assert torch.isfinite(out).all()
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


@pytest.mark.parametrize("paged", [True, False])
def test_oversized_cache_seqlens_are_truncated_and_append_nothing(paged):
    """A stale or oversized cache_seqlens entry (the host never sees the device-resident lengths) must not make any
    kernel index past the page-table row or the cache: such a length is truncated to the capacity and its append is
    dropped.  The cache and the table carry sentinel padding so that every access stays inside the allocations with
    or without the guard; the sentinels must come back untouched."""
    import flash_attn_npu as m
    gen = torch.Generator().manual_seed(77)
    b, h, hkv, d, page, dt = 3, 8, 2, 128, 64, torch.bfloat16
    cap_blocks = 4                                                   # capacity: 256 keys a sequence
    guard = 8                                                        # sentinel pages / table columns
    q = torch.randn(b, 1, h, d, generator=gen).to(dt)
    kn, vn = torch.randn(b, 1, hkv, d, generator=gen).to(dt), torch.randn(b, 1, hkv, d, generator=gen).to(dt)
    lens = torch.tensor([100, 256, 100000], dtype=torch.int32)      # fine, full (append would overflow), stale
    if paged:
        pool = b * cap_blocks
        kc = torch.randn(pool + guard, page, hkv, d, generator=gen).to(dt)
        vc = torch.randn(pool + guard, page, hkv, d, generator=gen).to(dt)
        big = torch.full((b, cap_blocks + guard), pool + guard - 1, dtype=torch.int32)     # sentinel columns name the last sentinel page
        big[:, :cap_blocks] = torch.arange(pool, dtype=torch.int32).reshape(b, cap_blocks)
        table = big[:, :cap_blocks]                                  # a view: row stride cap_blocks + guard, width cap_blocks
        assert table.stride(0) == cap_blocks + guard
    else:
        kc = torch.randn(b + 1, cap_blocks * page + guard * page, hkv, d, generator=gen).to(dt)
        vc = torch.randn(b + 1, cap_blocks * page + guard * page, hkv, d, generator=gen).to(dt)
        table = None
    kg, vg = kc.cuda(), vc.cuda()
    if paged:
        tg = big.cuda()[:, :cap_blocks]
        k_view, v_view = kg, vg
    else:
        tg = None
        k_view, v_view = kg[:b, :cap_blocks * page], vg[:b, :cap_blocks * page]     # capacity = 256 rows of a longer allocation
    out, lse = m.flash_attn_with_kvcache(q.cuda(), k_view, v_view, kn.cuda(), vn.cuda(), cache_seqlens=lens.cuda(),
                                         block_table=tg, causal=True, return_softmax_lse=True)
    torch.cuda.synchronize()
    k_after, v_after = kg.cpu(), vg.cpu()
    # sequence 0 appended one row at position 100; sequences 1 and 2 appended nothing; sentinels untouched
    exp_k, exp_v = kc.clone(), vc.clone()
    if paged:
        exp_k[int(big[0, 100 // page]), 100 % page], exp_v[int(big[0, 100 // page]), 100 % page] = kn[0, 0], vn[0, 0]
    else:
        exp_k[0, 100], exp_v[0, 100] = kn[0, 0], vn[0, 0]
    assert torch.equal(k_after.view(torch.int16), exp_k.view(torch.int16))
    assert torch.equal(v_after.view(torch.int16), exp_v.view(torch.int16))
    # sequence 0 is an ordinary call; the truncated ones attend to their 256 cached keys
    cap = cap_blocks * page
    for i, L in ((0, 101), (1, cap), (2, cap)):
        if paged:
            ki = orc.gather_paged(exp_k, big[i], L).unsqueeze(0)
            vi = orc.gather_paged(exp_v, big[i], L).unsqueeze(0)
        else:
            ki, vi = exp_k[i:i + 1, :L], exp_v[i:i + 1, :L]
        lp_o, _ = orc.attention_fwd(q[i:i + 1], ki, vi, d ** -0.5, True)
        f_o, f_l = orc.attention_fwd(q[i:i + 1].float(), ki.float(), vi.float(), d ** -0.5, True, data_type=torch.float32)
        assert_within(f"out[{i}]", out[i:i + 1].cpu(), lp_o, f_o)
        assert_lse(lse[i:i + 1], f_l)


@pytest.mark.parametrize("sq,h,hkv,kernel", [(1, 8, 2, "decode_splitkv_tma"), (4, 16, 2, "sm100_tcgen05_2q"), (70, 4, 2, "sm100_tcgen05_2q")])
def test_dense_cache_whose_capacity_is_not_a_multiple_of_the_tile(sq, h, hkv, kernel):
    """A dense cache of 333 rows: the last 128-key tile (32-key tile in the decode kernel) reaches past the capacity, the
    tile copy zero-fills those rows, and the rows between a sequence's length and the capacity hold NaN.  Sequences that
    end in the last tile, at the capacity itself and one row before it."""
    import flash_attn_npu as m
    import fa_b200_capi as capi
    gen = torch.Generator().manual_seed(333 + sq)
    b, cap, d, dt = 3, 333, 128, torch.bfloat16
    lens = [333, 332, 270]
    q = torch.randn(b, sq, h, d, generator=gen).to(dt)
    kc = torch.randn(b, cap, hkv, d, generator=gen).to(dt)
    vc = torch.randn(b, cap, hkv, d, generator=gen).to(dt)
    for i, L in enumerate(lens):
        kc[i, L:] = float("nan")
        vc[i, L:] = float("nan")
    lens_t = torch.tensor(lens, dtype=torch.int32)
    scale = d ** -0.5
    rk, rv = torch.nan_to_num(kc.clone()), torch.nan_to_num(vc.clone())
    lp_o, _ = orc.kvcache_fwd(q, rk.clone(), rv.clone(), lens_t, scale, causal=True)
    f_o, f_l = orc.kvcache_fwd(q.float(), rk.float(), rv.float(), lens_t, scale, causal=True)
    for ns in (0, 1):
        out, lse = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=lens_t.cuda(), softmax_scale=scale,
                                             causal=True, num_splits=ns, return_softmax_lse=True)
        torch.cuda.synchronize()
        assert capi.last_kernel() == kernel
        assert capi.lib.fa_debug_get(2) == 0
        assert torch.isfinite(out).all()
        assert_within("out", out.cpu(), lp_o, f_o)
        assert_lse(lse, f_l)
