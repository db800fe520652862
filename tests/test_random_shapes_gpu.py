"""Random ragged shapes: the default routing (tcgen05 forward and backward, split-KV decode) against the general
mma.sync kernels of the same library (both were checked against the oracle elsewhere; this sweep looks for
shape-dependent slips: partial tiles, windows that cut tiles, grouped heads, packed batches with empty sequences,
padded head dims, page sizes, appended chunks, forced split counts, one-CTA launches)."""
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


def _guarded(like):
    """A tensor of `like`'s shape that lies between sentinel elements (about four rows on each side): a kernel that
    writes past a row or past the tensor shows up as a changed sentinel instead of as a corrupted neighbour."""
    pad = 4 * like.shape[-1] * like.shape[-2]
    flat = torch.full((like.numel() + 2 * pad,), 777.0, dtype=like.dtype, device=like.device)
    return flat, flat[pad:pad + like.numel()].view(like.shape)


def _sentinels_intact(flat, view):
    pad = (flat.numel() - view.numel()) // 2
    return bool((flat[:pad] == 777.0).all() and (flat[pad + view.numel():] == 777.0).all())


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


def _cache_case(seed):
    """One random KV-cache call: shapes, features and tensors from the seed."""
    rnd = random.Random(seed)
    d = rnd.choice([32, 64, 64, 72, 96, 128, 128, 128, 160, 192, 256])
    hkv = rnd.choice([1, 2, 4])
    grp = rnd.choice([1, 2, 3, 4, 6, 8, 16])
    h = hkv * grp
    b = rnd.randint(1, 5)
    sq = rnd.choice([1, 1, 2, 3, 4, 4, 7, 8, 16, 17, 33, 64, 100, 130, 200, 300])
    paged = rnd.random() < 0.6
    page = rnd.choice([64, 128, 192, 256])
    cap = rnd.choice([256, 512, 768, 1024, 2048, 4096, 8192])
    if paged:
        cap = (cap + page - 1) // page * page
    append = rnd.random() < 0.5
    hi = cap - sq if append else cap
    if hi < 1:
        return None
    lens = [rnd.randint(0 if append else 1, hi) for _ in range(b)]
    if rnd.random() < 0.3:
        lens[0] = hi                                   # a sequence that fills the cache to its last row
    if rnd.random() < 0.2 and not append:
        lens[-1] = rnd.randint(1, min(hi, 40))         # one that is shorter than a tile (and than the chunk)
    mode = rnd.choice(["full", "causal", "causal", "window"])
    causal = mode == "causal"
    wl, wr = (rnd.randint(0, 600), rnd.choice([0, rnd.randint(0, 100)])) if mode == "window" else (-1, -1)
    softcap = rnd.choice([0.0, 0.0, 0.0, 20.0])
    use_alibi = rnd.random() < 0.15
    rotary = append and rnd.random() < 0.4 and d % 16 == 0
    nsplit = rnd.choice([0, 0, 0, 1, 3])
    dt = rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16])
    g = torch.Generator(device="cuda").manual_seed(5000 + seed)
    c = {"q": torch.randn(b, sq, h, d, device="cuda", generator=g).to(dt), "table": None, "kn": None, "vn": None,
         "cos": None, "sin": None, "alibi": None}
    if paged:
        nb = cap // page
        pool = nb * b + 3
        c["table"] = torch.randperm(pool, device="cuda", generator=g).int()[: nb * b].reshape(b, nb).contiguous()
        c["kc"] = torch.randn(pool, page, hkv, d, device="cuda", generator=g).to(dt)
        c["vc"] = torch.randn(pool, page, hkv, d, device="cuda", generator=g).to(dt)
    else:
        c["kc"] = torch.randn(b, cap, hkv, d, device="cuda", generator=g).to(dt)
        c["vc"] = torch.randn(b, cap, hkv, d, device="cuda", generator=g).to(dt)
    if append:
        c["kn"] = torch.randn(b, sq, hkv, d, device="cuda", generator=g).to(dt)
        c["vn"] = torch.randn(b, sq, hkv, d, device="cuda", generator=g).to(dt)
    c["lens"] = torch.tensor(lens, dtype=torch.int32, device="cuda")
    if rotary:
        rd = rnd.choice([d // 2, d]) // 16 * 16
        ang = torch.rand(cap, rd // 2, device="cuda", generator=g) * 6.28
        c["cos"], c["sin"] = ang.cos().to(dt), ang.sin().to(dt)
    c["interleaved"] = rnd.random() < 0.5
    if use_alibi:
        c["alibi"] = (torch.rand(h, device="cuda", generator=g) * 0.3).float()
    c.update(scale=d ** -0.5, causal=causal, wl=wl, wr=wr, softcap=softcap, nsplit=nsplit)
    c["tag"] = (f"seed {seed}: b{b} sq{sq} h{h}/{hkv} d{d} capacity {cap} paged {paged} page {page} lens {lens} append {append} "
                f"rotary {rotary} {mode} ({wl},{wr}) softcap {softcap} alibi {use_alibi} num_splits {nsplit} {dt}")
    return c


@pytest.mark.parametrize("block", range(12))
def test_kvcache_calls_random(block):
    """25 random flash_attn_with_kvcache calls a block (300 in all; head dims 32-256, query groups 1-16 including groups
    that cannot be stacked, 1-300 new tokens, dense and paged caches with pages of 64-256 tokens, append, rotary, windows,
    softcap, alibi, forced split counts): output, LSE and the cache after the call of the default routing against the
    general kernels.  Among them are one-sequence calls with a handful of new tokens against a cache of 256 rows (seed
    200: head dim 32, one CTA's worth of work), the smallest launches the routing has to place."""
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    bad, kernels = [], set()
    for seed in range(block * 25, block * 25 + 25):
        c = _cache_case(seed)
        if c is None:
            continue

        guards = []

        def call():
            k2, v2 = c["kc"].clone(), c["vc"].clone()
            flat, out_ = _guarded(c["q"])
            guards.append((flat, out_))
            out, lse = ext.fwd_kvcache(c["q"], k2, v2, c["kn"], c["vn"], c["lens"], c["cos"], c["sin"], None, None, c["table"],
                                       c["alibi"], out_, c["scale"], c["causal"], c["wl"], c["wr"], c["softcap"],
                                       c["interleaved"], c["nsplit"])
            return out, lse, k2, v2

        (o1, l1, k1, v1), n1 = _run(0, call)
        (o2, l2, k2, v2), n2 = _run(1, call)
        kernels.add(n1)
        assert not n2.startswith(("sm100", "decode")), n2
        assert capi.lib.fa_debug_get(2) == 0, c["tag"]
        msgs = []
        if not all(_sentinels_intact(f, o) for f, o in guards):
            msgs.append("a kernel wrote outside the output tensor")
        if not torch.equal(k1, k2) or not torch.equal(v1, v2):
            msgs.append("cache differs")
        a, r = o1.float(), o2.float()
        if not torch.equal(torch.isnan(a), torch.isnan(r)):
            msgs.append("nan pattern differs")
        mag = max(1.0, r[torch.isfinite(r)].abs().max().item() if torch.isfinite(r).any() else 1.0)
        err = (a - r).abs().nan_to_num(0).max().item()
        if err > 4 * 2 ** -8 * mag:
            msgs.append(f"out err {err:.4g} at magnitude {mag:.3g}")
        fin = torch.isfinite(l2)
        if not torch.equal(torch.isfinite(l1), fin):
            msgs.append("lse finiteness differs")
        elif fin.any() and (l1[fin] - l2[fin]).abs().max().item() > 1e-4 * max(1.0, l2[fin].abs().max().item()):
            msgs.append(f"lse err {(l1[fin] - l2[fin]).abs().max().item():.3g}")
        if msgs:
            bad.append(f"{c['tag']} [{n1}]: " + "; ".join(msgs))
    assert not bad, "\n".join(bad)
    assert kernels, "no case in this block"


@pytest.mark.parametrize("block", range(8))
def test_dense_and_packed_calls_any_head_dim_random(block):
    """25 random dense or packed forward + backward calls a block (200 in all): every head dim from 8 to 256 (padded by
    the tile copies), softcap, alibi, windows, packed batches whose query and key lengths differ."""
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    bad = []
    for seed in range(block * 25, block * 25 + 25):
        rnd = random.Random(seed)
        d = rnd.choice([8, 16, 24, 40, 64, 64, 80, 96, 104, 128, 128, 136, 160, 192, 224, 256])
        hkv = rnd.choice([1, 2, 3])
        h = hkv * rnd.choice([1, 2, 4, 8])
        packed = rnd.random() < 0.4
        mode = rnd.choice(["full", "causal", "causal", "window"])
        causal = mode == "causal"
        wl, wr = (rnd.randint(0, 300), rnd.randint(0, 300)) if mode == "window" else (-1, -1)
        softcap = rnd.choice([0.0, 0.0, 15.0])
        use_alibi = rnd.random() < 0.25
        dt = rnd.choice([torch.bfloat16, torch.float16])
        g = torch.Generator(device="cuda").manual_seed(9000 + seed)
        scale = d ** -0.5
        alibi = (torch.rand(h, device="cuda", generator=g) * 0.3).float() if use_alibi else None
        if packed:
            n = rnd.randint(1, 6)
            lq = [rnd.choice([0, 1, rnd.randint(2, 600)]) for _ in range(n)]
            lk = lq if rnd.random() < 0.5 else [rnd.choice([0, 1, rnd.randint(2, 800)]) for _ in range(n)]
            if sum(lq) == 0:
                lq[0] = 50
            if sum(lk) == 0:
                lk = list(lk)
                lk[0] = 60
            cuq = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32, device="cuda")
            cuk = torch.tensor([0] + list(torch.tensor(lk).cumsum(0)), dtype=torch.int32, device="cuda")
            q = torch.randn(sum(lq), h, d, device="cuda", generator=g).to(dt)
            k = torch.randn(sum(lk), hkv, d, device="cuda", generator=g).to(dt)
            v = torch.randn(sum(lk), hkv, d, device="cuda", generator=g).to(dt)
            tag = f"seed {seed}: packed lq {lq} lk {lk} h{h}/{hkv} d{d} {mode} ({wl},{wr}) softcap {softcap} alibi {use_alibi} {dt}"
        else:
            b = rnd.randint(1, 3)
            sq, sk = rnd.randint(1, 700), rnd.randint(1, 900)
            q = torch.randn(b, sq, h, d, device="cuda", generator=g).to(dt)
            k = torch.randn(b, sk, hkv, d, device="cuda", generator=g).to(dt)
            v = torch.randn(b, sk, hkv, d, device="cuda", generator=g).to(dt)
            tag = f"seed {seed}: dense b{b} sq{sq} sk{sk} h{h}/{hkv} d{d} {mode} ({wl},{wr}) softcap {softcap} alibi {use_alibi} {dt}"
        do = torch.randn(q.shape, device="cuda", generator=g).to(dt)

        guards = []

        def call():
            g4 = [_guarded(t) for t in (q, q, k, v)]
            guards.extend(g4)
            out_, dq, dk, dv = (x[1] for x in g4)
            if packed:
                out, lse, _, _ = ext.varlen_fwd(q, k, v, out_, cuq, cuk, None, None, None, alibi, max(lq), max(lk), 0.0, scale,
                                                False, causal, wl, wr, softcap, False, None)
            else:
                out, lse, _, _ = ext.fwd(q, k, v, out_, alibi, 0.0, scale, causal, wl, wr, softcap, False, None)
            if packed:
                ext.varlen_bwd(do, q, k, v, out, lse, dq, dk, dv, cuq, cuk, alibi, max(lq), max(lk), 0.0, scale, False, causal,
                               wl, wr, softcap, False, None, None)
            else:
                ext.bwd(do, q, k, v, out, lse, dq, dk, dv, alibi, 0.0, scale, causal, wl, wr, softcap, False, None, None)
            return out, lse, dq, dk, dv

        (o1, l1, dq1, dk1, dv1), b1 = _run(0, call)
        (o2, l2, dq2, dk2, dv2), b2 = _run(1, call)
        assert b2 == "generic_mma_bwd", b2
        assert b1.startswith("sm100_tcgen05_bwd") == (d <= 128), (tag, b1)
        assert capi.lib.fa_debug_get(2) == 0, tag
        msgs = []
        if not all(_sentinels_intact(f, o) for f, o in guards):
            msgs.append("a kernel wrote outside an output tensor")
        for name, t1, t2 in (("out", o1, o2), ("dq", dq1, dq2), ("dk", dk1, dk2), ("dv", dv1, dv2)):
            if torch.isnan(t1.float()).any():
                msgs.append(name + " has nan")
            try:
                _close(t1, t2, name)
            except AssertionError as e:
                msgs.append(str(e))
        fin = torch.isfinite(l2)
        if not torch.equal(torch.isfinite(l1), fin):
            msgs.append("lse finiteness differs")
        elif fin.any() and (l1[fin] - l2[fin]).abs().max().item() > 1e-4 * max(1.0, l2[fin].abs().max().item()):
            msgs.append("lse differs")
        if msgs:
            bad.append(tag + ": " + "; ".join(msgs))
    assert not bad, "\n".join(bad)


@pytest.mark.parametrize("block", range(8))
def test_small_cache_launches_random(block):
    """25 small flash_attn_with_kvcache launches a block (200 in all): one or two sequences, one to sixteen new tokens,
    dense caches whose capacity is not a multiple of the key tile (200, 300, 333, 1000 rows) or paged ones, lengths that
    end in the last tile, at the capacity and one row before it.  These are launches of one to a few CTAs with one to
    eight key tiles on the tcgen05 forward and on the decode kernel; default routing against the general kernels."""
    from flash_attn_npu import flash_attn_npu as ext
    import fa_b200_capi as capi
    bad = []
    for seed in range(block * 25, block * 25 + 25):
        rnd = random.Random(seed)
        d = rnd.choice([64, 64, 128, 128])
        hkv = rnd.choice([1, 1, 2])
        grp = rnd.choice([2, 4, 8, 16])
        h = hkv * grp
        b = rnd.choice([1, 1, 2])
        sq = rnd.choice([2, 3, 4, 4, 7, 8, 16])
        if rnd.random() < 0.3:
            sq = 1
        elif sq * grp <= 16:
            sq = 17 // grp + 1
        paged = rnd.random() < 0.4
        page = rnd.choice([64, 128, 256])
        cap = rnd.choice([256, 200, 300, 333, 512, 1000])
        lens = [rnd.randint(sq, cap) for _ in range(b)]
        if rnd.random() < 0.5:
            lens[0] = rnd.choice([86, 100, 128, min(249, cap), cap, cap - 1, max(sq, cap - 60)])
        causal = rnd.random() < 0.6
        nsplit = rnd.choice([0, 1, 1])
        dt = rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        g = torch.Generator(device="cuda").manual_seed(88000 + seed)
        q = torch.randn(b, sq, h, d, device="cuda", generator=g).to(dt)
        if paged:
            cap = (cap + page - 1) // page * page
            nb = cap // page
            pool = nb * b + 2
            table = torch.randperm(pool, device="cuda", generator=g).int()[: nb * b].reshape(b, nb).contiguous()
            kc = torch.randn(pool, page, hkv, d, device="cuda", generator=g).to(dt)
            vc = torch.randn(pool, page, hkv, d, device="cuda", generator=g).to(dt)
        else:
            table = None
            kc = torch.randn(b, cap, hkv, d, device="cuda", generator=g).to(dt)
            vc = torch.randn(b, cap, hkv, d, device="cuda", generator=g).to(dt)
        lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
        tag = f"seed {seed}: b{b} sq{sq} h{h}/{hkv} d{d} capacity {cap} paged {paged} page {page} lens {lens} causal {causal} num_splits {nsplit} {dt}"
        guards = []

        def call():
            flat, out_ = _guarded(q)
            guards.append((flat, out_))
            out, lse = ext.fwd_kvcache(q, kc, vc, None, None, lens_t, None, None, None, None, table, None, out_, d ** -0.5, causal,
                                       -1, -1, 0.0, False, nsplit)
            return out, lse

        (o1, l1), n1 = _run(0, call)
        (o2, l2), n2 = _run(1, call)
        assert n1 in ("sm100_tcgen05_2q", "decode_splitkv_tma"), (tag, n1)
        assert capi.lib.fa_debug_get(2) == 0, tag
        msgs = []
        if not all(_sentinels_intact(f, o) for f, o in guards):
            msgs.append("a kernel wrote outside the output tensor")
        try:
            _close(o1, o2, "out")
        except AssertionError as e:
            msgs.append(str(e))
        fin = torch.isfinite(l2)
        if not torch.equal(torch.isfinite(l1), fin):
            msgs.append("lse finiteness differs")
        elif fin.any() and (l1[fin] - l2[fin]).abs().max().item() > 1e-4 * max(1.0, l2[fin].abs().max().item()):
            msgs.append("lse differs")
        if msgs:
            bad.append(tag + f" [{n1}]: " + "; ".join(msgs))
    assert not bad, "\n".join(bad)
