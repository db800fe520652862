"""Every parameter tuple of the reference's own GPU-side tests, run against the CPU oracle.

The tuples live in tests/golden/reference_case_lists.json, extracted from the reference's test modules by
tests/golden/make_case_lists.py (tests/test_flash_attn_npu_v2.py:145-286, :436, :522; tests/test_flash_attn_npu_v2_bwd.py
:147-283; tests/test_flash_attn_npu_v3.py:148-303, :545, :622; tests/test_flash_attn_npu_v3_bwd.py).  Inputs follow the
reference's tests: uniform in [-5, 5] for the forward, [-1, 1] for the backward, page size 128, block tables that
number the pages consecutively.  The check is this repository's tolerance rule (tests/parity.py), which is
tighter than the reference's rtol = atol = 1e-2.  `--random-sample N` keeps N seeded cases per list."""
import json
import os

import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_lse, assert_within

pytestmark = pytest.mark.gpu
with open(os.path.join(os.path.dirname(__file__), "golden", "reference_case_lists.json")) as f:
    LISTS = json.load(f)
DT = {"bfloat16": torch.bfloat16, "float16": torch.float16}
PAGE = 128


def cases(module, fn):
    d = LISTS[module][fn]
    return [dict(zip(d["fields"], c)) for c in d["cases"]]


def ident(c):
    return "-".join(str(v) for v in c.values())


def api(version):
    if version == 2:
        import flash_attn_npu as m
    else:
        import flash_attn_npu_3 as m
    return m


def uniform(shape, lim, dt, gen=None):
    return ((torch.rand(shape, generator=gen) * 2 - 1) * lim).to(dt)


# ------------------------------------------------------------------------------------------------- forward, KV cache
def run_kvcache_bsnd(version, c, paged, num_splits=0):
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d = c["q_seqlen"], c["kv_seqlen"], c["head_size"]
    causal, win, cap = c["is_causal"], (c["window_size_left"], c["window_size_right"]), c["softcap"]
    q = uniform((b, sq, h, d), 5.0, dt)
    if paged:
        nb = (sk + PAGE - 1) // PAGE
        kc = uniform((max(64, nb * b), PAGE, hkv, d), 5.0, dt)
        vc = uniform((max(64, nb * b), PAGE, hkv, d), 5.0, dt)
        table = torch.arange(nb * b, dtype=torch.int32).reshape(b, nb)
    else:
        kc, vc, table = uniform((b, sk, hkv, d), 5.0, dt), uniform((b, sk, hkv, d), 5.0, dt), None
    lens = torch.full((b,), sk, dtype=torch.int32)
    scale = d ** -0.5
    lp_o, _ = orc.kvcache_fwd(q, kc.clone(), vc.clone(), lens, scale, block_table=table, causal=causal, window=win, softcap=cap)
    f_o, f_l = orc.kvcache_fwd(q.float(), kc.float(), vc.float(), lens, scale, block_table=table, causal=causal, window=win,
                               softcap=cap)
    m = api(version)
    kw = dict(cache_seqlens=lens.cuda(), softmax_scale=scale, causal=causal, window_size=win, softcap=cap,
              num_splits=num_splits, return_softmax_lse=True)
    kw["block_table" if version == 2 else "page_table"] = None if table is None else table.cuda()
    out, lse, *_ = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), **kw)
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v2", "test_fa_custom_ops"), ids=ident)
def test_v2_kvcache_list(c):
    run_kvcache_bsnd(2, c, bool(c["cache_mode"]))


def run_kvcache_tnd(c, paged, num_splits):
    """Packed queries against a paged cache (one length per sequence) or against packed keys (cache_mode 0): the
    v3 test's TND layout, with its seeded per-sequence lengths when `is_varied`."""
    import flash_attn_npu_3 as m
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d = c["q_seqlen"], c["kv_seqlen"], c["head_size"]
    causal, win, cap = c["is_causal"], (c["window_size_left"], c["window_size_right"]), c["softcap"]
    gen = torch.Generator().manual_seed(1234)
    if c["is_varied"]:
        qs = torch.randint(1, sq + 1, (b,), generator=gen).tolist()
        ks = [int(torch.randint(x, sk + 1, (1,), generator=gen)) for x in qs]
    else:
        qs, ks = [sq] * b, [sk] * b
    cu_q = torch.tensor([0] + torch.tensor(qs).cumsum(0).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + torch.tensor(ks).cumsum(0).tolist(), dtype=torch.int32)
    q = uniform((sum(qs), h, d), 5.0, dt, gen)
    scale = d ** -0.5
    if paged:
        nb = (sk + PAGE - 1) // PAGE
        kc = uniform((max(64, nb * b), PAGE, hkv, d), 5.0, dt, gen)
        vc = uniform((max(64, nb * b), PAGE, hkv, d), 5.0, dt, gen)
        table = torch.arange(nb * b, dtype=torch.int32).reshape(b, nb)
        kp = torch.cat([orc.gather_paged(kc, table[i], ks[i]) for i in range(b)])
        vp = torch.cat([orc.gather_paged(vc, table[i], ks[i]) for i in range(b)])
    else:
        kp, vp = uniform((sum(ks), hkv, d), 5.0, dt, gen), uniform((sum(ks), hkv, d), 5.0, dt, gen)
    # the reference normalises the windows against the longest key length of the call
    lp_o, _ = orc.attention_varlen_fwd(q, kp, vp, cu_q, cu_k, scale, causal, win, cap, max_seqlen_k=sk)
    f_o, f_l = orc.attention_varlen_fwd(q.float(), kp.float(), vp.float(), cu_q, cu_k, scale, causal, win, cap,
                                        data_type=torch.float32, max_seqlen_k=sk)
    if paged:
        out, lse, *_ = m.flash_attn_with_kvcache(q.cuda(), kc.cuda(), vc.cuda(), cache_seqlens=torch.tensor(ks, dtype=torch.int32).cuda(),
                                                 page_table=table.cuda(), cu_seqlens_q=cu_q.cuda(), max_seqlen_q=sq,
                                                 softmax_scale=scale, causal=causal, window_size=win, softcap=cap,
                                                 num_splits=num_splits, return_softmax_lse=True)
    else:
        out, lse = m.flash_attn_varlen_func(q.cuda(), kp.cuda(), vp.cuda(), cu_q.cuda(), cu_k.cuda(), sq, sk, softmax_scale=scale,
                                            causal=causal, window_size=win, softcap=cap, return_attn_probs=True)[:2]
    assert_within("out", out.cpu(), lp_o, f_o)
    assert_lse(lse, f_l)


@pytest.mark.parametrize("num_splits", [0, 2])
@pytest.mark.parametrize("cache_mode", [0, 1])
@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v3", "test_fa_custom_ops"), ids=ident)
def test_v3_kvcache_list(c, cache_mode, num_splits):
    # the reference's own skip rules (tests/test_flash_attn_npu_v3.py:310-318)
    if num_splits > 1 and not (cache_mode == 1 and c["layout"] == "TND"):
        pytest.skip("num_splits > 1 is exercised with a paged cache and packed queries")
    if c["is_varied"] and c["layout"] != "TND":
        pytest.skip("varied lengths need packed queries")
    if c["layout"] == "BSND":
        run_kvcache_bsnd(3, c, bool(cache_mode), num_splits)
    else:
        run_kvcache_tnd(c, bool(cache_mode), num_splits)


# ------------------------------------------------------------------------------------------------- forward, dense
def run_dense_fwd(version, c):
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d, causal, cap = c["q_seqlen"], c["kv_seqlen"], c["head_size"], c["is_causal"], c["softcap"]
    q, k, v = uniform((b, sq, h, d), 5.0, dt), uniform((b, sk, hkv, d), 5.0, dt), uniform((b, sk, hkv, d), 5.0, dt)
    scale = d ** -0.5
    lp_o, _ = orc.attention_fwd(q, k, v, scale, causal, (-1, -1), cap)
    f_o, f_l = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, (-1, -1), cap, data_type=torch.float32)
    m = api(version)
    ret = m.flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=causal, softcap=cap, return_attn_probs=c["return_attn_probs"])
    if c["return_attn_probs"]:
        assert len(ret) == (3 if version == 2 else 2)
        assert_lse(ret[1], f_l)
        ret = ret[0]
    assert_within("out", ret.cpu(), lp_o, f_o)


@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v2", "test_fa_fwd_custom_ops"), ids=ident)
def test_v2_dense_forward_list(c):
    run_dense_fwd(2, c)


@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v3", "test_fa_fwd_custom_ops"), ids=ident)
def test_v3_dense_forward_list(c):
    run_dense_fwd(3, c)


# ------------------------------------------------------------------------------------------------- forward, packed
def run_varlen_fwd(version, c):
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d = c["q_seqlen"], c["kv_seqlen"], c["head_size"]
    causal, win, cap = c["is_causal"], (c["window_size_left"], c["window_size_right"]), c["softcap"]
    q, k, v = uniform((b * sq, h, d), 5.0, dt), uniform((b * sk, hkv, d), 5.0, dt), uniform((b * sk, hkv, d), 5.0, dt)
    cu_q = torch.arange(b + 1, dtype=torch.int32) * sq
    cu_k = torch.arange(b + 1, dtype=torch.int32) * sk
    scale = d ** -0.5
    lp_o, _ = orc.attention_varlen_fwd(q, k, v, cu_q, cu_k, scale, causal, win, cap)
    f_o, f_l = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cu_q, cu_k, scale, causal, win, cap, data_type=torch.float32)
    m = api(version)
    ret = m.flash_attn_varlen_func(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), sq, sk, softmax_scale=scale,
                                   causal=causal, window_size=win, softcap=cap, return_attn_probs=True)
    assert_within("out", ret[0].cpu(), lp_o, f_o)
    assert_lse(ret[1], f_l)


@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v2", "test_fa_varlen_ops"), ids=ident)
def test_v2_varlen_forward_list(c):
    run_varlen_fwd(2, c)


@pytest.mark.parametrize("c", cases("test_flash_attn_npu_v3", "test_fa_varlen_ops"), ids=ident)
def test_v3_varlen_forward_list(c):
    run_varlen_fwd(3, c)


# ------------------------------------------------------------------------------------------------- backward
def run_dense_bwd(version, c):
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d, causal, cap = c["q_seqlen"], c["kv_seqlen"], c["head_size"], c["is_causal"], c["softcap"]
    win = (c.get("window_size_left", -1), c.get("window_size_right", -1))
    q, do = uniform((b, sq, h, d), 1.0, dt), uniform((b, sq, h, d), 1.0, dt)
    k, v = uniform((b, sk, hkv, d), 1.0, dt), uniform((b, sk, hkv, d), 1.0, dt)
    scale = d ** -0.5
    _, lse32 = orc.attention_fwd(q.float(), k.float(), v.float(), scale, causal, win, cap, data_type=torch.float32)
    lp = orc.attention_bwd(q, k, v, do, lse32, scale, causal, win, cap)
    f32 = orc.attention_bwd(q.float(), k.float(), v.float(), do.float(), lse32, scale, causal, win, cap)
    m = api(version)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = m.flash_attn_func(qc, kc, vc, softmax_scale=scale, causal=causal, window_size=win, softcap=cap)
    grads = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    for name, got, a, b_ in zip(("dq", "dk", "dv"), grads, lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)


def run_varlen_bwd(version, c):
    dt, b, h, hkv = DT[c["data_type"]], c["batch_size"], c["num_heads"], c["kv_heads"]
    sq, sk, d, causal, cap = c["q_seqlen"], c["kv_seqlen"], c["head_size"], c["is_causal"], c["softcap"]
    win = (c.get("window_size_left", -1), c.get("window_size_right", -1))
    q, do = uniform((b * sq, h, d), 1.0, dt), uniform((b * sq, h, d), 1.0, dt)
    k, v = uniform((b * sk, hkv, d), 1.0, dt), uniform((b * sk, hkv, d), 1.0, dt)
    cu_q = torch.arange(b + 1, dtype=torch.int32) * sq
    cu_k = torch.arange(b + 1, dtype=torch.int32) * sk
    scale = d ** -0.5
    _, lse32 = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cu_q, cu_k, scale, causal, win, cap, data_type=torch.float32)
    lp = orc.attention_varlen_bwd(q, k, v, do, lse32, cu_q, cu_k, scale, causal, win, cap)
    f32 = orc.attention_varlen_bwd(q.float(), k.float(), v.float(), do.float(), lse32, cu_q, cu_k, scale, causal, win, cap)
    m = api(version)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = m.flash_attn_varlen_func(qc, kc, vc, cu_q.cuda(), cu_k.cuda(), sq, sk, softmax_scale=scale, causal=causal,
                                   window_size=win, softcap=cap)
    grads = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    for name, got, a, b_ in zip(("dq", "dk", "dv"), grads, lp, f32):
        assert_within(name, got.cpu(), a, b_, roundings=3)


BWD = [(v, mod, fn, runner) for v, mod in ((2, "test_flash_attn_npu_v2_bwd"), (3, "test_flash_attn_npu_v3_bwd"))
       for fn, runner in (("test_fa_bsnd_bwd", run_dense_bwd), ("test_fa_bsnd_bwd_swa", run_dense_bwd),
                          ("test_fa_varlen_bwd", run_varlen_bwd), ("test_fa_varlen_bwd_swa", run_varlen_bwd))]


@pytest.mark.parametrize("version,runner,c", [(v, r, c) for v, mod, fn, r in BWD for c in cases(mod, fn)],
                         ids=[f"v{v}-{fn[8:]}-{ident(c)}" for v, mod, fn, r in BWD for c in cases(mod, fn)])
def test_backward_lists(version, runner, c):
    runner(version, c)
