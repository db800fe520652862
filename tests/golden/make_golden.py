"""Generate the golden fixtures in this folder from the reference's own Python goldens.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports `tests/test_flash_attn_npu_v2.py` (forward golden `ref_flash_attention`)
and `tests/fa_small_op_golden.py` (backward goldens) from the reference, with empty
stand-in modules for the device packages those test files import at the top, runs
them on seeded inputs and stores inputs (or their seeds) and outputs as `*.pt`.
The GPU box has no reference checkout; the tests read only these files.
"""
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root):
    for name in ("torch_npu", "flash_attn_npu"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.flash_attn_with_kvcache = m.flash_attn_func = m.flash_attn_varlen_func = None
            sys.modules[name] = m
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import test_flash_attn_npu_v2 as fwd_mod
    import fa_small_op_golden as bwd_mod
    return fwd_mod, bwd_mod


def ref_mask(sq, sk, causal, wl, wr):
    """Mask construction exactly as the reference test does it
    (tests/test_flash_attn_npu_v2.py:325-386), vectorised."""
    if sk > 0 and wl >= sk:
        wl = -1
    if sk > 0 and wr >= sk:
        wr = -1
    if causal:
        wr = 0
    is_causal = wl < 0 and wr == 0
    is_local = (wl >= 0 or wr > 0) and not is_causal
    if is_local:
        wl = sk if wl < 0 else wl
        wr = sk if wr < 0 else wr
    if is_causal:
        return torch.triu(torch.ones(sq, sk), diagonal=sk - sq + 1).bool(), False
    if is_local:
        pre, nxt = sk - sq - wl, sk - sq + wr
        i = torch.arange(sq).unsqueeze(1)
        j = torch.arange(sk).unsqueeze(0)
        return ((j - i) < pre) | ((j - i) > nxt), True
    return None, False


def ref_forward(fwd_mod, q, k, v, scale, causal, wl, wr, softcap, dt):
    """q (B,Sq,H,D) etc -> out (B,Sq,H,D), lse (B,H,Sq) via the reference golden."""
    b, sq, h, d = q.shape
    sk = k.shape[1]
    mask, local = ref_mask(sq, sk, causal, wl, wr)
    outs, lses = [], []
    for i in range(b):
        o, l = fwd_mod.ref_flash_attention(q[i], k[i], v[i], scale, mask, dt, softcap)
        o = o.reshape(sq, h, d)
        l = l.reshape(h, sq)
        if local and mask is not None:
            dead = mask.all(dim=-1)
            o[dead] = 0
            l[:, dead] = torch.inf
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def uniform(shape, lo, hi, dt, gen):
    return (lo + (hi - lo) * torch.rand(*shape, generator=gen)).to(dt)


def main(ref_root):
    fwd_mod, bwd_mod = load_reference(ref_root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- configuration 1: fp32, B2 S512 H8 D64 causal, N(0,1) seed 0 -----------------
    torch.manual_seed(0)
    q = torch.randn(2, 512, 8, 64)
    k = torch.randn(2, 512, 8, 64)
    v = torch.randn(2, 512, 8, 64)
    out, lse = ref_forward(fwd_mod, q, k, v, 1.0 / 8.0, True, -1, -1, 0.0, torch.float32)
    torch.save({"seed": 0, "shape": (2, 512, 8, 64), "causal": True, "scale": 0.125,
                "q_sum": q.double().sum().item(), "out": out.half(), "out_fp32_sample": out[0, ::37].clone(),
                "lse": lse}, os.path.join(HERE, "config1_fwd.pt"))

    # ---- forward matrix: (dtype, B, H, Hkv, Sq, Sk, D, causal, wl, wr, softcap) --------
    fwd_cases = [
        (torch.bfloat16, 1, 4, 4, 192, 192, 128, True, -1, -1, 0.0),
        (torch.float16, 2, 4, 2, 130, 130, 64, False, -1, -1, 0.0),
        (torch.bfloat16, 1, 6, 2, 2, 600, 128, True, -1, -1, 0.0),
        (torch.bfloat16, 1, 2, 1, 160, 160, 128, True, 64, 0, 0.0),
        (torch.float16, 1, 2, 2, 128, 192, 128, False, 32, 64, 0.0),
        (torch.bfloat16, 1, 4, 1, 96, 700, 64, True, -1, -1, 30.0),
        (torch.float16, 2, 2, 2, 200, 2, 128, False, 65, 412, 0.0),
        (torch.bfloat16, 1, 3, 1, 77, 150, 111 + 1, False, -1, -1, 0.0),
        (torch.bfloat16, 1, 2, 2, 64, 300, 256, True, -1, -1, 0.0),
        (torch.float16, 1, 2, 2, 100, 100, 128, False, 50, -30, 0.0),
    ]
    fixtures = []
    for idx, (dt, b, h, hkv, sq, sk, d, causal, wl, wr, cap) in enumerate(fwd_cases):
        gen = torch.Generator().manual_seed(1000 + idx)
        q = uniform((b, sq, h, d), -5, 5, dt, gen)
        k = uniform((b, sk, hkv, d), -5, 5, dt, gen)
        v = uniform((b, sk, hkv, d), -5, 5, dt, gen)
        out, lse = ref_forward(fwd_mod, q, k, v, d ** -0.5, causal, wl, wr, cap, dt)
        out32, _ = ref_forward(fwd_mod, q.float(), k.float(), v.float(), d ** -0.5, causal, wl, wr, cap,
                               torch.float32)
        fixtures.append({"q": q, "k": k, "v": v, "scale": d ** -0.5, "causal": causal, "window": (wl, wr),
                         "softcap": cap, "out": out, "out_fp32": out32.half(), "lse": lse})
    torch.save(fixtures, os.path.join(HERE, "fwd_cases.pt"))

    # ---- paged gather (block_table indexing) ------------------------------------------
    gen = torch.Generator().manual_seed(77)
    page, blocks, hkv, d, h = 16, 24, 2, 64, 4
    kc = uniform((blocks, page, hkv, d), -5, 5, torch.bfloat16, gen)
    vc = uniform((blocks, page, hkv, d), -5, 5, torch.bfloat16, gen)
    lens = [100, 37]
    perm = torch.randperm(blocks, generator=gen).int()
    table = torch.stack([perm[:8], perm[8:16]])
    q = uniform((2, 3, h, d), -5, 5, torch.bfloat16, gen)
    outs, lses = [], []
    for i, L in enumerate(lens):
        keys = torch.stack([kc[int(table[i][j // page]), j % page] for j in range(L)])
        vals = torch.stack([vc[int(table[i][j // page]), j % page] for j in range(L)])
        mask, _ = ref_mask(3, L, True, -1, -1)
        o, l = fwd_mod.ref_flash_attention(q[i], keys, vals, d ** -0.5, mask, torch.bfloat16, 0.0)
        outs.append(o.reshape(3, h, d))
        lses.append(l.reshape(h, 3))
    torch.save({"q": q, "k_cache": kc, "v_cache": vc, "block_table": table, "cache_seqlens": lens,
                "scale": d ** -0.5, "causal": True, "out": torch.stack(outs), "lse": torch.stack(lses)},
               os.path.join(HERE, "paged_case.pt"))

    # ---- backward matrix: (dtype, B, H, Hkv, Sq, Sk, D, causal, wl, wr, softcap) -------
    bwd_cases = [
        (torch.bfloat16, 1, 2, 2, 128, 128, 128, True, -1, -1, 0.0),
        (torch.float16, 2, 4, 2, 96, 160, 64, False, -1, -1, 0.0),
        (torch.bfloat16, 1, 4, 1, 100, 100, 128, True, 32, 0, 0.0),
        (torch.float16, 1, 2, 2, 64, 96, 64, False, 16, 24, 20.0),
        (torch.float32, 1, 2, 1, 80, 80, 64, True, -1, -1, 0.0),
    ]
    fixtures = []
    for idx, (dt, b, h, hkv, sq, sk, d, causal, wl, wr, cap) in enumerate(bwd_cases):
        gen = torch.Generator().manual_seed(2000 + idx)
        q = uniform((b, sq, h, d), -1, 1, dt, gen)
        k = uniform((b, sk, hkv, d), -1, 1, dt, gen)
        v = uniform((b, sk, hkv, d), -1, 1, dt, gen)
        do = uniform((b, sq, h, d), -1, 1, dt, gen)
        scale = d ** -0.5
        out, lse = ref_forward(fwd_mod, q, k, v, scale, causal, wl, wr, cap, dt)
        dq, dk, dv = bwd_mod.golden_bsnd_bwd_from_fwd(q, k, v, do, out, lse, h, hkv, scale, cap, 0.0,
                                                     causal, wl, wr, gtype=torch.float64)
        fixtures.append({"q": q, "k": k, "v": v, "dout": do, "lse": lse, "scale": scale, "causal": causal,
                         "window": (wl, wr), "softcap": cap, "dq": dq, "dk": dk, "dv": dv})
    torch.save(fixtures, os.path.join(HERE, "bwd_cases.pt"))

    # ---- varlen backward (TND) --------------------------------------------------------
    gen = torch.Generator().manual_seed(3000)
    lens_q, lens_k, h, hkv, d = [50, 0, 129], [70, 0, 129], 4, 2, 64
    tq, tk = sum(lens_q), sum(lens_k)
    q = uniform((tq, h, d), -1, 1, torch.bfloat16, gen)
    k = uniform((tk, hkv, d), -1, 1, torch.bfloat16, gen)
    v = uniform((tk, hkv, d), -1, 1, torch.bfloat16, gen)
    do = uniform((tq, h, d), -1, 1, torch.bfloat16, gen)
    lse = torch.full((h, tq), float("inf"))
    out = torch.zeros_like(q)
    oq = ok = 0
    for sq, sk in zip(lens_q, lens_k):
        if sq and sk:
            mask, _ = ref_mask(sq, sk, True, -1, -1)
            o, l = fwd_mod.ref_flash_attention(q[oq:oq + sq], k[ok:ok + sk], v[ok:ok + sk], d ** -0.5, mask,
                                               torch.bfloat16, 0.0)
            out[oq:oq + sq] = o.reshape(sq, h, d)
            lse[:, oq:oq + sq] = l.reshape(h, sq)
        oq += sq
        ok += sk
    dq, dk, dv = bwd_mod.golden_tnd_bwd_from_fwd(q, k, v, do, out, lse, h, hkv, lens_q, lens_k, d ** -0.5, 0.0,
                                                0.0, True, -1, -1, gtype=torch.float64)
    # the reference leaves rows of empty sequences uninitialised; none exist here (length 0)
    torch.save({"q": q, "k": k, "v": v, "dout": do, "lse": lse, "out": out, "lens_q": lens_q,
                "lens_k": lens_k, "scale": d ** -0.5, "causal": True, "dq": dq, "dk": dk, "dv": dv},
               os.path.join(HERE, "varlen_bwd_case.pt"))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
