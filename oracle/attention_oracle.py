"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference
arm may import this module, and only as the checker or as the timed CPU
baseline.  The product path (the CUDA kernels behind the C-ABI) never routes
through it.

What is restated here and where the reference defines it (paths inside the
reference project):

* forward golden   tests/test_flash_attn_npu_v2.py:84-143 (ref_flash_attention,
                   helpers :10-82): 512-key chunks, fp32 intermediates, scores
                   accumulated over 128-wide head-dim slices, soft mask -1e4,
                   P cast to the data type before P.V, row sum from fp32 P,
                   LSE = log(l) + m.
* masks            tests/test_flash_attn_npu_v2.py:325-341, :368-386
                   (window normalisation, bottom-right causal, local band) and
                   the fully-masked-row fix-up :421-427.
* paged gather     tests/test_flash_attn_npu_v2.py:391-411.
* backward golden  tests/fa_small_op_golden.py:207-265 (BSND) and :268-353
                   (TND), with :21-58 (window normalisation and mask),
                   :104-135 (P from LSE), :169-185 (dQ/dK/dV), :91-101 (GQA sum).
* split-KV combine csrc/ascend910/flash_attn_npu/CombineScale.hpp:165-316.

Pinned: `tests/golden/make_golden.py` imports the reference's own Python
goldens (from the reference checkout, with empty stand-ins for its device
modules), runs both on seeded inputs, and stores the reference outputs as
fixtures; tests/test_oracle.py checks this restatement against those fixtures.

PARITY UNPINNED parts (the reference rejects or lacks them, so there is no
reference code or test to pin against; they follow the flash-attn docstrings
the reference ships in flash_attn_npu/flash_attn_npu_interface.py:1459-1545):
rotary embedding, in-place KV append, alibi bias, int8 latent (MLA) decode.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

KV_CHUNK = 512      # keys per online-softmax step in the forward golden
DOT_SLICE = 128     # contraction slice of both matmuls in the forward golden
SOFT_MASK = -1e4    # forward golden's additive mask value
BWD_MASK = -40000.0  # backward golden's additive mask value


# --------------------------------------------------------------------------
# masks and window normalisation
# --------------------------------------------------------------------------
def normalize_window_fwd(seqlen_k: int, causal: bool, wl: int, wr: int):
    """Forward-side window normalisation (tests/test_flash_attn_npu_v2.py:325-341).

    Returns (wl, wr, is_causal, is_local); for local attention an unbounded
    side is replaced by seqlen_k.
    """
    if seqlen_k > 0 and wl >= seqlen_k:
        wl = -1
    if seqlen_k > 0 and wr >= seqlen_k:
        wr = -1
    if causal:
        wr = 0
    is_causal = wl < 0 and wr == 0
    is_local = (wl >= 0 or wr > 0) and not is_causal
    if is_local:
        if wl < 0:
            wl = seqlen_k
        if wr < 0:
            wr = seqlen_k
    return wl, wr, is_causal, is_local


def normalize_window_bwd(seqlen_q: int, seqlen_k: int, causal: bool, wl: int, wr: int):
    """Backward-side normalisation (tests/fa_small_op_golden.py:21-32)."""
    if wl >= seqlen_k - 1:
        wl = -1
    if wr >= seqlen_q - 1:
        wr = -1
    if causal:
        wr = 0
    is_causal = wl < 0 and wr == 0
    is_local = (wl >= 0 or wr >= 0) and not is_causal
    return wl, wr, is_causal, is_local


def fwd_mask(seqlen_q: int, seqlen_k: int, causal: bool, wl: int, wr: int) -> Optional[torch.Tensor]:
    """Boolean (Sq,Sk) mask, True = masked out, or None for full attention."""
    wl, wr, is_causal, is_local = normalize_window_fwd(seqlen_k, causal, wl, wr)
    if not (is_causal or is_local):
        return None
    i = torch.arange(seqlen_q).unsqueeze(1)
    j = torch.arange(seqlen_k).unsqueeze(0)
    rel = j - i - (seqlen_k - seqlen_q)          # key offset from the bottom-right diagonal
    if is_causal:
        return rel > 0
    return (rel < -wl) | (rel > wr)


def bwd_mask(seqlen_q: int, seqlen_k: int, causal: bool, wl: int, wr: int) -> Optional[torch.Tensor]:
    wl, wr, is_causal, is_local = normalize_window_bwd(seqlen_q, seqlen_k, causal, wl, wr)
    if not (is_causal or is_local):
        return None
    i = torch.arange(seqlen_q).unsqueeze(1)
    j = torch.arange(seqlen_k).unsqueeze(0)
    rel = j - i - (seqlen_k - seqlen_q)
    if is_causal:
        return rel > 0
    m = torch.zeros(seqlen_q, seqlen_k, dtype=torch.bool)
    if wr >= 0:
        m |= rel > wr
    if wl >= 0:
        m |= rel < -wl
    return m


# --------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------
def _sliced_group_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a: (Hkv, G, M, K) fp32-able, b: (Hkv, K, N). Contraction accumulated over
    DOT_SLICE-wide slices of K, like the golden's qkMM1 / pvMM2."""
    acc = None
    kdim = a.shape[-1]
    for s in range(0, kdim, DOT_SLICE):
        part = torch.matmul(a[..., s:s + DOT_SLICE].float(), b[:, None, s:s + DOT_SLICE, :].float())
        acc = part if acc is None else acc + part
    return acc


def fwd_one_sequence(q, k, v, scale: float, mask: Optional[torch.Tensor], data_type,
                     softcap: float = 0.0, bias: Optional[torch.Tensor] = None):
    """One sequence of the forward golden.

    q (Sq,H,D), k (Sk,Hkv,D), v (Sk,Hkv,Dv); mask bool (Sq,Sk) True = masked.
    `bias` (H,Sq,Sk) fp32 is added after scaling (alibi; not in the reference).
    Returns out (Sq,H,Dv) in data_type and lse (H,Sq) fp32.
    """
    sq, h, _ = q.shape
    sk, hkv, dv = v.shape
    g = h // hkv
    qh = q.permute(1, 0, 2).reshape(hkv, g, sq, -1)
    kt = k.permute(1, 2, 0)                       # (Hkv, D, Sk)
    vh = v.permute(1, 0, 2)                       # (Hkv, Sk, Dv)
    scale_t = torch.tensor(scale, dtype=torch.float32)
    run_max = run_sum = acc = None
    for start in range(0, sk, KV_CHUNK):
        stop = min(start + KV_CHUNK, sk)
        s = _sliced_group_matmul(qh, kt[:, :, start:stop]) * scale_t
        if softcap > 0.0:
            s = softcap * torch.tanh(s / softcap)
        if bias is not None:
            s = s + bias[:, :, start:stop].reshape(hkv, g, sq, stop - start)
        if mask is not None:
            s = s + mask[:sq, start:stop].float() * SOFT_MASK
        cmax = s.amax(dim=-1, keepdim=True)
        if run_max is None:
            new_max, decay = cmax, None
        else:
            new_max = torch.maximum(run_max, cmax)
            decay = torch.exp(run_max - new_max)
        p = torch.exp(s - new_max)
        psum = p.sum(dim=-1, keepdim=True)
        pv = _sliced_group_matmul(p.to(data_type), vh[:, start:stop, :])
        if decay is None:
            run_sum, acc = psum, pv
        else:
            run_sum = run_sum * decay + psum
            acc = acc * decay + pv
        run_max = new_max
    out = (acc / run_sum).reshape(h, sq, dv).permute(1, 0, 2)
    lse = (torch.log(run_sum) + run_max).reshape(h, sq).float()
    return out.to(data_type), lse


def _apply_fully_masked(out, lse, mask):
    """Rows whose window is empty give O = 0 and LSE = +inf
    (tests/test_flash_attn_npu_v2.py:421-427)."""
    if mask is None:
        return out, lse
    dead = mask.all(dim=-1)
    if dead.any():
        out = out.clone()
        lse = lse.clone()
        out[dead] = 0
        lse[:, dead] = float("inf")
    return out, lse


def alibi_bias(slopes: torch.Tensor, sq: int, sk: int) -> torch.Tensor:
    """-slope_h * |i + sk - sq - j|  (flash_attn_npu_interface.py:1531-1533). slopes (H,)."""
    i = torch.arange(sq).unsqueeze(1)
    j = torch.arange(sk).unsqueeze(0)
    dist = (i + sk - sq - j).abs().float()
    return -slopes.float().view(-1, 1, 1) * dist


def attention_fwd(q, k, v, scale: float, causal: bool = False, window=(-1, -1),
                  softcap: float = 0.0, data_type=None, alibi_slopes=None):
    """Dense BSND forward: q (B,Sq,H,D), k/v (B,Sk,Hkv,D). Returns out (B,Sq,H,Dv), lse (B,H,Sq)."""
    data_type = data_type or q.dtype
    b, sq, h, _ = q.shape
    sk = k.shape[1]
    mask = fwd_mask(sq, sk, causal, window[0], window[1])
    outs, lses = [], []
    for i in range(b):
        bias = None
        if alibi_slopes is not None:
            sl = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
            bias = alibi_bias(sl, sq, sk)
        if sk == 0:
            o = torch.zeros(sq, h, v.shape[-1], dtype=data_type)
            l = torch.full((h, sq), float("inf"))
        else:
            o, l = fwd_one_sequence(q[i], k[i], v[i], scale, mask, data_type, softcap, bias)
            o, l = _apply_fully_masked(o, l, mask)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def attention_varlen_fwd(q, k, v, cu_q: Sequence[int], cu_k: Sequence[int], scale: float,
                         causal: bool = False, window=(-1, -1), softcap: float = 0.0,
                         data_type=None, max_seqlen_k: Optional[int] = None):
    """Packed TND forward: q (Tq,H,D), k/v (Tk,Hkv,D). Returns out (Tq,H,Dv), lse (H,Tq).

    The window is normalised against max_seqlen_k like the reference host code
    (csrc/ascend910/flash_attn_npu/flash_api.cpp:936-956); the mask itself is
    per sequence.
    """
    data_type = data_type or q.dtype
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    h = q.shape[1]
    out = torch.zeros(q.shape[0], h, v.shape[-1], dtype=data_type)
    lse = torch.full((h, q.shape[0]), float("inf"))
    if max_seqlen_k is None:
        max_seqlen_k = max([cu_k[i + 1] - cu_k[i] for i in range(len(cu_k) - 1)] + [0])
    wl, wr = window
    if max_seqlen_k > 0 and wl >= max_seqlen_k:
        wl = -1
    if max_seqlen_k > 0 and wr >= max_seqlen_k:
        wr = -1
    for i in range(len(cu_q) - 1):
        sq, sk = cu_q[i + 1] - cu_q[i], cu_k[i + 1] - cu_k[i]
        if sq == 0 or sk == 0:
            continue
        mask = literal_mask(sq, sk, causal, wl, wr)
        o, l = fwd_one_sequence(q[cu_q[i]:cu_q[i + 1]], k[cu_k[i]:cu_k[i + 1]], v[cu_k[i]:cu_k[i + 1]],
                                scale, mask, data_type, softcap)
        o, l = _apply_fully_masked(o, l, mask)
        out[cu_q[i]:cu_q[i + 1]] = o
        lse[:, cu_q[i]:cu_q[i + 1]] = l
    return out, lse


def literal_mask(sq: int, sk: int, causal: bool, wl: int, wr: int) -> Optional[torch.Tensor]:
    """Mask for already-normalised windows: negative side = unbounded, causal forces wr = 0."""
    if causal:
        wr = 0
    if wl < 0 and wr < 0:
        return None
    i = torch.arange(sq).unsqueeze(1)
    j = torch.arange(sk).unsqueeze(0)
    rel = j - i - (sk - sq)
    m = torch.zeros(sq, sk, dtype=torch.bool)
    if wr >= 0:
        m |= rel > wr
    if wl >= 0:
        m |= rel < -wl
    return m


# --------------------------------------------------------------------------
# paged cache, rotary, append  (append / rotary: parity unpinned)
# --------------------------------------------------------------------------
def gather_paged(cache: torch.Tensor, block_table_row: torch.Tensor, length: int) -> torch.Tensor:
    """Token j of a sequence lives in block block_table[j // page], row j % page
    (tests/test_flash_attn_npu_v2.py:401-409). cache (blocks, page, Hkv, D) -> (length, Hkv, D)."""
    page = cache.shape[1]
    j = torch.arange(length)
    blocks = block_table_row.long()[j // page]
    return cache[blocks, j % page]


def rotary_tables(seqlen_ro: int, rotary_dim: int, base: float = 10000.0, dtype=torch.bfloat16):
    """cos/sin (seqlen_ro, rotary_dim/2) = cos/sin(pos * base^(-2j/rotary_dim)), fp32 then cast."""
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    ang = torch.outer(torch.arange(seqlen_ro, dtype=torch.float32), inv)
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                 interleaved: bool) -> torch.Tensor:
    """x (S,H,D), positions (S,) int. fp32 math with separately rounded products and
    one round-to-nearest-even back to x.dtype; dims >= rotary_dim pass through
    (flash_attn_npu_interface.py:1469-1474, :1527-1530)."""
    rd = cos.shape[-1] * 2
    c = cos[positions.long()].float().unsqueeze(1)   # (S,1,rd/2)
    s = sin[positions.long()].float().unsqueeze(1)
    xr = x[..., :rd].float()
    if interleaved:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
    else:
        x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
    o1 = x1 * c - x2 * s
    o2 = x1 * s + x2 * c
    if interleaved:
        rot = torch.stack((o1, o2), dim=-1).flatten(-2)
    else:
        rot = torch.cat((o1, o2), dim=-1)
    return torch.cat((rot.to(x.dtype), x[..., rd:]), dim=-1)


def kvcache_fwd(q, k_cache, v_cache, cache_seqlens, scale, *, k_new=None, v_new=None,
                rotary_cos=None, rotary_sin=None, rotary_interleaved=True, block_table=None,
                cache_batch_idx=None, causal=False, window=(-1, -1), softcap=0.0,
                alibi_slopes=None):
    """flash_attn_with_kvcache semantics. Mutates k_cache / v_cache in place when
    k_new / v_new are given. Returns out (B,Sq,H,Dv), lse (B,H,Sq)."""
    b, sq, h, _ = q.shape
    dt = q.dtype
    lens = [int(x) for x in cache_seqlens]
    s_new = 0 if k_new is None else k_new.shape[1]
    outs, lses = [], []
    max_sk = max(l + s_new for l in lens) if lens else 0
    wl, wr = window
    if max_sk > 0 and wl >= max_sk:
        wl = -1
    if max_sk > 0 and wr >= max_sk:
        wr = -1
    local = (wl >= 0 or wr >= 0) or causal
    for i in range(b):
        cb = i if cache_batch_idx is None else int(cache_batch_idx[i])
        L = lens[i]
        qi = q[i]
        if k_new is not None:
            kn, vn = k_new[i], v_new[i]
            if rotary_cos is not None:
                kn = apply_rotary(kn, rotary_cos, rotary_sin, L + torch.arange(s_new), rotary_interleaved)
            pos = L + torch.arange(s_new)
            if block_table is not None:
                page = k_cache.shape[1]
                blk = block_table[i].long()[pos // page]
                k_cache[blk, pos % page] = kn
                v_cache[blk, pos % page] = vn
            else:
                k_cache[cb, L:L + s_new] = kn
                v_cache[cb, L:L + s_new] = vn
        if rotary_cos is not None:
            qpos = L + torch.arange(sq) if local else torch.full((sq,), L)
            qi = apply_rotary(qi, rotary_cos, rotary_sin, qpos, rotary_interleaved)
        sk = L + s_new
        if block_table is not None:
            ki = gather_paged(k_cache, block_table[i], sk)
            vi = gather_paged(v_cache, block_table[i], sk)
        else:
            ki, vi = k_cache[cb, :sk], v_cache[cb, :sk]
        if sk == 0:
            outs.append(torch.zeros(sq, h, v_cache.shape[-1], dtype=dt))
            lses.append(torch.full((h, sq), float("inf")))
            continue
        mask = literal_mask(sq, sk, causal, wl, wr)
        bias = None
        if alibi_slopes is not None:
            sl = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
            bias = alibi_bias(sl, sq, sk)
        o, l = fwd_one_sequence(qi, ki, vi, scale, mask, dt, softcap, bias)
        o, l = _apply_fully_masked(o, l, mask)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


# --------------------------------------------------------------------------
# split-KV combine
# --------------------------------------------------------------------------
def combine_partials(o_partial: torch.Tensor, lse_partial: torch.Tensor, out_dtype=torch.bfloat16):
    """o_partial (nsplit, rows, Dv) fp32 (each already normalised), lse_partial (nsplit, rows).
    LSE = M + ln sum exp(lse_i - M); O = sum exp(lse_i - LSE) O_i (CombineScale.hpp:165-316).
    Splits that saw no key carry lse = -inf; rows with no key at all give O = 0, LSE = +inf."""
    m = lse_partial.amax(dim=0)
    safe_m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    total = torch.exp(lse_partial - safe_m).sum(dim=0)
    lse = safe_m + torch.log(total)
    w = torch.exp(lse_partial - lse)
    w = torch.where(torch.isfinite(w), w, torch.zeros_like(w))
    o = (w.unsqueeze(-1) * o_partial).sum(dim=0)
    dead = total == 0
    lse = torch.where(dead, torch.full_like(lse, float("inf")), lse)
    o[dead] = 0
    return o.to(out_dtype), lse


# --------------------------------------------------------------------------
# int8 latent (MLA) decode  (parity unpinned)
# --------------------------------------------------------------------------
def quantize_latent(x: torch.Tensor):
    """Per-token symmetric int8: scale = maxabs/127, q = round(x/scale) clamped to +-127."""
    scale = x.abs().amax(dim=-1).clamp_min(1e-12) / 127.0
    q = torch.round(x / scale.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
    return q, scale.float()


def mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, scale,
               kv_range=None):
    """q_nope (B,1,H,512), q_rope (B,1,H,64) bf16; latent_i8 (blocks,page,512) int8,
    scales (blocks,page) fp32, rope (blocks,page,64) bf16. K = [scale*latent (rounded to
    bf16) | rope], V = the same dequantised latent. Returns out (B,1,H,512) bf16, lse (B,H,1).
    kv_range=(lo,hi) restricts every sequence to tokens [lo,hi) and returns fp32 partials."""
    b, _, h, dl = q_nope.shape
    outs, lses = [], []
    for i in range(b):
        L = int(cache_seqlens[i])
        lo, hi = (0, L) if kv_range is None else (min(kv_range[0], L), min(kv_range[1], L))
        j = torch.arange(lo, hi)
        page = latent_i8.shape[1]
        blk = block_table[i].long()[j // page]
        lat = (latent_i8[blk, j % page].float() * scales[blk, j % page].unsqueeze(-1)).to(torch.bfloat16)
        kk = torch.cat((lat, rope[blk, j % page]), dim=-1).unsqueeze(1)      # (L,1,576)
        vv = lat.unsqueeze(1)                                                # (L,1,512)
        qq = torch.cat((q_nope[i], q_rope[i]), dim=-1)                       # (1,H,576)
        if hi <= lo:
            outs.append(torch.zeros(1, h, dl, dtype=torch.float32 if kv_range else torch.bfloat16))
            lses.append(torch.full((h, 1), float("-inf") if kv_range else float("inf")))
            continue
        o, l = fwd_one_sequence(qq, kk, vv, scale, None, torch.float32 if kv_range else torch.bfloat16)
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


# --------------------------------------------------------------------------
# backward
# --------------------------------------------------------------------------
def _bwd_one(q, k, v, dout, lse, scale, softcap, mask, gtype, bias=None):
    """q (H,Sq,D) in its own dtype, k/v (H,Sk,D) already broadcast over the group,
    lse (H,Sq) fp32. All returned in gtype. Follows tests/fa_small_op_golden.py:104-135,
    :169-185: the score recompute runs in the tensors' own dtype (so bf16 inputs give
    bf16-rounded scores), everything after it in gtype.  `bias` (H,Sq,Sk) fp32 is added to
    the scores after scaling and softcap, like the forward's (alibi; not in the reference,
    whose backward ignores the slopes); it is constant, so dS is unchanged in form."""
    cd = q.dtype
    s = torch.matmul(q.to(cd), k.to(cd).transpose(-1, -2)).to(torch.float32).mul(scale)
    factor = None
    if softcap > 0.0:
        t = torch.tanh(s.to(gtype) / softcap)
        factor = 1.0 - t * t
        s = softcap * torch.tanh(s / softcap)
    if bias is not None:
        s = s + bias
    if mask is not None:
        s = s + mask.to(torch.float32) * BWD_MASK
    p = torch.exp(s.to(gtype) - lse.to(torch.float32).to(gtype).unsqueeze(-1))
    if mask is not None:
        p = p.masked_fill(mask, 0.0)
    qg, kg, vg, dog = q.to(gtype), k.to(gtype), v.to(gtype), dout.to(gtype)
    dp = torch.matmul(dog, vg.transpose(-1, -2))
    dv = torch.matmul(p.transpose(-1, -2), dog)
    ds = (dp - (dp * p).sum(dim=-1, keepdim=True)) * p * scale
    if factor is not None:
        ds = ds * factor
    dq = torch.matmul(ds, kg)
    dk = torch.matmul(ds.transpose(-1, -2), qg)
    return dq, dk, dv


def attention_bwd(q, k, v, dout, lse, scale, causal=False, window=(-1, -1), softcap=0.0,
                  gtype=torch.float64, head_chunk: Optional[int] = None, alibi_slopes=None):
    """BSND backward golden. q/dout (B,Sq,H,D), k/v (B,Sk,Hkv,D), lse (B,H,Sq).
    Returns dq, dk, dv in q's dtype. `head_chunk` bounds memory by walking KV heads in
    groups (exact: heads are independent).  alibi_slopes (H,) or (B,H) as in attention_fwd."""
    b, sq, h, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    g = h // hkv
    mask = bwd_mask(sq, sk, causal, window[0], window[1])
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    step = head_chunk or hkv
    for i in range(b):
        for h0 in range(0, hkv, step):
            h1 = min(h0 + step, hkv)
            qs = q[i, :, h0 * g:h1 * g].permute(1, 0, 2)
            dos = dout[i, :, h0 * g:h1 * g].permute(1, 0, 2)
            ks = k[i, :, h0:h1].permute(1, 0, 2).repeat_interleave(g, dim=0)
            vs = v[i, :, h0:h1].permute(1, 0, 2).repeat_interleave(g, dim=0)
            bias = None
            if alibi_slopes is not None:
                sl = alibi_slopes if alibi_slopes.dim() == 1 else alibi_slopes[i]
                bias = alibi_bias(sl[h0 * g:h1 * g], sq, sk)
            dqi, dki, dvi = _bwd_one(qs, ks, vs, dos, lse[i, h0 * g:h1 * g], scale, softcap, mask, gtype, bias)
            dq[i, :, h0 * g:h1 * g] = dqi.permute(1, 0, 2).to(q.dtype)
            dk[i, :, h0:h1] = dki.reshape(h1 - h0, g, sk, d).sum(dim=1).permute(1, 0, 2).to(k.dtype)
            dv[i, :, h0:h1] = dvi.reshape(h1 - h0, g, sk, -1).sum(dim=1).permute(1, 0, 2).to(v.dtype)
    return dq, dk, dv


def attention_varlen_bwd(q, k, v, dout, lse, cu_q, cu_k, scale, causal=False, window=(-1, -1),
                         softcap=0.0, gtype=torch.float64):
    """TND backward golden. q/dout (Tq,H,D), k/v (Tk,Hkv,D), lse (H,Tq)."""
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    h, hkv = q.shape[1], k.shape[1]
    g = h // hkv
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    for i in range(len(cu_q) - 1):
        sq, sk = cu_q[i + 1] - cu_q[i], cu_k[i + 1] - cu_k[i]
        if sq == 0 or sk == 0:
            continue
        mask = bwd_mask(sq, sk, causal, window[0], window[1])
        qs = q[cu_q[i]:cu_q[i + 1]].permute(1, 0, 2)
        dos = dout[cu_q[i]:cu_q[i + 1]].permute(1, 0, 2)
        ks = k[cu_k[i]:cu_k[i + 1]].permute(1, 0, 2).repeat_interleave(g, dim=0)
        vs = v[cu_k[i]:cu_k[i + 1]].permute(1, 0, 2).repeat_interleave(g, dim=0)
        dqi, dki, dvi = _bwd_one(qs, ks, vs, dos, lse[:, cu_q[i]:cu_q[i + 1]], scale, softcap, mask, gtype)
        dq[cu_q[i]:cu_q[i + 1]] = dqi.permute(1, 0, 2).to(q.dtype)
        dk[cu_k[i]:cu_k[i + 1]] = dki.reshape(hkv, g, sk, -1).sum(dim=1).permute(1, 0, 2).to(k.dtype)
        dv[cu_k[i]:cu_k[i + 1]] = dvi.reshape(hkv, g, sk, -1).sum(dim=1).permute(1, 0, 2).to(v.dtype)
    return dq, dk, dv


# --------------------------------------------------------------------------
# tolerance rule
# --------------------------------------------------------------------------
LSE_FLOOR_REL = 1e-5   # fp32 re-association floor for LSE (the golden's own error is 0 there)
ABS_FLOOR = 1e-5


def tolerance(ref_lowp: torch.Tensor, ref_fp32: torch.Tensor, floor: float = ABS_FLOOR) -> float:
    """2 x max-abs(golden in low precision - golden in fp32), never below `floor`."""
    a, b = ref_lowp.float(), ref_fp32.float()
    fin = torch.isfinite(a) & torch.isfinite(b)
    err = (a[fin] - b[fin]).abs().max().item() if fin.any() else 0.0
    return max(2.0 * err, floor)


def lse_floor(lse: torch.Tensor) -> float:
    fin = lse[torch.isfinite(lse)]
    mag = fin.abs().max().item() if fin.numel() else 1.0
    return LSE_FLOOR_REL * max(1.0, mag)


def max_abs_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| over finite reference entries; non-finite entries must match exactly."""
    x, ref = x.float(), ref.float()
    fin = torch.isfinite(ref)
    if not torch.equal(x[~fin], ref[~fin]):
        return float("inf")
    return (x[fin] - ref[fin]).abs().max().item() if fin.any() else 0.0


# --------------------------------------------------------------------------
# seeded inputs of the five benchmark configurations
# --------------------------------------------------------------------------
def flops_fwd(seqlens_q, seqlens_k, hq, d, dv, causal):
    """4*Hq*Sq*Sk*D per sequence (D = (d+dv)/2), halved under a causal mask with Sq == Sk."""
    tot = 0.0
    for sq, sk in zip(seqlens_q, seqlens_k):
        f = 2.0 * hq * sq * sk * (d + dv)
        if causal:
            f *= 0.5 if sq == sk else max(0.0, 1.0 - sq / (2.0 * sk)) if sk >= sq else sk / (2.0 * sq)
        tot += f
    return tot
