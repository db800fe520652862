"""flash-attn-3 style Python API on top of the B200 library.

Public names, argument order, defaults and return conventions follow the reference's
flash_attn_npu_3/flash_attn_npu_interface.py: flash_attn_func :828, flash_attn_varlen_func :911,
flash_attn_qkvpacked_func :766, flash_attn_combine :961, flash_attn_with_kvcache :965,
get_scheduler_metadata :1129, the single forward custom op with 34 arguments :87-178 and the
backward op :286-342.  Ops are registered for CUDA.
"""
from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F

from . import flash_attn_npu_3 as _ext


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def round_multiple(x, m):
    return (x + m - 1) // m * m


def round_up_headdim(head_size: int) -> int:
    """Head-dim bucket of the kernels (64 / 96 / 128 / 192 / 256)."""
    for b in (64, 96, 128, 192, 256):
        if head_size <= b:
            return b
    return 256


def _pad_bwd_headdim(dout, q, k, v, out):
    og = dout.size(-1)
    target = round_multiple(max(t.size(-1) for t in (dout, q, k, v, out)), 64)
    pad = lambda t: t if t.size(-1) == target else F.pad(t, [0, target - t.size(-1)])  # noqa: E731
    return pad(dout), pad(q), pad(k), pad(v), pad(out), og


@torch.library.custom_op("flash_attn_npu_3::_flash_attn_forward", mutates_args=(), device_types="cuda")
def _flash_attn_forward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None,
    qv: Optional[torch.Tensor] = None, out_: Optional[torch.Tensor] = None,
    cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k: Optional[torch.Tensor] = None,
    cu_seqlens_k_new: Optional[torch.Tensor] = None,
    seqused_q: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None, max_seqlen_k: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None, kv_batch_idx: Optional[torch.Tensor] = None,
    leftpad_k: Optional[torch.Tensor] = None,
    rotary_cos: Optional[torch.Tensor] = None, rotary_sin: Optional[torch.Tensor] = None,
    seqlens_rotary: Optional[torch.Tensor] = None,
    q_descale: Optional[torch.Tensor] = None, k_descale: Optional[torch.Tensor] = None,
    v_descale: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None, causal: bool = False,
    window_size_left: int = -1, window_size_right: int = -1, attention_chunk: int = 0,
    softcap: float = 0.0, rotary_interleaved: bool = True,
    scheduler_metadata: Optional[torch.Tensor] = None, num_splits: int = 1,
    pack_gqa: Optional[bool] = None, sm_margin: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, k_new, v_new = [maybe_contiguous(x) for x in (q, k, k_new, v_new)]
    v = v.contiguous() if v.stride(-1) != 1 else v
    cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx = [
        maybe_contiguous(x) for x in (cu_seqlens_q, cu_seqlens_k, seqused_k, page_table, kv_batch_idx)]
    out, lse, out_accum, lse_accum = _ext.fwd(
        q, k, v, k_new, v_new, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
        max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
        q_descale, k_descale, v_descale, softmax_scale, causal, window_size_left, window_size_right,
        attention_chunk, softcap, rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin)
    if out_accum is None:
        out_accum = torch.empty((0,), device=out.device)
    if lse_accum is None:
        lse_accum = torch.empty((0,), device=out.device)
    if out_ is not None and out.data_ptr() == out_.data_ptr():
        out = out.clone()          # a custom op may not return an alias of its input
    return out, lse, out_accum, lse_accum


@torch.library.register_fake("flash_attn_npu_3::_flash_attn_forward")
def _flash_attn_forward_fake(q, k, v, k_new=None, v_new=None, qv=None, out_=None, cu_seqlens_q=None,
                             cu_seqlens_k=None, cu_seqlens_k_new=None, seqused_q=None, seqused_k=None,
                             max_seqlen_q=None, max_seqlen_k=None, page_table=None, kv_batch_idx=None,
                             leftpad_k=None, rotary_cos=None, rotary_sin=None, seqlens_rotary=None,
                             q_descale=None, k_descale=None, v_descale=None, softmax_scale=None, causal=False,
                             window_size_left=-1, window_size_right=-1, attention_chunk=0, softcap=0.0,
                             rotary_interleaved=True, scheduler_metadata=None, num_splits=1, pack_gqa=None,
                             sm_margin=0):
    dv = v.shape[-1]
    out = torch.empty(q.shape[:-1] + (dv,), dtype=q.dtype, device=q.device)
    if cu_seqlens_q is not None:
        lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device)
    else:
        lse = torch.empty((q.shape[0], q.shape[2], q.shape[1]), dtype=torch.float32, device=q.device)
    e = torch.empty((0,), device=q.device)
    return out, lse, e, e.clone()


@torch.library.custom_op("flash_attn_npu_3::_flash_attn_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_backward(
    dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
    softmax_lse: torch.Tensor,
    cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k: Optional[torch.Tensor] = None,
    sequed_q: Optional[torch.Tensor] = None, sequed_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None, max_seqlen_k: Optional[int] = None,
    dq: Optional[torch.Tensor] = None, dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None,
    softmax_scale: Optional[float] = None, is_causal: bool = False,
    window_size_left: int = -1, window_size_right: int = -1, softcap: float = 0.0,
    deterministic: bool = False, sm_margin: int = 0,
) -> torch.Tensor:
    dout, q, k, v, out = [maybe_contiguous(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                  sequed_q, sequed_k, max_seqlen_q, max_seqlen_k, softmax_scale, is_causal,
                                  window_size_left, window_size_right, softcap, deterministic, sm_margin)
    return softmax_d


@torch.library.register_fake("flash_attn_npu_3::_flash_attn_backward")
def _flash_attn_backward_fake(dout, q, k, v, out, softmax_lse, cu_seqlens_q=None, cu_seqlens_k=None, sequed_q=None,
                              sequed_k=None, max_seqlen_q=None, max_seqlen_k=None, dq=None, dk=None, dv=None,
                              softmax_scale=None, is_causal=False, window_size_left=-1, window_size_right=-1,
                              softcap=0.0, deterministic=False, sm_margin=0):
    if cu_seqlens_q is not None:
        return torch.empty((q.shape[1], q.shape[0] + 128 * (cu_seqlens_q.numel() - 1)), dtype=torch.float32,
                           device=q.device)
    return torch.empty((q.shape[0], q.shape[2], round_multiple(q.shape[1], 128)), dtype=torch.float32, device=q.device)


def _run_backward(ctx, dout, q, k, v, out, lse, cu_q=None, cu_k=None, max_q=None, max_k=None):
    assert ctx.attention_chunk == 0, "backward does not support attention_chunk"
    dout, q, k, v, out, og = _pad_bwd_headdim(dout, q, k, v, out)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _flash_attn_backward(dout, q, k, v, out, lse, cu_q, cu_k, None, None, max_q, max_k, dq, dk, dv,
                         ctx.softmax_scale, ctx.causal, ctx.window_size[0], ctx.window_size[1], ctx.softcap,
                         ctx.deterministic, ctx.sm_margin)
    return dq[..., :og], dk[..., :og], dv[..., :og]


def _stash(ctx, softmax_scale, causal, window_size, attention_chunk, softcap, deterministic, sm_margin):
    ctx.softmax_scale, ctx.causal, ctx.window_size = softmax_scale, causal, window_size
    ctx.attention_chunk, ctx.softcap, ctx.deterministic, ctx.sm_margin = attention_chunk, softcap, deterministic, sm_margin


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, qv=None, q_descale=None, k_descale=None, v_descale=None,
                window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1, pack_gqa=None,
                deterministic=False, sm_margin=0, return_softmax=False, scheduler_metadata=None):
        if softmax_scale is None:
            softmax_scale = (q.shape[-1] + (qv.shape[-1] if qv is not None else 0)) ** (-0.5)
        out, lse, *_ = _flash_attn_forward(
            q, k, v, None, None, qv, None, None, None, None, None, None, None, None, None, None, None, None, None,
            None, q_descale, k_descale, v_descale, softmax_scale, causal=causal, window_size_left=window_size[0],
            window_size_right=window_size[1], attention_chunk=attention_chunk, softcap=softcap,
            scheduler_metadata=scheduler_metadata, num_splits=num_splits, pack_gqa=pack_gqa, sm_margin=sm_margin)
        ctx.save_for_backward(q, k, v, out, lse)
        _stash(ctx, softmax_scale, causal, window_size, attention_chunk, softcap, deterministic, sm_margin)
        return (out, lse) if return_softmax else out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _run_backward(ctx, dout, q, k, v, out, lse)
        return (dq, dk, dv) + (None,) * 15


class FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, max_seqlen_q, max_seqlen_k,
                softmax_scale, causal, qv=None, q_descale=None, k_descale=None, v_descale=None,
                window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1, pack_gqa=None,
                deterministic=False, sm_margin=0, return_softmax=False, scheduler_metadata=None):
        if softmax_scale is None:
            softmax_scale = (q.shape[-1] + (qv.shape[-1] if qv is not None else 0)) ** (-0.5)
        out, lse, *_ = _flash_attn_forward(
            q, k, v, None, None, qv, None, cu_seqlens_q, cu_seqlens_k, None, seqused_q, seqused_k, max_seqlen_q,
            max_seqlen_k, None, None, None, None, None, None, q_descale, k_descale, v_descale, softmax_scale,
            causal=causal, window_size_left=window_size[0], window_size_right=window_size[1],
            attention_chunk=attention_chunk, softcap=softcap, scheduler_metadata=scheduler_metadata,
            num_splits=num_splits, pack_gqa=pack_gqa, sm_margin=sm_margin)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k)
        ctx.max_seqlen_q, ctx.max_seqlen_k = max_seqlen_q, max_seqlen_k
        _stash(ctx, softmax_scale, causal, window_size, attention_chunk, softcap, deterministic, sm_margin)
        return (out, lse) if return_softmax else out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = _run_backward(ctx, dout, q, k, v, out, lse, cu_q, cu_k, ctx.max_seqlen_q, ctx.max_seqlen_k)
        return (dq, dk, dv) + (None,) * 21


class FlashAttnQKVPackedFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, softmax_scale, causal, q_descale=None, k_descale=None, v_descale=None,
                window_size=(-1, -1), attention_chunk=0, softcap=0.0, deterministic=False, num_heads_q=None,
                sm_margin=0, return_softmax=False):
        if qkv.dim() == 5:
            assert qkv.shape[-3] == 3
            q, k, v = qkv.unbind(dim=-3)
        else:
            assert qkv.dim() == 4 and num_heads_q is not None
            hk = (qkv.shape[2] - num_heads_q) // 2
            q, k, v = qkv.split([num_heads_q, hk, hk], dim=-2)
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, lse, *_ = _flash_attn_forward(
            q, k, v, None, None, None, None, None, None, None, None, None, None, None, None, None, None, None, None,
            None, q_descale, k_descale, v_descale, softmax_scale, causal=causal, window_size_left=window_size[0],
            window_size_right=window_size[1], attention_chunk=attention_chunk, softcap=softcap, sm_margin=sm_margin)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.ndim = qkv.dim()
        _stash(ctx, softmax_scale, causal, window_size, attention_chunk, softcap, deterministic, sm_margin)
        return (out, lse) if return_softmax else out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _run_backward(ctx, dout, q, k, v, out, lse)
        dqkv = torch.stack((dq, dk, dv), dim=-3) if ctx.ndim == 5 else torch.cat((dq, dk, dv), dim=-2)
        return (dqkv,) + (None,) * 12


def flash_attn_qkvpacked_func(qkv, softmax_scale=None, causal=False, q_descale=None, k_descale=None, v_descale=None,
                              window_size=(-1, -1), attention_chunk=0, softcap=0.0, deterministic=False,
                              num_heads_q=None, sm_margin=0, return_attn_probs=False):
    """qkv (batch, seqlen, 3, nheads, headdim), or (batch, seqlen, nheads_q + 2 nheads_k, headdim)
    with num_heads_q; see flash_attn_func."""
    return FlashAttnQKVPackedFunc.apply(qkv, softmax_scale, causal, q_descale, k_descale, v_descale, window_size,
                                        attention_chunk, softcap, deterministic, num_heads_q, sm_margin,
                                        return_attn_probs)


def flash_attn_func(q, k, v, softmax_scale=None, causal=False, qv=None, q_descale=None, k_descale=None,
                    v_descale=None, window_size=(-1, -1), attention_chunk=0, softcap=0.0, num_splits=1,
                    pack_gqa=None, deterministic=False, sm_margin=0, return_attn_probs=False,
                    scheduler_metadata=None):
    """Differentiable attention: q (batch, seqlen_q, nheads, headdim), k/v (batch, seqlen_k, nheads_k,
    headdim); bottom-right aligned causal / window masks, softcap, GQA.  qv, FP8 descales and
    attention_chunk are rejected.  Returns out, or (out, softmax_lse (batch, nheads, seqlen_q))."""
    return FlashAttnFunc.apply(q, k, v, softmax_scale, causal, qv, q_descale, k_descale, v_descale, window_size,
                               attention_chunk, softcap, num_splits, pack_gqa, deterministic, sm_margin,
                               return_attn_probs, scheduler_metadata)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, seqused_q=None,
                           seqused_k=None, softmax_scale=None, causal=False, qv=None, q_descale=None,
                           k_descale=None, v_descale=None, window_size=(-1, -1), attention_chunk=0, softcap=0.0,
                           num_splits=1, pack_gqa=None, deterministic=False, sm_margin=0, return_attn_probs=False,
                           scheduler_metadata=None):
    """Packed-sequence attention: q (total_q, nheads, headdim), k/v (total_k, nheads_k, headdim) with int32
    prefix sums.  Returns out, or (out, softmax_lse (nheads, total_q))."""
    return FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, max_seqlen_q,
                                     max_seqlen_k, softmax_scale, causal, qv, q_descale, k_descale, v_descale,
                                     window_size, attention_chunk, softcap, num_splits, pack_gqa, deterministic,
                                     sm_margin, return_attn_probs, scheduler_metadata)


def flash_attn_combine(out_partial, lse_partial, out=None, out_dtype=None):
    """LSE-weighted merge of split-KV partial results: out_partial (nsplit, ..., dv) fp32 (each already
    normalised), lse_partial (nsplit, ...) -> (out, lse)."""
    return _ext.fwd_combine(out_partial, lse_partial, out, out_dtype)


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, qv=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx: Optional[torch.Tensor] = None,
                            cache_leftpad: Optional[torch.Tensor] = None,
                            page_table: Optional[torch.Tensor] = None,
                            cu_seqlens_q: Optional[torch.Tensor] = None,
                            cu_seqlens_k_new: Optional[torch.Tensor] = None,
                            max_seqlen_q: Optional[int] = None, rotary_seqlens: Optional[torch.Tensor] = None,
                            q_descale=None, k_descale=None, v_descale=None, softmax_scale=None, causal=False,
                            window_size=(-1, -1), attention_chunk=0, softcap=0.0, rotary_interleaved=True,
                            scheduler_metadata=None, num_splits=0, pack_gqa=None, sm_margin=0,
                            return_softmax_lse=False):
    """Inference attention against a dense or paged KV cache, with optional in-place append of k / v and
    rotary embedding; same semantics as the v2 flash_attn_with_kvcache.  q may be packed (total_q, nheads,
    headdim) with cu_seqlens_q and max_seqlen_q.  scheduler_metadata (from get_scheduler_metadata) is
    accepted; the call never synchronises with the host either way.  Returns out, or (out, softmax_lse, ...)."""
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    if softmax_scale is None:
        softmax_scale = (q.shape[-1] + (qv.shape[-1] if qv is not None else 0)) ** (-0.5)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        nb = q.shape[0] if cu_seqlens_q is None else cu_seqlens_q.numel() - 1
        cache_seqlens = torch.full((nb,), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    out, lse, *rest = _flash_attn_forward(
        q, k_cache, v_cache, k, v, qv, None, cu_seqlens_q, None, cu_seqlens_k_new, None, cache_seqlens,
        max_seqlen_q, None, page_table, cache_batch_idx, cache_leftpad, rotary_cos, rotary_sin, rotary_seqlens,
        q_descale, k_descale, v_descale, softmax_scale, causal=causal, window_size_left=window_size[0],
        window_size_right=window_size[1], attention_chunk=attention_chunk, softcap=softcap,
        rotary_interleaved=rotary_interleaved, scheduler_metadata=scheduler_metadata, num_splits=num_splits,
        pack_gqa=pack_gqa, sm_margin=sm_margin)
    return (out, lse, *rest) if return_softmax_lse else out


def get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim,
                           cache_seqlens: torch.Tensor, qkv_dtype=torch.bfloat16, headdim_v=None,
                           cu_seqlens_q: Optional[torch.Tensor] = None,
                           cu_seqlens_k_new: Optional[torch.Tensor] = None,
                           cache_leftpad: Optional[torch.Tensor] = None, page_size: Optional[int] = None,
                           max_seqlen_k_new=0, causal=False, window_size=(-1, -1), attention_chunk=0,
                           has_softcap=False, num_splits=0, pack_gqa=None, sm_margin=0):
    """Device-side split plan for flash_attn_with_kvcache, computed without a host synchronisation."""
    cache_seqlens = maybe_contiguous(cache_seqlens)
    if headdim_v is None:
        headdim_v = headdim
    return _ext.get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads_q, num_heads_kv, headdim,
                                       headdim_v, qkv_dtype, cache_seqlens, cu_seqlens_q, None, cu_seqlens_k_new,
                                       None, cache_leftpad, page_size, max_seqlen_k_new, causal, window_size[0],
                                       window_size[1], attention_chunk, has_softcap, num_splits, pack_gqa, sm_margin)


def flash_attn_mla_with_kvcache(q_nope, q_rope, latent_cache_i8, latent_scales, rope_cache, cache_seqlens, page_table,
                                softmax_scale=None, num_splits=0, return_softmax_lse=False):
    """Decode step of multi-head latent attention against a paged, int8-quantised latent cache (an addition of
    this library).  q_nope (batch, 1, nheads, 512) and q_rope (batch, 1, nheads, 64) bf16; latent_cache_i8
    (num_blocks, page, 512) int8 with latent_scales (num_blocks, page) fp32 (key = value = scale * int8 row,
    rounded to bf16); rope_cache (num_blocks, page, 64) bf16 is the positional part of the keys; all query heads
    share the one KV head.  softmax_scale defaults to 576 ** -0.5.  Returns out (batch, 1, nheads, 512) bf16,
    or (out, softmax_lse (batch, nheads, 1))."""
    if softmax_scale is None:
        softmax_scale = (q_nope.shape[-1] + q_rope.shape[-1]) ** (-0.5)
    out, lse = _ext.mla_decode(q_nope, q_rope, latent_cache_i8, latent_scales, rope_cache, page_table, cache_seqlens,
                               softmax_scale, num_splits)
    return (out, lse) if return_softmax_lse else out
