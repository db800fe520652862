"""flash-attn-2 style Python API on top of the B200 library.

Same public names, argument order, defaults and return conventions as the reference's
flash_attn_npu/flash_attn_npu_interface.py (flash_attn_func :1109, flash_attn_varlen_func
:1344, flash_attn_with_kvcache :1438, the four packed variants :972-1341, the autograd
classes :432-969 and the four custom ops :71-429).  Ops are registered for CUDA.
"""
from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F

from . import flash_attn_npu as _ext

_BWD_ALIGN = 64   # the backward pads the head dim to a multiple of 64 (reference :23-44)


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def round_multiple(x, m):
    return (x + m - 1) // m * m


def _pad_last(t, target):
    return t if t.size(-1) == target else F.pad(t, [0, target - t.size(-1)])


def _pad_bwd_headdim(dout, q, k, v, out):
    og = dout.size(-1)
    target = round_multiple(max(t.size(-1) for t in (dout, q, k, v, out)), _BWD_ALIGN)
    return tuple(_pad_last(t, target) for t in (dout, q, k, v, out)) + (og,)


def _pad_fwd_headdim(q, k, v):
    og = q.size(-1)
    if og % 8 != 0:
        q, k, v = (F.pad(t, [0, 8 - og % 8]) for t in (q, k, v))
    return q, k, v, og


_custom_op = torch.library.custom_op
_register_fake = torch.library.register_fake


# ------------------------------------------------------------------------------------------
# custom ops (torch.compile sees these; the fakes give shapes only)
# ------------------------------------------------------------------------------------------
@_custom_op("flash_attn_npu::_flash_attn_forward", mutates_args=(), device_types="cuda")
def _flash_attn_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dropout_p: float, softmax_scale: float,
                        causal: bool, window_size_left: int, window_size_right: int, softcap: float,
                        alibi_slopes: Optional[torch.Tensor], return_softmax: bool
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    out, lse, s_dmask, rng = _ext.fwd(q, k, v, None, alibi_slopes, dropout_p, softmax_scale, causal,
                                      window_size_left, window_size_right, softcap, return_softmax, None)
    return out, lse, s_dmask, rng


@_register_fake("flash_attn_npu::_flash_attn_forward")
def _flash_attn_forward_fake(q, k, v, dropout_p, softmax_scale, causal, window_size_left, window_size_right,
                             softcap, alibi_slopes, return_softmax):
    b, sq, h, _ = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    p = torch.empty((0,), dtype=q.dtype, device=q.device)
    if return_softmax:
        p = torch.empty((b, h, round_multiple(sq, 128), round_multiple(k.shape[1], 128)), dtype=q.dtype, device=q.device)
    return out, lse, p, torch.empty((2,), dtype=torch.int64, device=q.device)


@_custom_op("flash_attn_npu::_flash_attn_varlen_forward", mutates_args=(), device_types="cuda")
def _flash_attn_varlen_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                               cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, dropout_p: float,
                               softmax_scale: float, causal: bool, window_size_left: int = -1,
                               window_size_right: int = -1, softcap: float = 0.0,
                               alibi_slopes: Optional[torch.Tensor] = None, return_softmax: bool = False,
                               block_table: Optional[torch.Tensor] = None, leftpad_k: Optional[torch.Tensor] = None,
                               seqused_k: Optional[torch.Tensor] = None, zero_tensors: bool = False
                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    out, lse, s_dmask, rng = _ext.varlen_fwd(q, k, v, None, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k,
                                             block_table, alibi_slopes, max_seqlen_q, max_seqlen_k, dropout_p,
                                             softmax_scale, zero_tensors, causal, window_size_left,
                                             window_size_right, softcap, return_softmax, None)
    return out, lse, s_dmask, rng


@_register_fake("flash_attn_npu::_flash_attn_varlen_forward")
def _flash_attn_varlen_forward_fake(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                                    softmax_scale, causal, window_size_left=-1, window_size_right=-1, softcap=0.0,
                                    alibi_slopes=None, return_softmax=False, block_table=None, leftpad_k=None,
                                    seqused_k=None, zero_tensors=False):
    total_q, h, _ = q.shape
    b = cu_seqlens_q.numel() - 1
    out = torch.empty_like(q)
    lse = torch.empty((h, total_q), dtype=torch.float32, device=q.device)
    p = torch.empty((0,), dtype=q.dtype, device=q.device)
    if return_softmax:
        p = torch.empty((b, h, round_multiple(max_seqlen_q, 128), round_multiple(max_seqlen_k, 128)),
                        dtype=q.dtype, device=q.device)
    return out, lse, p, torch.empty((2,), dtype=torch.int64, device=q.device)


@_custom_op("flash_attn_npu::_flash_attn_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                         softmax_lse: torch.Tensor, dq: Optional[torch.Tensor], dk: Optional[torch.Tensor],
                         dv: Optional[torch.Tensor], dropout_p: float, softmax_scale: float, causal: bool,
                         window_size_left: int, window_size_right: int, softcap: float,
                         alibi_slopes: Optional[torch.Tensor], deterministic: bool,
                         rng_state: Optional[torch.Tensor] = None) -> torch.Tensor:
    dout, q, k, v, out = [maybe_contiguous(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, alibi_slopes, dropout_p,
                                  softmax_scale, causal, window_size_left, window_size_right, softcap,
                                  deterministic, None, rng_state)
    return softmax_d


@_register_fake("flash_attn_npu::_flash_attn_backward")
def _flash_attn_backward_fake(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale, causal,
                              window_size_left, window_size_right, softcap, alibi_slopes, deterministic,
                              rng_state=None):
    b, sq, h, _ = q.shape
    return torch.empty((b, h, round_multiple(sq, 128)), device=q.device, dtype=torch.float32)


@_custom_op("flash_attn_npu::_flash_attn_varlen_backward", mutates_args=("dq", "dk", "dv"), device_types="cuda")
def _flash_attn_varlen_backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                out: torch.Tensor, softmax_lse: torch.Tensor, dq: Optional[torch.Tensor],
                                dk: Optional[torch.Tensor], dv: Optional[torch.Tensor], cu_seqlens_q: torch.Tensor,
                                cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, dropout_p: float,
                                softmax_scale: float, causal: bool, window_size_left: int, window_size_right: int,
                                softcap: float, alibi_slopes: Optional[torch.Tensor], deterministic: bool,
                                rng_state: Optional[torch.Tensor] = None, zero_tensors: bool = False) -> torch.Tensor:
    dout, q, k, v, out = [maybe_contiguous(x) for x in (dout, q, k, v, out)]
    _, _, _, softmax_d = _ext.varlen_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                         alibi_slopes, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                                         zero_tensors, causal, window_size_left, window_size_right, softcap,
                                         deterministic, None, rng_state)
    return softmax_d


@_register_fake("flash_attn_npu::_flash_attn_varlen_backward")
def _flash_attn_varlen_backward_fake(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                     max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, causal, window_size_left,
                                     window_size_right, softcap, alibi_slopes, deterministic, rng_state=None,
                                     zero_tensors=False):
    total_q, h, _ = q.shape
    b = cu_seqlens_q.numel() - 1
    return torch.empty((h, total_q + 128 * b), device=q.device, dtype=torch.float32)


_wrapped_flash_attn_forward = _flash_attn_forward
_wrapped_flash_attn_varlen_forward = _flash_attn_varlen_forward
_wrapped_flash_attn_backward = _flash_attn_backward
_wrapped_flash_attn_varlen_backward = _flash_attn_varlen_backward


# ------------------------------------------------------------------------------------------
# autograd
# ------------------------------------------------------------------------------------------
def _dense_forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                   deterministic, return_softmax, is_grad):
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k, v, og = _pad_fwd_headdim(q, k, v)
    out_padded, lse, s_dmask, rng = _wrapped_flash_attn_forward(
        q, k, v, dropout_p, softmax_scale, causal=causal, window_size_left=window_size[0],
        window_size_right=window_size[1], softcap=softcap, alibi_slopes=alibi_slopes,
        return_softmax=return_softmax and dropout_p > 0)
    if is_grad:
        ctx.save_for_backward(q, k, v, out_padded, lse, rng)
        ctx.dropout_p, ctx.softmax_scale, ctx.causal = dropout_p, softmax_scale, causal
        ctx.window_size, ctx.softcap, ctx.alibi_slopes, ctx.deterministic = window_size, softcap, alibi_slopes, deterministic
    return out_padded[..., :og], lse, s_dmask


def _dense_backward(ctx, dout, dq=None, dk=None, dv=None):
    q, k, v, out, lse, rng = ctx.saved_tensors
    dout, q, k, v, out, og = _pad_bwd_headdim(dout, q, k, v, out)
    if dq is None or dq.size(-1) != q.size(-1):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        views = None
    else:
        views = True
    _wrapped_flash_attn_backward(dout, q, k, v, out, lse, dq, dk, dv, ctx.dropout_p, ctx.softmax_scale, ctx.causal,
                                 ctx.window_size[0], ctx.window_size[1], ctx.softcap, ctx.alibi_slopes,
                                 ctx.deterministic, rng_state=rng)
    return dq[..., :og], dk[..., :og], dv[..., :og], views


def _varlen_forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, dropout_p, softmax_scale, causal, window_size,
                    softcap, alibi_slopes, deterministic, return_softmax, block_table, is_grad):
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    q, k, v, og = _pad_fwd_headdim(q, k, v)
    out_padded, lse, s_dmask, rng = _wrapped_flash_attn_varlen_forward(
        q, k, v, cu_q, cu_k, max_q, max_k, dropout_p, softmax_scale, causal=causal,
        window_size_left=window_size[0], window_size_right=window_size[1], softcap=softcap,
        alibi_slopes=alibi_slopes, return_softmax=return_softmax and dropout_p > 0, block_table=block_table)
    if is_grad:
        ctx.save_for_backward(q, k, v, out_padded, lse, cu_q, cu_k, rng)
        ctx.dropout_p, ctx.max_seqlen_q, ctx.max_seqlen_k = dropout_p, max_q, max_k
        ctx.softmax_scale, ctx.causal, ctx.window_size = softmax_scale, causal, window_size
        ctx.softcap, ctx.alibi_slopes, ctx.deterministic = softcap, alibi_slopes, deterministic
    return out_padded[..., :og], lse, s_dmask


def _varlen_backward(ctx, dout):
    q, k, v, out, lse, cu_q, cu_k, rng = ctx.saved_tensors
    dout, q, k, v, out, og = _pad_bwd_headdim(dout, q, k, v, out)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    _wrapped_flash_attn_varlen_backward(dout, q, k, v, out, lse, dq, dk, dv, cu_q, cu_k, ctx.max_seqlen_q,
                                        ctx.max_seqlen_k, ctx.dropout_p, ctx.softmax_scale, ctx.causal,
                                        ctx.window_size[0], ctx.window_size[1], ctx.softcap, ctx.alibi_slopes,
                                        ctx.deterministic, rng_state=rng)
    return dq[..., :og], dk[..., :og], dv[..., :og]


def _needs_grad(enabled, *ts):
    return enabled and any(t.requires_grad for t in ts)


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                return_softmax, is_grad_enabled):
        out, lse, s_dmask = _dense_forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                                           alibi_slopes, deterministic, return_softmax,
                                           _needs_grad(is_grad_enabled, q, k, v))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv, _ = _dense_backward(ctx, dout)
        return (dq, dk, dv) + (None,) * 9


class FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                causal, window_size, softcap, alibi_slopes, deterministic, return_softmax, block_table,
                is_grad_enabled):
        out, lse, s_dmask = _varlen_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                            dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                            deterministic, return_softmax, block_table,
                                            _needs_grad(is_grad_enabled, q, k, v))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv = _varlen_backward(ctx, dout)
        return (dq, dk, dv) + (None,) * 14


class FlashAttnQKVPackedFunc(torch.autograd.Function):
    """qkv (B,S,3,H,D): the three gradients are written into one packed buffer."""

    @staticmethod
    def forward(ctx, qkv, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                return_softmax, is_grad_enabled):
        q, k, v = qkv[:, :, 0].detach(), qkv[:, :, 1].detach(), qkv[:, :, 2].detach()
        out, lse, s_dmask = _dense_forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                                           alibi_slopes, deterministic, return_softmax,
                                           _needs_grad(is_grad_enabled, qkv))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        q = ctx.saved_tensors[0]
        dqkv = torch.empty(q.shape[:2] + (3,) + q.shape[2:], dtype=q.dtype, device=q.device)
        dq, dk, dv, used = _dense_backward(ctx, dout, dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2])
        if not used:
            dqkv = torch.stack((dq, dk, dv), dim=2)
        else:
            dqkv = dqkv[..., :dout.shape[-1]]
        return (dqkv,) + (None,) * 9


class FlashAttnKVPackedFunc(torch.autograd.Function):
    """q (B,Sq,H,D), kv (B,Sk,2,Hkv,D)."""

    @staticmethod
    def forward(ctx, q, kv, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                return_softmax, is_grad_enabled):
        k, v = kv[:, :, 0].detach(), kv[:, :, 1].detach()
        out, lse, s_dmask = _dense_forward(ctx, q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                                           alibi_slopes, deterministic, return_softmax,
                                           _needs_grad(is_grad_enabled, q, kv))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv, _ = _dense_backward(ctx, dout)
        return (dq, torch.stack((dk, dv), dim=2)) + (None,) * 9


class FlashAttnVarlenQKVPackedFunc(torch.autograd.Function):
    """qkv (T,3,H,D) with cu_seqlens."""

    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, dropout_p, softmax_scale, causal, window_size, softcap,
                alibi_slopes, deterministic, return_softmax, is_grad_enabled):
        q, k, v = qkv[:, 0].detach(), qkv[:, 1].detach(), qkv[:, 2].detach()
        out, lse, s_dmask = _varlen_forward(ctx, q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, dropout_p,
                                            softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                                            return_softmax, None, _needs_grad(is_grad_enabled, qkv))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv = _varlen_backward(ctx, dout)
        return (torch.stack((dq, dk, dv), dim=1),) + (None,) * 11


class FlashAttnVarlenKVPackedFunc(torch.autograd.Function):
    """q (Tq,H,D), kv (Tk,2,Hkv,D) with cu_seqlens."""

    @staticmethod
    def forward(ctx, q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale,
                causal, window_size, softcap, alibi_slopes, deterministic, return_softmax, is_grad_enabled):
        k, v = kv[:, 0].detach(), kv[:, 1].detach()
        out, lse, s_dmask = _varlen_forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                            dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                            deterministic, return_softmax, None, _needs_grad(is_grad_enabled, q, kv))
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        dq, dk, dv = _varlen_backward(ctx, dout)
        return (dq, torch.stack((dk, dv), dim=1)) + (None,) * 13


# ------------------------------------------------------------------------------------------
# public functions
# ------------------------------------------------------------------------------------------
def flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                              softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """Attention over a packed qkv (batch, seqlen, 3, nheads, headdim); see flash_attn_func."""
    return FlashAttnQKVPackedFunc.apply(qkv, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                        deterministic, return_attn_probs, torch.is_grad_enabled())


def flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                             softcap=0.0, alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """q (batch, seqlen_q, nheads, headdim), kv (batch, seqlen_k, 2, nheads_k, headdim); see flash_attn_func."""
    return FlashAttnKVPackedFunc.apply(q, kv, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                       deterministic, return_attn_probs, torch.is_grad_enabled())


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """Scaled dot-product attention, differentiable.

    q (batch, seqlen_q, nheads, headdim); k, v (batch, seqlen_k, nheads_k, headdim) with
    nheads % nheads_k == 0 (MQA/GQA: query head h reads KV head h // (nheads / nheads_k)).
    softmax_scale defaults to headdim ** -0.5.  causal masks are aligned to the bottom-right
    corner: key j is visible to query i iff j <= i + seqlen_k - seqlen_q.  window_size
    (left, right) keeps keys in [i + seqlen_k - seqlen_q - left, i + seqlen_k - seqlen_q + right];
    -1 means unbounded.  softcap > 0 applies softcap * tanh(score / softcap).  alibi_slopes
    (nheads,) or (batch, nheads) fp32 adds -slope * |i + seqlen_k - seqlen_q - j| (forward only).
    Rows without any visible key give zeros.  dropout_p must be 0.

    Returns out (batch, seqlen_q, nheads, headdim), or (out, softmax_lse (batch, nheads, seqlen_q),
    S_dmask (empty)) when return_attn_probs is set.
    """
    return FlashAttnFunc.apply(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                               deterministic, return_attn_probs, torch.is_grad_enabled())


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p=0.0, softmax_scale=None, causal=False,
                                     window_size=(-1, -1), softcap=0.0, alibi_slopes=None, deterministic=False,
                                     return_attn_probs=False):
    """Packed-sequence attention over qkv (total, 3, nheads, headdim); see flash_attn_varlen_func."""
    return FlashAttnVarlenQKVPackedFunc.apply(qkv, cu_seqlens, max_seqlen, dropout_p, softmax_scale, causal,
                                              window_size, softcap, alibi_slopes, deterministic, return_attn_probs,
                                              torch.is_grad_enabled())


def flash_attn_varlen_kvpacked_func(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                                    softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                                    alibi_slopes=None, deterministic=False, return_attn_probs=False):
    """q (total_q, nheads, headdim), kv (total_k, 2, nheads_k, headdim); see flash_attn_varlen_func."""
    return FlashAttnVarlenKVPackedFunc.apply(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                             dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                                             deterministic, return_attn_probs, torch.is_grad_enabled())


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                           softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                           deterministic=False, return_attn_probs=False, block_table=None):
    """Attention over sequences packed along the token axis, differentiable.

    q (total_q, nheads, headdim), k/v (total_k, nheads_k, headdim); cu_seqlens_q / cu_seqlens_k
    are int32 (batch + 1,) prefix sums; max_seqlen_q / max_seqlen_k bound the lengths.  Masking,
    scaling, softcap and GQA as in flash_attn_func, applied per sequence.  With block_table,
    k/v are a paged cache (num_blocks, page, nheads_k, headdim) (forward only).
    Returns out (total_q, nheads, headdim) or (out, softmax_lse (nheads, total_q), S_dmask).
    """
    return FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p,
                                     softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic,
                                     return_attn_probs, block_table, torch.is_grad_enabled())


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens: Optional[Union[int, torch.Tensor]] = None,
                            cache_batch_idx: Optional[torch.Tensor] = None,
                            cache_leftpad: Optional[torch.Tensor] = None,
                            block_table: Optional[torch.Tensor] = None, softmax_scale=None, causal=False,
                            window_size=(-1, -1), softcap=0.0, rotary_interleaved=True, alibi_slopes=None,
                            num_splits=0, return_softmax_lse=False):
    """Inference attention against a KV cache (no backward).

    q (batch, seqlen_q, nheads, headdim).  k_cache / v_cache are (batch_cache, seqlen_cache,
    nheads_k, headdim), or (num_blocks, page_block_size, nheads_k, headdim) together with an int32
    block_table (batch, max_blocks_per_seq).  cache_seqlens (int or int32 (batch,)) gives the number
    of valid keys per sequence.  If k and v (batch, seqlen_new, nheads_k, headdim) are given they
    are written into the cache IN PLACE at positions cache_seqlens .. cache_seqlens + seqlen_new - 1
    and attention runs over the extended cache.  rotary_cos / rotary_sin (seqlen_ro, rotary_dim / 2)
    rotate the new keys at those positions and the queries at cache_seqlens + i when the call is
    causal or windowed, else at cache_seqlens; rotary_interleaved pairs dims (0,1),(2,3).. instead
    of (i, i + rotary_dim/2).  cache_batch_idx selects cache rows for a dense cache.
    num_splits: 0 = choose automatically, 1 = no split of the key axis, n = n splits.
    Masking, softcap, alibi and GQA as in flash_attn_func.  cache_leftpad is not supported.
    Returns out, or (out, softmax_lse (batch, nheads, seqlen_q)) with return_softmax_lse.
    """
    assert k_cache.stride(-1) == 1, "k_cache must have contiguous last dimension"
    assert v_cache.stride(-1) == 1, "v_cache must have contiguous last dimension"
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if cache_seqlens is not None and isinstance(cache_seqlens, int):
        cache_seqlens = torch.full((q.shape[0],), cache_seqlens, dtype=torch.int32, device=k_cache.device)
    cache_seqlens = maybe_contiguous(cache_seqlens)
    cache_batch_idx = maybe_contiguous(cache_batch_idx)
    block_table = maybe_contiguous(block_table)
    out, lse = _ext.fwd_kvcache(q, k_cache, v_cache, k, v, cache_seqlens, rotary_cos, rotary_sin, cache_batch_idx,
                                cache_leftpad, block_table, alibi_slopes, None, softmax_scale, causal,
                                window_size[0], window_size[1], softcap, rotary_interleaved, num_splits)
    return (out, lse) if return_softmax_lse else out
