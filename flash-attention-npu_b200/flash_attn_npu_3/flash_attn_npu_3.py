"""The extension module of the v3 API: `fwd`, `bwd`, `get_scheduler_metadata` with the
positional signatures of the reference's pybind module
(csrc/ascend910/flash_attn_npu_3/flash_api.cpp:829-835; fwd :60-96, bwd :573-596,
get_scheduler_metadata :506-530) plus `fwd_combine`, which the reference's Python calls
(flash_attn_npu_3/flash_attn_npu_interface.py:961) but its module never defines."""
from typing import Optional

import torch

import fa_b200_capi as capi
from fa_b200_capi import CombineParams, SchedParams, check, lib, ptr
from flash_attn_npu import flash_attn_npu as _v2


def _reject(cond, what):
    if cond:
        raise RuntimeError(f"FlashAttention on B200 does not support {what}")


def fwd(q, k, v, k_new, v_new, qv, out_, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q, seqused_k,
        max_seqlen_q, max_seqlen_k, page_table, kv_batch_idx, leftpad_k, rotary_cos, rotary_sin, seqlens_rotary,
        q_descale, k_descale, v_descale, softmax_scale, is_causal, window_size_left, window_size_right,
        attention_chunk, softcap, is_rotary_interleaved, scheduler_metadata, num_splits, pack_gqa, sm_margin):
    """mha_fwd (csrc/ascend910/flash_attn_npu_3/flash_api.cpp:60-504): one entry for dense,
    packed, paged and KV-cache calls -> [out, softmax_lse, out_accum, softmax_lse_accum].
    The same features are rejected as there (:149-161): qv, FP8 descales, attention_chunk,
    leftpad_k, seqused_q, cu_seqlens_k_new, seqlens_rotary."""
    _reject(qv is not None, "qv")
    _reject(q_descale is not None or k_descale is not None or v_descale is not None, "FP8 descale")
    _reject(attention_chunk != 0, "attention_chunk")
    _reject(leftpad_k is not None, "leftpad_k")
    _reject(seqused_q is not None, "seqused_q")
    _reject(cu_seqlens_k_new is not None, "cu_seqlens_k_new")
    _reject(seqlens_rotary is not None, "seqlens_rotary")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    cache_like = page_table is not None or seqused_k is not None or k_new is not None or kv_batch_idx is not None
    if cache_like:
        # The kernels read the lengths themselves, so the call is sync-free with or without the blob; with it the
        # split-KV decode takes each sequence's keys per split from the device-side plan (flash_api.cpp:248-267
        # takes its tiling from the blob in the same way).
        out, lse = _v2.kvcache_forward(q, k, v, k_new, v_new, seqused_k, rotary_cos, rotary_sin, kv_batch_idx,
                                       page_table, None, out_, softmax_scale, is_causal, window_size_left,
                                       window_size_right, softcap, is_rotary_interleaved,
                                       num_splits if num_splits is not None else 0,
                                       cu_seqlens_q=cu_seqlens_q, max_seqlen_q=max_seqlen_q,
                                       sched_meta=scheduler_metadata)
        return [out, lse, None, None]
    if cu_seqlens_q is not None:
        out, lse, _, _ = _v2.varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, None, None, None, None,
                                        max_seqlen_q, max_seqlen_k, 0.0, softmax_scale, False, is_causal,
                                        window_size_left, window_size_right, softcap, False, None)
        return [out, lse, None, None]
    out, lse, _, _ = _v2.fwd(q, k, v, out_, None, 0.0, softmax_scale, is_causal, window_size_left,
                             window_size_right, softcap, False, None)
    return [out, lse, None, None]


def bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k,
        max_seqlen_q, max_seqlen_k, softmax_scale, is_causal, window_size_left, window_size_right, softcap,
        deterministic, sm_margin):
    """mha_bwd (csrc/ascend910/flash_attn_npu_3/flash_api.cpp:573-827) -> [dq, dk, dv, softmax_d]."""
    _reject(seqused_q is not None or seqused_k is not None, "seqused_q / seqused_k in the backward pass")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if cu_seqlens_q is not None:
        return _v2.varlen_bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, None,
                              max_seqlen_q, max_seqlen_k, 0.0, softmax_scale, False, is_causal, window_size_left,
                              window_size_right, softcap, deterministic, None, None)
    return _v2.bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, None, 0.0, softmax_scale, is_causal,
                   window_size_left, window_size_right, softcap, deterministic, None, None)


def get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                           qkv_dtype, seqused_k, cu_seqlens_q, cu_seqlens_k, cu_seqlens_k_new, seqused_q,
                           leftpad_k, page_size, max_seqlen_k_new, is_causal, window_size_left, window_size_right,
                           attention_chunk, has_softcap, num_splits, pack_gqa, sm_margin):
    """get_scheduler_metadata (csrc/ascend910/flash_attn_npu_3/flash_api.cpp:506-571): a device
    tensor holding the KV split plan computed on the device from the device-resident lengths.
    Returned as uint8 like the reference's blob."""
    capi.require_cuda(seqused_k)
    n = lib.fa_scheduler_metadata_ints(batch_size)
    meta = torch.empty((n,), dtype=torch.int32, device=seqused_k.device)
    p = SchedParams()
    p.seqused_k, p.cu_seqlens_q = seqused_k.data_ptr(), ptr(cu_seqlens_q)
    p.b, p.sq, p.sk, p.hq, p.hkv = batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k
    p.d, p.dv, p.page_size, p.s_new = headdim, headdim_v, page_size or 0, max_seqlen_k_new or 0
    p.causal, p.window_left, p.window_right = int(is_causal), window_size_left, window_size_right
    p.num_splits = num_splits or 0
    p.meta = meta.data_ptr()
    p.stream = capi.stream_ptr(seqused_k.device)
    with torch.cuda.device(seqused_k.device):
        check(lib.fa_scheduler_metadata(p))
    return meta.view(torch.uint8)


def fwd_combine(out_partial, lse_partial, out=None, out_dtype=None):
    """LSE-weighted combine. out_partial (nsplit, ..., dv) fp32, lse_partial (nsplit, ...) fp32
    -> (out (..., dv), lse (...))."""
    capi.require_cuda(out_partial, lse_partial)
    nsplit = out_partial.shape[0]
    dv = out_partial.shape[-1]
    # the partials of one split must be dense; the splits themselves may lie any distance apart (the receive buffer
    # of an all-gather holds [O | LSE] of every rank back to back)
    op = out_partial if out_partial.dtype == torch.float32 and out_partial[0].is_contiguous() else out_partial.contiguous().float()
    lp = lse_partial if lse_partial.dtype == torch.float32 and lse_partial[0].is_contiguous() else lse_partial.contiguous().float()
    rows = lp[0].numel()
    out_dtype = out_dtype or (out.dtype if out is not None else torch.float32)
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out_dtype]
    res = torch.empty(out_partial.shape[1:], dtype=out_dtype, device=op.device)
    lse = torch.empty(lse_partial.shape[1:], dtype=torch.float32, device=op.device)
    c = CombineParams()
    c.o_partial, c.lse_partial = op.data_ptr(), lp.data_ptr()
    c.o_split_stride, c.o_row_stride, c.lse_split_stride = op.stride(0), dv, lp.stride(0)
    c.o, c.o_stride, c.lse = res.data_ptr(), dv, lse.data_ptr()
    c.nsplit, c.rows, c.dv, c.out_dtype = nsplit, rows, dv, code
    c.stream = capi.stream_ptr(op.device)
    with torch.cuda.device(op.device):
        check(lib.fa_combine(c))
    if out is not None:
        out.copy_(res)
        res = out
    return res, lse


def mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale,
               num_splits=0, kv_range=None, partials=None):
    """int8 latent (MLA) paged decode, seqlen_q = 1, one shared KV head (no counterpart in the reference).
    q_nope (B,1,H,512) / q_rope (B,1,H,64) bf16; latent_i8 (blocks,page,512) int8; scales (blocks,page)
    fp32; rope (blocks,page,64) bf16 -> [out (B,1,H,512) bf16, lse (B,H,1) fp32].  With kv_range and
    partials=(o fp32 (B*H,512), lse fp32 (B*H)) only fp32 partial results over that key range are left."""
    from fa_b200_capi import MlaParams
    capi.require_cuda(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens)
    if q_nope.dtype != torch.bfloat16 or q_rope.dtype != torch.bfloat16 or rope.dtype != torch.bfloat16:
        raise RuntimeError("MLA decode takes bf16 queries and rope cache")
    if latent_i8.dtype != torch.int8 or scales.dtype != torch.float32:
        raise RuntimeError("MLA decode takes an int8 latent cache with fp32 per-token scales")
    b, sq, h, dl = q_nope.shape
    if sq != 1 or dl != 512 or q_rope.shape[-1] != 64 or latent_i8.shape[-1] != 512 or rope.shape[-1] != 64:
        raise RuntimeError("MLA decode expects seqlen_q 1, a 512-dim latent and a 64-dim rope part")
    if block_table.dtype != torch.int32 or cache_seqlens.dtype != torch.int32:
        raise RuntimeError("block_table and cache_seqlens must be int32")
    latent_i8, scales, rope = latent_i8.contiguous(), scales.contiguous(), rope.contiguous()
    block_table = block_table.contiguous()
    p = MlaParams()
    p.q_nope, p.q_rope = q_nope.data_ptr(), q_rope.data_ptr()
    p.q_nope_stride_b, p.q_nope_stride_h = q_nope.stride(0), q_nope.stride(2)
    p.q_rope_stride_b, p.q_rope_stride_h = q_rope.stride(0), q_rope.stride(2)
    p.latent, p.scales, p.rope = latent_i8.data_ptr(), scales.data_ptr(), rope.data_ptr()
    p.block_table, p.block_table_stride, p.page_size = block_table.data_ptr(), block_table.stride(0), latent_i8.shape[1]
    p.cache_seqlens = cache_seqlens.data_ptr()
    out = torch.empty((b, 1, h, 512), dtype=torch.bfloat16, device=q_nope.device)
    lse = torch.empty((b, h, 1), dtype=torch.float32, device=q_nope.device)
    p.o, p.o_stride_b, p.o_stride_h, p.lse = out.data_ptr(), out.stride(0), out.stride(2), lse.data_ptr()
    p.b, p.hq, p.scale, p.num_splits = b, h, softmax_scale, num_splits
    if kv_range is not None:
        p.kv_begin, p.kv_end = int(kv_range[0]), int(kv_range[1])
    if partials is not None:
        p.partials_only = 1
        p.o_partial, p.lse_partial = partials[0].data_ptr(), partials[1].data_ptr()
    ws = capi.workspace(lib.fa_mla_workspace_bytes(p), q_nope.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.stream = capi.stream_ptr(q_nope.device)
    with torch.cuda.device(q_nope.device):
        check(lib.fa_mla_decode(p))
    return [out, lse]
