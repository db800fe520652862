"""The extension module of the v2 API: `fwd`, `varlen_fwd`, `fwd_kvcache`, `bwd`,
`varlen_bwd` with the positional signatures and return lists of the reference's pybind
module (csrc/ascend910/flash_attn_npu/flash_api.cpp:1330-1338), implemented as calls
into libfa_b200.so.  torch allocates outputs and workspaces; the library computes.

Argument errors are raised as RuntimeError like the reference's TORCH_CHECKs
(flash_api.cpp:386-420, :658-682, :884-934).  Unlike the reference, alibi slopes,
rotary embedding, in-place append of new k/v, paged varlen and forced split counts are
implemented rather than rejected; dropout, return_softmax, leftpad_k stay rejected.
"""
from typing import List, Optional

import torch
import torch.nn.functional as F

import fa_b200_capi as capi
from fa_b200_capi import FwdParams, BwdParams, tensor4, ptr, check, lib


def _dtype_code(t):
    if t.dtype not in capi.DTYPES:
        raise RuntimeError("FlashAttention only supports FP16 and BF16 data types")
    return capi.DTYPES[t.dtype]


def _common_checks(q, k, v, softcap, what="key"):
    capi.require_cuda(q, k, v)
    if k.dtype != q.dtype:
        raise RuntimeError(f"query and {what} must have the same dtype")
    if v.dtype != q.dtype:
        raise RuntimeError("query and value must have the same dtype")
    for t in (q, k, v):
        if t.stride(-1) != 1:
            raise RuntimeError("Input tensor must have contiguous last dimension")
    if softcap < 0.0:
        raise RuntimeError("softcap must be non-negative (0.0 disables softcap)")


def _alibi(p, alibi_slopes, batch, nheads):
    if alibi_slopes is None:
        return None
    a = alibi_slopes.to(torch.float32).contiguous()
    if a.shape not in ((nheads,), (batch, nheads)):
        raise RuntimeError("alibi_slopes must have shape (nheads,) or (batch_size, nheads)")
    p.alibi_slopes = a.data_ptr()
    p.alibi_stride_b = 0 if a.dim() == 1 else a.stride(0)
    return a


def _pad8(t):
    d = t.size(-1)
    return t if d % 8 == 0 else F.pad(t, [0, 8 - d % 8])


def fwd(q, k, v, out_, alibi_slopes_, p_dropout, softmax_scale, is_causal, window_size_left,
        window_size_right, softcap, return_softmax, gen_) -> List[torch.Tensor]:
    """mha_fwd (flash_api.cpp:639-846). q (B,Sq,H,D), k/v (B,Sk,Hkv,D) ->
    [out, softmax_lse (B,H,Sq) fp32, p (empty), rng_state (int64[2])]."""
    _common_checks(q, k, v, softcap)
    if p_dropout != 0.0:
        raise RuntimeError("FlashAttention on B200 does not support dropout.")
    if return_softmax:
        raise RuntimeError("FlashAttention on B200 does not support return_softmax.")
    batch, sq, hq, d_og = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    if batch <= 0:
        raise RuntimeError("batch size must be positive")
    if d_og > 256:
        raise RuntimeError("FlashAttention only supports head dimension at most 256")
    if hq % hkv != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    q, k, v = _pad8(q), _pad8(k), _pad8(v)
    d = q.size(-1)
    out = torch.empty_like(q) if (out_ is None or d != d_og) else out_
    lse = torch.empty((batch, hq, sq), dtype=torch.float32, device=q.device)
    p = FwdParams()
    p.q, p.k, p.v, p.o = tensor4(q), tensor4(k), tensor4(v), tensor4(out)
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = lse.stride(0), lse.stride(1), lse.stride(2)
    p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv = batch, sq, sk, hq, hkv, d, v.size(-1)
    p.scale, p.softcap = softmax_scale, softcap
    p.causal, p.window_left, p.window_right = int(is_causal), window_size_left, window_size_right
    p.dtype = _dtype_code(q)
    p.num_splits = 1
    keep = _alibi(p, alibi_slopes_, batch, hq)
    p.stream = capi.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        check(lib.fa_fwd(p))
    del keep
    if d != d_og:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
            out = out_
    empty_p = torch.empty((0,), dtype=q.dtype, device=q.device)
    rng_state = torch.zeros((2,), dtype=torch.int64, device=q.device)
    return [out, lse, empty_p, rng_state]


def varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k_, leftpad_k_, block_table_,
               alibi_slopes_, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors,
               is_causal, window_size_left, window_size_right, softcap, return_softmax, gen_):
    """mha_varlen_fwd (flash_api.cpp:848-1089). q (Tq,H,D), k/v (Tk,Hkv,D) or a paged cache
    (blocks,page,Hkv,D) with block_table -> [out, softmax_lse (H,Tq), p, rng_state]."""
    _common_checks(q, k, v, softcap)
    if p_dropout != 0.0:
        raise RuntimeError("FlashAttention on B200 does not support dropout.")
    if return_softmax:
        raise RuntimeError("FlashAttention on B200 does not support return_softmax.")
    if leftpad_k_ is not None:
        raise RuntimeError("FlashAttention on B200 does not support leftpad_k.")
    if cu_seqlens_q.dtype != torch.int32 or (cu_seqlens_k is not None and cu_seqlens_k.dtype != torch.int32):
        raise RuntimeError("cu_seqlens must have dtype int32")
    total_q, hq, d_og = q.shape
    paged = block_table_ is not None
    hkv = k.shape[-2]
    if d_og > 256:
        raise RuntimeError("FlashAttention only supports head dimension at most 256")
    if hq % hkv != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    q, k, v = _pad8(q), _pad8(k), _pad8(v)
    d = q.size(-1)
    batch = cu_seqlens_q.numel() - 1
    out = torch.empty_like(q) if (out_ is None or d != d_og) else out_
    if zero_tensors:
        out.zero_()
    lse = torch.full((hq, total_q), float("inf"), dtype=torch.float32, device=q.device)
    p = FwdParams()
    p.q, p.o = tensor4(q, packed=True), tensor4(out, packed=True)
    if paged:
        p.k, p.v = tensor4(k), tensor4(v)
        if block_table_.dtype != torch.int32 or block_table_.stride(-1) != 1:
            raise RuntimeError("block_table must be int32 with contiguous last dimension")
        p.block_table, p.block_table_stride, p.page_size = block_table_.data_ptr(), block_table_.stride(0), k.shape[1]
        p.kv_entries = min(k.shape[0], v.shape[0])
        p.seqused_k = ptr(seqused_k_)
        p.num_splits = 0
    else:
        p.k, p.v = tensor4(k, packed=True), tensor4(v, packed=True)
        p.seqused_k = None
        p.num_splits = 1
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = 0, lse.stride(0), lse.stride(1)
    p.cu_seqlens_q, p.cu_seqlens_k = cu_seqlens_q.data_ptr(), ptr(cu_seqlens_k)
    p.b, p.sq, p.sk, p.total_q = batch, max_seqlen_q, max_seqlen_k, total_q
    p.total_k = 0 if paged else k.shape[0]
    p.hq, p.hkv, p.d, p.dv = hq, hkv, d, v.size(-1)
    p.scale, p.softcap = softmax_scale, softcap
    p.causal, p.window_left, p.window_right = int(is_causal), window_size_left, window_size_right
    p.dtype = _dtype_code(q)
    keep = _alibi(p, alibi_slopes_, batch, hq)
    ws = capi.workspace(lib.fa_fwd_workspace_bytes(p), q.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.stream = capi.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        check(lib.fa_varlen_fwd(p))
    del keep
    if d != d_og:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
            out = out_
    empty_p = torch.empty((0,), dtype=q.dtype, device=q.device)
    rng_state = torch.zeros((2,), dtype=torch.int64, device=q.device)
    return [out, lse, empty_p, rng_state]


def kvcache_forward(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_,
                    block_table_, alibi_slopes_, out_, softmax_scale, is_causal, window_size_left,
                    window_size_right, softcap, is_rotary_interleaved, num_splits,
                    cu_seqlens_q=None, max_seqlen_q=None, kv_range=None, partials=None, sched_meta=None):
    """Shared by the v2 and v3 kvcache entry points.  q (B,Sq,H,D) or packed (Tq,H,D) with
    cu_seqlens_q.  kv_range=(begin,end) and partials=(o fp32, lse fp32) select the
    cross-device KV-sharded mode, where fp32 partial results are left for a later combine.
    sched_meta: the device blob of get_scheduler_metadata (uint8 or int32 view); the split-KV decode kernels take
    every sequence's keys per split from it (a blob built for another batch, split count or for other lengths is
    ignored on the device, so a stale blob costs balance, never correctness)."""
    _common_checks(q, kcache, vcache, softcap, what="key_cache")
    packed_q = cu_seqlens_q is not None
    if packed_q:
        total_q, hq, d_og = q.shape
        batch = cu_seqlens_q.numel() - 1
        sq = int(max_seqlen_q)
    else:
        batch, sq, hq, d_og = q.shape
        total_q = 0
    paged = block_table_ is not None
    hkv = kcache.shape[2]
    if batch <= 0:
        raise RuntimeError("batch size must be positive")
    if d_og > 256:
        raise RuntimeError("FlashAttention only supports head dimension at most 256")
    if hq % hkv != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    if seqlens_k_ is not None and seqlens_k_.dtype != torch.int32:
        raise RuntimeError("seqlens_k must have dtype int32")
    if paged and (block_table_.dtype != torch.int32 or block_table_.stride(-1) != 1):
        raise RuntimeError("block_table must have dtype int32 and contiguous last dimension")
    if d_og % 8 != 0:
        if k_ is not None:
            raise RuntimeError("appending k/v needs a head dimension that is a multiple of 8")
        q, kcache, vcache = _pad8(q), _pad8(kcache), _pad8(vcache)
    d = q.size(-1)
    out = torch.empty_like(q) if (out_ is None or d != d_og) else out_
    p = FwdParams()
    if packed_q:
        lse = torch.full((hq, total_q), float("inf"), dtype=torch.float32, device=q.device)
        p.q, p.o = tensor4(q, packed=True), tensor4(out, packed=True)
        p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = 0, lse.stride(0), lse.stride(1)
        p.cu_seqlens_q, p.total_q = cu_seqlens_q.data_ptr(), total_q
    else:
        lse = torch.empty((batch, hq, sq), dtype=torch.float32, device=q.device)
        p.q, p.o = tensor4(q), tensor4(out)
        p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = lse.stride(0), lse.stride(1), lse.stride(2)
    p.lse = lse.data_ptr()
    p.k, p.v = tensor4(kcache), tensor4(vcache)
    p.kv_entries = min(kcache.shape[0], vcache.shape[0])
    s_new = 0
    if k_ is not None:
        if v_ is None:
            raise RuntimeError("k and v must be passed together")
        if seqlens_k_ is None:
            raise RuntimeError("seqlens_k must be passed when appending k and v")
        if k_.dtype != q.dtype or v_.dtype != q.dtype:
            raise RuntimeError("new k/v must have the query's dtype")
        p.k_new, p.v_new = tensor4(k_), tensor4(v_)
        s_new = k_.shape[1]
    p.s_new = s_new
    if paged:
        p.block_table, p.block_table_stride, p.page_size = block_table_.data_ptr(), block_table_.stride(0), kcache.shape[1]
        sk = block_table_.shape[1] * kcache.shape[1]
    else:
        sk = kcache.shape[1]
    p.seqused_k = ptr(seqlens_k_)
    p.cache_batch_idx = ptr(cache_batch_idx_)
    if rotary_cos_ is not None:
        if k_ is None:
            raise RuntimeError("rotary embedding is only applied when k and v are passed in")
        rc = rotary_cos_.to(q.dtype).contiguous()
        rs = rotary_sin_.to(q.dtype).contiguous()
        p.rotary_cos, p.rotary_sin = rc.data_ptr(), rs.data_ptr()
        p.rotary_dim, p.seqlen_ro = rc.shape[1] * 2, rc.shape[0]
        p.rotary_interleaved = int(is_rotary_interleaved)
    p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv = batch, sq, sk, hq, hkv, d, vcache.size(-1)
    p.scale, p.softcap = softmax_scale, softcap
    p.causal, p.window_left, p.window_right = int(is_causal), window_size_left, window_size_right
    p.dtype = _dtype_code(q)
    p.num_splits = num_splits
    if kv_range is not None:
        p.kv_begin, p.kv_end = int(kv_range[0]), int(kv_range[1])
    if partials is not None:
        p.partials_only = 1
        p.o_partial, p.lse_partial = partials[0].data_ptr(), partials[1].data_ptr()
    if sched_meta is not None:
        capi.require_cuda(sched_meta)
        if sched_meta.dtype not in (torch.uint8, torch.int32) or not sched_meta.is_contiguous():
            raise RuntimeError("scheduler_metadata must be the contiguous uint8 / int32 tensor get_scheduler_metadata returned")
        if sched_meta.numel() * sched_meta.element_size() < 4 * lib.fa_scheduler_metadata_ints(batch) or sched_meta.data_ptr() % 4:
            raise RuntimeError("scheduler_metadata is too small for this batch size")
        p.sched_meta = sched_meta.data_ptr()
    keep = _alibi(p, alibi_slopes_, batch, hq)
    ws = capi.workspace(lib.fa_fwd_workspace_bytes(p), q.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.stream = capi.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        check(lib.fa_fwd_kvcache(p))
    del keep
    if d != d_og:
        out = out[..., :d_og]
        if out_ is not None:
            out_.copy_(out)
            out = out_
    return out, lse


def fwd_kvcache(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_, cache_batch_idx_,
                leftpad_k_, block_table_, alibi_slopes_, out_, softmax_scale, is_causal,
                window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits):
    """mha_fwd_kvcache (flash_api.cpp:356-637) -> [out, softmax_lse (B,H,Sq)]."""
    if leftpad_k_ is not None:
        raise RuntimeError("FlashAttention on B200 does not support leftpad_k")
    if num_splits < 0:
        raise RuntimeError("num_splits must be >= 0")
    out, lse = kvcache_forward(q, kcache, vcache, k_, v_, seqlens_k_, rotary_cos_, rotary_sin_,
                               cache_batch_idx_, block_table_, alibi_slopes_, out_, softmax_scale, is_causal,
                               window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits)
    return [out, lse]


def _bwd_common(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, alibi_slopes_, p_dropout, softmax_scale,
                is_causal, wl, wr, softcap, deterministic, cu_q=None, cu_k=None, max_sq=0, max_sk=0):
    capi.require_cuda(dout, q, k, v, out, softmax_lse)
    if softcap < 0.0:
        raise RuntimeError("softcap must be non-negative (0.0 disables softcap)")
    if p_dropout != 0.0:
        raise RuntimeError("FlashAttention on B200 does not support dropout.")
    packed = cu_q is not None
    d_og = q.size(-1)
    if d_og % 8 != 0:
        raise RuntimeError("backward needs a head dimension that is a multiple of 8 (the Python API pads it)")
    dq = torch.empty_like(q) if dq_ is None else dq_
    dk = torch.empty_like(k) if dk_ is None else dk_
    dv = torch.empty_like(v) if dv_ is None else dv_
    p = BwdParams()
    names = ("dout", "q", "k", "v", "o", "dq", "dk", "dv")
    for name, t in zip(names, (dout, q, k, v, out, dq, dk, dv)):
        if t.stride(-1) != 1:
            raise RuntimeError("Input tensor must have contiguous last dimension")
        setattr(p, name, tensor4(t, packed=packed))
    if packed:
        total_q, hq, _ = q.shape
        total_k, hkv, _ = k.shape
        if softmax_lse.dim() != 2:
            raise RuntimeError("mha_varlen_bwd: softmax_lse for TND must be a 2D tensor.")
        if softmax_lse.shape != (hq, total_q):
            raise RuntimeError("mha_varlen_bwd: softmax_lse must have shape (nheads, total_q)")
        batch = cu_q.numel() - 1
        p.cu_seqlens_q, p.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
        p.b, p.sq, p.sk, p.total_q, p.total_k = batch, max_sq, max_sk, total_q, total_k
        p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = 0, softmax_lse.stride(0), softmax_lse.stride(1)
        softmax_d = torch.empty((hq, total_q + 128 * batch), dtype=torch.float32, device=q.device)
    else:
        batch, sq, hq, _ = q.shape
        sk, hkv = k.shape[1], k.shape[2]
        if softmax_lse.shape != (batch, hq, sq):
            raise RuntimeError("softmax_lse must have shape (batch, nheads, seqlen_q)")
        p.b, p.sq, p.sk = batch, sq, sk
        p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = softmax_lse.stride(0), softmax_lse.stride(1), softmax_lse.stride(2)
        softmax_d = torch.empty((batch, hq, (sq + 127) // 128 * 128), dtype=torch.float32, device=q.device)
    if softmax_lse.dtype != torch.float32:
        raise RuntimeError("softmax_lse must be fp32")
    if hq % hkv != 0:
        raise RuntimeError("Number of heads in key/value must divide number of heads in query")
    p.lse = softmax_lse.data_ptr()
    p.hq, p.hkv, p.d, p.dv_dim = hq, hkv, q.size(-1), v.size(-1)
    p.scale, p.softcap = softmax_scale, softcap
    p.causal, p.window_left, p.window_right = int(is_causal), wl, wr
    p.dtype = _dtype_code(q)
    p.deterministic = int(deterministic)
    keep = _alibi(p, alibi_slopes_, batch, hq)
    ws = capi.workspace(lib.fa_bwd_workspace_bytes(p), q.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    p.stream = capi.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        check(lib.fa_varlen_bwd(p) if packed else lib.fa_bwd(p))
    return [dq, dk, dv, softmax_d]


def bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, alibi_slopes_, p_dropout, softmax_scale, is_causal,
        window_size_left, window_size_right, softcap, deterministic, gen_, rng_state):
    """mha_bwd (flash_api.cpp:1279-1328) -> [dq, dk, dv, softmax_d]."""
    return _bwd_common(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, alibi_slopes_, p_dropout, softmax_scale,
                       is_causal, window_size_left, window_size_right, softcap, deterministic)


def varlen_bwd(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, cu_seqlens_q, cu_seqlens_k, alibi_slopes_,
               max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal,
               window_size_left, window_size_right, softcap, deterministic, gen_, rng_state):
    """mha_varlen_bwd (flash_api.cpp:1092-1277) -> [dq, dk, dv, softmax_d]."""
    res = _bwd_common(dout, q, k, v, out, softmax_lse, dq_, dk_, dv_, alibi_slopes_, p_dropout, softmax_scale,
                      is_causal, window_size_left, window_size_right, softcap, deterministic,
                      cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k)
    return res
