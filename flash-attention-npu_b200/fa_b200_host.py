"""Attention for operands that live in pinned HOST memory: the batch is streamed through the GPU in chunks on three
CUDA streams (host-to-device copies, the flash_attn_func forward + backward, device-to-host copies), so that the
two PCIe directions and the kernels overlap.  A chunk is one batch entry with all of its heads, which is one
CONTIGUOUS range of every operand: each tensor of a chunk moves with a single multi-megabyte asynchronous copy
(a chunk of 4096 x 32 x 128 bf16 is 32 MiB a tensor).  A chunk's forward starts when q, k and v have arrived (dout
follows while it runs) and its output leaves while the backward runs, which keeps the pipeline's fill and drain
short.  `kv_heads_per_chunk` > 0 cuts a batch entry further into groups of KV heads (pitched copies of
heads x headdim wide rows): smaller chunks fill the pipeline faster but move through the copy engines as many short
rows, which some hosts handle badly.  Each chunk goes through the public `flash_attn_func`; nothing here touches the
kernels.  The reference has no counterpart (its tensors are created on the device)."""
import torch

import fa_b200_capi as _capi
import flash_attn_npu as _fa


class HostPipeline:
    """Reusable streams for `fwd_bwd` and `copy_only`; one instance per device."""

    def __init__(self, device, kv_heads_per_chunk=0):
        self.device = torch.device(device)
        self.kv_heads_per_chunk = kv_heads_per_chunk
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def _copy(self, dst, src, stream):
        """dst, src: (seqlen, heads, headdim) views of equal shape, last two dimensions dense.  One contiguous
        asynchronous copy when both sides are dense, otherwise a pitched copy of heads x headdim wide rows."""
        s, h, d = src.shape
        width = h * d * src.element_size()
        if dst.is_contiguous() and src.is_contiguous():
            with torch.cuda.stream(stream):
                dst.copy_(src, non_blocking=True)
            return
        _capi.check(_capi.lib.fa_copy_2d_async(dst.data_ptr(), dst.stride(0) * dst.element_size(), src.data_ptr(),
                                               src.stride(0) * src.element_size(), width, s, stream.cuda_stream))

    def _check(self, tensors):
        for t in tensors:
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("host pipeline operands must be pinned host tensors")
            if t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != t.shape[3]:
                raise ValueError("host pipeline operands are (batch, seqlen, heads, headdim) with dense heads")

    def _chunks(self, b, hkv):
        step = self.kv_heads_per_chunk or hkv
        return [(i, g0, min(hkv, g0 + step)) for i in range(b) for g0 in range(0, hkv, step)]

    def fwd_bwd(self, q, k, v, dout, out, dq, dk, dv, causal=False, softmax_scale=None, window_size=(-1, -1),
                run_kernels=True):
        """q, k, v, dout: pinned host tensors (batch, seqlen, heads, headdim); out, dq, dk, dv: pinned host tensors
        that receive the results.  Returns after queueing everything; the caller's current stream waits for the
        last copy, so an event recorded on it afterwards marks the end of the whole step.  `run_kernels=False`
        moves the same bytes through the same streams without launching anything (the copy floor of the box)."""
        self._check((q, k, v, dout, out, dq, dk, dv))
        b, sq, hq, d = q.shape
        sk, hkv = k.shape[1], k.shape[2]
        if hq % hkv:
            raise ValueError("query heads must be a multiple of KV heads")
        group = hq // hkv
        dev_, dt = self.device, q.dtype
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.device(self.device):
            for i, g0, g1 in self._chunks(b, hkv):
                hq0, hq1 = g0 * group, g1 * group
                with torch.cuda.stream(self.s_in):
                    qd = torch.empty(1, sq, hq1 - hq0, d, dtype=dt, device=dev_)
                    kd = torch.empty(1, sk, g1 - g0, k.shape[3], dtype=dt, device=dev_)
                    vd = torch.empty(1, sk, g1 - g0, v.shape[3], dtype=dt, device=dev_)
                    dod = torch.empty(1, sq, hq1 - hq0, dout.shape[3], dtype=dt, device=dev_)
                    self._copy(qd[0], q[i, :, hq0:hq1], self.s_in)
                    self._copy(kd[0], k[i, :, g0:g1], self.s_in)
                    self._copy(vd[0], v[i, :, g0:g1], self.s_in)
                    qkv_ready = torch.cuda.Event()
                    qkv_ready.record(self.s_in)
                    self._copy(dod[0], dout[i, :, hq0:hq1], self.s_in)
                    do_ready = torch.cuda.Event()
                    do_ready.record(self.s_in)
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(qkv_ready)
                    for t in (qd, kd, vd, dod):
                        t.record_stream(self.s_run)
                    if run_kernels:
                        qd.requires_grad_(True)
                        kd.requires_grad_(True)
                        vd.requires_grad_(True)
                        o = _fa.flash_attn_func(qd, kd, vd, causal=causal, softmax_scale=softmax_scale,
                                                window_size=window_size)
                    else:
                        o = qd
                    fwd_done = torch.cuda.Event()
                    fwd_done.record(self.s_run)
                    self.s_run.wait_event(do_ready)
                    grads = torch.autograd.grad(o, (qd, kd, vd), dod) if run_kernels else (dod, kd, vd)
                    bwd_done = torch.cuda.Event()
                    bwd_done.record(self.s_run)
                with torch.cuda.stream(self.s_out):
                    od = o.detach()
                    for t in (od,) + tuple(grads):
                        t.record_stream(self.s_out)
                    self.s_out.wait_event(fwd_done)
                    self._copy(out[i, :, hq0:hq1], od[0], self.s_out)
                    self.s_out.wait_event(bwd_done)
                    self._copy(dq[i, :, hq0:hq1], grads[0][0], self.s_out)
                    self._copy(dk[i, :, g0:g1], grads[1][0], self.s_out)
                    self._copy(dv[i, :, g0:g1], grads[2][0], self.s_out)
        cur.wait_stream(self.s_out)

    def copy_only(self, q, k, v, dout, out, dq, dk, dv):
        """The copies of `fwd_bwd` without the kernels: same bytes, same chunks, same streams and dependencies."""
        self.fwd_bwd(q, k, v, dout, out, dq, dk, dv, run_kernels=False)
