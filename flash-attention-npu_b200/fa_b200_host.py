"""Attention for operands that live in pinned HOST memory: the batch is streamed through the GPU in chunks of one
batch entry x a group of KV heads on three CUDA streams (host-to-device copies, the flash_attn_func forward +
backward, device-to-host copies), so that the two PCIe directions and the kernels overlap.  A chunk's forward starts
when q, k and v have arrived (dout follows while it runs) and its output leaves while the backward runs, which keeps
the pipeline's fill and drain short.  Head groups are moved with pitched copies straight between the pinned tensors
and contiguous device chunks.  Each chunk goes through the public `flash_attn_func`; nothing here touches the
kernels.  The reference has no counterpart (its tensors are created on the device)."""
import torch

import fa_b200_capi as _capi
import flash_attn_npu as _fa


class HostPipeline:
    """Reusable streams for `fwd_bwd`; one instance per device.  `kv_heads_per_chunk` = 0 picks 8 KV heads a chunk
    (a chunk of 4096 x 8 x 128 bf16 is 8 MiB a tensor: long enough for the copy engines, short enough to fill the
    pipeline quickly)."""

    def __init__(self, device, kv_heads_per_chunk=0):
        self.device = torch.device(device)
        self.kv_heads_per_chunk = kv_heads_per_chunk
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def _copy_heads(self, dst, src, stream):
        """dst, src: (seqlen, heads, headdim) views of equal shape, last two dimensions dense."""
        s, h, d = src.shape
        width = h * d * src.element_size()
        _capi.check(_capi.lib.fa_copy_2d_async(dst.data_ptr(), dst.stride(0) * dst.element_size(), src.data_ptr(),
                                               src.stride(0) * src.element_size(), width, s, stream.cuda_stream))

    def fwd_bwd(self, q, k, v, dout, out, dq, dk, dv, causal=False, softmax_scale=None, window_size=(-1, -1)):
        """q, k, v, dout: pinned host tensors (batch, seqlen, heads, headdim); out, dq, dk, dv: pinned host tensors
        that receive the results.  Returns after queueing everything; the caller's current stream waits for the
        last copy, so an event recorded on it afterwards marks the end of the whole step."""
        for t in (q, k, v, dout, out, dq, dk, dv):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("host pipeline operands must be pinned host tensors")
            if t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != t.shape[3]:
                raise ValueError("host pipeline operands are (batch, seqlen, heads, headdim) with dense heads")
        b, sq, hq, d = q.shape
        sk, hkv = k.shape[1], k.shape[2]
        if hq % hkv:
            raise ValueError("query heads must be a multiple of KV heads")
        group = hq // hkv
        step = self.kv_heads_per_chunk or min(hkv, 8)
        dev_, dt = self.device, q.dtype
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.device(self.device):
            for i in range(b):
                for g0 in range(0, hkv, step):
                    g1 = min(hkv, g0 + step)
                    hq0, hq1 = g0 * group, g1 * group
                    with torch.cuda.stream(self.s_in):
                        qd = torch.empty(1, sq, hq1 - hq0, d, dtype=dt, device=dev_)
                        kd = torch.empty(1, sk, g1 - g0, k.shape[3], dtype=dt, device=dev_)
                        vd = torch.empty(1, sk, g1 - g0, v.shape[3], dtype=dt, device=dev_)
                        dod = torch.empty(1, sq, hq1 - hq0, dout.shape[3], dtype=dt, device=dev_)
                        self._copy_heads(qd[0], q[i, :, hq0:hq1], self.s_in)
                        self._copy_heads(kd[0], k[i, :, g0:g1], self.s_in)
                        self._copy_heads(vd[0], v[i, :, g0:g1], self.s_in)
                        qkv_ready = torch.cuda.Event()
                        qkv_ready.record(self.s_in)
                        self._copy_heads(dod[0], dout[i, :, hq0:hq1], self.s_in)
                        do_ready = torch.cuda.Event()
                        do_ready.record(self.s_in)
                    with torch.cuda.stream(self.s_run):
                        self.s_run.wait_event(qkv_ready)
                        for t in (qd, kd, vd, dod):
                            t.record_stream(self.s_run)
                        qd.requires_grad_(True)
                        kd.requires_grad_(True)
                        vd.requires_grad_(True)
                        o = _fa.flash_attn_func(qd, kd, vd, causal=causal, softmax_scale=softmax_scale,
                                                window_size=window_size)
                        fwd_done = torch.cuda.Event()
                        fwd_done.record(self.s_run)
                        self.s_run.wait_event(do_ready)
                        grads = torch.autograd.grad(o, (qd, kd, vd), dod)
                        bwd_done = torch.cuda.Event()
                        bwd_done.record(self.s_run)
                    with torch.cuda.stream(self.s_out):
                        od = o.detach()
                        for t in (od,) + tuple(grads):
                            t.record_stream(self.s_out)
                        self.s_out.wait_event(fwd_done)
                        self._copy_heads(out[i, :, hq0:hq1], od[0], self.s_out)
                        self.s_out.wait_event(bwd_done)
                        self._copy_heads(dq[i, :, hq0:hq1], grads[0][0], self.s_out)
                        self._copy_heads(dk[i, :, g0:g1], grads[1][0], self.s_out)
                        self._copy_heads(dv[i, :, g0:g1], grads[2][0], self.s_out)
        cur.wait_stream(self.s_out)
