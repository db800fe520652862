"""Attention for operands that live in pinned HOST memory: the batch is streamed through the GPU one entry at a
time on three CUDA streams (host-to-device copies, the flash_attn_func forward + backward, device-to-host copies),
so that the two PCIe directions and the kernels overlap.  Each chunk goes through the public `flash_attn_func`;
nothing here touches the kernels.  The reference has no counterpart (its tensors are created on the device)."""
import torch

import flash_attn_npu as _fa


class HostPipeline:
    """Reusable streams for `fwd_bwd`; one instance per device."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def fwd_bwd(self, q, k, v, dout, out, dq, dk, dv, causal=False, softmax_scale=None, window_size=(-1, -1)):
        """q, k, v, dout: pinned host tensors (batch, seqlen, heads, headdim); out, dq, dk, dv: pinned host tensors
        that receive the results.  Returns after queueing everything; the caller's current stream waits for the
        last copy, so an event recorded on it afterwards marks the end of the whole step."""
        for t in (q, k, v, dout, out, dq, dk, dv):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("host pipeline operands must be pinned host tensors")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for i in range(q.shape[0]):
            with torch.cuda.stream(self.s_in):
                dev = [t[i:i + 1].to(self.device, non_blocking=True) for t in (q, k, v, dout)]
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                for t in dev:
                    t.record_stream(self.s_run)
                qd, kd, vd, dod = dev
                qd.requires_grad_(True)
                kd.requires_grad_(True)
                vd.requires_grad_(True)
                o = _fa.flash_attn_func(qd, kd, vd, causal=causal, softmax_scale=softmax_scale, window_size=window_size)
                grads = torch.autograd.grad(o, (qd, kd, vd), dod)
                done = torch.cuda.Event()
                done.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for src, dst in zip((o.detach(),) + tuple(grads), (out, dq, dk, dv)):
                    src.record_stream(self.s_out)
                    dst[i:i + 1].copy_(src, non_blocking=True)
        cur.wait_stream(self.s_out)
