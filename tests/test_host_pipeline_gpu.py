"""The pinned-host streaming helper gives the same results as one call on device-resident tensors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_device_call():
    import fa_b200_host
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(9)
    b, s, h, hk, d = 3, 512, 8, 2, 128
    q = torch.randn(b, s, h, d, generator=g).bfloat16().pin_memory()
    k = torch.randn(b, s, hk, d, generator=g).bfloat16().pin_memory()
    v = torch.randn(b, s, hk, d, generator=g).bfloat16().pin_memory()
    do = torch.randn(b, s, h, d, generator=g).bfloat16().pin_memory()
    out, dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (q, q, k, v))
    pipe = fa_b200_host.HostPipeline("cuda:0")
    pipe.fwd_bwd(q, k, v, do, out, dq, dk, dv, causal=True)
    torch.cuda.synchronize()
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = fa.flash_attn_func(qd, kd, vd, causal=True)
    gq, gk, gv = torch.autograd.grad(o, (qd, kd, vd), do.cuda())
    assert torch.equal(out, o.detach().cpu())
    assert torch.equal(dq, gq.cpu()) and torch.equal(dk, gk.cpu()) and torch.equal(dv, gv.cpu())


def test_host_pipeline_rejects_pageable_memory():
    import fa_b200_host
    t = torch.zeros(1, 128, 1, 64, dtype=torch.bfloat16)
    pipe = fa_b200_host.HostPipeline("cuda:0")
    with pytest.raises(ValueError):
        pipe.fwd_bwd(t, t, t, t, t, t, t, t)
