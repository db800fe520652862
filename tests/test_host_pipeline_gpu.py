"""The pinned-host streaming helper gives the same results as one call on device-resident tensors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_heads_per_chunk", [0, 1])
def test_host_pipeline_matches_device_call(kv_heads_per_chunk):
    import fa_b200_host
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(9)
    b, s, h, hk, d = 3, 512, 8, 2, 128
    q = torch.randn(b, s, h, d, generator=g).bfloat16().pin_memory()
    k = torch.randn(b, s, hk, d, generator=g).bfloat16().pin_memory()
    v = torch.randn(b, s, hk, d, generator=g).bfloat16().pin_memory()
    do = torch.randn(b, s, h, d, generator=g).bfloat16().pin_memory()
    out, dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (q, q, k, v))
    pipe = fa_b200_host.HostPipeline("cuda:0", kv_heads_per_chunk)
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


def test_first_call_of_a_fresh_thread_whose_allocations_come_from_the_cache():
    """A worker thread (an autograd worker, a serving thread) whose first CUDA-related action is the attention call:
    its output allocations are served from the framework's cache, so the library itself has to make the device's
    context current before it encodes tensor maps."""
    import threading
    import flash_attn_npu as fa
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(1, 512, 4, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(1, 512, 4, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(1, 512, 4, 128, device="cuda", generator=g).bfloat16()
    ref = fa.flash_attn_func(q, k, v, causal=True)       # also leaves blocks of the right sizes in the cache
    torch.cuda.synchronize()
    keep = ref.clone()
    del ref
    res = {}

    def work():
        try:
            qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
            o = fa.flash_attn_func(qd, kd, vd, causal=True)
            res["grads"] = torch.autograd.grad(o, (qd, kd, vd), torch.ones_like(o))
            res["out"] = o.detach()
        except Exception as exc:                          # surfaced below, in the test's thread
            res["error"] = exc

    for _ in range(3):                                    # three fresh threads
        res.clear()
        t = threading.Thread(target=work)
        t.start()
        t.join()
        torch.cuda.synchronize()
        assert "error" not in res, res.get("error")
        assert torch.equal(res["out"], keep)
        assert all(torch.isfinite(x.float()).all() for x in res["grads"])
