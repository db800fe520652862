"""CUDA-graph capture and replay of the KV-cache call, as the reference does with its device graphs
(tests/test_flash_attn_npu_v3_graph.py:56-123).  The library never synchronises or reads device memory on
the host, so lengths that change between replays are picked up from the device tensors."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("with_metadata", [False, True])
def test_kvcache_decode_graph_replay(with_metadata):
    import flash_attn_npu_3 as fa3
    gen = torch.Generator().manual_seed(17)
    b, h, hkv, d, page, nblk = 4, 16, 4, 128, 64, 40
    kc = torch.randn(b * nblk, page, hkv, d, generator=gen).bfloat16().cuda()
    vc = torch.randn(b * nblk, page, hkv, d, generator=gen).bfloat16().cuda()
    table = torch.randperm(b * nblk, generator=gen).int().reshape(b, nblk).cuda()
    q = torch.randn(b, 1, h, d, generator=gen).bfloat16().cuda()
    kn = torch.randn(b, 1, hkv, d, generator=gen).bfloat16().cuda()
    vn = torch.randn(b, 1, hkv, d, generator=gen).bfloat16().cuda()
    lens = torch.tensor([100, 900, 2000, 5], dtype=torch.int32).cuda()
    meta = None
    if with_metadata:
        meta = fa3.get_scheduler_metadata(b, 1, nblk * page, h, hkv, d, lens, page_size=page, causal=True)

    def call():
        return fa3.flash_attn_with_kvcache(q, kc, vc, kn, vn, cache_seqlens=lens, page_table=table, causal=True,
                                           scheduler_metadata=meta)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()                                   # warm-up outside capture (first-use set-up of the kernels)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = call()
    for step_lens in ([101, 901, 2001, 6], [300, 10, 2500, 77]):
        lens.copy_(torch.tensor(step_lens, dtype=torch.int32))
        q.copy_(torch.randn(b, 1, h, d, generator=gen).bfloat16())
        kn.copy_(torch.randn(b, 1, hkv, d, generator=gen).bfloat16())
        kr, vr = kc.cpu(), vc.cpu()
        ref, _ = orc.kvcache_fwd(q.cpu(), kr, vr, step_lens, d ** -0.5, k_new=kn.cpu(), v_new=vn.cpu(),
                                 block_table=table.cpu(), causal=True)
        graph.replay()
        torch.cuda.synchronize()
        assert (out.cpu().float() - ref.float()).abs().max().item() <= 2 ** -6
        assert torch.equal(kc.cpu().view(torch.int16), kr.view(torch.int16))      # the replay appended in place
