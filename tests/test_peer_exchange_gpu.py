"""The exchange-and-combine kernel of the KV-sharded decode on one GPU: the other ranks are played by the test, which
writes their partials and flags before the launch, so no launch ever waits for another one.  The two-GPU run of the
same kernel is in test_multigpu_gpu.py."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fill(ex, epoch, gen, dead_rank=None):
    """Random partials for every rank of call `epoch` (rank 0's through the tensors a decode would fill)."""
    os_, ls_ = [], []
    for r in range(ex.world):
        o, l, _ = ex.views(r, epoch)
        o.copy_(torch.randn(ex.rows, ex.dv, generator=gen).to(o.device))
        lse = torch.randn(ex.rows, generator=gen) * 3
        lse[::7] = -math.inf if r == 1 else lse[::7]                  # rows for which rank 1 saw no key
        if r == dead_rank:
            lse[:] = -math.inf
            o.fill_(float("nan"))                                     # never read: its weight is 0
        l.copy_(lse.to(l.device))
        os_.append(o.clone())
        ls_.append(l.clone())
    return torch.stack(os_), torch.stack(ls_)


def _signal_as_peers(ex, epoch):
    _, _, flags = ex.views(0, epoch)
    flags.view(torch.int32)[1:ex.world] = epoch


@pytest.mark.parametrize("world,rows,dv,dtype", [(2, 48, 128, torch.bfloat16), (3, 37, 64, torch.float16),
                                                 (8, 2048, 512, torch.bfloat16), (16, 5, 256, torch.float32)])
def test_peer_combine_equals_combine_of_gathered_partials(world, rows, dv, dtype):
    import fa_b200_sharding as sh
    import fa_b200_capi as capi
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(world * 1000 + rows)
    ex = sh.PeerExchange(rows, dv, dev, local_world=world)
    try:
        for call in range(4):                                         # both slots, twice
            po, pl = ex.partials()
            assert po.shape == (rows, dv) and pl.shape == (rows,)
            go, gl = _fill(ex, ex.epoch, gen, dead_rank=2 if world > 2 and call == 1 else None)
            _signal_as_peers(ex, ex.epoch)
            out, lse = ex.combine(dtype)
            assert capi.last_kernel() == "peer_combine"
            ex.check()
            ref, ref_lse = ext3.fwd_combine(go, gl, None, dtype)
            assert torch.equal(lse, ref_lse)
            assert (out.float() - ref.float()).abs().max().item() <= (1e-6 if dtype == torch.float32 else 2 ** -8)
            assert not torch.isnan(out.float()).any()
    finally:
        ex.close()


def test_peer_combine_gives_up_after_its_time_limit_and_the_context_stays_usable():
    """A flag that nothing sets: the wait runs out, the kernel reports the missing rank and writes nothing."""
    import fa_b200_sharding as sh
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    ex = sh.PeerExchange(16, 128, dev, local_world=3, timeout_ms=20)
    try:
        ex.partials()
        _fill(ex, ex.epoch, gen)
        _, _, flags = ex.views(0, ex.epoch)
        flags.view(torch.int32)[1] = ex.epoch                         # rank 1 signalled, rank 2 never does
        ex.combine(torch.bfloat16)
        with pytest.raises(RuntimeError, match="rank 2"):
            ex.check()
        # the next call (other slot) with all signals present works
        ex.partials()
        go, gl = _fill(ex, ex.epoch, gen)
        _signal_as_peers(ex, ex.epoch)
        out, lse = ex.combine(torch.float32)
        ex.check()
        w = torch.softmax(gl, dim=0)
        ref = (torch.nan_to_num(w).unsqueeze(-1) * go).sum(0)
        assert (out - ref).abs().max().item() < 1e-5
    finally:
        ex.close()


def test_peer_combine_rejects_bad_arguments():
    import fa_b200_sharding as sh
    with pytest.raises(RuntimeError):
        sh.PeerExchange(4, 30, torch.device("cuda", 0), local_world=2)      # dv not a multiple of 4
    with pytest.raises(RuntimeError):
        sh.PeerExchange(4, 32, torch.device("cuda", 0), local_world=17)     # more ranks than the kernel takes
