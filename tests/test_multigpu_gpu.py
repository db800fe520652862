"""Key-range sharded decode over 2 GPUs against the single-GPU result: with an NCCL all-gather of the (O, LSE)
partials followed by a combine, and with the one kernel that exchanges them over peer memory and combines.
Skipped when fewer than two GPUs are visible."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import fa_b200_sharding as sh
        import flash_attn_npu as fa
        import flash_attn_npu_3 as fa3
        from oracle import attention_oracle as orc
        dev = torch.device("cuda", rank)
        gen = torch.Generator().manual_seed(5)                # identical data on every rank
        b, h, hkv, d, page = 3, 16, 4, 128, 64
        lens = [1000, 130, 4000]
        nblk = [(l + page - 1) // page for l in lens]
        pool = sum(nblk)
        perm = torch.randperm(pool, generator=gen).int()
        table = torch.zeros(b, max(nblk), dtype=torch.int32)
        off = 0
        for i, n in enumerate(nblk):
            table[i, :n] = perm[off:off + n]
            off += n
        kc = torch.randn(pool, page, hkv, d, generator=gen).bfloat16().to(dev)
        vc = torch.randn(pool, page, hkv, d, generator=gen).bfloat16().to(dev)
        q = torch.randn(b, 1, h, d, generator=gen).bfloat16().to(dev)
        lens_t = torch.tensor(lens, dtype=torch.int32, device=dev)
        full, full_lse = fa.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens_t, block_table=table.to(dev),
                                                    return_softmax_lse=True)
        out, lse = sh.sharded_kvcache_decode(q, kc, vc, lens_t, table.to(dev), d ** -0.5, max(lens), page)
        assert (out.float() - full.float()).abs().max().item() <= 2 ** -7
        assert (lse - full_lse).abs().max().item() < 1e-4
        # int8 latent decode, sequences sharded over the key range
        lat, sc = orc.quantize_latent(torch.randn(pool, page, 512, generator=gen))
        rope = torch.randn(pool, page, 64, generator=gen).bfloat16()
        qn = torch.randn(b, 1, 128, 512, generator=gen).bfloat16().to(dev)
        qr = torch.randn(b, 1, 128, 64, generator=gen).bfloat16().to(dev)
        args = (qn, qr, lat.to(dev), sc.to(dev), rope.to(dev))
        mfull, mlse = fa3.flash_attn_mla_with_kvcache(*args, lens_t, table.to(dev), return_softmax_lse=True)
        mout, mlse2 = sh.sharded_mla_decode(*args, table.to(dev), lens_t, 576 ** -0.5, max(lens), page)
        assert (mout.float() - mfull.float()).abs().max().item() <= 2 ** -7
        assert (mlse2 - mlse).abs().max().item() < 1e-4
        # the same two calls with the partials exchanged and combined by one kernel over peer memory; several
        # calls so that both slots of the exchange buffers are reused
        ex = sh.PeerExchange(b * h, d, dev)
        mex = sh.PeerExchange(b * 128, 512, dev)
        for it in range(5):
            qi = (q.float() * (1.0 + 0.25 * it)).bfloat16()
            ref_o, ref_l = sh.sharded_kvcache_decode(qi, kc, vc, lens_t, table.to(dev), d ** -0.5, max(lens), page)
            o2, l2 = sh.sharded_kvcache_decode(qi, kc, vc, lens_t, table.to(dev), d ** -0.5, max(lens), page,
                                               exchange=ex)
            ex.check()
            assert torch.equal(o2, ref_o), (o2.float() - ref_o.float()).abs().max().item()
            assert (l2 - ref_l).abs().max().item() < 1e-6
            m2, ml2 = sh.sharded_mla_decode(*args, table.to(dev), lens_t, 576 ** -0.5, max(lens), page, exchange=mex)
            mex.check()
            assert (m2.float() - mfull.float()).abs().max().item() <= 2 ** -7
            assert (ml2 - mlse).abs().max().item() < 1e-4
        import fa_b200_capi as capi
        assert capi.last_kernel() == "peer_combine"
        ex.close()
        mex.close()
        torch.cuda.synchronize()
        dist.barrier()
        torch.save({"ok": True}, os.path.join(tmp, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_kv_sharded_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29700 + (os.getpid() % 200)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all(os.path.exists(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(2))
