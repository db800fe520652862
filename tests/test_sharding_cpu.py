"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world_size 2): item balancing, key-range
sharding, and the all-gather of packed (O, LSE) partials followed by the combine (checked with the oracle's
combine on gathered buffers, since the CUDA combine needs a GPU)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fa_b200_sharding as sh
from oracle import attention_oracle as orc


def test_balance_items_is_deterministic_and_balanced():
    gen = torch.Generator().manual_seed(3)
    lens = torch.randint(256, 8193, (16,), generator=gen).tolist()
    items, costs = sh.varlen_items(lens, kv_heads=8)
    assert len(items) == 128
    for world in (1, 2, 4, 8):
        bins = sh.balance_items(costs, world)
        assert sorted(i for b in bins for i in b) == list(range(128))
        loads = [sum(costs[i] for i in b) for b in bins]
        assert max(loads) <= sum(loads) / world + max(costs) + 1e-6      # greedy bound
        assert bins == sh.balance_items(costs, world)


def test_kv_shard_ranges_cover_and_align():
    for max_len, world, align in ((131072, 8, 256), (5000, 4, 64), (100, 8, 256)):
        ranges = [sh.kv_shard_range(max_len, r, world, align) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] >= max_len
        for (a, b), (c, d) in zip(ranges, ranges[1:]):
            assert b == c and a % align == 0 and b % align == 0


def _worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                                   # same data on every rank
        h, d, L = 4, 64, 700
        q = torch.randn(1, 1, h, d).bfloat16()
        k = torch.randn(1, L, 1, d).bfloat16()
        v = torch.randn(1, L, 1, d).bfloat16()
        lo, hi = sh.kv_shard_range(L, rank, world, 64)
        hi = min(hi, L)
        if hi > lo:
            o, l = orc.attention_fwd(q, k[:, lo:hi], v[:, lo:hi], 0.125, data_type=torch.float32)
            po, pl = o.reshape(h, d), l.reshape(h)
        else:
            po, pl = torch.zeros(h, d), torch.full((h,), float("-inf"))
        go, gl = sh.all_gather_partials(po, pl)
        assert go.shape == (world, h, d) and gl.shape == (world, h)
        out, lse = orc.combine_partials(go, gl, torch.float32)
        full, full_lse = orc.attention_fwd(q, k, v, 0.125, data_type=torch.float32)
        assert (out - full.reshape(h, d)).abs().max().item() < 1e-5
        assert (lse - full_lse.reshape(h)).abs().max().item() < 1e-5
        # a rank that never joins is detected by the others through a short timeout, not by hanging:
        # here every rank joined, so a barrier completes
        dist.barrier()
        torch.save({"ok": True}, os.path.join(tmp, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_all_gather_of_partials_and_combine_over_two_gloo_ranks(tmp_path):
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all(os.path.exists(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(2))


def test_partial_buffer_views_share_one_allocation():
    buf = sh.PartialBuffer(5, 8, "cpu", 1)
    buf.o.copy_(torch.arange(40, dtype=torch.float32).view(5, 8))
    buf.lse.copy_(torch.arange(5, dtype=torch.float32) + 100)
    assert buf.o.data_ptr() == buf.send.data_ptr() and buf.lse.data_ptr() == buf.send.data_ptr() + 5 * 8 * 4
    go, gl = buf.gather()
    assert go.shape == (1, 5, 8) and gl.shape == (1, 5)
    assert torch.equal(go[0], buf.o) and torch.equal(gl[0], buf.lse)
    assert go[0].is_contiguous() and gl[0].is_contiguous() and buf.floats % 64 == 0


def test_group_items_makes_rectangular_calls():
    items = sh.dense_items(4, 32)
    assert len(items) == 128
    for world in (1, 2, 4, 8):
        bins = sh.balance_items([1.0] * len(items), world)
        assert sorted(i for b in bins for i in b) == list(range(128))
        for mine in bins:
            assert len(mine) == 128 // world
            groups = sh.group_items([items[i] for i in mine])
            # equal costs deal the heads round-robin: every batch entry gets the same heads -> one call per rank
            assert len(groups) == 1 and len(groups[0][0]) == 4 and len(groups[0][1]) == 32 // world
    groups = sh.group_items([(0, 1), (0, 2), (1, 1), (2, 2), (2, 1)])
    assert groups == [((0, 2), (1, 2)), ((1,), (1,))]


def test_decode_shard_plan_cuts_long_sequences_by_their_own_length():
    gen = torch.Generator().manual_seed(5)
    lens = torch.randint(4096, 131073, (64,), generator=gen).tolist()
    page, thr = 256, 32768
    one = sh.decode_shard_plan(lens, 1, page, thr)
    assert one["long"] == [] and one["short"] == [list(range(64))]
    for world in (2, 4, 8):
        plan = sh.decode_shard_plan(lens, world, page, thr)
        longs = plan["long"]
        assert all(lens[i] > thr for i in longs)
        owned = sorted(i for r in range(world) for i in plan["short"][r])
        assert owned == [i for i in range(64) if lens[i] <= thr]
        for k, i in enumerate(longs):
            n = (lens[i] + page - 1) // page
            ranges = [plan["pages"][r][k] for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert sum(plan["tokens"][r][k] for r in range(world)) == lens[i]
            assert max(b - a for a, b in ranges) - min(b - a for a, b in ranges) <= 1
        loads = [sum(plan["tokens"][r]) + sum(lens[i] for i in plan["short"][r]) for r in range(world)]
        assert max(loads) - min(loads) <= thr
