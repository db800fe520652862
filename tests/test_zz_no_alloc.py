"""fa_fwd_kvcache_static: the KV-cache forward for callers that cannot allocate scratch memory
(a serving loop with a sealed memory pool, a plugin that must not call the allocator inside a step).
Called straight through the C-ABI and compared with fa_fwd_kvcache on the same inputs, twice in a row:
the built-in pool is shared and keeps the previous call's contents, so the second call must not be
disturbed by the first.  A third call repeats the second and checks the property the entry point exists for: the
device's free memory and the framework's allocation counter are the same before and after it (the first calls may
still make the driver load kernel images, which takes memory once).  Collected last so that a failure here cannot hide
any other test."""
import pytest
import torch

import fa_b200_capi as capi
from fa_b200_capi import FwdParams, tensor4

pytestmark = pytest.mark.gpu


def build_params(q, kc, vc, table, lens, out, lse, num_splits):
    b, sq, hq, d = q.shape
    p = FwdParams()
    p.q, p.k, p.v, p.o = tensor4(q), tensor4(kc), tensor4(vc), tensor4(out)
    p.kv_entries = kc.shape[0]
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h, p.lse_stride_s = lse.stride(0), lse.stride(1), lse.stride(2)
    p.block_table, p.block_table_stride, p.page_size = table.data_ptr(), table.stride(0), kc.shape[1]
    p.seqused_k = lens.data_ptr()
    p.b, p.sq, p.sk, p.hq, p.hkv, p.d, p.dv = b, sq, table.shape[1] * kc.shape[1], hq, kc.shape[2], d, d
    p.scale, p.causal, p.window_left, p.window_right, p.dtype = d ** -0.5, 1, -1, -1, 1
    p.num_splits = num_splits
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_static_scratch_matches_caller_workspace_twice_in_a_row():
    torch.manual_seed(31)
    b, hq, hkv, d, page = 5, 16, 4, 128, 64
    blocks_per_seq = 40
    kc = torch.randn(b * blocks_per_seq, page, hkv, d, device="cuda").bfloat16()
    vc = torch.randn(b * blocks_per_seq, page, hkv, d, device="cuda").bfloat16()
    table = torch.randperm(b * blocks_per_seq, device="cuda").int().reshape(b, blocks_per_seq)
    rounds = (([2500, 64, 1, 1999, 777], 6), ([900, 2560, 333, 5, 1500], 0), ([900, 2560, 333, 5, 1500], 0))
    for round_, (lens_list, splits) in enumerate(rounds):
        lens = torch.tensor(lens_list, dtype=torch.int32, device="cuda")
        q = torch.randn(b, 2, hq, d, device="cuda").bfloat16()
        ref_out, new_out = torch.empty_like(q), torch.empty_like(q)
        ref_lse = torch.empty(b, hq, 2, device="cuda")
        new_lse = torch.empty(b, hq, 2, device="cuda")
        p = build_params(q, kc, vc, table, lens, ref_out, ref_lse, splits)
        need = capi.lib.fa_fwd_workspace_bytes(p)
        assert 0 < need <= capi.lib.fa_static_scratch_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        p.workspace, p.workspace_bytes = ws.data_ptr(), need
        assert capi.lib.fa_fwd_kvcache(p) == 0, capi.lib.fa_last_error()
        p2 = build_params(q, kc, vc, table, lens, new_out, new_lse, splits)      # no workspace given
        torch.cuda.synchronize()
        free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        assert capi.lib.fa_fwd_kvcache_static(p2) == 0, capi.lib.fa_last_error()
        torch.cuda.synchronize()
        if round_ == 2:
            assert torch.cuda.mem_get_info()[0] == free_before, "device memory in use changed across the call"
            assert torch.cuda.memory_allocated() == held_before
        # same tolerance as the other KV-cache tests (2^-6 on bf16 outputs, 1e-4 on LSE)
        assert (new_out.float() - ref_out.float()).abs().max().item() <= 2 ** -6, f"call {round_}"
        fin = torch.isfinite(ref_lse)            # rows without a visible key carry LSE = +inf in both
        assert torch.equal(new_lse[~fin], ref_lse[~fin]), f"call {round_}"
        assert (new_lse[fin] - ref_lse[fin]).abs().max().item() <= 1e-4, f"call {round_}"


def test_static_scratch_refuses_oversized_requests():
    b, hq, d = 512, 64, 128
    q = torch.empty(b, 1, hq, d, device="cuda", dtype=torch.bfloat16)
    kc = torch.empty(4, 256, 8, d, device="cuda", dtype=torch.bfloat16)
    table = torch.zeros(b, 128, dtype=torch.int32, device="cuda")
    lens = torch.ones(b, dtype=torch.int32, device="cuda")
    out, lse = torch.empty_like(q), torch.empty(b, hq, 1, device="cuda")
    p = build_params(q, kc, kc, table, lens, out, lse, 64)
    assert capi.lib.fa_fwd_workspace_bytes(p) > capi.lib.fa_static_scratch_bytes()
    assert capi.lib.fa_fwd_kvcache_static(p) == 6
    msg = capi.lib.fa_last_error().decode()
    assert "built-in pool holds" in msg and str(capi.lib.fa_static_scratch_bytes()) in msg
