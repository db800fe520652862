"""Multi-GPU partitioning of the attention path: one process per GPU, torch.distributed for the plumbing.

Prefill / training and ordinary decode shard independent (sequence x KV head) items across ranks with no
data-path collective (`balance_items`).  Long-context decode shards the KEY RANGE of every sequence:
rank r attends to keys [r*span, (r+1)*span), leaves fp32 partial (O, LSE) and one all-gather over NVLink
brings every rank's partials into local memory, where the LSE-weighted combine kernel merges them
(`sharded_kvcache_decode`, `sharded_mla_decode`).  The reference has no multi-device code; the combine math
is its split-KV combine (csrc/ascend910/flash_attn_npu/CombineScale.hpp:165-316)."""
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def balance_items(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Greedy longest-first bin packing: item indices per rank, deterministic (ties by index)."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * world_size
    bins: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        bins[r].append(i)
        loads[r] += costs[i]
    return [sorted(b) for b in bins]


def varlen_items(seqlens: Sequence[int], kv_heads: int, causal: bool = True) -> Tuple[List[Tuple[int, int]], List[float]]:
    """(sequence, KV head) work items of a packed batch and their cost (~ L^2, halved under a causal mask)."""
    items, costs = [], []
    for s, L in enumerate(seqlens):
        for h in range(kv_heads):
            items.append((s, h))
            costs.append(float(L) * float(L) * (0.5 if causal else 1.0))
    return items, costs


def kv_shard_range(max_len: int, rank: int, world_size: int, align: int) -> Tuple[int, int]:
    """Key range of `rank` when [0, max_len) is cut into world_size spans that are multiples of `align`."""
    span = (max_len + world_size * align - 1) // (world_size * align) * align
    return rank * span, (rank + 1) * span


def pack_partials(o_partial: torch.Tensor, lse_partial: torch.Tensor) -> torch.Tensor:
    """(rows, dv) fp32 + (rows,) fp32 -> (rows, dv + 1): one buffer, one collective."""
    return torch.cat((o_partial, lse_partial.unsqueeze(-1)), dim=-1).contiguous()


def unpack_partials(buf: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(world, rows, dv + 1) -> (world, rows, dv), (world, rows)."""
    return buf[..., :-1].contiguous(), buf[..., -1].contiguous()


def all_gather_partials(o_partial: torch.Tensor, lse_partial: torch.Tensor, group=None):
    """All-gather every rank's (O, LSE) partials into local memory. Returns (world, rows, dv), (world, rows)."""
    world = dist.get_world_size(group)
    mine = pack_partials(o_partial, lse_partial)
    out = torch.empty((world * mine.shape[0], mine.shape[1]), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(out, mine, group=group)      # rank-major concatenation along dim 0
    return unpack_partials(out.view(world, mine.shape[0], mine.shape[1]))


def sharded_kvcache_decode(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale, max_len, page_size,
                           causal=False, group=None, out_dtype=None):
    """flash_attn_with_kvcache (seqlen_q small, no append) with the key range sharded over the ranks of `group`.
    Every rank holds q and the cache blocks of its own key range (block_table entries outside it are never
    dereferenced).  Returns out (B, Sq, H, Dv) and lse (B, H, Sq), identical on all ranks."""
    from flash_attn_npu import flash_attn_npu as ext
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, sq, h, _ = q.shape
    dv = v_cache.shape[-1]
    rows = b * sq * h
    po = torch.empty(rows, dv, dtype=torch.float32, device=q.device)
    pl = torch.empty(rows, dtype=torch.float32, device=q.device)
    ext.kvcache_forward(q, k_cache, v_cache, None, None, cache_seqlens, None, None, None, block_table, None, None,
                        softmax_scale, causal, -1, -1, 0.0, False, 0,
                        kv_range=kv_shard_range(max_len, rank, world, page_size), partials=(po, pl))
    go, gl = all_gather_partials(po, pl, group)
    out, lse = ext3.fwd_combine(go, gl, None, out_dtype or q.dtype)
    return out.reshape(b, sq, h, dv), lse.reshape(b, sq, h).permute(0, 2, 1).contiguous()


def sharded_mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, max_len,
                       page_size, group=None):
    """int8 latent decode with the key range sharded over the ranks of `group` (BASELINE configuration 5):
    partial (O, LSE) per rank, one all-gather, local combine.  Returns out (B,1,H,512) bf16, lse (B,H,1)."""
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, _, h, dl = q_nope.shape
    po = torch.empty(b * h, dl, dtype=torch.float32, device=q_nope.device)
    pl = torch.empty(b * h, dtype=torch.float32, device=q_nope.device)
    ext3.mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, 0,
                    kv_range=kv_shard_range(max_len, rank, world, page_size), partials=(po, pl))
    go, gl = all_gather_partials(po, pl, group)
    out, lse = ext3.fwd_combine(go, gl, None, torch.bfloat16)
    return out.reshape(b, 1, h, dl), lse.reshape(b, h, 1)
