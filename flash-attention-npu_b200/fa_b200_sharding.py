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


class _DeviceMemory:
    """Lets torch view raw device memory owned by the CUDA library (no copy, no ownership)."""

    def __init__(self, address: int, floats: int):
        self.__cuda_array_interface__ = {"shape": (floats,), "typestr": "<f4", "data": (address, False), "version": 2}


class PeerExchange:
    """Exchange buffers for the KV-sharded decode without a library collective: every rank's fp32 partial (O, LSE)
    stay in a buffer of its own that the other ranks have mapped (CUDA IPC), and `combine` runs the one kernel that
    signals the peers, waits for them (at most `timeout_ms`) and sums all ranks' partials with loads over NVLink.
    All ranks must make the same sequence of `partials()` / `combine()` calls, on one stream each.

    `local_world=n` builds n buffers inside this process instead (rank 0, no process group): single-GPU tests use it
    and play the other ranks by writing their slots and flags themselves."""

    def __init__(self, rows: int, dv: int, device, group=None, timeout_ms: int = 1000, local_world: int = 0):
        import ctypes as C
        import fa_b200_capi as capi
        self._capi, self._C = capi, C
        self.rows, self.dv, self.device, self.group, self.timeout_ms = int(rows), int(dv), torch.device(device), group, timeout_ms
        self.local = local_world > 0
        self.rank = 0 if self.local else dist.get_rank(group)
        self.world = local_world if self.local else dist.get_world_size(group)
        if self.world > capi.MAX_PEERS:
            raise RuntimeError(f"at most {capi.MAX_PEERS} ranks")
        if dv % 4:
            raise RuntimeError("dv must be a multiple of 4")
        up = lambda n: (n + 255) // 256 * 256
        self.o_bytes, self.l_bytes = up(self.rows * self.dv * 4), up(self.rows * 4)
        self.slot_bytes = self.o_bytes + self.l_bytes + 256          # partial O | partial LSE | flags
        self.owned, self.opened, self.ptrs = [], [], []
        with torch.cuda.device(self.device):
            if self.local:
                for _ in range(self.world):
                    self.ptrs.append(self._create()[0])
            else:
                mine, handle = self._create()
                handles = [None] * self.world
                dist.all_gather_object(handles, handle, group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.ptrs.append(mine)
                        continue
                    p = C.c_void_p()
                    capi.check(capi.lib.fa_peer_buffer_open(h, C.byref(p)))
                    self.opened.append(p.value)
                    self.ptrs.append(p.value)
                dist.barrier(group=group)                             # every buffer is mapped before its first use
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = 0

    def _create(self):
        C, capi = self._C, self._capi
        p, h = C.c_void_p(), C.create_string_buffer(capi.PEER_HANDLE_BYTES)
        capi.check(capi.lib.fa_peer_buffer_create(2 * self.slot_bytes, C.byref(p), h))
        self.owned.append(p.value)
        return p.value, h.raw

    def _slot(self, epoch: int) -> int:
        return (epoch & 1) * self.slot_bytes

    def views(self, rank: int, epoch: int):
        """(partial O (rows, dv), partial LSE (rows), flags as fp32 words) of `rank`'s slot for call `epoch`."""
        base = self.ptrs[rank] + self._slot(epoch)
        with torch.cuda.device(self.device):
            o = torch.as_tensor(_DeviceMemory(base, self.rows * self.dv), device=self.device).view(self.rows, self.dv)
            l = torch.as_tensor(_DeviceMemory(base + self.o_bytes, self.rows), device=self.device)
            f = torch.as_tensor(_DeviceMemory(base + self.o_bytes + self.l_bytes, 64), device=self.device)
        return o, l, f

    def partials(self):
        """Starts the next call: the (O, LSE) tensors this rank's decode has to fill."""
        self.epoch += 1
        o, l, _ = self.views(self.rank, self.epoch)
        return o, l

    def combine(self, out_dtype=torch.bfloat16):
        """Signal, bounded wait, combine over peer memory -> out (rows, dv), lse (rows).  `check()` reports a timeout."""
        C, capi = self._C, self._capi
        out = torch.empty(self.rows, self.dv, dtype=out_dtype, device=self.device)
        lse = torch.empty(self.rows, dtype=torch.float32, device=self.device)
        c = capi.PeerCombineParams()
        c.rank, c.world = self.rank, self.world
        for r, p in enumerate(self.ptrs):
            c.peers[r] = p
        c.slot_offset = self._slot(self.epoch)
        c.lse_offset = c.slot_offset + self.o_bytes
        c.flag_offset = c.lse_offset + self.l_bytes
        c.epoch, c.timeout_ms = self.epoch, self.timeout_ms
        c.rows, c.dv = self.rows, self.dv
        c.out_dtype = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out_dtype]
        c.o, c.o_stride, c.lse, c.status = out.data_ptr(), self.dv, lse.data_ptr(), self.status.data_ptr()
        c.stream = capi.stream_ptr(self.device)
        with torch.cuda.device(self.device):
            capi.check(capi.lib.fa_peer_combine(c))
        return out, lse

    def check(self):
        """Synchronises; raises if a peer's signal did not arrive within the limit since the last check."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"peer exchange: no signal from rank {code - 1} within {self.timeout_ms} ms")

    def close(self):
        capi = self._capi
        torch.cuda.synchronize(self.device)
        if not self.local:
            dist.barrier(group=self.group)                            # nobody reads a buffer that is about to go
        with torch.cuda.device(self.device):
            for p in self.opened:
                capi.check(capi.lib.fa_peer_buffer_close(p))
            for p in self.owned:
                capi.check(capi.lib.fa_peer_buffer_destroy(p))
        self.opened, self.owned, self.ptrs = [], [], []


def sharded_kvcache_decode(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale, max_len, page_size,
                           causal=False, group=None, out_dtype=None, exchange=None):
    """flash_attn_with_kvcache (seqlen_q small, no append) with the key range sharded over the ranks of `group`.
    Every rank holds q and the cache blocks of its own key range (block_table entries outside it are never
    dereferenced).  Returns out (B, Sq, H, Dv) and lse (B, H, Sq), identical on all ranks.  With `exchange`
    (a PeerExchange of rows = B*Sq*H) the partials are exchanged and combined by one kernel over peer memory
    instead of an NCCL all-gather followed by a combine."""
    from flash_attn_npu import flash_attn_npu as ext
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, sq, h, _ = q.shape
    dv = v_cache.shape[-1]
    rows = b * sq * h
    if exchange is not None:
        po, pl = exchange.partials()
    else:
        po = torch.empty(rows, dv, dtype=torch.float32, device=q.device)
        pl = torch.empty(rows, dtype=torch.float32, device=q.device)
    ext.kvcache_forward(q, k_cache, v_cache, None, None, cache_seqlens, None, None, None, block_table, None, None,
                        softmax_scale, causal, -1, -1, 0.0, False, 0,
                        kv_range=kv_shard_range(max_len, rank, world, page_size), partials=(po, pl))
    if exchange is not None:
        out, lse = exchange.combine(out_dtype or q.dtype)
    else:
        go, gl = all_gather_partials(po, pl, group)
        out, lse = ext3.fwd_combine(go, gl, None, out_dtype or q.dtype)
    return out.reshape(b, sq, h, dv), lse.reshape(b, sq, h).permute(0, 2, 1).contiguous()


def sharded_mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, max_len,
                       page_size, group=None, exchange=None):
    """int8 latent decode with the key range sharded over the ranks of `group` (benchmark configuration 5):
    partial (O, LSE) per rank, one all-gather, local combine.  Returns out (B,1,H,512) bf16, lse (B,H,1)."""
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, _, h, dl = q_nope.shape
    if exchange is not None:
        po, pl = exchange.partials()
    else:
        po = torch.empty(b * h, dl, dtype=torch.float32, device=q_nope.device)
        pl = torch.empty(b * h, dtype=torch.float32, device=q_nope.device)
    ext3.mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, 0,
                    kv_range=kv_shard_range(max_len, rank, world, page_size), partials=(po, pl))
    if exchange is not None:
        out, lse = exchange.combine(torch.bfloat16)
    else:
        go, gl = all_gather_partials(po, pl, group)
        out, lse = ext3.fwd_combine(go, gl, None, torch.bfloat16)
    return out.reshape(b, 1, h, dl), lse.reshape(b, h, 1)
