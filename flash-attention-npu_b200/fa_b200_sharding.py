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


def dense_items(batch: int, kv_heads: int) -> List[Tuple[int, int]]:
    """(batch entry, KV head) work items of a dense batch; a KV head carries its whole query-head group."""
    return [(b, h) for b in range(batch) for h in range(kv_heads)]


def group_items(items: Sequence[Tuple[int, int]]) -> List[Tuple[Tuple[int, ...], Tuple[int, ...]]]:
    """Turns a rank's (outer, head) items into as few rectangular calls as possible: outer indices (batch entries
    or sequences) that own the same set of heads are put into one (outers, heads) group."""
    heads_of = {}
    for o, h in items:
        heads_of.setdefault(o, []).append(h)
    groups = {}
    for o in sorted(heads_of):
        groups.setdefault(tuple(sorted(heads_of[o])), []).append(o)
    return [(tuple(outers), heads) for heads, outers in sorted(groups.items(), key=lambda kv: (kv[1][0], kv[0]))]


def split_pages(n_pages: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous page ranges [g*n/N, (g+1)*n/N) of one sequence, one per rank (some may be empty)."""
    return [(g * n_pages // world_size, (g + 1) * n_pages // world_size) for g in range(world_size)]


def decode_shard_plan(seqlens: Sequence[int], world_size: int, page_size: int, long_threshold: int):
    """Long-context decode plan.  Sequences of at most `long_threshold` keys stay whole and are spread over the
    ranks by length (longest first, on top of the load the long ones put on every rank); a longer sequence is cut
    into `world_size` contiguous page ranges, one per rank, whose partial (O, LSE) are exchanged and combined.
    With one rank nothing is cut.  Returns a dict:
      short[r]      sequence indices rank r owns whole
      long          indices of the cut sequences (the same order on every rank)
      pages[r][k]   (first page, end page) of long sequence k on rank r
      tokens[r][k]  keys of long sequence k that lie in that range"""
    n = len(seqlens)
    if world_size == 1:
        return {"short": [list(range(n))], "long": [], "pages": [[]], "tokens": [[]]}
    long_ids = [i for i in range(n) if seqlens[i] > long_threshold]
    short_ids = [i for i in range(n) if seqlens[i] <= long_threshold]
    pages = [[] for _ in range(world_size)]
    tokens = [[] for _ in range(world_size)]
    loads = [0.0] * world_size
    for i in long_ids:
        L = int(seqlens[i])
        for r, (p0, p1) in enumerate(split_pages((L + page_size - 1) // page_size, world_size)):
            t = max(0, min(L, p1 * page_size) - p0 * page_size)
            pages[r].append((p0, p1))
            tokens[r].append(t)
            loads[r] += t
    short = [[] for _ in range(world_size)]
    for i in sorted(short_ids, key=lambda j: (-seqlens[j], j)):
        r = min(range(world_size), key=lambda j: (loads[j], j))
        short[r].append(i)
        loads[r] += seqlens[i]
    return {"short": [sorted(x) for x in short], "long": long_ids, "pages": pages, "tokens": tokens}


class PartialBuffer:
    """Send buffer of one rank for the all-gather of split partials: fp32 (rows, dv) partial O followed by the
    (rows) partial LSE in ONE allocation, so that the decode kernels write straight into what the collective sends
    and nothing is packed or unpacked.  `gather()` returns strided views of the receive buffer that the combine
    kernel reads in place."""

    def __init__(self, rows: int, dv: int, device, world_size: int):
        self.rows, self.dv, self.world = int(rows), int(dv), int(world_size)
        self.floats = (self.rows * (self.dv + 1) + 63) // 64 * 64      # every rank's part starts 256-byte aligned
        self.send = torch.empty(self.floats, dtype=torch.float32, device=device)
        self.recv = torch.empty(self.world * self.floats, dtype=torch.float32, device=device)
        self.o = self.send[: self.rows * self.dv].view(self.rows, self.dv)
        self.lse = self.send[self.rows * self.dv: self.rows * (self.dv + 1)]

    def gather(self, group=None):
        """One all-gather; returns (world, rows, dv) and (world, rows) views of the receive buffer."""
        if self.world == 1:
            self.recv.copy_(self.send)
        else:
            dist.all_gather_into_tensor(self.recv, self.send, group=group)
        r = self.recv.view(self.world, self.floats)
        return (r[:, : self.rows * self.dv].view(self.world, self.rows, self.dv),
                r[:, self.rows * self.dv: self.rows * (self.dv + 1)])


def all_gather_partials(o_partial: torch.Tensor, lse_partial: torch.Tensor, group=None):
    """All-gather of (O, LSE) partials that do not live in a PartialBuffer (one staging copy).
    Returns (world, rows, dv), (world, rows)."""
    world = dist.get_world_size(group)
    buf = PartialBuffer(o_partial.shape[0], o_partial.shape[1], o_partial.device, world)
    buf.o.copy_(o_partial)
    buf.lse.copy_(lse_partial)
    return buf.gather(group)


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

    def combine(self, out_dtype=torch.bfloat16, row_begin: int = 0, row_end: int = None):
        """Signal, bounded wait, combine over peer memory -> out (rows, dv), lse (rows).  `check()` reports a timeout.
        With a row range only rows [row_begin, row_end) are combined (and returned): when every rank needs the
        result of its OWN sequences only, each combines its own range and the bytes that cross NVLink drop by the
        number of ranks.  All ranks still make the call (the signals are per call, not per row)."""
        C, capi = self._C, self._capi
        row_end = self.rows if row_end is None else row_end
        n = max(0, row_end - row_begin)
        out = torch.empty(n, self.dv, dtype=out_dtype, device=self.device)
        lse = torch.empty(n, dtype=torch.float32, device=self.device)
        c = capi.PeerCombineParams()
        c.rank, c.world = self.rank, self.world
        for r, p in enumerate(self.ptrs):
            c.peers[r] = p
        slot = self._slot(self.epoch)
        c.slot_offset = slot + row_begin * self.dv * 4
        c.lse_offset = slot + self.o_bytes + row_begin * 4
        c.flag_offset = slot + self.o_bytes + self.l_bytes
        c.epoch, c.timeout_ms = self.epoch, self.timeout_ms
        c.rows, c.dv = n, self.dv
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
                           causal=False, group=None, out_dtype=None, exchange=None, buffer=None):
    """flash_attn_with_kvcache (seqlen_q small, no append) with the key range sharded over the ranks of `group`.
    Every rank holds q and the cache blocks of its own key range (block_table entries outside it are never
    dereferenced).  Returns out (B, Sq, H, Dv) and lse (B, H, Sq), identical on all ranks.  With `exchange`
    (a PeerExchange of rows = B*Sq*H) the partials are exchanged and combined by one kernel over peer memory;
    otherwise the decode writes them into a PartialBuffer (`buffer`, made here when not given), one NCCL
    all-gather brings every rank's buffer into local memory and the combine kernel reads them in place."""
    from flash_attn_npu import flash_attn_npu as ext
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, sq, h, _ = q.shape
    dv = v_cache.shape[-1]
    rows = b * sq * h
    if exchange is not None:
        po, pl = exchange.partials()
    else:
        buffer = buffer or PartialBuffer(rows, dv, q.device, world)
        po, pl = buffer.o, buffer.lse
    ext.kvcache_forward(q, k_cache, v_cache, None, None, cache_seqlens, None, None, None, block_table, None, None,
                        softmax_scale, causal, -1, -1, 0.0, False, 0,
                        kv_range=kv_shard_range(max_len, rank, world, page_size), partials=(po, pl))
    if exchange is not None:
        out, lse = exchange.combine(out_dtype or q.dtype)
    else:
        go, gl = buffer.gather(group)
        out, lse = ext3.fwd_combine(go, gl, None, out_dtype or q.dtype)
    return out.reshape(b, sq, h, dv), lse.reshape(b, sq, h).permute(0, 2, 1).contiguous()


def sharded_mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, max_len=None,
                       page_size=None, group=None, exchange=None, buffer=None):
    """int8 latent decode of sequences whose keys are spread over the ranks of `group` (benchmark configuration
    5): partial (O, LSE) per rank, exchange, combine.  Returns out (B,1,H,512) bf16, lse (B,H,1), identical on
    all ranks.  Two ways to say which keys a rank holds:
      * `max_len` given: every rank passes the full table and lengths and attends to the key range
        kv_shard_range(max_len, rank, world, page_size) of every sequence;
      * `max_len` None: `block_table` / `cache_seqlens` already describe only this rank's pages and key count of
        every sequence (decode_shard_plan), which lets each sequence be cut in proportion to its own length."""
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, _, h, dl = q_nope.shape
    if exchange is not None:
        po, pl = exchange.partials()
    else:
        buffer = buffer or PartialBuffer(b * h, dl, q_nope.device, world)
        po, pl = buffer.o, buffer.lse
    rng = kv_shard_range(max_len, rank, world, page_size) if max_len is not None else None
    ext3.mla_decode(q_nope, q_rope, latent_i8, scales, rope, block_table, cache_seqlens, softmax_scale, 0,
                    kv_range=rng, partials=(po, pl))
    if exchange is not None:
        out, lse = exchange.combine(torch.bfloat16)
    else:
        go, gl = buffer.gather(group)
        out, lse = ext3.fwd_combine(go, gl, None, torch.bfloat16)
    return out.reshape(b, 1, h, dl), lse.reshape(b, h, 1)
