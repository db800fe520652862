"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl reference]

Headline (`value`): benchmark configuration 2, flash_attn_func forward + backward in bf16, batch 4, seqlen 4096,
32 query heads, 32 KV heads, headdim 128, causal, softmax_scale 1/sqrt(128), synthetic N(0,1) inputs.  One step =
one forward + one backward over that batch.  The metric is fwd+bwd TFLOP/s with the standard FlashAttention
accounting (forward 4*B*H*S*S*D/2 under the causal mask, backward 2.5 x forward).

With N > 1 ranks (one process per GPU) the batch is PARTITIONED: its 128 (batch entry x KV head) items are dealt
to the ranks (fa_b200_sharding.balance_items), every rank runs forward + backward of its own items, there is no
data-path collective, and `value` is the whole batch's flop over the slowest rank's time (strong scaling).  The
other configurations run the same way in the same process and are reported beside it: 3 (packed forward,
(sequence x KV head) items balanced by L^2), 4 (paged decode, sequences balanced by length), 5 (int8 latent
decode: sequences of at most 32768 keys spread over the ranks, longer ones cut into one page range per rank whose
partial (O, LSE) are exchanged, by an NCCL all-gather and by one kernel over peer memory, and combined).  Every rank
checks a sample of each configuration's results against the CPU oracle; a miss makes the process exit non-zero.

`--impl reference` times the CPU oracle (a port of the reference's Python goldens; the reference's device code
needs an Ascend toolchain) on a bounded sample of the same workload.  Prints one JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "flash-attention-npu_b200"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

B, S, H, HKV, D = 4, 4096, 32, 32, 128
SCALE = D ** -0.5
WORKLOAD = "config2: flash_attn_func fwd+bwd bf16 B4 S4096 Hq32 Hkv32 D128 causal"
FWD_FLOPS = 4.0 * B * H * S * S * D / 2.0
BWD_FLOPS = 2.5 * FWD_FLOPS
STEP_FLOPS = FWD_FLOPS + BWD_FLOPS
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126e6

# DRAM bytes of one dK/dV launch at B2 S4096 H32 D128 causal in the committed ncu capture of that kernel
# (dram__bytes_read.sum 278.8 MB + dram__bytes_write.sum 1203.7 MB, of which 1107 MB are the dS tiles it hands to the dQ
# kernel); the traffic grows in proportion to the batch
DKDV_TRAFFIC_B2 = 278.7e6 + 1204.2e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML in a thread while the timed region runs
    (a polling nvidia-smi process was seen to stall kernel launches for milliseconds)."""

    def __init__(self, index, period=0.01):
        self.index, self.period = index, period
        self.samples, self.stop_flag, self.thread, self.h = [], False, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.smax = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:                                     # NVML missing: report that, do not fail the bench
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                clk = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.time(), clk, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.nv is not None and self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)

    def window(self, t0, t1):
        """Median SM MHz of the samples taken in [t0, t1] (None when the window was shorter than a sample)."""
        inside = [c for ts, c, _ in self.samples if t0 <= ts <= t1]
        return statistics.median(inside) if inside else None

    def summary(self, t0, t1):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        inside = [(c, r) for ts, c, r in self.samples if t0 <= ts <= t1] or [(c, r) for _, c, r in self.samples[-2:]]
        reasons = sorted(n for n, bit in names.items() if any(r & bit for _, r in inside))
        return {"sm_mhz": statistics.median(c for c, _ in inside) if inside else None, "sm_max_mhz": self.smax,
                "reasons": reasons, "samples": len(inside)}


def cpu_oracle_sample(heads=2, batch=1):
    """The CPU oracle on `batch` batch entries and `heads` heads of the workload (forward fp32 math on bf16
    inputs, backward in float64 like the reference golden).  Returns (TFLOP/s, seconds, cores, text)."""
    from oracle import attention_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(batch, S, heads, D, generator=g).bfloat16() for _ in range(4))
    t0 = time.perf_counter()
    out, lse = orc.attention_fwd(q, k, v, SCALE, causal=True)
    orc.attention_bwd(q, k, v, do, lse, SCALE, causal=True, head_chunk=1)
    dt = time.perf_counter() - t0
    flops = STEP_FLOPS * heads * batch / (B * H)
    return flops / dt / 1e12, dt, cores, f"{batch} of {B} batch entries x {heads} of {H} heads of the workload, fwd + bwd"


def run_reference(args, rank):
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup):
        cpu_oracle_sample(1)
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, dt, cores, sample = cpu_oracle_sample(2)
        vals.append((v, dt))
    wall = time.perf_counter() - t_all
    value = sum(STEP_FLOPS * 2 / (B * H) for _ in vals) / sum(dt for _, dt in vals) / 1e12
    line = {
        "impl": "reference", "metric": "fwd_bwd_attention_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "note": "CPU oracle (port of the reference's torch goldens) on the host cores"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------
# small helpers
# ---------------------------------------------------------------------------------------------------------------
class Dist:
    """Rank bookkeeping plus the two collectives the bench itself needs (barrier, max over ranks)."""

    def __init__(self, rank, world, dev):
        self.rank, self.world, self.dev = rank, world, dev

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, values):
        """Element-wise max over the ranks of a list of floats."""
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def all_ok(self, ok):
        t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item()) == 0


def bind_to_gpu_numa_node(local):
    """Pins this process to the cores of the NUMA node its GPU hangs off, so that pinned host buffers allocated
    afterwards are local to the GPU's PCIe root.  Best effort; returns the previous affinity (or None)."""
    try:
        props = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        old = os.sched_getaffinity(0)
        new = cpus & old
        if new:
            os.sched_setaffinity(0, new)
            return old
    except Exception:
        pass
    return None


def _time_calls(call, iters, warm=3):
    for _ in range(warm):
        call()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        call()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def _paged_tables(lens_tokens, page, gen):
    """Block table of a pool that holds exactly the pages of these sequences, in a seeded random order."""
    nblk = [(int(n) + page - 1) // page for n in lens_tokens]
    pool = sum(nblk)
    perm = torch.randperm(max(pool, 1), generator=gen).int()
    table = torch.zeros(max(len(nblk), 1), max(nblk + [1]), dtype=torch.int32)
    off = 0
    for i, n in enumerate(nblk):
        table[i, :n] = perm[off:off + n]
        off += n
    return table, pool, nblk


def _worst(results):
    """Summary of a list of parity results: ok flag and the entry closest to (or furthest beyond) its tolerance."""
    if not results:
        return {"ok": True, "checked": 0}
    w = max(results, key=lambda r: r["err"] / r["tol"] if r["tol"] > 0 else (0.0 if r["err"] == 0 else float("inf")))
    return {"ok": all(r["ok"] for r in results), "checked": len(results), "worst": w["name"], "err": w["err"],
            "tol": w["tol"], "two_x_golden": w["two_x_golden"], "floor": w["floor"], "binding": w["binding"]}


# ---------------------------------------------------------------------------------------------------------------
# configuration 2: the headline
# ---------------------------------------------------------------------------------------------------------------
def config2_leg(args, dd, ext, capi, sampler):
    import fa_b200_sharding as sh
    import parity
    from oracle import attention_oracle as orc
    dev, rank, world = dd.dev, dd.rank, dd.world
    items = sh.dense_items(B, HKV)
    bins = sh.balance_items([1.0] * len(items), world)
    groups = sh.group_items([items[i] for i in bins[rank]])
    G = H // HKV
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def make_set():
        calls = []
        for batches, heads in groups:
            nb, nh = len(batches), len(heads)
            t = {n: torch.randn(nb, S, hh, D, device=dev, generator=gen).bfloat16()
                 for n, hh in (("q", nh * G), ("k", nh), ("v", nh), ("do", nh * G))}
            t["dq"], t["dk"], t["dv"] = torch.empty_like(t["q"]), torch.empty_like(t["k"]), torch.empty_like(t["v"])
            calls.append(t)
        return calls

    # Between timed iterations the inputs must not stay in L2: a rank's share shrinks with N, so the steps rotate
    # over as many independent input sets as it takes to put at least 2 x L2 of inputs between two uses of a set.
    in_bytes = sum(len(bs) * S * len(hs) * D * 2 * (2 * G + 2) for bs, hs in groups)
    nsets = max(1, int(-(-2 * L2_BYTES // in_bytes)))
    sets = [make_set() for _ in range(nsets)]

    def step(calls):
        res = []
        for t in calls:
            out, lse, _, _ = ext.fwd(t["q"], t["k"], t["v"], None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
            ext.bwd(t["do"], t["q"], t["k"], t["v"], out, lse, t["dq"], t["dk"], t["dv"], None, 0.0, SCALE, True, -1, -1,
                    0.0, False, None, None)
            res.append((out, lse))
        return res

    for i in range(args.warmup):
        step(sets[i % nsets])
    t0 = sets[0][0]
    out, lse, _, _ = ext.fwd(t0["q"], t0["k"], t0["v"], None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
    fwd_kernel = capi.last_kernel()
    ext.bwd(t0["do"], t0["q"], t0["k"], t0["v"], out, lse, t0["dq"], t0["dk"], t0["dv"], None, 0.0, SCALE, True, -1, -1, 0.0,
            False, None, None)
    bwd_kernel = capi.last_kernel()

    # ---- per-kernel durations: a few eager steps with events lent to the library (not the headline) ----------
    nev, nb_steps = 8, min(args.steps, 10)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(nev)] for _ in range(2 * nb_steps)]
    for row in evs:
        for e in row:
            e.record()
    torch.cuda.synchronize()
    arr_t = ctypes.c_void_p * nev
    arrays = [arr_t(*[e.cuda_event for e in row]) for row in evs]
    used = [0] * (2 * nb_steps)
    for i in range(nb_steps):
        t = sets[i % nsets][0]
        capi.lib.fa_set_kernel_events(arrays[2 * i], nev)
        out, lse, _, _ = ext.fwd(t["q"], t["k"], t["v"], None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
        used[2 * i] = capi.lib.fa_kernel_events_used()
        capi.lib.fa_set_kernel_events(arrays[2 * i + 1], nev)
        ext.bwd(t["do"], t["q"], t["k"], t["v"], out, lse, t["dq"], t["dk"], t["dv"], None, 0.0, SCALE, True, -1, -1, 0.0,
                False, None, None)
        used[2 * i + 1] = capi.lib.fa_kernel_events_used()
    capi.lib.fa_set_kernel_events(None, 0)
    torch.cuda.synchronize()
    fwd_ms = statistics.mean(evs[2 * i][0].elapsed_time(evs[2 * i][used[2 * i] - 1]) for i in range(nb_steps))
    bwd_parts = [statistics.mean(evs[2 * i + 1][j - 1].elapsed_time(evs[2 * i + 1][j]) for i in range(nb_steps))
                 for j in range(1, used[1])]
    launches_per_step = (used[0] - 1 + used[1] - 1) * len(groups)

    # ---- device-timed region: R repeats of exactly K steps, each step a CUDA-graph replay (no host work between
    # launches); the max over ranks of every repeat, then the median over the repeats --------------------------
    timed_as = "cuda graph replay of one step"
    graphs = []
    try:
        for calls in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step(calls)
            g.replay()
            graphs.append(g)
        torch.cuda.synchronize()
        run = [g.replay for g in graphs]
    except Exception as exc:                                   # fall back to eager launches
        timed_as = "eager launches (graph capture failed: %s)" % str(exc)[:80]
        torch.cuda.synchronize()
        run = [(lambda c=calls: step(c)) for calls in sets]
    rep_ms, rep_win = [], []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for r in range(args.repeats):
        dd.barrier()
        w0 = time.time()
        start.record()
        for i in range(args.steps):
            run[i % nsets]()
        stop.record()
        dd.barrier()
        rep_win.append((w0, time.time()))
        rep_ms.append(start.elapsed_time(stop) / args.steps)
    rep_ms = dd.max(rep_ms)
    ms = statistics.median(rep_ms)

    # ---- parity of one of this rank's items against the CPU oracle ------------------------------------------------
    res = step(sets[0])
    torch.cuda.synchronize()
    t, (out, lse) = sets[0][0], res[0]
    hs = slice(0, G)
    qs, ks, vs, dos = (t[n][0:1, :, sl].cpu() for n, sl in (("q", hs), ("k", slice(0, 1)), ("v", slice(0, 1)), ("do", hs)))
    lp_o, _ = orc.attention_fwd(qs, ks, vs, SCALE, True)
    f_o, f_l = orc.attention_fwd(qs.float(), ks.float(), vs.float(), SCALE, True, data_type=torch.float32)
    checks = [parity.check_within("out", out[0:1, :, hs].cpu(), lp_o, f_o), parity.check_lse(lse[0:1, hs].cpu(), f_l)]
    lp = orc.attention_bwd(qs, ks, vs, dos, f_l, SCALE, True, head_chunk=1)
    f32 = orc.attention_bwd(qs.float(), ks.float(), vs.float(), dos.float(), f_l, SCALE, True, head_chunk=1)
    for name, got, a, b_ in zip(("dq", "dk", "dv"), (t["dq"][0:1, :, hs], t["dk"][0:1, :, 0:1], t["dv"][0:1, :, 0:1]), lp, f32):
        checks.append(parity.check_within(name, got.cpu(), a, b_, roundings=3))
    batches, heads = groups[0]
    par = _worst(checks)
    par["item"] = f"batch entry {batches[0]}, KV head {heads[0]} of rank {rank}"

    return {"ms": ms, "rep_ms": rep_ms, "rep_win": rep_win, "fwd_ms": fwd_ms, "bwd_parts": bwd_parts,
            "launches_per_step": launches_per_step, "fwd_kernel": fwd_kernel, "bwd_kernel": bwd_kernel,
            "timed_as": timed_as, "nsets": nsets, "groups": groups, "in_bytes": in_bytes, "parity": par, "sets": sets}


def replicated_leg(args, dd, ext):
    """Every rank runs the WHOLE batch of configuration 2 (weak scaling, what a data-parallel trainer does): shows
    that the GPUs of one box do not slow each other down; no partition involved."""
    dev = dd.dev
    gen = torch.Generator(device=dev).manual_seed(4321 + dd.rank)
    q, k, v, do = (torch.randn(B, S, hh, D, device=dev, generator=gen).bfloat16() for hh in (H, HKV, HKV, H))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def step():
        out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
        ext.bwd(do, q, k, v, out, lse, dq, dk, dv, None, 0.0, SCALE, True, -1, -1, 0.0, False, None, None)

    for _ in range(3):
        step()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    g.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dd.barrier()
    start.record()
    for _ in range(args.steps):
        g.replay()
    stop.record()
    dd.barrier()
    ms = dd.max([start.elapsed_time(stop) / args.steps])[0]
    return {"what": "every rank runs the whole batch (weak scaling, no partition)", "ms_per_step": ms,
            "value": STEP_FLOPS * dd.world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}


def e2e_leg(args, dd, sets, groups):
    """The same step through the public API with pinned HOST operands: every step copies the rank's q, k, v, dout to
    the device and out, dq, dk, dv back, inside the timed region (fa_b200_host.HostPipeline, one batch entry a
    chunk, contiguous copies).  Also times the copies alone (same bytes, streams and chunks, no kernels)."""
    import fa_b200_host
    dev = dd.dev
    calls = sets[0]
    host = [{n: t[n].cpu().pin_memory() for n in ("q", "k", "v", "do")} for t in calls]
    outs = [{n: torch.empty(h[m].shape, dtype=h[m].dtype).pin_memory() for n, m in (("out", "q"), ("dq", "q"), ("dk", "k"), ("dv", "v"))}
            for h in host]
    pipe = fa_b200_host.HostPipeline(dev, args.e2e_kv_heads)

    def one(run_kernels):
        for h, o in zip(host, outs):
            pipe.fwd_bwd(h["q"], h["k"], h["v"], h["do"], o["out"], o["dq"], o["dk"], o["dv"], causal=True,
                         softmax_scale=SCALE, run_kernels=run_kernels)

    def timed(run_kernels, n):
        one(run_kernels)
        dd.barrier()
        per = []
        for _ in range(n):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            one(run_kernels)
            e.record()
            torch.cuda.synchronize()
            per.append(s.elapsed_time(e))
        dd.barrier()
        return per

    n = max(args.e2e_steps, 3)
    floor = timed(False, max(5, n // 2))               # first: it leaves copies of the inputs in the result buffers
    full = timed(True, n)
    # check what came back against the device-resident run of the same set
    torch.cuda.synchronize()
    same = all(torch.equal(o["dq"], t["dq"].cpu()) and torch.equal(o["dk"], t["dk"].cpu()) and torch.equal(o["dv"], t["dv"].cpu())
               for o, t in zip(outs, calls))
    med, mn, fl = dd.max([statistics.median(full), min(full), statistics.median(floor)])
    h2d = sum(x.numel() * 2 for h in host for x in h.values())
    d2h = sum(x.numel() * 2 for o in outs for x in o.values())
    del host, outs
    return {"median_ms": med, "min_ms": mn, "copy_floor_ms": fl, "steps": n, "h2d": h2d, "d2h": d2h,
            "same_as_device_resident_run": same}


# ---------------------------------------------------------------------------------------------------------------
# configuration 3: packed forward, (sequence x KV head) items
# ---------------------------------------------------------------------------------------------------------------
def config3_leg(dd, iters=10):
    import flash_attn_npu as fa
    import fa_b200_capi as capi
    import fa_b200_sharding as sh
    import parity
    from oracle import attention_oracle as orc
    dev, rank, world = dd.dev, dd.rank, dd.world
    g = torch.Generator().manual_seed(3)
    hq, hkv, d = 32, 8, 128
    G = hq // hkv
    lens = torch.randint(256, 8193, (16,), generator=g).tolist()
    items, costs = sh.varlen_items(lens, hkv)
    bins = sh.balance_items(costs, world)
    mine = [items[i] for i in bins[rank]]
    groups = sh.group_items(mine)                      # (sequences, KV heads) rectangles of this rank
    gen = torch.Generator(device=dev).manual_seed(300 + rank)
    calls = []
    for seqs, heads in groups:
        ls = [lens[s] for s in seqs]
        cu = torch.zeros(len(ls) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(torch.tensor(ls), 0)
        total, nh = int(cu[-1]), len(heads)
        calls.append({"q": torch.randn(total, nh * G, d, device=dev, generator=gen).bfloat16(),
                      "k": torch.randn(total, nh, d, device=dev, generator=gen).bfloat16(),
                      "v": torch.randn(total, nh, d, device=dev, generator=gen).bfloat16(),
                      "cu": cu.to(dev), "cu_h": cu, "mx": max(ls), "seqs": seqs, "heads": heads})

    def run():
        return [fa.flash_attn_varlen_func(c["q"], c["k"], c["v"], c["cu"], c["cu"], c["mx"], c["mx"], causal=True,
                                          return_attn_probs=True) for c in calls]

    dd.barrier()
    ms = dd.max([_time_calls(run, iters)])[0]
    kern = capi.last_kernel()
    # parity: this rank's shortest item
    res = run()
    torch.cuda.synchronize()
    ci, si = min(((ci, si) for ci, c in enumerate(calls) for si in range(len(c["seqs"]))),
                 key=lambda x: lens[calls[x[0]]["seqs"][x[1]]])
    c = calls[ci]
    a, e = int(c["cu_h"][si]), int(c["cu_h"][si + 1])
    qs, ks, vs = c["q"][a:e, 0:G].cpu().unsqueeze(0), c["k"][a:e, 0:1].cpu().unsqueeze(0), c["v"][a:e, 0:1].cpu().unsqueeze(0)
    lp_o, _ = orc.attention_fwd(qs, ks, vs, d ** -0.5, True)
    f_o, f_l = orc.attention_fwd(qs.float(), ks.float(), vs.float(), d ** -0.5, True, data_type=torch.float32)
    out, lse = res[ci][0], res[ci][1]
    par = _worst([parity.check_within("out", out[a:e, 0:G].cpu().unsqueeze(0), lp_o, f_o),
                  parity.check_lse(lse[0:G, a:e].cpu().unsqueeze(0), f_l)])
    par["item"] = f"sequence {c['seqs'][si]} (L={e - a}), KV head {c['heads'][0]} of rank {rank}"
    flops = float(sum(4.0 * hq * n * n * d / 2.0 for n in lens))
    loads = [sum(costs[i] for i in b) for b in bins]
    peaks = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": "config3: flash_attn_varlen_func fwd bf16 16 seqs L~U[256,8192] Hq32 Hkv8 D128 causal",
            "partition": f"{len(items)} (sequence x KV head) items dealt longest-first by L^2; rank 0 runs "
                         f"{len(groups)} calls; heaviest rank carries {max(loads) / (sum(loads) / world):.3f} x the mean",
            "ms": ms, "value": tf, "unit": "TFLOP/s", "flops": flops, "tokens": int(sum(lens)), "kernel": kern,
            "frac_of_measured_bf16": tf / (world * peaks["bf16_tflops"]), "frac_of_nominal_2250": tf / (world * 2250.0),
            "parity": par}


# ---------------------------------------------------------------------------------------------------------------
# configuration 4: paged decode with append + rotary, sequences dealt to the ranks
# ---------------------------------------------------------------------------------------------------------------
def config4_leg(dd, iters=10):
    import flash_attn_npu as fa
    import fa_b200_capi as capi
    import fa_b200_sharding as sh
    import parity
    from oracle import attention_oracle as orc
    dev, rank, world = dd.dev, dd.rank, dd.world
    g = torch.Generator().manual_seed(4)
    b, hq, hkv, d, page = 128, 32, 8, 128, 256
    lens_all = torch.randint(1024, 32769, (b,), generator=g, dtype=torch.int32)
    bins = sh.balance_items([float(x) for x in lens_all], world)
    mine = bins[rank]
    lens = lens_all[mine]
    nb = len(mine)
    table, pool, nblk = _paged_tables((lens + 1).tolist(), page, torch.Generator().manual_seed(40 + rank))
    gen = torch.Generator(device=dev).manual_seed(400 + rank)
    kc = torch.randn(pool, page, hkv, d, device=dev, generator=gen).bfloat16()
    vc = torch.randn(pool, page, hkv, d, device=dev, generator=gen).bfloat16()
    q = torch.randn(nb, 1, hq, d, device=dev, generator=gen).bfloat16()
    kn = torch.randn(nb, 1, hkv, d, device=dev, generator=gen).bfloat16()
    vn = torch.randn(nb, 1, hkv, d, device=dev, generator=gen).bfloat16()
    cos_h, sin_h = orc.rotary_tables(32800, d)
    cos, sin = cos_h.to(dev), sin_h.to(dev)
    lens_d, table_d = lens.to(dev), table.to(dev)

    def call():
        return fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens_d,
                                          block_table=table_d, causal=True, rotary_interleaved=False,
                                          return_softmax_lse=True)

    dd.barrier()
    ms = dd.max([_time_calls(call, iters)])[0]
    kern = capi.last_kernel()
    out, lse = call()
    torch.cuda.synchronize()
    # parity: appended rows bit for bit on every sequence of the rank, the two shortest against the oracle
    qh, knh, vnh = q.cpu(), kn.cpu(), vn.cpu()
    kn_rot = torch.stack([orc.apply_rotary(knh[i], cos_h, sin_h, torch.tensor([int(lens[i])]), False) for i in range(nb)])
    blk = table[torch.arange(nb), (lens // page).long()].long().to(dev)
    row = (lens % page).long().to(dev)
    bit_exact = bool(torch.equal(kc[blk, row].cpu().view(torch.int16), kn_rot[:, 0].view(torch.int16)) and
                     torch.equal(vc[blk, row].cpu().view(torch.int16), vnh[:, 0].view(torch.int16)))
    checks = []
    for i in torch.argsort(lens).tolist()[:2]:
        L = int(lens[i]) + 1
        ki = orc.gather_paged(kc, table_d[i], L).cpu().unsqueeze(0)
        vi = orc.gather_paged(vc, table_d[i], L).cpu().unsqueeze(0)
        qi = orc.apply_rotary(qh[i], cos_h, sin_h, torch.tensor([L - 1]), False).unsqueeze(0)
        lp_o, _ = orc.attention_fwd(qi, ki, vi, d ** -0.5, True)
        f_o, f_l = orc.attention_fwd(qi.float(), ki.float(), vi.float(), d ** -0.5, True, data_type=torch.float32)
        checks += [parity.check_within("out", out[i:i + 1].cpu(), lp_o, f_o), parity.check_lse(lse[i:i + 1].cpu(), f_l)]
    par = _worst(checks)
    par["append_bit_exact"] = bit_exact
    par["ok"] = par["ok"] and bit_exact
    tokens = int((lens_all + 1).sum())
    bytes_ = tokens * hkv * d * 2 * 2 + b * hq * d * 2 * 2 + int(((lens_all + page) // page).sum()) * 4 + b * hkv * d * 2 * 2
    peaks = measured_peaks()
    gbs = bytes_ / (ms * 1e-3) / 1e9
    loads = [float(sum(lens_all[i] for i in bn)) for bn in bins]
    return {"workload": "config4: paged decode bf16 B128 Sq1 Hq32 Hkv8 D128 page256 L~U[1024,32768], append+rotary",
            "partition": f"128 sequences dealt longest-first by length, every rank holds the pages of its own; heaviest "
                         f"rank carries {max(loads) / (sum(loads) / world):.3f} x the mean",
            "ms": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": bytes_, "kernel": kern,
            "frac_of_measured_hbm": gbs / (world * peaks["hbm_gbs"]), "frac_of_nominal_8000": gbs / (world * 8000.0),
            "cache_gb_this_rank": pool * page * hkv * d * 2 * 2 / 1e9, "parity": par}


# ---------------------------------------------------------------------------------------------------------------
# configuration 5: int8 latent decode; long sequences cut over the ranks with an exchange of partials
# ---------------------------------------------------------------------------------------------------------------
LONG_THRESHOLD = 32768


def _latent_rows(n_tokens, seed, dev):
    """Seeded cache rows of one (sequence, rank range): N(0,1) latent quantised per token to int8 + fp32 scale, and
    the bf16 positional part.  The same seed and size give the same rows on every GPU of the box."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(n_tokens, 512, device=dev, generator=gen)
    sc = x.abs().amax(dim=-1).clamp_min(1e-12) / 127.0
    lat = torch.round(x / sc.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
    rope = torch.randn(n_tokens, 64, device=dev, generator=gen).bfloat16()
    return lat, sc.float(), rope


def _fill_pages(lat, sc, rope, pages, rows, page):
    """Scatters `rows` (lat, scale, rope of n tokens) into the pool pages `pages` (a sequence's pages in order)."""
    n = rows[0].shape[0]
    j = torch.arange(n, device=lat.device)
    blk = pages.to(lat.device).long()[j // page]
    lat[blk, j % page], sc[blk, j % page], rope[blk, j % page] = rows


def config5_leg(dd, iters=10):
    import torch.distributed as dist
    import flash_attn_npu_3 as fa3
    from flash_attn_npu_3 import flash_attn_npu_3 as ext3
    import fa_b200_capi as capi
    import fa_b200_sharding as sh
    import parity
    from oracle import attention_oracle as orc
    dev, rank, world = dd.dev, dd.rank, dd.world
    g = torch.Generator().manual_seed(5)
    b, hq, dl, dr, page = 64, 128, 512, 64, 256
    scale = 576 ** -0.5
    lens = torch.randint(4096, 131073, (b,), generator=g, dtype=torch.int32).tolist()
    plan = sh.decode_shard_plan(lens, world, page, LONG_THRESHOLD)
    shorts, longs = plan["short"][rank], plan["long"]
    # identical queries on every rank (a long sequence's query is needed by all of them)
    gq = torch.Generator(device=dev).manual_seed(50)
    qn_all = torch.randn(b, 1, hq, dl, device=dev, generator=gq).bfloat16()
    qr_all = torch.randn(b, 1, hq, dr, device=dev, generator=gq).bfloat16()
    # local batch: the sequences owned whole, then this rank's page range of every cut sequence
    tok_local = [lens[i] for i in shorts] + [plan["tokens"][rank][k] for k in range(len(longs))]
    table, pool, nblk = _paged_tables(tok_local, page, torch.Generator().manual_seed(60 + rank))
    lat = torch.zeros(max(pool, 1), page, dl, dtype=torch.int8, device=dev)
    sc = torch.ones(max(pool, 1), page, dtype=torch.float32, device=dev)
    rope = torch.zeros(max(pool, 1), page, dr, dtype=torch.bfloat16, device=dev)
    for j, i in enumerate(shorts):
        _fill_pages(lat, sc, rope, table[j, :nblk[j]], _latent_rows(lens[i], 5000 + i, dev), page)
    for k, i in enumerate(longs):
        j = len(shorts) + k
        if tok_local[j] > 0:
            _fill_pages(lat, sc, rope, table[j, :nblk[j]], _latent_rows(tok_local[j], 5000 + i + 1000 * (rank + 1), dev), page)
    ns, nl = len(shorts), len(longs)
    table_d = table.to(dev)
    lens_d = torch.tensor(tok_local if tok_local else [0], dtype=torch.int32, device=dev)
    ids_s = torch.tensor(shorts, dtype=torch.long, device=dev)
    ids_l = torch.tensor(longs, dtype=torch.long, device=dev)
    qn_s, qr_s = qn_all[ids_s].contiguous(), qr_all[ids_s].contiguous()
    qn_l, qr_l = qn_all[ids_l].contiguous(), qr_all[ids_l].contiguous()
    tab_s, len_s = table_d[:ns].contiguous(), lens_d[:ns].contiguous()
    tab_l, len_l = table_d[ns:ns + nl].contiguous(), lens_d[ns:ns + nl].contiguous()

    def whole():                                       # sequences owned whole: one ordinary call
        if ns == 0:
            return None
        return fa3.flash_attn_mla_with_kvcache(qn_s, qr_s, lat, sc, rope, len_s, tab_s, softmax_scale=scale,
                                               return_softmax_lse=True)

    buf = sh.PartialBuffer(nl * hq, dl, dev, world) if nl else None
    ex = sh.PeerExchange(nl * hq, dl, dev) if (nl and world > 1) else None

    def cut_partials_only():
        ext3.mla_decode(qn_l, qr_l, lat, sc, rope, tab_l, len_l, scale, 0, partials=(buf.o, buf.lse))

    def cut_nccl():
        return sh.sharded_mla_decode(qn_l, qr_l, lat, sc, rope, tab_l, len_l, scale, buffer=buf)

    def cut_peer():
        return sh.sharded_mla_decode(qn_l, qr_l, lat, sc, rope, tab_l, len_l, scale, exchange=ex)

    own0, own1 = rank * nl // world, (rank + 1) * nl // world          # cut sequences whose result THIS rank keeps

    def cut_peer_own_rows():
        po, pl = ex.partials()
        ext3.mla_decode(qn_l, qr_l, lat, sc, rope, tab_l, len_l, scale, 0, partials=(po, pl))
        return ex.combine(torch.bfloat16, own0 * hq, own1 * hq)

    variants = {}
    if nl:
        variants = {"decode_only_ms": lambda: (whole(), cut_partials_only()),
                    "nccl_allgather_combine_ms": lambda: (whole(), cut_nccl()),
                    "peer_exchange_combine_ms": lambda: (whole(), cut_peer()),
                    "peer_exchange_own_rows_ms": lambda: (whole(), cut_peer_own_rows())}
    else:
        variants = {"decode_only_ms": whole}
    times = {}
    for name, fn in variants.items():
        dd.barrier()
        times[name] = dd.max([_time_calls(fn, iters)])[0]
    kern = capi.last_kernel() if not nl else "mla_int8_tcgen05_pair + combine"
    # ---- parity -----------------------------------------------------------------------------------------------------
    checks, same = [], None

    def oracle_rows(seq, rows):
        lat_h, sc_h, rope_h = (r.cpu() for r in rows)
        L = lat_h.shape[0]
        n = (L + page - 1) // page
        pad = n * page - L
        li = torch.cat((lat_h, torch.zeros(pad, dl, dtype=torch.int8))).reshape(n, page, dl)
        si = torch.cat((sc_h, torch.ones(pad))).reshape(n, page)
        ri = torch.cat((rope_h, torch.zeros(pad, dr, dtype=torch.bfloat16))).reshape(n, page, dr)
        t1 = torch.arange(n, dtype=torch.int32).unsqueeze(0)
        return orc.mla_decode(qn_all[seq:seq + 1].cpu(), qr_all[seq:seq + 1].cpu(), li, si, ri, t1, [L], scale)

    def flat(name, got, ref, tol):
        err = orc.max_abs_err(got, ref)
        return {"name": name, "err": err, "two_x_golden": 0.0, "floor": tol, "tol": tol, "binding": "floor", "ok": bool(err <= tol)}

    if ns:
        o_s, l_s = whole()
        j = min(range(ns), key=lambda x: lens[shorts[x]])
        r_o, r_l = oracle_rows(shorts[j], _latent_rows(lens[shorts[j]], 5000 + shorts[j], dev))
        checks += [flat("out (whole sequence)", out_cpu(o_s[j:j + 1]), r_o, 2 ** -7), parity.check_lse(l_s[j:j + 1].cpu(), r_l)]
    if nl:
        o_n, l_n = cut_nccl()
        if ex is not None:
            o_p, l_p = cut_peer()
            o_own, _ = cut_peer_own_rows()
            ex.check()
            same = bool(torch.equal(o_n, o_p)) and bool(torch.equal(o_own, o_n[own0:own1].reshape(-1, dl)))
        # every rank checks a different cut sequence (the shortest ones): all its ranges are regenerated from the seeds
        order = sorted(range(nl), key=lambda x: lens[longs[x]])
        k = order[rank % nl]
        i = longs[k]
        parts = [_latent_rows(plan["tokens"][r][k], 5000 + i + 1000 * (r + 1), dev) for r in range(world) if plan["tokens"][r][k] > 0]
        rows = tuple(torch.cat([p[x] for p in parts]) for x in range(3))
        r_o, r_l = oracle_rows(i, rows)
        checks += [flat(f"out (sequence of {lens[i]} keys cut over {world} ranks)", out_cpu(o_n[k:k + 1]), r_o, 2 ** -7),
                   parity.check_lse(l_n[k:k + 1].cpu(), r_l)]
    par = _worst(checks)
    if same is not None:
        par["nccl_and_peer_kernel_identical"] = same
        par["ok"] = par["ok"] and same
    if ex is not None:
        ex.close()
    tokens = int(sum(lens))
    bytes_ = tokens * (dl + dr * 2 + 4) + b * hq * (dl + dr) * 2 + b * hq * dl * 2 + sum((n + page - 1) // page for n in lens) * 4
    flops = 2.0 * tokens * hq * (dl + dr + dl)
    peaks = measured_peaks()
    key = "nccl_allgather_combine_ms" if nl else "decode_only_ms"
    ms = times[key]
    gbs = bytes_ / (ms * 1e-3) / 1e9
    res = {"workload": "config5: int8 latent decode B64 Sq1 Hq128 Hkv1 (512 int8 + 64 bf16) page256 L~U[4096,131072]",
           "partition": (f"{b - nl} sequences of at most {LONG_THRESHOLD} keys dealt to the ranks whole, {nl} longer ones cut "
                         f"into {world} page ranges each; partial (O, LSE) of the cut ones exchanged" if world > 1 else
                         "one rank holds every sequence whole"),
           "ms": ms, "timed": key, "value": gbs, "unit": "GB/s", "algorithmic_bytes": bytes_, "kernel": kern,
           "frac_of_measured_hbm": gbs / (world * peaks["hbm_gbs"]), "frac_of_nominal_8000": gbs / (world * 8000.0),
           "tflops": flops / (ms * 1e-3) / 1e12, "tensor_time_bound_ms": flops / (world * peaks["bf16_tflops"] * 1e12) * 1e3,
           "hbm_time_bound_ms": bytes_ / (world * peaks["hbm_gbs"] * 1e9) * 1e3, "parity": par}
    res["roofline_frac"] = max(res["tensor_time_bound_ms"], res["hbm_time_bound_ms"]) / ms
    sharded = None
    if nl:
        rows = nl * hq
        sharded = dict(times)
        sharded.update({"what": f"{nl} sequences of more than {LONG_THRESHOLD} keys cut over {world} ranks, {b - nl} shorter ones whole; "
                                "max over ranks of (whole-sequence call + cut-sequence call + exchange + combine)",
                        "identical_results": same, "partial_rows": rows, "exchange_bytes_per_rank": rows * (dl + 1) * 4,
                        "exchange_cost_us": {"nccl": 1e3 * (times["nccl_allgather_combine_ms"] - times["decode_only_ms"]),
                                             "peer_kernel": 1e3 * (times["peer_exchange_combine_ms"] - times["decode_only_ms"]),
                                             "peer_kernel_own_rows": 1e3 * (times["peer_exchange_own_rows_ms"] - times["decode_only_ms"])},
                        "own_rows": "every rank combines only the cut sequences whose result it keeps (1/N of the rows): "
                                    "the all-gather variants leave every result on every rank"})
    return res, sharded


def out_cpu(t):
    return t.detach().cpu()


# ---------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="the K-step timed region is run this many times; the median is reported")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-decode", action="store_true", help="skip configurations 3, 4 and 5")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg")
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--e2e-kv-heads", type=int, default=0,
                    help="KV heads per chunk of the end-to-end leg's host pipeline (0 = a whole batch entry, contiguous copies)")
    ap.add_argument("--profile-case", default=None, choices=["fwd", "bwd", "decode", "mla", "fwd256", "decode4", "decode4s"],
                    help="run two calls of one kernel on a small case (for a profiler capture) and exit")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return 0
    if args.profile_case:
        profile_case(args.profile_case)
        return 0
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # several ranks on one host: keep each rank (and the pinned buffers it allocates) on its GPU's NUMA node
    old_affinity = bind_to_gpu_numa_node(local) if world > 1 else None
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) // (1 if old_affinity else world)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    import fa_b200_capi as capi
    from flash_attn_npu import flash_attn_npu as ext
    dd = Dist(rank, world, dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    c2 = config2_leg(args, dd, ext, capi, sampler)
    if rank == 0:
        sampler.stop()
    rep = replicated_leg(args, dd, ext) if world > 1 else None
    e2e = None
    if not args.no_e2e:
        e2e = e2e_leg(args, dd, c2["sets"], c2["groups"])
    c2.pop("sets")
    torch.cuda.empty_cache()
    c3 = c4 = c5 = sharded = None
    if not args.no_decode:
        c3 = config3_leg(dd)
        torch.cuda.empty_cache()
        c4 = config4_leg(dd)
        torch.cuda.empty_cache()
        c5, sharded = config5_leg(dd)
        torch.cuda.empty_cache()
    legs = {"config2": c2["parity"], "config3": c3 and c3["parity"], "config4": c4 and c4["parity"], "config5": c5 and c5["parity"]}
    mine_ok = all(p["ok"] for p in legs.values() if p)
    if not mine_ok:
        print(f"rank {rank}: parity check failed: " + json.dumps({k: v for k, v in legs.items() if v and not v["ok"]}), file=sys.stderr)
    all_ok = dd.all_ok(mine_ok)
    per_config_ok = {k: (dd.all_ok(v["ok"]) if v else None) for k, v in legs.items()}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0 if all_ok else 3
    if old_affinity:
        os.sched_setaffinity(0, old_affinity)
    peaks = measured_peaks()
    ms, fwd_ms, bwd_parts = c2["ms"], c2["fwd_ms"], c2["bwd_parts"]
    bwd_ms = sum(bwd_parts)
    share = 1.0 / world                                    # rank 0's part of the batch (equal item costs)
    parts = [("fwd:" + c2["fwd_kernel"], fwd_ms, FWD_FLOPS * share)]
    names = ["bwd:delta", "bwd:dk_dv", "bwd:dq"] if len(bwd_parts) == 3 else [f"bwd:{j}" for j in range(len(bwd_parts))]
    # flops per backward launch: the dK/dV pass computes S, dP, dV, dK (4 GEMMs); the dQ pass multiplies the dS tiles the
    # dK/dV pass left in the workspace (1 GEMM), or recomputes S and dP first (3) when the call takes that path
    unit = FWD_FLOPS * share / 2.0
    five = c2["bwd_kernel"].endswith("5gemm")
    flops_of = {"bwd:delta": 0.0, "bwd:dk_dv": 4 * unit, "bwd:dq": (1 if five else 3) * unit}
    for n, t in zip(names, bwd_parts):
        parts.append((n, t, flops_of.get(n, BWD_FLOPS * share)))
    dom = max(parts, key=lambda x: x[1])
    sustained = ms * args.steps * args.repeats > 1500.0
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    achieved = dom[2] / (dom[1] * 1e-3) / 1e12
    w_all = (c2["rep_win"][0][0], c2["rep_win"][-1][1])
    clocks = sampler.summary(*w_all)
    clocks["sm_mhz_per_repeat"] = [sampler.window(a, b_) for a, b_ in c2["rep_win"]]
    value = STEP_FLOPS / (ms * 1e-3) / 1e12
    line = {
        "metric": "fwd_bwd_attention_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "partition": (f"the 128 (batch entry x KV head) items dealt to {world} ranks, {128 // world} each, no collective"
                                 if world > 1 else "one rank runs the whole batch"),
                   "l2": (f"steps rotate over {c2['nsets']} independent input sets of {c2['in_bytes'] / 2**20:.0f} MiB each per rank, "
                          "so at least 2 x L2 of inputs pass between two uses of a set" if c2["nsets"] > 1 else
                          f"inputs larger than L2 ({c2['in_bytes'] / 2**20:.0f} MiB of q,k,v,dout per rank)"),
                   "seed": 1234, "timed_as": c2["timed_as"], "fwd_kernel": c2["fwd_kernel"], "bwd_kernel": c2["bwd_kernel"],
                   "repeats": args.repeats, "value_is": "median over the repeats of (max over ranks of a repeat's ms per step)"},
        "repeats_ms_per_step": c2["rep_ms"],
        "frac_of_n_x_measured_peak": value / (world * peak),
        "fwd_tflops": FWD_FLOPS * share / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": BWD_FLOPS * share / (bwd_ms * 1e-3) / 1e12,
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "kernels_ms": {n: t for n, t, _ in parts},
        "roofline": {"bound": "tensor", "kernel": dom[0], "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak,
                     "traffic": DKDV_TRAFFIC_B2 * (B / 2.0) * share if dom[0] == "bwd:dk_dv" else None,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of the same kernel on the "
                                       "B2 case, scaled by the batch entries x heads one launch covers",
                     "peak_source": peaks["_source"] + (" sustained" if sustained else " burst") + " cuBLAS bf16",
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "per_rank": "rank 0's launches", "flops_counted": "executed by that launch (dK/dV pass: 4 GEMMs; dQ pass: 1 GEMM over the stored dS "
                                                                        "tiles, so the backward executes the algorithm's 5)" if five else
                                                        "executed by that launch (this call recomputes S and dP in the dQ pass: 7 GEMMs for 5)",
                     "fwd_frac": FWD_FLOPS * share / (fwd_ms * 1e-3) / 1e12 / peak,
                     "bwd_frac_algorithmic": BWD_FLOPS * share / (bwd_ms * 1e-3) / 1e12 / peak},
        "gpu_launches": c2["launches_per_step"] * args.steps * args.repeats,
        "clocks": clocks,
        "parity_at_n": {k: ("ok" if v else "FAILED") for k, v in per_config_ok.items() if v is not None},
        "parity_detail_rank0": {k: v for k, v in legs.items() if v},
    }
    if e2e is not None:
        line["e2e"] = {"value": STEP_FLOPS / (e2e["median_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"] * world, "d2h_bytes_per_step": e2e["d2h"] * world,
                       "ms_per_step": e2e["median_ms"], "min_ms_per_step": e2e["min_ms"], "copy_floor_ms": e2e["copy_floor_ms"],
                       "over_copy_floor": e2e["median_ms"] / e2e["copy_floor_ms"], "steps": e2e["steps"],
                       "same_as_device_resident_run": e2e["same_as_device_resident_run"],
                       "how": "pinned host operands of the rank's items, one batch entry a chunk, contiguous copies, three streams; "
                              "median over the steps, max over ranks"}
    if rep is not None:
        line["replicated"] = rep
    if c3 is not None:
        line["varlen_fwd"] = c3
    if c4 is not None:
        line["paged_decode"] = c4
    if c5 is not None:
        line["mla_decode"] = c5
    if sharded is not None:
        line["kv_sharded_decode"] = sharded
    if not args.no_cpu and world == 1:
        v_cpu, dt, cores, sample = cpu_oracle_sample(H, 2)      # 10-30 s of host work
        line["cpu_baseline"] = {"value": v_cpu, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                                "seconds": dt}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0 if all_ok else 3


def profile_case(name):
    """Two calls of one kernel family on a case small enough for a full profiler capture (a few hundred MB on the
    device, inputs still larger than L2 where the kernel is memory-bound)."""
    import fa_b200_capi as capi
    import flash_attn_npu as fa
    import flash_attn_npu_3 as fa3
    from flash_attn_npu import flash_attn_npu as ext
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    if name in ("fwd", "bwd", "fwd256"):
        b, s, h, d = (2, 4096, 32, 128) if name != "fwd256" else (2, 4096, 16, 256)
        q, k, v, do = (torch.randn(b, s, h, d, device=dev).bfloat16() for _ in range(4))
        for _ in range(2):
            out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, d ** -0.5, True, -1, -1, 0.0, False, None)
            if name == "bwd":
                ext.bwd(do, q, k, v, out, lse, None, None, None, None, 0.0, d ** -0.5, True, -1, -1, 0.0, False, None, None)
    else:
        page = 256
        # decode4: 4 new tokens under a query group of 6 (24 stacked rows a KV head; the group cannot be stacked into
        # the tcgen05 tiles) on the decode kernel's 17-64-row form; decode4s: a group of 8 (32 stacked rows) on the
        # tcgen05 forward with the group in the tile rows and the keys split over CTAs
        b = 16
        lo, hi = (1024, 32769) if name in ("decode", "decode4", "decode4s") else (4096, 65537)
        lens = torch.randint(lo, hi, (b,), generator=g, dtype=torch.int32)
        table, pool, _ = _paged_tables((lens + 1).tolist(), page, g)
        lens_d, table_d = lens.to(dev), table.to(dev)
        if name in ("decode", "decode4", "decode4s"):
            hq, hkv, d = (32, 8, 128) if name == "decode" else ((48, 8, 128) if name == "decode4" else (64, 8, 128))
            sq = 1 if name == "decode" else 4
            kc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
            vc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
            q = torch.randn(b, sq, hq, d, device=dev, dtype=torch.bfloat16)
            print("cached tokens", int(lens.sum()), "algorithmic bytes", int(lens.sum()) * hkv * d * 4)
            for _ in range(2):
                fa.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens_d, block_table=table_d, causal=True)
        else:
            hq, dl, dr = 128, 512, 64
            lat = torch.randint(-127, 128, (pool, page, dl), device=dev, dtype=torch.int8)
            scales = torch.rand(pool, page, device=dev, dtype=torch.float32) * 0.02 + 0.001
            rope = torch.randn(pool, page, dr, device=dev, dtype=torch.bfloat16)
            qn = torch.randn(b, 1, hq, dl, device=dev, dtype=torch.bfloat16)
            qr = torch.randn(b, 1, hq, dr, device=dev, dtype=torch.bfloat16)
            print("cached tokens", int(lens.sum()), "algorithmic bytes", int(lens.sum()) * (dl + 2 * dr + 4))
            for _ in range(2):
                fa3.flash_attn_mla_with_kvcache(qn, qr, lat, scales, rope, lens_d, table_d)
    torch.cuda.synchronize()
    print("profile case", name, "kernel", capi.last_kernel(), "error flag", capi.lib.fa_debug_get(2))


if __name__ == "__main__":
    sys.exit(main())
