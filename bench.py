"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1 and per rank for N > 1, weak scaling): benchmark configuration 2,
flash_attn_func forward + backward in bf16, batch 4, seqlen 4096, 32 query heads,
32 KV heads, headdim 128, causal, softmax_scale 1/sqrt(128); q/k/v/dout i.i.d. N(0,1)
from a seed (synthetic).  One step = one forward + one backward over that batch.
The metric is fwd+bwd TFLOP/s with the standard FlashAttention accounting
(forward 4*B*H*S*S*D/2 under the causal mask, backward 2.5 x forward).

`--impl reference` times the CPU oracle (a port of the reference's Python goldens; the
reference's device code needs an Ascend toolchain) on a bounded sample of the same workload.
Prints one JSON line on rank 0.
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
for p in (ROOT, os.path.join(ROOT, "flash-attention-npu_b200")):
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


# DRAM bytes of one dK/dV launch at B2 S4096 H32 D128 causal from the committed ncu capture (271.1 MB read + 108.6 MB
# written); the traffic grows in proportion to the batch
DKDV_TRAFFIC_B2 = 379.7e6


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
    """Samples SM clock, power and throttle reasons through NVML in a thread while the timed region runs
    (a polling nvidia-smi process was seen to stall kernel launches for milliseconds)."""

    def __init__(self, index, period=0.02):
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

    def stop(self, t0, t1):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.stop_flag = True
        self.thread.join(timeout=1.0)
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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU oracle (port of the reference's torch goldens) on host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-decode", action="store_true", help="skip the paged-decode side measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-kv-heads", type=int, default=0,
                    help="KV heads per chunk of the end-to-end leg's host pipeline (0 = the pipeline's default)")
    ap.add_argument("--sharded-decode", action="store_true",
                    help="with 2 or more GPUs: also time the key-range sharded decode, NCCL all-gather + combine "
                         "against the one kernel that exchanges the partials over peer memory")
    ap.add_argument("--profile-case", default=None, choices=["fwd", "bwd", "decode", "mla"],
                    help="run two calls of one kernel on a small case (for a profiler capture) and exit")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.profile_case:
        profile_case(args.profile_case)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    import fa_b200_capi as capi
    import flash_attn_npu as fa
    from flash_attn_npu import flash_attn_npu as ext

    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randn(B, S, hh, D, generator=g).bfloat16().pin_memory() for hh in (H, HKV, HKV, H)]
    q, k, v, do = (t.to(dev) for t in host)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def step():
        out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
        ext.bwd(do, q, k, v, out, lse, dq, dk, dv, None, 0.0, SCALE, True, -1, -1, 0.0, False, None, None)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    fwd_kernel = None
    out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
    fwd_kernel = capi.last_kernel()
    ext.bwd(do, q, k, v, out, lse, dq, dk, dv, None, 0.0, SCALE, True, -1, -1, 0.0, False, None, None)
    bwd_kernel = capi.last_kernel()

    # ---- per-kernel durations: a few eager steps with events lent to the library (not the headline) --------
    nev = 8
    nb_steps = min(args.steps, 10)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(nev)] for _ in range(2 * nb_steps)]
    for row in evs:
        for e in row:
            e.record()
    torch.cuda.synchronize()
    arr_t = ctypes.c_void_p * nev
    arrays = [arr_t(*[e.cuda_event for e in row]) for row in evs]
    used = [0] * (2 * nb_steps)
    for i in range(nb_steps):
        capi.lib.fa_set_kernel_events(arrays[2 * i], nev)
        out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, SCALE, True, -1, -1, 0.0, False, None)
        used[2 * i] = capi.lib.fa_kernel_events_used()
        capi.lib.fa_set_kernel_events(arrays[2 * i + 1], nev)
        ext.bwd(do, q, k, v, out, lse, dq, dk, dv, None, 0.0, SCALE, True, -1, -1, 0.0, False, None, None)
        used[2 * i + 1] = capi.lib.fa_kernel_events_used()
    capi.lib.fa_set_kernel_events(None, 0)
    torch.cuda.synchronize()

    # ---- device-timed region: K steps replayed from a CUDA graph of one step (no host work between launches)
    timed_as = "cuda graph replay of one step"
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        graph.replay()
        torch.cuda.synchronize()
    except Exception as exc:  # fall back to eager launches
        graph = None
        timed_as = "eager launches (graph capture failed: %s)" % str(exc)[:80]
        torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0 = time.time()
    start.record()
    for i in range(args.steps):
        run_step()
    stop.record()
    barrier()
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms = start.elapsed_time(stop) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    # per-kernel durations (ms), averaged over the eager steps
    fwd_ms = statistics.mean(evs[2 * i][0].elapsed_time(evs[2 * i][used[2 * i] - 1]) for i in range(nb_steps))
    bwd_parts = []
    nb = used[1]
    for j in range(1, nb):
        bwd_parts.append(statistics.mean(evs[2 * i + 1][j - 1].elapsed_time(evs[2 * i + 1][j]) for i in range(nb_steps)))
    bwd_ms = sum(bwd_parts)
    launches = (used[0] - 1 + used[1] - 1) * args.steps

    # ---- end to end through the public API with host buffers ---------------------------------------------
    e2e_steps = max(2, min(args.steps, 5))
    hq, hk, hv, hdo = host
    out_h, gq_h, gk_h, gv_h = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (hq, hq, hk, hv))

    import fa_b200_host
    pipe = fa_b200_host.HostPipeline(dev, args.e2e_kv_heads)

    def e2e_step():
        # pinned host operands in, pinned host results out: chunks of one batch entry x a head group on three streams
        pipe.fwd_bwd(hq, hk, hv, hdo, out_h, gq_h, gk_h, gv_h, causal=True, softmax_scale=SCALE)

    e2e_step()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    h2d = sum(t.numel() * 2 for t in host)
    d2h = sum(t.numel() * 2 for t in (out_h, gq_h, gk_h, gv_h))

    sharded = None
    if world > 1 and args.sharded_decode:
        sharded = kv_sharded_decode_side_measurement(dev, rank, world)
    decode = varlen = mla = None
    if rank == 0 and not args.no_decode:
        # side measurements of the other single-GPU configurations; none may take the headline down
        try:
            decode = paged_decode_side_measurement(dev)
        except Exception as exc:
            decode = {"error": str(exc)[:200]}
        try:
            varlen = varlen_side_measurement(dev)
        except Exception as exc:
            varlen = {"error": str(exc)[:200]}
        try:
            mla = mla_side_measurement(dev)
        except Exception as exc:
            mla = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = measured_peaks()
    # dominant kernel = the longest single launch of the step
    parts = [("fwd:" + fwd_kernel, fwd_ms, FWD_FLOPS)]
    names = ["bwd:delta", "bwd:dk_dv", "bwd:dq"] if len(bwd_parts) == 3 else [f"bwd:{j}" for j in range(len(bwd_parts))]
    # flops per backward launch: dK/dV pass recomputes S and dP (2) and does dV, dK (2); dQ pass S, dP, dQ (3)
    unit = FWD_FLOPS / 2.0
    flops_of = {"bwd:delta": 0.0, "bwd:dk_dv": 4 * unit, "bwd:dq": 3 * unit}
    for n, t in zip(names, bwd_parts):
        parts.append((n, t, flops_of.get(n, BWD_FLOPS)))
    dom = max(parts, key=lambda x: x[1])
    sustained = ms * args.steps > 1500.0
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    achieved = dom[2] / (dom[1] * 1e-3) / 1e12
    line = {
        "metric": "fwd_bwd_attention_tflops", "value": STEP_FLOPS * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu": "one full batch per rank, no collective",
                   "l2": "inputs larger than L2 (q,k,v,dout 128 MiB each)", "seed": 1234, "timed_as": timed_as,
                   "fwd_kernel": fwd_kernel, "bwd_kernel": bwd_kernel},
        "fwd_tflops": FWD_FLOPS / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": BWD_FLOPS / (bwd_ms * 1e-3) / 1e12,
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "kernels_ms": {n: t for n, t, _ in parts},
        "roofline": {"bound": "tensor", "kernel": dom[0], "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": DKDV_TRAFFIC_B2 * (B / 2.0) if dom[0] == "bwd:dk_dv" else None,
                     "traffic_source": "ncu dram__bytes_read+write of the B2 case of the same kernel "
                                       "(profiles/bwd_sm100_kernels_B2_S4096_H32_D128_causal.md) scaled by batch",
                     "peak_source": peaks["_source"] + (" sustained" if sustained else " burst") + " cuBLAS bf16",
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "fwd_frac": FWD_FLOPS / (fwd_ms * 1e-3) / 1e12 / peak},
        "e2e": {"value": STEP_FLOPS * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if decode is not None:
        line["paged_decode"] = decode
    if varlen is not None:
        line["varlen_fwd"] = varlen
    if mla is not None:
        line["mla_decode"] = mla
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


def paged_decode_side_measurement(dev, iters=10):
    """Benchmark configuration 4 (paged decode, B128 Hq32 Hkv8 D128 page 256, lengths U[1024,32768], append +
    rotary) timed with CUDA events; reports achieved HBM GB/s over the algorithmic bytes (K and V rows read
    once, 4096 B per cached token and KV head set, plus q / out / table / appended rows)."""
    import flash_attn_npu as fa
    g = torch.Generator().manual_seed(4)
    b, hq, hkv, d, page = 128, 32, 8, 128, 256
    lens = torch.randint(1024, 32769, (b,), generator=g, dtype=torch.int32)
    nblk = (lens + 1 + page - 1) // page
    pool = int(nblk.sum())
    perm = torch.randperm(pool, generator=g).int()
    table = torch.zeros(b, int(nblk.max()), dtype=torch.int32)
    off = 0
    for i in range(b):
        n = int(nblk[i])
        table[i, :n] = perm[off:off + n]
        off += n
    kc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
    q = torch.randn(b, 1, hq, d, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(b, 1, hkv, d, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(b, 1, hkv, d, device=dev, dtype=torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(32800, dtype=torch.float32), inv)
    cos, sin = torch.cos(ang).bfloat16().to(dev), torch.sin(ang).bfloat16().to(dev)
    lens_d, table_d = lens.to(dev), table.to(dev)

    def call():
        return fa.flash_attn_with_kvcache(q, kc, vc, kn, vn, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens_d,
                                          block_table=table_d, causal=True, rotary_interleaved=False)

    for _ in range(3):
        call()
    import fa_b200_capi as capi
    kern = capi.last_kernel()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        call()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / iters
    tokens = int((lens + 1).sum())
    bytes_ = tokens * hkv * d * 2 * 2 + b * hq * d * 2 * 2 + table.numel() * 4 + b * hkv * d * 2 * 2
    peaks = measured_peaks()
    gbs = bytes_ / (ms * 1e-3) / 1e9
    return {"workload": "config4: paged decode bf16 B128 Sq1 Hq32 Hkv8 D128 page256 L~U[1024,32768], append+rotary",
            "ms": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": bytes_, "kernel": kern,
            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8000": gbs / 8000.0,
            "cache_gb": pool * page * hkv * d * 2 * 2 / 1e9}


def kv_sharded_decode_side_measurement(dev, rank, world, iters=20):
    """Long-context decode with the key range of every sequence cut over the ranks (B8 Hq32 Hkv8 D128 page 256,
    131072 keys a sequence; every rank holds only the cache blocks of its own range).  Times, max over ranks:
    the decode kernels alone (fp32 partials), the call with an NCCL all-gather of the partials + combine, and the
    call with the kernel that exchanges them over peer memory and combines."""
    import torch.distributed as dist
    import fa_b200_sharding as sh
    from flash_attn_npu import flash_attn_npu as ext
    g = torch.Generator().manual_seed(7)
    b, hq, hkv, d, page, length = 8, 32, 8, 128, 256, 131072
    lo, hi = sh.kv_shard_range(length, rank, world, page)
    own = (min(hi, length) - lo) // page
    table = torch.zeros(b, length // page, dtype=torch.int32)
    perm = torch.randperm(b * own, generator=g).int().view(b, own)
    table[:, lo // page:lo // page + own] = perm
    kc = torch.randn(b * own, page, hkv, d, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(b * own, page, hkv, d, device=dev, dtype=torch.bfloat16)
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().to(dev)
    lens = torch.full((b,), length, dtype=torch.int32, device=dev)
    table = table.to(dev)
    ex = sh.PeerExchange(b * hq, d, dev)
    po = torch.empty(b * hq, d, dtype=torch.float32, device=dev)
    pl = torch.empty(b * hq, dtype=torch.float32, device=dev)

    def partial_only():
        ext.kvcache_forward(q, kc, vc, None, None, lens, None, None, None, table, None, None, d ** -0.5, False, -1, -1,
                            0.0, False, 0, kv_range=(lo, hi), partials=(po, pl))

    def with_nccl():
        return sh.sharded_kvcache_decode(q, kc, vc, lens, table, d ** -0.5, length, page)

    def with_peers():
        return sh.sharded_kvcache_decode(q, kc, vc, lens, table, d ** -0.5, length, page, exchange=ex)

    a, _ = with_nccl()
    c, _ = with_peers()
    ex.check()
    same = bool(torch.equal(a, c))
    res = {}
    for name, fn in (("decode_only_ms", partial_only), ("nccl_allgather_combine_ms", with_nccl),
                     ("peer_exchange_combine_ms", with_peers)):
        dist.barrier()
        t = torch.tensor([_time_calls(fn, iters)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = t.item()
    ex.check()
    ex.close()
    bytes_ = b * own * page * hkv * d * 2 * 2
    res.update({"workload": f"decode bf16 B8 Sq1 Hq32 Hkv8 D128 page256 L131072, keys cut over {world} ranks",
                "identical_results": same, "cache_gb_per_rank": bytes_ / 1e9,
                "decode_gbs_per_rank": bytes_ / (res["decode_only_ms"] * 1e-3) / 1e9,
                "exchange_cost_us": {"nccl": 1e3 * (res["nccl_allgather_combine_ms"] - res["decode_only_ms"]),
                                     "peer_kernel": 1e3 * (res["peer_exchange_combine_ms"] - res["decode_only_ms"])}})
    return res


def profile_case(name):
    """Two calls of one kernel family on a case small enough for a full profiler capture (a few hundred MB on the
    device, inputs still larger than L2 where the kernel is memory-bound)."""
    import fa_b200_capi as capi
    import flash_attn_npu as fa
    import flash_attn_npu_3 as fa3
    from flash_attn_npu import flash_attn_npu as ext
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    if name in ("fwd", "bwd"):
        b, s, h, d = 2, 4096, 32, 128
        q, k, v, do = (torch.randn(b, s, h, d, device=dev).bfloat16() for _ in range(4))
        for _ in range(2):
            out, lse, _, _ = ext.fwd(q, k, v, None, None, 0.0, d ** -0.5, True, -1, -1, 0.0, False, None)
            if name == "bwd":
                ext.bwd(do, q, k, v, out, lse, None, None, None, None, 0.0, d ** -0.5, True, -1, -1, 0.0, False, None, None)
    else:
        page = 256
        b = 16
        lo, hi = (1024, 32769) if name == "decode" else (4096, 65537)
        lens = torch.randint(lo, hi, (b,), generator=g, dtype=torch.int32)
        nblk = (lens + page) // page
        pool = int(nblk.sum())
        perm = torch.randperm(pool, generator=g).int()
        table = torch.zeros(b, int(nblk.max()), dtype=torch.int32)
        off = 0
        for i in range(b):
            n = int(nblk[i])
            table[i, :n] = perm[off:off + n]
            off += n
        lens_d, table_d = lens.to(dev), table.to(dev)
        if name == "decode":
            hq, hkv, d = 32, 8, 128
            kc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
            vc = torch.randn(pool, page, hkv, d, device=dev, dtype=torch.bfloat16)
            q = torch.randn(b, 1, hq, d, device=dev, dtype=torch.bfloat16)
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


def varlen_side_measurement(dev, iters=10):
    """Benchmark configuration 3 (packed forward, 16 sequences with lengths U[256,8192], Hq32 Hkv8 D128,
    causal): forward TFLOP/s over the unmasked half of every sequence's score matrix."""
    import flash_attn_npu as fa
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(3)
    hq, hkv, d = 32, 8, 128
    lens = torch.randint(256, 8193, (16,), generator=g)
    cu = torch.zeros(17, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    total, mx = int(cu[-1]), int(lens.max())
    q = torch.randn(total, hq, d, device=dev, dtype=torch.bfloat16)
    k = torch.randn(total, hkv, d, device=dev, dtype=torch.bfloat16)
    v = torch.randn(total, hkv, d, device=dev, dtype=torch.bfloat16)
    cu_d = cu.to(dev)
    ms = _time_calls(lambda: fa.flash_attn_varlen_func(q, k, v, cu_d, cu_d, mx, mx, causal=True), iters)
    flops = float(sum(4.0 * hq * int(n) * int(n) * d / 2.0 for n in lens))
    peaks = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": "config3: flash_attn_varlen_func fwd bf16 16 seqs L~U[256,8192] Hq32 Hkv8 D128 causal",
            "ms": ms, "value": tf, "unit": "TFLOP/s", "flops": flops, "tokens": total, "kernel": capi.last_kernel(),
            "frac_of_measured_bf16": tf / peaks["bf16_tflops"], "frac_of_nominal_2250": tf / 2250.0}


def mla_side_measurement(dev, iters=10):
    """Benchmark configuration 5 (latent-attention decode, B64 Sq1 Hq128 against one latent head: 512 int8 +
    fp32 scale + 64 bf16 positional values per cached token, page 256, lengths U[4096,131072]): achieved HBM
    GB/s over 644 B per cached token plus q / out / table."""
    import flash_attn_npu_3 as fa3
    import fa_b200_capi as capi
    g = torch.Generator().manual_seed(5)
    b, hq, dl, dr, page = 64, 128, 512, 64, 256
    lens = torch.randint(4096, 131073, (b,), generator=g, dtype=torch.int32)
    nblk = (lens + page - 1) // page
    pool = int(nblk.sum())
    perm = torch.randperm(pool, generator=g).int()
    table = torch.zeros(b, int(nblk.max()), dtype=torch.int32)
    off = 0
    for i in range(b):
        n = int(nblk[i])
        table[i, :n] = perm[off:off + n]
        off += n
    lat = torch.randint(-127, 128, (pool, page, dl), device=dev, dtype=torch.int8)
    scales = torch.rand(pool, page, device=dev, dtype=torch.float32) * 0.02 + 0.001
    rope = torch.randn(pool, page, dr, device=dev, dtype=torch.bfloat16)
    qn = torch.randn(b, 1, hq, dl, device=dev, dtype=torch.bfloat16)
    qr = torch.randn(b, 1, hq, dr, device=dev, dtype=torch.bfloat16)
    lens_d, table_d = lens.to(dev), table.to(dev)
    ms = _time_calls(lambda: fa3.flash_attn_mla_with_kvcache(qn, qr, lat, scales, rope, lens_d, table_d), iters)
    tokens = int(lens.sum())
    bytes_ = tokens * (dl + dr * 2 + 4) + b * hq * (dl + dr) * 2 + b * hq * dl * 2 + table.numel() * 4
    flops = 2.0 * tokens * hq * (dl + dr + dl)
    peaks = measured_peaks()
    gbs = bytes_ / (ms * 1e-3) / 1e9
    return {"workload": "config5: int8 latent decode B64 Sq1 Hq128 Hkv1 (512 int8 + 64 bf16) page256 L~U[4096,131072]",
            "ms": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": bytes_, "kernel": capi.last_kernel(),
            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8000": gbs / 8000.0,
            "tflops": flops / (ms * 1e-3) / 1e12, "tensor_time_bound_ms": flops / (peaks["bf16_tflops"] * 1e12) * 1e3,
            "hbm_time_bound_ms": bytes_ / (peaks["hbm_gbs"] * 1e9) * 1e3}


if __name__ == "__main__":
    main()
