"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Workload ("stack64_p32768_b128x16"): the 64-layer attention stack of the
Qwen3-32B forward over a shared prefix of 32768 tokens resident in paged f16 KV
plus 128 branches x 16 packed suffix tokens (2048 query tokens), Q/K/V per layer
seeded bf16 N(0,1) (seed = layer index). One step = all 64 layers: fused
QK-RMSNorm + RoPE + KV write of the suffix tokens, then shared-prefix +
own-suffix attention. With N GPUs the KV heads are sharded (8/N KV heads and
their 64/N query heads per rank) and the per-head outputs are all-gathered
after every layer (copy-engine copies into peer-mapped buffers plus flags,
overlapped with the next layer; --gather nccl keeps the NCCL baseline).

value      suffix tokens per second through the 64-layer stack, inputs resident
           in HBM, device-timed (CUDA events on the launching stream), max over
           ranks.
e2e        the same through the host-buffer C-ABI entry: per layer, q/k/v come
           from pinned host memory and the output goes back to pinned host
           memory, copies (and at N > 1 the exchange) inside the timed region.
parity_check  after the timed region: rows of the last layer against the CPU
           oracle (at N > 1: every rank's gathered buffer); the run fails when
           it does.
roofline   the tensor-core attention kernel: algorithmic FLOPs per launch
           (4*128 per query-head row and visible key) / its mean device time,
           against the measured bf16 peak of MEASURED_PEAKS.json.
cpu_baseline  the CPU oracle (OpenMP, all host threads) on a bounded sample of
           the same workload.
Synthetic data throughout; there is no dataset for this path.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, HKV, D, L = 64, 8, 128, 64
PREFIX, BRANCHES, SUFFIX = 32768, 128, 16
TOKENS = BRANCHES * SUFFIX
WORKLOAD = "stack64_p32768_b128x16"
METRIC = "attn_suffix_tokens_per_s"
UNIT = "tokens/s"
# visible (query-head row, key) pairs per layer * 4*D FLOPs
PAIRS_PER_HEAD = TOKENS * PREFIX + BRANCHES * (SUFFIX * (SUFFIX + 1) // 2)
FLOPS_PER_LAYER = 4 * D * H * PAIRS_PER_HEAD
FLOPS_PER_STEP = FLOPS_PER_LAYER * L
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch at N = 1, from an
# ncu capture of `--case stack_layer_p32768_b128x16` (207.4 MB read + 54.0 MB written;
# algorithmic bytes 218 MB). A constant, not re-measured per run; at N > 1 the per-rank
# share (1/N of the KV heads) is reported and marked as scaled.
ATTENTION_DRAM_BYTES_PER_LAUNCH = 261.3e6


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"],
                    tflops_sustained=p["bf16_tflops_sustained"], source="measured")
    except Exception:
        return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0,
                    source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU during a timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=float(np.median(sm)) if sm else None,
                    sm_max_mhz=float(max(mx)) if mx else None,
                    samples=len(sm), reasons=sorted(reasons))


def shard_inputs(torch, layer, rank, n_gpus, device):
    """Seeded bf16 N(0,1) q/k/v of one layer, sliced to this rank's heads."""
    g = torch.Generator(device="cpu").manual_seed(layer)
    q = torch.randn(TOKENS, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(TOKENS, HKV, D, generator=g).to(torch.bfloat16)
    v = torch.randn(TOKENS, HKV, D, generator=g).to(torch.bfloat16)
    from sera_c_b200 import sharding
    return sharding.slice_heads(q, k, v, rank, n_gpus)


def bind_to_gpu_cpus(torch, device):
    """Multi-rank runs: keep this process (and so its pinned host buffers, by
    first touch) on the CPUs NVML lists as local to its GPU. Eight ranks that
    copy from host memory of the wrong socket share one inter-socket link.
    Returns the number of CPUs kept, or None when NVML gives no answer."""
    try:
        import pynvml
        pynvml.nvmlInit()
        pr = torch.cuda.get_device_properties(device)
        bus = "%08X:%02X:%02X.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, m in enumerate(words) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def run_ours(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = args.gpus
    if world != n_gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run"
                         % (n_gpus, world))
    if HKV % n_gpus:
        raise SystemExit("KV-head sharding needs --gpus in {1,2,4,8}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = bind_to_gpu_cpus(torch, device) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    entry.build()
    pkg = entry.load_package()
    from sera_c_b200 import sharding
    hq, hk = H // n_gpus, HKV // n_gpus
    n_prefix_pages = PREFIX // 16
    num_pages = n_prefix_pages + BRANCHES + 8

    rt = pkg.Runtime(num_layers=L, n_heads=hq, n_kv_heads=hk, max_positions=PREFIX + 64,
                     max_tokens=TOKENS, num_pages=num_pages, device=local)
    rt.enable_timing(4 * L * (args.steps + args.warmup) + 64)
    # resident prefix: seeded f16 N(0,1) in a randomly permuted page table
    perm = np.random.default_rng(1).permutation(num_pages).astype(np.uint32)
    rt.alloc_pages(num_pages)
    rt.free_pages(perm[n_prefix_pages:])
    prefix = pkg.Prefix(rt, PREFIX, pages=perm[:n_prefix_pages])
    kp, vp = rt.pool()
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    for l in range(L):
        kp[l].normal_(generator=gen)
        vp[l].normal_(generator=gen)
    torch.cuda.synchronize()
    prefix.set_resident(PREFIX)
    prefix.seal()
    bset = pkg.BranchSet(prefix, BRANCHES, SUFFIX)
    handles = [bset.acquire() for _ in range(BRANCHES)]
    plan = pkg.PackPlan(prefix, bset, [(h, SUFFIX) for h in handles])

    # per-layer inputs: pinned host copies (e2e leg) and device copies (value leg)
    hq_, hk_, hv_, dq_, dk_, dv_ = [], [], [], [], [], []
    for l in range(L):
        q, k, v = shard_inputs(torch, l, rank, n_gpus, device)
        hq_.append(q.pin_memory()); hk_.append(k.pin_memory()); hv_.append(v.pin_memory())
        dq_.append(hq_[-1].to(device)); dk_.append(hk_[-1].to(device)); dv_.append(hv_[-1].to(device))
    out_local = [torch.zeros(TOKENS, hq, D, dtype=torch.bfloat16, device=device) for _ in range(2)]
    out_full = [torch.zeros(n_gpus, TOKENS, hq, D, dtype=torch.bfloat16, device=device)
                for _ in range(2)] if world > 1 else None
    out_host = torch.zeros(TOKENS, hq, D, dtype=torch.bfloat16).pin_memory()
    stream = rt.torch_stream()

    fused = world > 1 and args.gather == "copy"
    GD = max(2, args.gather_depth)
    pg = (sharding.PeerGather(TOKENS, hq, D, torch.bfloat16, device, depth=GD)
          if fused else None)

    def step_device():
        if fused:
            # each layer writes this rank's slot of its gathered buffer; copy
            # engines push the slot to the other ranks on a side stream and
            # publish flags; a buffer is reused GD layers later, only after every
            # rank's rows of the layer it held have arrived here (device-side
            # flag wait, no collective): with GD buffers a rank may run GD - 1
            # layers ahead of the slowest one. Sequence numbers are
            # step-relative; the device-side counter advanced at the end makes
            # every step (or graph replay) publish fresh ones
            for l in range(L):
                if l >= GD:
                    rt.wait_gathered(pg.peers(l), l - GD + 1)
                plan.attention_layer_gathered(l, dq_[l], dk_[l], dv_[l], pg.peers(l), l + 1)
            for l in range(max(0, L - GD), L):
                rt.wait_gathered(pg.peers(l), l + 1)
            rt.gather_advance(L)
            return
        works = [None, None]
        for l in range(L):
            b = l & 1
            if works[b] is not None:
                works[b].wait()          # out_local[b] is free again (stream wait)
            plan.attention_layer(l, dq_[l], dk_[l], dv_[l], out_local[b])
            if world > 1 and args.gather == "nccl":
                works[b] = sharding.all_gather_heads(out_local[b], out_full[b], async_op=True)
        for w in works:
            if w is not None:
                w.wait()

    def step_host():
        if fused:
            # the whole step as a host caller sees it: host buffers in, the
            # exchange between the ranks, this rank's rows back to the host
            for l in range(L):
                if l >= GD:
                    rt.wait_gathered(pg.peers(l), l - GD + 1)
                plan.attention_layer_gathered_host(l, hq_[l], hk_[l], hv_[l], pg.peers(l),
                                                   l + 1, out_host)
            for l in range(max(0, L - GD), L):
                rt.wait_gathered(pg.peers(l), l + 1)
            rt.gather_advance(L)
            return
        for l in range(L):
            plan.attention_layer_host(l, hq_[l], hk_[l], hv_[l], out_host)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, drain=None):
        with torch.cuda.stream(stream):
            barrier()     # ranks enter together: the device-side gather waits are bounded (~1 s)
            for _ in range(warmup):
                fn()
            barrier()
            rt.phase_times()                      # rewind the per-kernel events
            launches0 = rt.stats().kernel_launches
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            if drain:
                drain()          # copy-out streams: the last result must be on the host
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            phases = rt.phase_times()
            launches = rt.stats().kernel_launches - launches0
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        n = torch.tensor([float(launches)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(n, op=dist.ReduceOp.SUM)
        return float(t.item()), phases, int(n.item())

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    use_graph = args.graph == "on" or (args.graph == "auto" and fused)
    if use_graph and world > 1 and args.gather == "nccl":
        raise SystemExit("--graph on records this library's calls only: use --gather copy|none")
    if use_graph:
        # the 64-layer step recorded once and replayed as one graph launch;
        # per-kernel times then come from a short eager pass after the timed region
        with torch.cuda.stream(stream):
            barrier()
            for _ in range(2):
                step_device()
            barrier()
            rt.graph_begin()
            step_device()
            graph = rt.graph_end()
        ms, _, launches = timed(graph.launch, args.steps, args.warmup)
        clocks = sampler.stop() if sampler else None
        _, phases, _ = timed(step_device, args.steps, 1)
        graph.close()
    else:
        ms, phases, launches = timed(step_device, args.steps, args.warmup)
        clocks = sampler.stop() if sampler else None
    ms_e2e, _, _ = timed(step_host, args.steps, args.warmup, drain=rt.synchronize)
    e2e_steps = args.steps
    rt.synchronize()
    status = rt.stats().device_status
    parity = parity_check(torch, dist, pkg, rt, plan, pg, kp, vp, perm[:n_prefix_pages],
                          dq_[L - 1], dk_[L - 1], dv_[L - 1], rank, world, device, stream)
    if world > 1:
        flag = torch.tensor([1.0 if parity["ok"] else 0.0], dtype=torch.float64, device=device)
        worst = torch.tensor([parity["max_normalised"]], dtype=torch.float64, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        parity["ok"] = bool(flag.item() > 0.5)
        parity["max_normalised"] = float(worst.item())

    result = None
    if rank == 0:
        peaks = measured_peaks()
        ms_per_step = ms / args.steps
        value = TOKENS / (ms_per_step * 1e-3)
        attn_ms, attn_n = phases["attention"]
        per_launch_ms = attn_ms / max(attn_n, 1)
        flops_per_launch = FLOPS_PER_LAYER / n_gpus
        achieved = flops_per_launch / (per_launch_ms * 1e-3) / 1e12
        peak = peaks["tflops_sustained"]
        e2e_ms_per_step = ms_e2e / e2e_steps
        qkv_bytes = L * TOKENS * (H + 2 * HKV) * D * 2
        out_bytes = L * TOKENS * H * D * 2
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 operands, fp32 accumulate (bf16 in/out, f16 KV)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": L, "prefix_tokens": PREFIX,
                       "branches": BRANCHES, "suffix_tokens_per_branch": SUFFIX,
                       "heads": "%d/%d x %d" % (H, HKV, D), "kv": "paged f16, page 16, permuted table",
                       "sharding": "kv_heads/%d + all-gather per layer (%s)" % (
                           n_gpus, args.gather if n_gpus > 1 else "single GPU"),
                       "l2": "inputs larger than L2 (8.6 GB of KV per step)",
                       "host_cpus_bound_to_gpu": numa},
            "tflops": FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12,
            "e2e": {"value": TOKENS / (e2e_ms_per_step * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": qkv_bytes, "d2h_bytes_per_step": out_bytes,
                    "ms_per_step": e2e_ms_per_step},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"kernel": "attention_tc_kernel", "bound": "tensor",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "traffic": ATTENTION_DRAM_BYTES_PER_LAUNCH / n_gpus,
                         "traffic_unit": "bytes per launch: one ncu capture at N = 1"
                                         + (", scaled by 1/N (not re-measured)" if n_gpus > 1 else ""),
                         "peak_source": "%s bf16 sustained" % peaks["source"],
                         "ms_per_launch": per_launch_ms, "launches": attn_n,
                         "flops_per_launch": flops_per_launch},
            "kernel_ms_per_step": {k: v[0] / args.steps for k, v in phases.items()},
            "exposed_exchange_ms_per_step": phases["gather_wait"][0] / args.steps,
            "parity_check": parity,
            "launch_mode": ("one CUDA graph per step; per-kernel times from an eager pass "
                            "of the same step after the timed region") if use_graph
                           else "eager; per-kernel times from the timed region",
            "device_status": status,
        }
    for o in (plan, bset, prefix):
        o.close()
    rt.close()
    del kp, vp
    torch.cuda.empty_cache()
    if rank == 0:
        if n_gpus == 1 and not args.no_extra:
            result["extra"] = run_extras(pkg, torch, device)
        if n_gpus == 1 and not args.no_cpu:
            result["cpu_baseline"] = cpu_baseline(target_s=args.cpu_seconds)
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit("parity_check failed: %s" % json.dumps(parity))


def parity_check(torch, dist, pkg, rt, plan, pg, kp, vp, prefix_pages, q, k, v, rank,
                 world, device, stream):
    """Outside the timed region: the last layer once more, a handful of its rows
    against the CPU oracle (ref math: src/q3_forward.cu:418-525). At N > 1 every
    rank compares ALL ranks' rows as they arrived in its gathered buffer with
    the oracle rows computed by their owners, so the exchange is checked too.
    Error measure: |got - oracle| less half a bf16 ulp of the oracle value
    (output rounding), absolute and normalised by max |oracle|; both <= 2e-3."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import q3_oracle as oracle
    layer = L - 1
    toks = [0, 15, 16, 31, TOKENS // 2 + 5, TOKENS - 17, TOKENS - 1]
    hq, hk = q.shape[1], k.shape[1]
    with torch.cuda.stream(stream):
        torch.cuda.synchronize()
        if pg is not None:
            dist.barrier()
            plan.attention_layer_gathered(layer, q, k, v, pg.peers(0), 1)
            rt.wait_gathered(pg.peers(0), 1)
            rt.gather_advance(1)
            rt.synchronize()
            dist.barrier()
            got = pg.bufs[0][:, toks].float().cpu().numpy()          # [world, n, hq, D]
        else:
            out = torch.zeros(TOKENS, hq, D, dtype=torch.bfloat16, device=device)
            plan.attention_layer(layer, q, k, v, out)
            rt.synchronize()
            got = out[toks].float().cpu().numpy()[None]
    idx = torch.from_numpy(prefix_pages.astype(np.int64)).to(device)
    kpre = np.ascontiguousarray(kp[layer][:, idx].permute(1, 2, 0, 3).reshape(PREFIX, hk, D)
                                .float().cpu().numpy())
    vpre = np.ascontiguousarray(vp[layer][:, idx].permute(1, 2, 0, 3).reshape(PREFIX, hk, D)
                                .float().cpu().numpy())
    ones = np.ones(D, np.float32)
    pos = (PREFIX + np.tile(np.arange(SUFFIX), BRANCHES)).astype(np.uint32)
    qn = oracle.rms_norm(q.float().cpu().numpy(), ones, 1e-6)
    kn = oracle.rms_norm(k.float().cpu().numpy(), ones, 1e-6)
    qn, kn = oracle.rope(qn, kn, 0, pos, oracle.inv_freq(1e6, D))
    vn = v.float().cpu().numpy()
    scale = np.float32(1 / np.sqrt(D))
    ref = np.zeros((len(toks), hq, D), np.float32)
    for i, t in enumerate(toks):
        b, lp = t // SUFFIX, t % SUFFIX
        keys = np.concatenate([kpre, kn[b * SUFFIX:b * SUFFIX + lp + 1]])
        vals = np.concatenate([vpre, vn[b * SUFFIX:b * SUFFIX + lp + 1]])
        ref[i] = oracle.attention(np.ascontiguousarray(qn[t:t + 1]), keys, vals, PREFIX + lp,
                                  PREFIX + lp + 1, scale)[0]
    if world > 1 and pg is not None:
        mine = torch.from_numpy(ref).to(device)
        allref = torch.zeros((world,) + ref.shape, dtype=torch.float32, device=device)
        dist.all_gather_into_tensor(allref.view(-1), mine.view(-1))
        ref_all = allref.cpu().numpy()
    else:
        ref_all = ref[None]
    r64 = ref_all.astype(np.float64)
    e = np.maximum(np.abs(got.astype(np.float64) - r64) - np.abs(r64) * 2.0 ** -8, 0.0)
    max_abs, norm = float(e.max()), float(e.max() / np.abs(r64).max())
    ok = bool(np.isfinite(got).all() and max_abs <= 2e-3 and norm <= 2e-3)
    return {"layer": layer, "rows": int(got.shape[0] * got.shape[1] * got.shape[2]),
            "tokens": toks, "ranks_checked": int(got.shape[0]), "max_abs": max_abs,
            "max_normalised": norm, "tolerance": 2e-3,
            "against": "CPU oracle of the reference kernels, same bf16/f16 inputs", "ok": ok}


def _time_calls(torch, rt, fn, reps, warmup=3):
    stream = rt.torch_stream()
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        rt.phase_times()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, rt.phase_times()


def case_prefill(pkg, torch, device, T=4096, reps=20):
    """Causal GQA prefill of T tokens, one layer (fused norm+rope+KV write, then
    attention over the pages just written)."""
    peaks = measured_peaks()
    g = torch.Generator(device=device).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=device).to(torch.bfloat16)
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=HKV, max_positions=T,
                     max_tokens=T, num_pages=T // 16 + 4, device=device.index)
    rt.enable_timing(16 * reps + 64)
    prefix = pkg.Prefix(rt, T)
    q, k, v = rnd(T, H, D), rnd(T, HKV, D), rnd(T, HKV, D)
    out = torch.zeros(T, H, D, dtype=torch.bfloat16, device=device)
    ms, ph = _time_calls(torch, rt, lambda: prefix.prefill_layer(0, q, k, v, out), reps)
    flops = 4 * D * H * (T * (T + 1) // 2)
    k_ms = ph["attention"][0] / max(ph["attention"][1], 1)
    w_ms = ph["kvwrite"][0] / max(ph["kvwrite"][1], 1)
    res = {"tokens": T, "ms": ms, "tflops": flops / ms / 1e9, "tokens_per_s": T / ms * 1e3,
           "attention_kernel_ms": k_ms, "attention_kernel_tflops": flops / k_ms / 1e9,
           "frac_of_bf16_burst_peak": flops / k_ms / 1e9 / peaks["tflops_burst"],
           "kvwrite_ms": w_ms, "kvwrite_algorithmic_bytes": T * (H + 2 * HKV) * D * 2 * 2,
           "kvwrite_gbs": T * (H + 2 * HKV) * D * 2 * 2 / 1e6 / w_ms,
           "kvwrite_frac_of_hbm_peak": T * (H + 2 * HKV) * D * 2 * 2 / 1e6 / w_ms / peaks["hbm_gbs"]}
    prefix.close()
    rt.close()
    return res


def case_cascade(pkg, torch, device, P=8192, B=64, n=24, reps=20, n_kv_heads=HKV,
                 permute=False):
    """Shared-prefix + packed-suffix attention, one layer, prefix resident; pages
    in the pool's allocation order, or (`permute`) in a random order."""
    peaks = measured_peaks()
    g = torch.Generator(device=device).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=device).to(torch.bfloat16)
    S = B * n
    ppb = (n + 15) // 16
    rt = pkg.Runtime(num_layers=1, n_heads=8 * n_kv_heads, n_kv_heads=n_kv_heads, max_positions=P + n + 8,
                     max_tokens=S, num_pages=P // 16 + ppb * B + 4, device=device.index)
    rt.enable_timing(16 * reps + 64)
    if permute:
        num_pages = P // 16 + ppb * B + 4
        perm = np.random.default_rng(1).permutation(num_pages).astype(np.uint32)
        rt.alloc_pages(num_pages)
        rt.free_pages(perm[P // 16:])
        prefix = pkg.Prefix(rt, P, pages=perm[:P // 16])
    else:
        prefix = pkg.Prefix(rt, P)
    kp, vp = rt.pool()
    kp.normal_(generator=g)
    vp.normal_(generator=g)
    prefix.set_resident(P)
    prefix.seal()
    bset = pkg.BranchSet(prefix, B, n)
    plan = pkg.PackPlan(prefix, bset, [(bset.acquire(), n) for _ in range(B)])
    q, k, v = rnd(S, 8 * n_kv_heads, D), rnd(S, n_kv_heads, D), rnd(S, n_kv_heads, D)
    out = torch.zeros(S, 8 * n_kv_heads, D, dtype=torch.bfloat16, device=device)
    ms, ph = _time_calls(torch, rt, lambda: plan.attention_layer(0, q, k, v, out), reps)
    flops = 4 * D * 8 * n_kv_heads * (S * P + B * n * (n + 1) // 2)
    k_ms = ph["attention"][0] / max(ph["attention"][1], 1)
    res = {"prefix": P, "branches": B, "suffix": n, "kv_heads": n_kv_heads,
           "pages": "random order" if permute else "allocation order", "ms": ms,
           "suffix_tokens_per_s": S / ms * 1e3, "tflops": flops / ms / 1e9,
           "attention_kernel_ms": k_ms, "attention_kernel_tflops": flops / k_ms / 1e9,
           "frac_of_bf16_burst_peak": flops / k_ms / 1e9 / peaks["tflops_burst"],
           "kvwrite_ms": ph["kvwrite"][0] / max(ph["kvwrite"][1], 1)}
    for o in (plan, bset, prefix):
        o.close()
    rt.close()
    return res


def case_decode(pkg, torch, device, n_seqs=256, reps=20):
    """Paged decode: n_seqs sequences, ctx uniform in [1024, 16384]
    (numpy default_rng(1)), randomly permuted pages, one query token each."""
    peaks = measured_peaks()
    g = torch.Generator(device=device).manual_seed(0)
    ctx = np.random.default_rng(1).integers(1024, 16385, 256).astype(np.uint32)[:n_seqs]
    n_pages = (ctx + 15) // 16
    total = int(n_pages.sum())
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=HKV, max_positions=16400,
                     max_tokens=n_seqs, num_pages=total + 4, device=device.index)
    rt.enable_timing(16 * reps + 64)
    kp, vp = rt.pool()
    kp.normal_(generator=g)
    vp.normal_(generator=g)
    perm = np.random.default_rng(2).permutation(total).astype(np.uint32)
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.uint32)
    plan = pkg.DecodePlan(rt, ctx, indptr, perm)
    q = torch.randn(n_seqs, H, D, generator=g, device=device).to(torch.bfloat16)
    out = torch.zeros(n_seqs, H, D, dtype=torch.bfloat16, device=device)
    ms, ph = _time_calls(torch, rt, lambda: plan.attention_layer(0, q, None, None, out), reps)
    kv_bytes = int(ctx.sum()) * 2 * HKV * D * 2
    alg_bytes = kv_bytes + 2 * n_seqs * H * D * 2 + 4 * (total + n_seqs + 1)
    res = {"sequences": n_seqs, "ms": ms, "sum_ctx": int(ctx.sum()),
           "algorithmic_bytes": alg_bytes, "gbs": alg_bytes / ms / 1e6,
           "frac_of_hbm_peak": alg_bytes / ms / 1e6 / peaks["hbm_gbs"],
           "seq_tokens_per_s": n_seqs / ms * 1e3,
           "decode_kernels_ms": ph["decode"][0] / reps}
    plan.close()
    rt.close()
    return res


CASES = {
    "prefill_4096": lambda pkg, torch, dev, reps: case_prefill(pkg, torch, dev, 4096, reps),
    "cascade_p8192_b64x24": lambda pkg, torch, dev, reps: case_cascade(pkg, torch, dev, 8192, 64, 24, reps),
    "stack_layer_p32768_b128x16": lambda pkg, torch, dev, reps: case_cascade(pkg, torch, dev, PREFIX, BRANCHES, SUFFIX, reps),
    "stack_layer_1kvhead": lambda pkg, torch, dev, reps: case_cascade(pkg, torch, dev, PREFIX, BRANCHES, SUFFIX, reps, 1),
    "stack_layer_permuted_pages": lambda pkg, torch, dev, reps: case_cascade(pkg, torch, dev, PREFIX, BRANCHES, SUFFIX, reps, permute=True),
    "decode_256seq": lambda pkg, torch, dev, reps: case_decode(pkg, torch, dev, 256, reps),
    "decode_64seq": lambda pkg, torch, dev, reps: case_decode(pkg, torch, dev, 64, reps),
}


def random_q4k_weight(torch, n_features, k, device, seed=0):
    """Synthetic resident Q4_K weight [n_features][k/256 blocks of 144 bytes]:
    random scales, mins and quants; d, dmin (the two f16 at the head of each
    block) drawn so that the weights are O(0.1)."""
    g = torch.Generator(device=device).manual_seed(seed)
    nb = n_features * (k // 256)
    w = torch.randint(0, 256, (nb, 144), generator=g, device=device, dtype=torch.uint8)
    d = (torch.rand(nb, generator=g, device=device) * 0.004 + 0.0004).to(torch.float16)
    dmin = (torch.rand(nb, generator=g, device=device) * 0.002).to(torch.float16)
    w[:, 0:2] = d.view(torch.uint8).view(nb, 2)
    w[:, 2:4] = dmin.view(torch.uint8).view(nb, 2)
    return w.view(n_features, -1)


def random_q6k_weight(torch, n_features, k, device, seed=0):
    """Synthetic Q6_K weight [n_features][k/256 blocks of 210 bytes]; d (the f16
    at the end of each block) drawn so that the weights are O(0.1)."""
    g = torch.Generator(device=device).manual_seed(seed)
    nb = n_features * (k // 256)
    w = torch.randint(0, 256, (nb, 210), generator=g, device=device, dtype=torch.uint8)
    d = (torch.rand(nb, generator=g, device=device) * 0.002 + 0.0002).to(torch.float16)
    w[:, 208:210] = d.view(torch.uint8).view(nb, 2)
    return w.view(n_features, -1)


def case_q4k_linear(pkg, torch, device, M=2048, N=(H + 2 * HKV) * D, K=5120, reps=20,
                    tiled=True, qtype=12):
    """Resident Q4_K projection next to the attention path (q/k/v projection of
    Qwen3-32B as one [10240, 5120] weight, or the output projection
    [5120, 8192]): f16 activations in, bf16 out, one kernel. Six weight copies
    are cycled so that every call reads its weight from HBM, not L2."""
    from sera_c_b200 import q4_linear
    peaks = measured_peaks()
    lin = q4_linear.Q4Linear(device.index, M, N, K)
    geo = q4_linear.bind_geometry(K, N, qtype=qtype)
    copies = max(2, int(200e6 // geo.weight_bytes) + 1)
    make = random_q4k_weight if qtype == 12 else random_q6k_weight
    ws = [make(torch, N, K, device, seed=i) for i in range(copies)]
    if tiled:   # one-time re-layout (q3_cuda_q4k_linear_pack), not timed
        packed = [lin.pack(geo, w) for w in ws]
        ws, geo = [t for t, _ in packed], packed[0][1]
    g = torch.Generator(device=device).manual_seed(1)
    x = torch.randn(M, K, generator=g, device=device).to(torch.float16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    for i in range(3):
        lin.linear_f16(geo, ws[i % copies], x, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        lin.linear_f16(geo, ws[i % copies], x, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    flops = 2.0 * M * N * K
    tf = flops / (ms * 1e-3) / 1e12
    return {"ms": ms, "tflops": tf, "frac_of_burst_peak": tf / peaks["tflops_burst"],
            "tokens_per_s": M / (ms * 1e-3), "M": M, "N": N, "K": K,
            "weight_bytes": int(geo.weight_bytes), "status": lin.status(),
            "weight_layout": "tiled (packed once)" if tiled else "GGUF row-major",
            "algorithmic_bytes": int(geo.weight_bytes + M * K * 2 + M * N * 2),
            "gbs": (geo.weight_bytes + M * K * 2 + M * N * 2) / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": (geo.weight_bytes + M * K * 2 + M * N * 2) / (ms * 1e-3) / 1e9
                                / peaks["hbm_gbs"]}


def case_qkv_fused(pkg, torch, device, T=4096, K=5120, reps=20):
    """Prefill of T tokens of one layer starting from the layer's input rows:
    the three Q4_K projections + norm/RoPE/KV-write kernel + attention (the
    sequence of the reference's run_layer with this library's kernels) against
    the projection whose epilogue does the norm, the rotation and the page write
    (q3_prefix_prefill_layer_projected: two launches, no q/k/v tensors). Weights
    in the tiled order, three weight sets cycled so that they come from HBM."""
    from sera_c_b200 import q4_linear
    lin = q4_linear.Q4Linear(device.index, T, H * D, K)
    sets = []
    for i in range(3):
        ws, geos = [], []
        for j, n in enumerate((H, HKV, HKV)):
            geo = q4_linear.bind_geometry(K, n * D)
            t, tgeo = lin.pack(geo, random_q4k_weight(torch, n * D, K, device, seed=10 * i + j))
            ws.append(t)
            geos.append(tgeo)
        sets.append((ws, geos, pkg.qkv_weights(ws[0], ws[1], ws[2], K, geos[0].qtype)))
    g = torch.Generator(device=device).manual_seed(1)
    x = (torch.randn(T, K, generator=g, device=device) * 0.02).to(torch.float16)
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=HKV, max_positions=T,
                     max_tokens=T, num_pages=T // 16 + 4, device=device.index)
    rt.enable_timing(32 * reps + 64)
    prefix = pkg.Prefix(rt, T)
    q = torch.empty(T, H, D, dtype=torch.bfloat16, device=device)
    k = torch.empty(T, HKV, D, dtype=torch.bfloat16, device=device)
    v = torch.empty(T, HKV, D, dtype=torch.bfloat16, device=device)
    out_a = torch.zeros(T, H, D, dtype=torch.bfloat16, device=device)
    out_b = torch.zeros(T, H, D, dtype=torch.bfloat16, device=device)
    stream = rt.stream_ptr
    it = [0]

    def unfused():
        ws, geos, _ = sets[it[0] % 3]
        it[0] += 1
        for w, geo, o in zip(ws, geos, (q, k, v)):
            lin.linear_f16(geo, w, x, out=o.view(T, -1), stream=stream)
        prefix.prefill_layer(0, q, k, v, out_a)

    def fused():
        _, _, W = sets[it[0] % 3]
        it[0] += 1
        prefix.prefill_layer_projected(0, W, x, out_b)

    ms_u, _ = _time_calls(torch, rt, unfused, reps)
    ms_f, ph = _time_calls(torch, rt, fused, reps)
    it[0] = 0
    unfused()
    it[0] = 0
    fused()
    torch.cuda.synchronize()
    diff = float((out_a.float() - out_b.float()).abs().max())
    flops = 2.0 * T * (H + 2 * HKV) * D * K + 4 * D * H * (T * (T + 1) // 2)
    res = {"tokens": T, "hidden": K, "unfused_ms": ms_u, "fused_ms": ms_f,
           "speedup": ms_u / ms_f, "fused_tflops": flops / ms_f / 1e9,
           "fused_projection_kernel_ms": ph["kvwrite"][0] / max(ph["kvwrite"][1], 1),
           "attention_kernel_ms": ph["attention"][0] / max(ph["attention"][1], 1),
           "max_abs_diff_between_the_two_paths": diff,
           "launches_per_layer": {"unfused": 5, "fused": 2},
           "status": lin.status()}
    prefix.close()
    rt.close()
    return res


CASES["qkv_fused_prefill_4096"] = lambda pkg, torch, dev, reps: case_qkv_fused(pkg, torch, dev, 4096, reps=reps)
CASES["qkv_fused_prefill_2048"] = lambda pkg, torch, dev, reps: case_qkv_fused(pkg, torch, dev, 2048, reps=reps)


CASES.update({
    "q4k_qkv_2048": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 2048, reps=reps),
    "q4k_qkv_4096": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 4096, reps=reps),
    "q4k_oproj_2048": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 2048, 5120, 8192, reps),
    "q4k_qkv_16": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 16, reps=reps,
                                                               tiled=False),
    "q4k_qkv_1": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 1, reps=reps,
                                                              tiled=False),
    "q4k_qkv_16_tile_kernel": lambda pkg, torch, dev, reps: case_q4k_linear(pkg, torch, dev, 16,
                                                                           reps=reps),
    "q6k_v_4096": lambda pkg, torch, dev, reps: case_q4k_linear(
        pkg, torch, dev, 4096, 1024, 5120, reps, qtype=14),
    "q4k_qkv_4096_gguf_layout": lambda pkg, torch, dev, reps: case_q4k_linear(
        pkg, torch, dev, 4096, reps=reps, tiled=False),
})


def case_q4k_mmvq(pkg, torch, device, M=1, N=(H + 2 * HKV) * D, K=5120, reps=50):
    """The fp32 reference surface (q3_cuda_q4k_linear) on a decode-size batch: the
    reference's 8-bit-activation arithmetic, bound by the weight bytes."""
    from sera_c_b200 import q4_linear
    peaks = measured_peaks()
    lin = q4_linear.Q4Linear(device.index, max(M, 16), N, K)
    geo = q4_linear.bind_geometry(K, N)
    copies = max(2, int(200e6 // geo.weight_bytes) + 1)
    ws = [random_q4k_weight(torch, N, K, device, seed=i) for i in range(copies)]
    g = torch.Generator(device=device).manual_seed(1)
    x = torch.randn(M, K, generator=g, device=device)
    out = torch.empty(M, N, dtype=torch.float32, device=device)
    for i in range(3):
        lin.linear_f32(geo, ws[i % copies], x, out=out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        lin.linear_f32(geo, ws[i % copies], x, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    nbytes = geo.weight_bytes + M * K * 4 + M * N * 4
    return {"ms": ms, "M": M, "N": N, "K": K, "algorithmic_bytes": int(nbytes),
            "gbs": nbytes / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "path": lin_path(M), "launches_per_call": 2}


def lin_path(m):
    from sera_c_b200 import q4_linear
    return q4_linear._L().q3_cuda_q4k_linear_path_for_batch(m).decode()


CASES.update({
    "q4k_qkv_fp32_1": lambda pkg, torch, dev, reps: case_q4k_mmvq(pkg, torch, dev, 1, reps=reps),
    "q4k_qkv_fp32_8": lambda pkg, torch, dev, reps: case_q4k_mmvq(pkg, torch, dev, 8, reps=reps),
})


def case_fp32_surface_cascade(pkg, torch, device, P=8192, B=64, n=24, reps=10):
    """The reference's own fp32 entry points (rms_norm, rope_positions,
    attention_segmented; fp32 contiguous slabs, descriptors in host memory as
    its caller keeps them) served by this library after
    q3_cuda_attention_native_init: the sequence the reference's
    run_layer_packed executes, timed as the same-box reference kernels are."""
    import ctypes
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _gpu_harness as harness
    L = harness.fp32_surface(pkg.lib_path())
    lib = pkg.lib()
    err = ctypes.create_string_buffer(256)
    f32 = torch.float32
    S = B * n
    g = torch.Generator(device=device).manual_seed(0)
    qs = torch.randn(S, H, D, generator=g, dtype=f32, device=device)
    ks = torch.randn(S, HKV, D, generator=g, dtype=f32, device=device)
    pk = torch.randn(1, P, HKV, D, generator=g, dtype=f32, device=device)
    pv = torch.randn(1, P, HKV, D, generator=g, dtype=f32, device=device)
    sk = torch.randn(B, 1, n, HKV * D, generator=g, dtype=f32, device=device)
    sv = torch.randn(B, 1, n, HKV * D, generator=g, dtype=f32, device=device)
    tb = np.repeat(np.arange(B, dtype=np.uint32), n)
    tl = np.tile(np.arange(n, dtype=np.uint32), B)
    pos = torch.from_numpy((tl + P).astype(np.int32)).to(device)
    ones = torch.ones(D, dtype=f32, device=device)
    ifr = torch.tensor((1.0 / (1e6 ** (np.arange(D // 2) * 2.0 / D))).astype(np.float32),
                       device=device)
    o = torch.zeros_like(qs)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    scale = float(1.0 / np.sqrt(D))

    def ck(ok):
        if not ok:
            raise RuntimeError(err.value.decode())

    def run():
        ck(L.q3_cuda_rms_norm(p(qs), p(ones), S * H, D, 1e-6, p(qs), None, err, 256))
        ck(L.q3_cuda_rms_norm(p(ks), p(ones), S * HKV, D, 1e-6, p(ks), None, err, 256))
        ck(L.q3_cuda_rope_positions(p(qs), p(ks), S, H, HKV, D, p(pos), p(ifr), None, err, 256))
        ck(L.q3_cuda_attention_segmented(p(qs), p(pk), p(pv), P, P, p(sk), p(sv), n, 1, 0,
                                         ctypes.c_void_p(tb.ctypes.data),
                                         ctypes.c_void_p(tl.ctypes.data), S, H, HKV, D, scale,
                                         p(o), None, err, 256))

    pkg._call(lib.q3_cuda_attention_native_init, device.index, S, P + B * 32, H, HKV)
    try:
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        path = lib.q3_cuda_attention_last_path().decode()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        pkg._call(lib.q3_cuda_attention_native_synchronize, device.index)
        ms = e0.elapsed_time(e1) / reps
    finally:
        lib.q3_cuda_attention_native_shutdown(device.index)
    pairs = S * P + B * n * (n + 1) // 2
    return {"ms": ms, "tflops": 4 * D * H * pairs / (ms * 1e-3) / 1e12,
            "suffix_tokens_per_s": S / (ms * 1e-3), "path": path,
            "note": "fp32 norm + rope + attention_segmented per call; the attention call "
                    "converts q and the K/V slabs to f16 pages, builds its schedule on the "
                    "host and runs the tensor-core kernel"}


CASES["fp32_surface_cascade_p8192_b64x24"] = \
    lambda pkg, torch, dev, reps: case_fp32_surface_cascade(pkg, torch, dev, reps=reps)


def run_extras(pkg, torch, device):
    """The other single-GPU configurations of the benchmark definition, one
    layer each: causal prefill (TFLOP/s), 8192-prefix cascade (tokens/s),
    paged decode (GB/s). Device-timed, inputs resident."""
    return {name: CASES[name](pkg, torch, device, 20)
            for name in ("prefill_4096", "cascade_p8192_b64x24", "decode_256seq",
                         "q4k_qkv_2048", "fp32_surface_cascade_p8192_b64x24")}


def run_case(args):
    """One small single-layer case on its own (used for profiler captures)."""
    import torch
    import __graft_entry__ as entry
    entry.build()
    pkg = entry.load_package()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    print(json.dumps({"case": args.case, **CASES[args.case](pkg, torch, device, args.reps)}))


def host_cores():
    """Host threads this process may use (its CPU affinity, else the core count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample(n_branches, threads=None):
    """One layer of the workload restricted to `n_branches` branches (16 tokens
    each, full 32768-token prefix) through the CPU oracle. Returns seconds.
    The thread count is always set explicitly: a launcher that exports
    OMP_NUM_THREADS=1 (torch.distributed.run does) must not turn the CPU arm
    into a one-core run."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import q3_oracle as oracle
    oracle.set_threads(threads or host_cores())
    rng = np.random.default_rng(0)
    S = n_branches * SUFFIX
    q = rng.standard_normal((S, H, D), dtype=np.float32)
    k = rng.standard_normal((S, HKV, D), dtype=np.float32)
    v = rng.standard_normal((S, HKV, D), dtype=np.float32)
    pk = rng.standard_normal((1, PREFIX, HKV, D), dtype=np.float32)
    pv = rng.standard_normal((1, PREFIX, HKV, D), dtype=np.float32)
    tb = np.repeat(np.arange(n_branches, dtype=np.uint32), SUFFIX)
    tl = np.tile(np.arange(SUFFIX, dtype=np.uint32), n_branches)
    pos = (PREFIX + tl).astype(np.uint32)
    ones = np.ones(D, np.float32)
    ifreq = oracle.inv_freq(1e6, D)
    t0 = time.perf_counter()
    qn = oracle.rms_norm(q, ones, 1e-6)
    kn = oracle.rms_norm(k, ones, 1e-6)
    qn, kn = oracle.rope(qn, kn, 0, pos, ifreq)
    sk = np.zeros((n_branches, 1, SUFFIX, HKV * D), np.float32)
    sv = np.zeros_like(sk)
    oracle.kv_scatter(sk, sv, kn, v, tb, tl, SUFFIX, 1, 0)
    oracle.attention_segmented(qn, pk, pv, PREFIX, PREFIX, sk, sv, SUFFIX, 1, 0, tb, tl,
                               HKV, np.float32(1 / np.sqrt(D)))
    return time.perf_counter() - t0, oracle.threads()


def cpu_baseline(target_s=15.0):
    t1, threads = cpu_sample(1)
    nb = int(max(1, min(BRANCHES, target_s / max(t1, 1e-3))))
    t = t1 if nb == 1 else cpu_sample(nb)[0]
    tokens = nb * SUFFIX
    return {"value": tokens / (t * L), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "1 of %d layers, %d of %d branches x %d tokens over the full %d-token "
                      "prefix, fp32 contiguous KV, %.1f s; scaled by the layer count"
                      % (L, nb, BRANCHES, SUFFIX, PREFIX, t)}


def reference_gpu_kernels():
    """The reference's own CUDA kernels (compiled unchanged for sm_100a into
    oracle/_ref/libq3ref.so) timed on this box in their own layout (fp32
    contiguous slabs): prefill at 4096 tokens, the 8192-token-prefix cascade
    case and one layer of the 64-layer workload. Reported beside the CPU number
    of the reference arm; none of this repository's kernels run here."""
    import ctypes
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _gpu_harness as harness
    path = os.path.join(ROOT, "oracle", "_ref", "libq3ref.so")
    if not torch.cuda.is_available() or not os.path.exists(path):
        return {"unavailable": "no GPU or oracle/_ref/libq3ref.so not built"}
    R = harness.fp32_surface(path)
    err = ctypes.create_string_buffer(256)
    f32 = torch.float32
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    scale = float(1.0 / np.sqrt(D))
    ifr = torch.tensor((1.0 / (1e6 ** (np.arange(D // 2) * 2.0 / D))).astype(np.float32),
                       device=dev)
    ones = torch.ones(D, dtype=f32, device=dev)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    def ck(ok):
        if not ok:
            raise RuntimeError(err.value.decode())

    def timeit(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    res = {}
    # prefill: rms_norm(q), rms_norm(k), rope, attention over the call's own rows
    T = 4096
    q = torch.randn(T, H, D, generator=g, dtype=f32, device=dev)
    k = torch.randn(T, HKV, D, generator=g, dtype=f32, device=dev)
    v = torch.randn(T, HKV, D, generator=g, dtype=f32, device=dev)
    out = torch.zeros_like(q)

    def prefill():
        ck(R.q3_cuda_rms_norm(p(q), p(ones), T * H, D, 1e-6, p(q), None, err, 256))
        ck(R.q3_cuda_rms_norm(p(k), p(ones), T * HKV, D, 1e-6, p(k), None, err, 256))
        ck(R.q3_cuda_rope(p(q), p(k), T, H, HKV, D, 0, p(ifr), None, err, 256))
        ck(R.q3_cuda_attention(p(q), p(k), p(v), T, H, HKV, D, 0, None, 0, scale, p(out),
                               None, err, 256))
    ms = timeit(prefill, 3)
    pairs = T * (T + 1) // 2
    res["prefill_4096"] = {"ms": ms, "tflops": 4 * D * H * pairs / (ms * 1e-3) / 1e12,
                           "tokens_per_s": T / (ms * 1e-3)}
    del q, k, v, out

    def cascade(P, B, n, reps):
        S = B * n
        qs = torch.randn(S, H, D, generator=g, dtype=f32, device=dev)
        ks = torch.randn(S, HKV, D, generator=g, dtype=f32, device=dev)
        pk = torch.randn(1, P, HKV, D, generator=g, dtype=f32, device=dev)
        pv = torch.randn(1, P, HKV, D, generator=g, dtype=f32, device=dev)
        sk = torch.randn(B, 1, n, HKV * D, generator=g, dtype=f32, device=dev)
        sv = torch.randn(B, 1, n, HKV * D, generator=g, dtype=f32, device=dev)
        tb = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(n)
        tl = torch.arange(n, dtype=torch.int32, device=dev).repeat(B)
        pos = (tl + P).to(torch.int32)
        o = torch.zeros_like(qs)

        def run():
            ck(R.q3_cuda_rms_norm(p(qs), p(ones), S * H, D, 1e-6, p(qs), None, err, 256))
            ck(R.q3_cuda_rms_norm(p(ks), p(ones), S * HKV, D, 1e-6, p(ks), None, err, 256))
            ck(R.q3_cuda_rope_positions(p(qs), p(ks), S, H, HKV, D, p(pos), p(ifr), None,
                                        err, 256))
            ck(R.q3_cuda_attention_segmented(p(qs), p(pk), p(pv), P, P, p(sk), p(sv), n, 1, 0,
                                             p(tb), p(tl), S, H, HKV, D, scale, p(o), None,
                                             err, 256))
        ms = timeit(run, reps)
        pairs = S * P + B * n * (n + 1) // 2
        return {"ms": ms, "tflops": 4 * D * H * pairs / (ms * 1e-3) / 1e12,
                "suffix_tokens_per_s": S / (ms * 1e-3)}
    res["cascade_p8192_b64x24"] = cascade(8192, 64, 24, 3)
    res["stack_layer_p32768_b128x16"] = cascade(PREFIX, BRANCHES, SUFFIX, 2)
    res["stack64_tokens_per_s_extrapolated"] = TOKENS / (
        res["stack_layer_p32768_b128x16"]["ms"] * 1e-3 * L)
    # the reference's Q4_K linear (Q8_1 activation quantisation + MMQ) on the q/k/v shape
    qpath = os.path.join(ROOT, "oracle", "_ref", "libq3q4ref.so")
    if os.path.exists(qpath):
        import __graft_entry__ as entry
        entry.load_package()
        from sera_c_b200 import _lib
        Q = _lib.bind_linear(ctypes.CDLL(qpath))
        M, N, K = 2048, (H + 2 * HKV) * D, 5120
        geo = _lib.LinearGeometry()
        ck(Q.q3_q4_linear_bind_geometry(12, K, N, ctypes.byref(geo), err, 256))
        ck(Q.q3_cuda_q4k_linear_init(0, M, N, K, err, 256))
        arena = torch.empty(max(int(Q.q3_cuda_q4k_linear_workspace_bytes()), 256),
                            dtype=torch.uint8, device=dev)
        ck(Q.q3_cuda_q4k_linear_set_workspace(arena.data_ptr(), arena.numel(), err, 256))
        w = random_q4k_weight(torch, N, K, dev)
        x = torch.randn(M, K, generator=g, dtype=f32, device=dev)
        o = torch.zeros(M, N, dtype=f32, device=dev)
        ms = timeit(lambda: ck(Q.q3_cuda_q4k_linear(ctypes.byref(geo), w.data_ptr(),
                                                    x.data_ptr(), M, o.data_ptr(), None, None,
                                                    err, 256)), 5)
        res["q4k_qkv_2048"] = {"ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12,
                               "tokens_per_s": M / (ms * 1e-3)}
    res["note"] = ("reference SIMT kernels, fp32 contiguous KV, norm + rope + attention per "
                   "call, scatter of the suffix rows not timed (file-static in the reference)")
    return res


def python_path_baseline():
    """The reference's Python path for this arithmetic: the HuggingFace Qwen3
    functions its oracle scripts execute (RMSNorm, rotary embedding,
    apply_rotary_pos_emb, repeat_kv) plus torch SDPA, on CPU in fp32 with all
    host threads (ref: tools/qwen3_q4_oracle.py:88-92,151-154). Configuration 1
    in full, prefill at 4096 tokens, the 8192-token-prefix cascade case, a
    32-sequence subset of the decode configuration and one layer of the stack
    with a reduced prefix; one repeat each after a small warm-up."""
    try:
        import torch
        from transformers.models.qwen3 import modeling_qwen3 as m
        from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
    except Exception as e:  # the third-party modules are not part of this repository
        return {"unavailable": "transformers/torch import failed: %s" % e}
    torch.set_num_threads(host_cores())
    cfg = Qwen3Config(hidden_size=H * D, num_attention_heads=H, num_key_value_heads=HKV,
                      head_dim=D, rope_theta=1e6, max_position_embeddings=1 << 17,
                      num_hidden_layers=1, intermediate_size=64, vocab_size=16)
    qn, kn, rot = m.Qwen3RMSNorm(D, eps=1e-6), m.Qwen3RMSNorm(D, eps=1e-6), m.Qwen3RotaryEmbedding(cfg)
    gen = torch.Generator().manual_seed(0)

    def run(P, B, n):
        """P resident-equivalent prefix tokens + B branches of n tokens; B == 0: causal prefill of P."""
        T = P + B * n
        q = torch.randn(1, T, H, D, generator=gen)
        k = torch.randn(1, T, HKV, D, generator=gen)
        v = torch.randn(1, T, HKV, D, generator=gen)
        pos = torch.cat([torch.arange(P)] + [torch.arange(P, P + n)] * B)[None]
        t0 = time.perf_counter()
        with torch.no_grad():
            rows = slice(0, T) if B == 0 else slice(P, T)   # cascade: only the suffix rows query
            qs = qn(q[:, rows]).transpose(1, 2)
            ks = kn(k).transpose(1, 2)
            vs = v.transpose(1, 2)
            cos, sin = rot(vs, pos)
            qs, _ = m.apply_rotary_pos_emb(qs, qs, cos[:, rows], sin[:, rows])
            ks, _ = m.apply_rotary_pos_emb(ks, ks, cos, sin)
            kk, vv = m.repeat_kv(ks, H // HKV), m.repeat_kv(vs, H // HKV)
            if B == 0:
                torch.nn.functional.scaled_dot_product_attention(qs, kk, vv, is_causal=True)
            else:
                S = B * n
                br = torch.arange(S) // n
                lp = torch.arange(S) % n
                mask = torch.zeros(S, T, dtype=torch.bool)
                mask[:, :P] = True
                mask[:, P:] = (br[:, None] == br[None, :]) & (lp[None, :] <= lp[:, None])
                torch.nn.functional.scaled_dot_product_attention(qs, kk, vv, attn_mask=mask)
        return time.perf_counter() - t0

    def decode(ctx_lens):
        """One query token per sequence over its own context (paged decode's arithmetic)."""
        t0 = time.perf_counter()
        with torch.no_grad():
            for c in ctx_lens:
                c = int(c)
                q = torch.randn(1, 1, H, D, generator=gen)
                k = torch.randn(1, c, HKV, D, generator=gen)
                v = torch.randn(1, c, HKV, D, generator=gen)
                qs = qn(q).transpose(1, 2)
                ks = kn(k).transpose(1, 2)
                cos, sin = rot(v, torch.arange(c)[None])
                qs, _ = m.apply_rotary_pos_emb(qs, qs, cos[:, -1:], sin[:, -1:])
                ks, _ = m.apply_rotary_pos_emb(ks, ks, cos, sin)
                kk, vv = m.repeat_kv(ks, H // HKV), m.repeat_kv(v.transpose(1, 2), H // HKV)
                torch.nn.functional.scaled_dot_product_attention(qs, kk, vv)
        return time.perf_counter() - t0

    res = {"cores": torch.get_num_threads()}
    # configuration 1 in full: 256-token prefix + 3 branches x 8 tokens
    run(64, 2, 4)
    t = run(256, 3, 8)
    res["config1_p256_b3x8"] = {"ms": t * 1e3, "suffix_tokens_per_s": 24 / t,
                                "note": "prefix rows are computed too (280 query rows)"}
    run(400, 0, 0)
    t = run(4096, 0, 0)
    res["prefill_4096"] = {"ms": t * 1e3, "tokens_per_s": 4096 / t,
                           "tflops": 4 * D * H * (4096 * 4097 // 2) / t / 1e12}
    run(800, 8, 24)
    t = run(8192, 64, 24)
    res["cascade_p8192_b64x24"] = {
        "ms": t * 1e3, "suffix_tokens_per_s": 1536 / t,
        "tflops": 4 * D * H * (1536 * 8192 + 64 * 300) / t / 1e12,
        "note": "includes norm + rope of the 8192 prefix keys, which the GPU path keeps resident"}
    # configuration 4 on a 32-sequence subset (the first 32 of the seeded context lengths;
    # random data generation is inside the time, about a tenth of it)
    ctx = np.random.default_rng(1).integers(1024, 16385, 256)[:32]
    decode(ctx[:2])
    t = decode(ctx)
    res["decode_32_of_256_sequences"] = {
        "ms": t * 1e3, "seq_tokens_per_s": 32 / t, "sum_ctx": int(ctx.sum()),
        "note": "32 of the 256 sequences, norm + rope of every context key included "
                "(the GPU path keeps them resident)"}
    # configuration 5: one layer, prefix reduced from 32768 to 4096 tokens, all 128 x 16
    # suffix tokens; scaled by 8 (attention work is linear in the prefix) and by 64 layers
    t = run(4096, BRANCHES, SUFFIX)
    res["stack_layer_p4096_of_32768_b128x16"] = {
        "ms": t * 1e3, "suffix_tokens_per_s": TOKENS / t,
        "stack64_tokens_per_s_extrapolated": TOKENS / (t * 8 * L),
        "note": "one of 64 layers, prefix 4096 of 32768 tokens; extrapolation = x8 for the "
                "prefix, x64 for the layers"}
    return res


def run_reference(args):
    """The reference arm: the path's CPU implementation (the oracle port of the
    reference kernels; the reference ships no CPU attention of its own) on all
    host threads. Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    times = []
    t1, threads = cpu_sample(1)
    # a step = a bounded sample sized to a few seconds
    nb = int(max(1, min(BRANCHES, 4.0 / max(t1, 1e-3))))
    for i in range(args.warmup + args.steps):
        t, _ = cpu_sample(nb)
        if i >= args.warmup:
            times.append(t)
    t = float(np.mean(times))
    tokens = nb * SUFFIX
    value = tokens / (t * L)
    # the same port on one thread (one branch of one layer), for the scalar figure
    t_single, _ = cpu_sample(1, threads=1)
    single = {"value": SUFFIX / (t_single * L), "unit": UNIT, "cores": 1, "kind": "port",
              "sample": "1 of %d layers, 1 of %d branches x %d tokens, %.1f s"
                        % (L, BRANCHES, SUFFIX, t_single)}
    sample = ("1 of %d layers, %d of %d branches x %d tokens over the full %d-token prefix "
              "per step; scaled by the layer count" % (L, nb, BRANCHES, SUFFIX, PREFIX))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 (double accumulation)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": L, "prefix_tokens": PREFIX,
                   "branches": BRANCHES, "suffix_tokens_per_branch": SUFFIX},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "cpu_baseline_single_thread": single,
        **({} if args.no_ref_gpu else {"reference_gpu_kernels": reference_gpu_kernels(),
                                       "python_path_cpu": python_path_baseline()})}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the single-layer prefill / cascade / decode lines")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="--impl reference: skip timing the reference's own CUDA kernels")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="record the 64-layer step once and replay it as one CUDA graph "
                         "(auto: at N > 1 with the copy-engine gather, where it measured "
                         "5.7 %% faster at 8 GPUs; off at N = 1, where it changes nothing and "
                         "per-kernel times then come from the timed region itself)")
    ap.add_argument("--gather", default="copy", choices=["copy", "nccl", "none"],
                    help="per-layer output all-gather at N > 1: 'copy' = copy-engine copies "
                         "of this rank's rows into the other ranks' buffers plus flags, on a "
                         "side stream (default), 'nccl' = all_gather_into_tensor overlapped on "
                         "a side stream, 'none' = skipped (diagnostic)")
    ap.add_argument("--gather-depth", type=int, default=3,
                    help="gathered buffers per rank at N > 1 (a rank may run depth - 1 layers "
                         "ahead of the slowest)")
    ap.add_argument("--case", choices=sorted(CASES), default=None,
                    help="run only this single-layer case (for profiler captures)")
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
