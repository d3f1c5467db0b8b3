#!/usr/bin/env python
"""Benchmark of the attention hot path: one JSON line on stdout (rank 0).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c5|c2|c4]

A "step" is one call of ``dot_product_attention`` over one batch of seeded
synthetic inputs.  The default workload is the configuration the headline
metric is quoted on: bf16 causal self-attention, E = 4096, nheads = 32
(d = 128), L = 4096, batch = 8 per GPU, scores discarded (x-only).  With N > 1
every rank runs the same per-GPU work on its own batch slice (weak scaling; the
(batch, head) units are independent, so no collective is on the data path).

* ``value``: whole-job TFLOP/s with inputs resident in HBM (CUDA events on the
  launching stream, max over ranks); FLOPs are algorithmic:
  2·(d+dv)·P·H·B with P = L(L+1)/2 for causal.
* ``e2e``: the same metric through the public API from pinned HOST buffers,
  H2D of q, k, v and D2H of x inside the timed region.
* ``roofline``: algorithmic FLOP/s of the fused kernel against the measured
  dense-bf16 peak of this pool (MEASURED_PEAKS.json).
* ``cpu_baseline``: the CPU restatement of the reference's operation sequence
  (the oracle), timed on this host's cores on a bounded sample.
``--impl reference`` times only that CPU path (NNlib.jl itself is Julia, which
is not installed here) with all host threads; a step there is one bounded
sample of the workload.

Beside the line's own numbers (default workload only, ``--no-extras`` skips them):
* ``strong_c5``: the long-context configuration (bf16 causal, L = 32768, 128
  (batch, head) units) with its units partitioned over the N ranks
  (``rank_rects``), per-rank time, aggregate TFLOP/s and, for N > 1, the time of
  all 128 units on rank 0 alone measured in the same run.
* ``sharded_driver`` (N > 1): the same 128 units through ``ShardedAttention`` —
  ONE process, one host thread per device, inputs in pinned host memory.
* ``host_copy_ceiling``: the end-to-end step's copies alone (same bytes, same
  two copy streams, no kernels) on all ranks at once: what the host side allows.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "attention TFLOP/s per B200 (bf16 causal, L=4096, d=128); % of dense TC peak"

WORKLOADS = {
    # name: dtype, E, H, Lq, Lkv, B(per GPU), causal, extras
    "c3": dict(desc="decoder causal self-attention (Llama-7B shape): bf16 E=4096 nheads=32 d=128 L=4096 batch=8, "
                    "mask=make_causal_mask(q), x only",
               dtype="bf16", E=4096, H=32, Lq=4096, Lkv=4096, B=8, causal=True),
    "c5": dict(desc="long-context causal: bf16 E=2048 nheads=16 d=128 L=32768 batch=8 (128 units)",
               dtype="bf16", E=2048, H=16, Lq=32768, Lkv=32768, B=8, causal=True),
    "c2": dict(desc="encoder self-attention (BERT-base shape): bf16 E=768 nheads=12 d=64 L=512 batch=32, "
                    "key-padding mask, scores returned",
               dtype="bf16", E=768, H=12, Lq=512, Lkv=512, B=32, causal=False, padmask=True, alpha=True),
    "c3f32": dict(desc="config 3's shape in Float32 on the TF32 tensor-core path (set_math_mode('fast')): E=4096 nheads=32 "
                       "d=128 L=4096 batch=2, causal, x only",
                  dtype="f32", E=4096, H=32, Lq=4096, Lkv=4096, B=2, causal=True, fast_math=True),
    "c4": dict(desc="cross-attention with additive bias: fp16 q(1024,256,16) kv(1024,2048,16) nheads=16 d=64, "
                    "bias f16 (Lkv,Lq,H,B), dropout 0.1",
               dtype="f16", E=1024, H=16, Lq=256, Lkv=2048, B=16, causal=False, bias=True, dropout=0.1),
}


def algorithmic_flops(w) -> float:
    d = w["E"] // w["H"]
    P = w["Lq"] * (w["Lq"] + 1) // 2 if w["causal"] else w["Lq"] * w["Lkv"]
    return 2.0 * (d + d) * P * w["H"] * w["B"]


def algorithmic_bytes(w, esz: int) -> float:
    """Bytes one step must move: q, k, v, x once, plus bias, mask and the scores where the workload has them."""
    n = (w["E"] * w["Lq"] * 2 + w["E"] * w["Lkv"] * 2) * w["B"] * esz
    if w.get("bias"):
        n += w["Lkv"] * w["Lq"] * w["H"] * w["B"] * esz
    if w.get("padmask"):
        n += w["Lkv"] * w["B"]
    if w.get("alpha"):
        n += w["Lkv"] * w["Lq"] * w["H"] * w["B"] * esz
    return float(n)


# stdout carries the JSON line and nothing else: libraries that print there (NCCL's version banner) are
# sent to stderr by pointing file descriptor 1 at it; the line itself goes to the saved descriptor
_json_out = None


def claim_stdout():
    global _json_out
    if _json_out is None:
        sys.stdout.flush()
        _json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(obj):
    out = _json_out if _json_out is not None else sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def config_of(args, w, world):
    """The `config` object of the JSON line: the same for both arms."""
    return {"workload": args.workload + ": " + w["desc"], "per_gpu_batch": w["B"], "global_batch": w["B"] * world,
            "sharding": "batch slices per rank, no collective"}


def profile_traffic(workload, w, esz):
    """DRAM bytes of one launch of the dominant kernel from the ncu capture summarised under profiles/: the
    read bytes of the (smaller) captured case scaled by the units processed, plus the algorithmic bytes of x
    (part of x is still in L2 when a small capture ends, so its written figure undercounts)."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.exists():
        return None
    t = json.loads(p.read_text()).get(workload)
    if not t:
        return None
    x_bytes = w["E"] * w["Lq"] * w["B"] * esz
    return t["dram_bytes_read"] * (w["B"] / t["capture_batch"]) + x_bytes


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return dict(bf16=j["bf16_tflops"], bf16_sustained=j.get("bf16_tflops_sustained"), hbm=j["hbm_gbs"],
                    source="measured (MEASURED_PEAKS.json)")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback (earlier measurement on this pool)")


# --------------------------------------------------------------------------
# clocks sampled during the timed region
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()   # the exact process this object started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        busy = [s for s in sm if s >= 0.5 * max(sm)]
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------
# CPU path (oracle) on a bounded sample
# --------------------------------------------------------------------------
def host_threads() -> int:
    """Host cores this process may use."""
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def claim_host_threads():
    """Give the BLAS behind numpy every core this process may use.  Launchers such as torchrun export
    OMP_NUM_THREADS=1 to their children, which would silently turn the CPU arm into a one-thread run; must be
    called before numpy is first imported."""
    n = str(host_threads())
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = n


def blas_threads_in_use() -> int:
    """Threads the BLAS that numpy loaded really runs with (threadpoolctl), else the cores we may use."""
    try:
        from threadpoolctl import threadpool_info
        counts = [int(i["num_threads"]) for i in threadpool_info() if i.get("user_api") == "blas"]
        if counts:
            return max(counts)
    except Exception:
        pass
    return host_threads()


def cpu_sample(w, budget_s: float = 20.0):
    """Time the CPU restatement of the reference's op sequence on a slice of the
    workload (whole heads of one batch element), sized from a one-head probe to
    take roughly ``budget_s``.  Returns (TFLOP/s, BLAS threads, description, seconds of the timed sample)."""
    import numpy as np
    from oracle import attention_oracle as O
    d = w["E"] // w["H"]
    rng = np.random.default_rng(1234)

    def run(nh):
        q = rng.standard_normal((d * nh, w["Lq"], 1), dtype=np.float32)
        k = rng.standard_normal((d * nh, w["Lkv"], 1), dtype=np.float32)
        v = rng.standard_normal((d * nh, w["Lkv"], 1), dtype=np.float32)
        mask = O.make_causal_mask(q) if w["causal"] else None
        t0 = time.perf_counter()
        O.dot_product_attention(q, k, v, mask=mask, nheads=nh)
        return time.perf_counter() - t0

    t1 = run(1)
    nh = int(max(1, min(w["H"], budget_s / max(t1, 1e-3))))
    t = run(nh) if nh > 1 else t1
    cores = blas_threads_in_use()
    P = w["Lq"] * (w["Lq"] + 1) // 2 if w["causal"] else w["Lq"] * w["Lkv"]
    flops = 2.0 * (d + d) * P * nh
    return flops / t / 1e12, cores, (f"{nh} head(s) of one batch element of the workload "
                                     f"({t:.2f} s, Float32, numpy/OpenBLAS, {cores} BLAS threads)"), t


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, secs = [], []
    desc = ""
    cores = host_threads()
    budget = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for it in range(args.warmup + args.steps):
        v, cores, desc, t = cpu_sample(w, budget_s=budget)
        if it >= args.warmup:
            vals.append(v)
            secs.append(t)
    value = statistics.mean(vals)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # a step of this arm is one bounded sample of the workload (see `cpu_baseline.sample`); this is its time
        "ms_per_step": 1e3 * statistics.mean(secs),
        "ms_per_step_full_workload_extrapolated": 1e3 * algorithmic_flops(w) / (value * 1e12),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(args, w, world),
        "note": "NNlib.jl is Julia (not installed here): the CPU restatement of its operation sequence "
                "(oracle/attention_oracle.py) is timed instead, on rank 0 only, one bounded sample per step",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(out)


# --------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------
def gpu_host_locality(torch, local):
    """NUMA node and CPU list the kernel reports for GPU `local` (sysfs, read only), and how many NUMA nodes
    this process can see.  Returns a dict for the JSON line; binds nothing."""
    info = {"numa_nodes_visible": None, "gpu_numa_node": None, "gpu_local_cpus": None}
    try:
        nodes = [p for p in Path("/sys/devices/system/node").glob("node[0-9]*")]
        info["numa_nodes_visible"] = len(nodes)
    except OSError:
        pass
    try:
        pr = torch.cuda.get_device_properties(local)
        bus = "%04x:%02x:%02x.0" % (getattr(pr, "pci_domain_id", 0), pr.pci_bus_id, pr.pci_device_id)
        base = Path("/sys/bus/pci/devices") / bus
        info["gpu_numa_node"] = int((base / "numa_node").read_text().strip())
        info["gpu_local_cpus"] = (base / "local_cpulist").read_text().strip()
    except (OSError, ValueError, AttributeError):
        pass
    return info


def parse_cpulist(text):
    cpus = set()
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_near_gpu(info):
    """Run this rank (and therefore place the pinned buffers it allocates from now on: first touch) on the
    CPUs next to its GPU, when the machine has more than one NUMA node and says which CPUs those are."""
    if not info.get("gpu_local_cpus") or (info.get("numa_nodes_visible") or 1) < 2:
        return "not bound: one NUMA node visible" if (info.get("numa_nodes_visible") or 1) < 2 else "not bound"
    try:
        want = parse_cpulist(info["gpu_local_cpus"]) & os.sched_getaffinity(0)
        if want:
            os.sched_setaffinity(0, want)
            return f"bound to {len(want)} CPUs of NUMA node {info['gpu_numa_node']}"
    except (OSError, ValueError, AttributeError):
        pass
    return "not bound"


def run_ours(args, w):
    import torch
    import torch.distributed as dist

    import nnlib_jl_b200 as nb
    from nnlib_jl_b200 import _lib
    from nnlib_jl_b200.shard import ShardedAttention, rank_rects

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    locality = gpu_host_locality(torch, local)
    locality["binding"] = bind_near_gpu(locality)      # before any pinned allocation
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    tdtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[w["dtype"]]
    E, H, Lq, Lkv, B = w["E"], w["H"], w["Lq"], w["Lkv"], w["B"]
    # seeded synthetic inputs; every rank owns its own batch slice of a global batch of B*world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    q = nb.jl_empty((E, Lq, B), tdtype, dev); q.normal_(generator=g)
    k = nb.jl_empty((E, Lkv, B), tdtype, dev); k.normal_(generator=g)
    v = nb.jl_empty((E, Lkv, B), tdtype, dev); v.normal_(generator=g)
    kwargs = dict(nheads=H)
    bias = None
    if w.get("causal"):
        # the reference's own call: the Bool matrix is built once, outside the timed region, and passed as mask=
        kwargs["mask"] = nb.make_causal_mask(q)
    if w.get("padmask"):
        lens = torch.randint(Lkv // 2, Lkv + 1, (B,), generator=g, device=dev)
        m = (torch.arange(Lkv, device=dev)[None, :] < lens[:, None])            # (B, Lkv) row-major
        kwargs["mask"] = m.reshape(B, 1, 1, Lkv).permute(3, 2, 1, 0)            # (Lkv,1,1,B) column-major
    if w.get("bias"):
        bias = nb.jl_empty((Lkv, Lq, H, B), tdtype, dev); bias.normal_(0.0, 0.5, generator=g)
    if w.get("fast_math"):
        nb.set_math_mode("fast")
    want_alpha = bool(w.get("alpha"))
    if want_alpha:
        # the workload returns the scores: ask for them with x (one library call) instead of rebuilding them lazily
        nb.set_scores_mode("eager")

    def step():
        if w.get("dropout"):
            kwargs["fdrop"] = nb.PhiloxDropout(w["dropout"], seed=0xB200, offset=0)
        y, a = nb.dot_product_attention(q, k, v, bias, **kwargs)
        if want_alpha and not isinstance(a, torch.Tensor):
            a.materialize()
        return y

    if args.backward:
        # side measurement, not the bench line: the pullback of the same call (dq, dk, dv from dx)
        fd = nb.PhiloxDropout(w["dropout"], seed=0xB200, offset=0) if w.get("dropout") else nb.identity
        _, _, back = nb.dot_product_attention_pullback(q, k, v, bias, mask=kwargs.get("mask"), nheads=H, fdrop=fd)
        dx = nb.jl_empty((E, Lq, B), tdtype, dev); dx.normal_(generator=g)

        def step():
            return back(dx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    nb.device_health(dev)

    # ---- device-resident timing -------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.nnlib_b200_launch_count()
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    launches = lib.nnlib_b200_launch_count() - launches0
    ms_total = ev0.elapsed_time(ev1)
    nb.device_health(dev)

    # ---- end-to-end timing from pinned host buffers ------------------------
    if args.no_e2e or args.backward:
        if rank == 0:
            sampler.stop()
            # the backward is counted as five products per score tile against the forward's two
            fl = algorithmic_flops(w) * (2.5 if args.backward else 1.0)
            note = "backward only (--backward)" if args.backward else "kernel-only run (--no-e2e)"
            line = {"note": note + ": not a bench line", "ms_per_step": ms_total / args.steps,
                    "tflops": fl / (ms_total / args.steps * 1e-3) / 1e12, "gpu_launches": int(launches)}
            if args.backward:
                line["backward_path"] = {_lib.PATH_UMMA: "tcgen05", _lib.PATH_SIMT: "cuda-core"}.get(back.path)
            emit(line)
        if world > 1:
            dist.destroy_process_group()
        return
    hq, hk, hv = (torch.empty(t.permute(2, 1, 0).shape, dtype=tdtype).pin_memory() for t in (q, k, v))
    for h, t in ((hq, q), (hk, k), (hv, v)):
        h.copy_(t.permute(2, 1, 0))
    hx = torch.empty((B, Lq, E), dtype=tdtype).pin_memory()
    dq, dk, dv = (nb.jl_empty(t.shape, tdtype, dev) for t in (q, k, v))

    if bias is None and not w.get("padmask") and not w.get("dropout") and not want_alpha:
        # plain / causal: the library's host-buffer pipeline (batch chunks; H2D, kernels and D2H overlap)
        pipe = nb.HostPipelinedAttention(E, E, Lq, Lkv, B, tdtype, nheads=H, mask=kwargs.get("mask"), chunk=1, device=dev)
        e2e_path = ("HostPipelinedAttention: batch chunks of 1, the last one in 4 query ranges; H2D / kernels / D2H "
                    "overlapped")

        def e2e_step():
            pipe(hq, hk, hv, hx)
    else:
        e2e_path = "H2D copies, dot_product_attention, D2H copy on one stream"

        def e2e_step():
            dq.permute(2, 1, 0).copy_(hq, non_blocking=True)
            dk.permute(2, 1, 0).copy_(hk, non_blocking=True)
            dv.permute(2, 1, 0).copy_(hv, non_blocking=True)
            if w.get("dropout"):
                kwargs["fdrop"] = nb.PhiloxDropout(w["dropout"], seed=0xB200, offset=0)
            y, a = nb.dot_product_attention(dq, dk, dv, bias, **kwargs)
            if want_alpha and not isinstance(a, torch.Tensor):
                a.materialize()
            hx.copy_(y.permute(2, 1, 0), non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks = sampler.stop() if rank == 0 else None
    nb.device_health(dev)

    # ---- the same copies without the kernels: what the host side allows -------
    ceiling = None
    extras = (args.workload == "c3" and args.batch == 0 and not args.no_extras)
    if extras:
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        xdev = nb.jl_empty((E, Lq, B), tdtype, dev)

        def copies():
            with torch.cuda.stream(s_in):
                dq.permute(2, 1, 0).copy_(hq, non_blocking=True)
                dk.permute(2, 1, 0).copy_(hk, non_blocking=True)
                dv.permute(2, 1, 0).copy_(hv, non_blocking=True)
            with torch.cuda.stream(s_out):
                hx.copy_(xdev.permute(2, 1, 0), non_blocking=True)

        copies()
        barrier()
        cur = torch.cuda.current_stream()
        c0.record(cur)
        s_in.wait_event(c0); s_out.wait_event(c0)
        for _ in range(5):
            copies()
        cur.wait_stream(s_in); cur.wait_stream(s_out)
        c1.record(cur)
        barrier()
        ceiling = c0.elapsed_time(c1) / 5

    # ---- north_star's multi-GPU split: the 128 units of the long-context configuration over the ranks ------
    strong = None
    sharded = None
    if extras:
        del dq, dk, dv
        c5 = WORKLOADS["c5"]
        E5, H5, L5, B5 = c5["E"], c5["H"], c5["Lq"], c5["B"]
        d5 = E5 // H5
        rects = rank_rects(B5, H5, rank, world)
        unit_flops = 2.0 * (d5 + d5) * (L5 * (L5 + 1) // 2)
        cm = nb.CausalMask()            # the Bool matrix would be 1 GiB at this length
        probs = []
        for r in rects:
            gq = torch.Generator(device=dev).manual_seed(5000 + r.b0 * H5 + r.h0)
            ts = [nb.jl_empty((r.nh * d5, L5, r.nb), tdtype, dev) for _ in range(3)]
            for t in ts:
                t.normal_(generator=gq)
            probs.append((r, ts))

        def strong_step():
            for r, (tq, tk, tv) in probs:
                nb.dot_product_attention(tq, tk, tv, mask=cm, nheads=r.nh)

        for _ in range(2):
            strong_step()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_strong = 5
        barrier()
        s0.record()
        for _ in range(n_strong):
            strong_step()
        s1.record()
        barrier()
        strong_ms = s0.elapsed_time(s1) / n_strong
        nb.device_health(dev)
        del probs
        t_all = torch.tensor([strong_ms], dtype=torch.float64, device=dev)
        if world > 1:
            gathered = [torch.zeros_like(t_all) for _ in range(world)]
            dist.all_gather(gathered, t_all)
            per_rank = [float(t.item()) for t in gathered]
        else:
            per_rank = [strong_ms]
        strong = {"workload": "c5: " + c5["desc"], "units_total": B5 * H5,
                  "units_per_rank": [sum(r.units for r in rank_rects(B5, H5, rr, world)) for rr in range(world)],
                  "ms_per_step_per_rank": per_rank, "ms_per_step": max(per_rank),
                  "tflops": unit_flops * B5 * H5 / (max(per_rank) * 1e-3) / 1e12, "scaling": "strong",
                  "partition": "rank_rects(8, 16, rank, world): contiguous, balanced unit ranges; no collective"}

        # all 128 units on rank 0 alone, and through the one-process driver, while the other ranks wait on the host
        store = dist.distributed_c10d._get_default_store() if world > 1 else None
        if world > 1 and rank != 0:
            torch.cuda.synchronize()
            store.wait(["bench_rank0_done"])
        elif world > 1:
            torch.cuda.synchronize()
            try:
                gq = torch.Generator(device=dev).manual_seed(5000)
                tq, tk, tv = (nb.jl_empty((E5, L5, B5), tdtype, dev) for _ in range(3))
                for t in (tq, tk, tv):
                    t.normal_(generator=gq)
                for _ in range(2):
                    nb.dot_product_attention(tq, tk, tv, mask=cm, nheads=H5)
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(3):
                    nb.dot_product_attention(tq, tk, tv, mask=cm, nheads=H5)
                a1.record()
                torch.cuda.synchronize()
                t1 = a0.elapsed_time(a1) / 3
                strong["ms_per_step_one_gpu_same_run"] = t1
                strong["efficiency_vs_one_gpu"] = t1 / (world * strong["ms_per_step"])
                # one process, one host thread per device, inputs and output in pinned host memory
                hq5, hk5, hv5 = (t.permute(2, 1, 0).cpu().pin_memory().permute(2, 1, 0) for t in (tq, tk, tv))
                del tq, tk, tv
                drv = ShardedAttention([f"cuda:{i}" for i in range(world)])
                hx5 = torch.empty((B5, L5, E5), dtype=tdtype, pin_memory=True).permute(2, 1, 0)
                drv(hq5, hk5, hv5, mask=cm, nheads=H5, out=hx5)     # creates the contexts, warms the allocator
                ts = []
                for _ in range(3):
                    t0 = time.perf_counter()
                    drv(hq5, hk5, hv5, mask=cm, nheads=H5, out=hx5)  # returns after every device has synchronised
                    ts.append(1e3 * (time.perf_counter() - t0))
                h2d5 = 3 * E5 * L5 * B5 * 2
                sharded = {"driver": "ShardedAttention: one process, one host thread per device, pinned host "
                                     "inputs and output (copies inside the timed call)",
                           "devices": world, "ms_per_call": min(ts), "ms_per_call_all": ts,
                           "tflops": unit_flops * B5 * H5 / (min(ts) * 1e-3) / 1e12,
                           "h2d_bytes_per_call": h2d5, "d2h_bytes_per_call": h2d5 // 3,
                           "timing": "host clock around the call (it joins its threads after a device synchronise)"}
            finally:
                store.set("bench_rank0_done", "1")
        if world > 1:
            dist.barrier()

    # ---- max over ranks -----------------------------------------------------
    times = torch.tensor([ms_total, e2e_ms, ceiling if ceiling is not None else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, ceiling_ms = times.tolist()
    ms_step = ms_total / args.steps
    flops_gpu = algorithmic_flops(w)
    value = flops_gpu * world / (ms_step * 1e-3) / 1e12
    e2e_value = flops_gpu * world / (e2e_ms * 1e-3) / 1e12
    esz = torch.empty(0, dtype=tdtype).element_size()
    h2d_bytes = (q.numel() + k.numel() + v.numel()) * esz
    d2h_bytes = Lq * E * B * esz

    if rank == 0:
        peaks = measured_peaks()
        per_gpu = value / world
        out = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": config_of(args, w, world),
            # every step reads and writes the same arrays: what one step touches must not fit in L2
            "notes": {"l2": ("arrays one step touches (q, k, v, x%s = %.0f MB per GPU) %s the 126 MB L2"
                             % (", bias / mask / scores" if algorithmic_bytes(w, esz) > h2d_bytes + d2h_bytes else "",
                                algorithmic_bytes(w, esz) / 1e6,
                                "larger than" if algorithmic_bytes(w, esz) > 126e6 else "SMALLER than")),
                      "kernel_path": "tcgen05",
                      "mask": "make_causal_mask(q) built once before the timed region and passed as mask= "
                              "(recognised as unmodified, never read)" if w.get("causal") else None},
            "per_gpu_tflops": per_gpu,
            "pct_of_dense_bf16_peak": 100.0 * per_gpu / peaks["bf16"],
            "clocks": clocks,
            "ms_times_sm_mhz": (ms_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "path": e2e_path,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "h2d_GBps_per_rank": h2d_bytes / (e2e_ms * 1e-3) / 1e9},
            "host": locality,
            "gpu_launches": int(launches),
        }
        if ceiling is not None:
            out["host_copy_ceiling"] = {
                "ms_per_step": ceiling_ms, "what": "the e2e step's copies alone (H2D q,k,v and D2H x on two streams, "
                "no kernels), all ranks at once, max over ranks",
                "h2d_GBps_per_rank": h2d_bytes / (ceiling_ms * 1e-3) / 1e9,
                "aggregate_GBps": world * (h2d_bytes + d2h_bytes) / (ceiling_ms * 1e-3) / 1e9,
                "e2e_over_ceiling": e2e_ms / ceiling_ms}
        if strong is not None:
            out["strong_c5"] = strong
        if sharded is not None:
            out["sharded_driver"] = sharded
        if w["causal"]:
            # long causal sequences: the fused kernel is bound by the tensor cores
            out["roofline"] = {
                "bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16"], "unit": "TFLOP/s",
                "frac": per_gpu / peaks["bf16"], "peak_source": peaks["source"] + ", burst",
                "frac_of_sustained": (per_gpu / peaks["bf16_sustained"]) if peaks["bf16_sustained"] else None,
                "kernel": "attn_fwd_umma_kernel", "algorithmic_flops_per_launch": flops_gpu,
                # dram__bytes_read + write of one launch, from the ncu capture listed in profiles/traffic.json
                "traffic": profile_traffic(args.workload, w, esz),
                "algorithmic_bytes_per_launch": algorithmic_bytes(w, esz)}
        else:
            # short sequences with bias / mask / scores returned: bound by HBM traffic (all launches of a step)
            nbytes = algorithmic_bytes(w, esz)
            gbs = nbytes / (ms_step * 1e-3) / 1e9
            out["roofline"] = {
                "bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                "peak_source": peaks["source"], "kernel": "attn_fwd_umma_kernel + attn_scores_umma_kernel"
                if (want_alpha and launches > args.steps) else ("attn_short_kernel" if want_alpha else
                                                                  "attn_fwd_umma_kernel"),
                "algorithmic_bytes_per_step": nbytes,
                "traffic": profile_traffic(args.workload, w, esz)}
        if world == 1 and not args.no_cpu:
            v_cpu, cores, desc, _ = cpu_sample(w, budget_s=args.cpu_budget)
            out["cpu_baseline"] = {"value": v_cpu, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}
        emit(out)
    if world > 1:
        dist.destroy_process_group()


def run_softmax(args):
    """Side measurement, not the bench line: the stand-alone softmax / logsoftmax kernels on the sizes the
    reference's GPU softmax benchmark quotes (benchmark/cuda_softmax/README.md, Float32, dims = 1 and 2) plus one
    HBM-sized array; algorithmic bytes = one read and one write per element."""
    import torch

    import nnlib_jl_b200 as nb
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    rows = []
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)       # larger than the 126 MB L2
    for shape, dims, dt in [((32000, 64), 1, torch.float32), ((10000, 100), 1, torch.float32),
                            ((1000, 1000), 1, torch.float32), ((256, 1000), 1, torch.float32),
                            ((256, 10, 32), 2, torch.float32), ((8192, 16384), 1, torch.float32),
                            ((4096, 32768), 1, torch.bfloat16), ((512, 512, 384), 1, torch.bfloat16)]:
        x = nb.jl_empty(shape, dt, dev); x.normal_()
        dy = nb.jl_empty(shape, dt, dev); dy.normal_()
        y = nb.softmax.softmax(x, dims=dims)
        for name, fn in (("softmax", lambda: nb.softmax.softmax(x, dims=dims)),
                         ("softmax_pullback", lambda: nb.softmax.softmax_pullback(dy, y, dims=dims))):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(max(3, args.steps)):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            us = statistics.median(ts) * 1e3
            nbytes = x.numel() * x.element_size() * (2 if name == "softmax" else 3)
            rows.append({"op": name, "size": list(shape), "dims": dims, "dtype": str(dt).replace("torch.", ""),
                         "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                         "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm"], 3)})
    emit({"note": "stand-alone softmax kernels (--softmax): not a bench line; L2 flushed between launches",
          "hbm_peak_GBps": peaks["hbm"], "rows": rows})


def run_batched_mul(args):
    """Side measurement, not the bench line: batched_mul of BFloat16 arrays on the tcgen05 product kernel,
    4096 x 4096 x 4096 x 8 (inputs 512 MB: larger than L2) in the four transpose combinations plus the two
    products of the attention path at config-3 size; algorithmic FLOPs 2·M·N·K·batch against the measured
    dense-bf16 peak."""
    import torch

    import nnlib_jl_b200 as nb
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    rows = []
    dt = torch.bfloat16
    cases = [("NN", 4096, 4096, 4096, 8), ("TN", 4096, 4096, 4096, 8), ("NT", 4096, 4096, 4096, 8),
             ("TT", 4096, 4096, 4096, 8), ("NN", 8192, 8192, 8192, 1),
             ("NN", 4096, 4096, 128, 64),      # logits = batched_mul(kt, qt) at L = 4096, d = 128 (64 units)
             ("NN", 128, 4096, 4096, 64)]      # x = batched_mul(vt, alpha)
    for tr, M, N, K, nbt in cases:
        A = nb.jl_empty((M, K, nbt) if tr[0] == "N" else (K, M, nbt), dt, dev); A.normal_()
        B = nb.jl_empty((K, N, nbt) if tr[1] == "N" else (N, K, nbt), dt, dev); B.normal_()
        Cm = nb.jl_empty((M, N, nbt), dt, dev)
        opA = A if tr[0] == "N" else nb.batched_transpose(A)
        opB = B if tr[1] == "N" else nb.batched_transpose(B)
        for _ in range(3):
            nb.batched_mul_(Cm, opA, opB)
        n = max(3, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            nb.batched_mul_(Cm, opA, opB)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        tf = 2.0 * M * N * K * nbt / (ms * 1e-3) / 1e12
        rows.append({"trans": tr, "M": M, "N": N, "K": K, "batch": nbt, "ms": round(ms, 4), "tflops": round(tf, 1),
                     "frac_of_bf16_peak": round(tf / peaks["bf16"], 3)})
        del A, B, Cm
    nb.device_health(dev)
    emit({"note": "batched_mul on the tcgen05 product kernel (--batched-mul): not a bench line", "dtype": "bf16",
          "bf16_peak_tflops": peaks["bf16"], "peak_source": peaks["source"] + ", burst", "rows": rows})


def run_decode(args):
    """Side measurement, not the bench line: few queries against a long key / value history (bf16, d = 128,
    CausalMask(offset = Lkv - Lq)): the split-key forward against the ordinary forward on the same call.  The
    work is the one pass over K and V: algorithmic bytes = 2 bytes x (d + dv) x Lkv x H x B, against the
    measured HBM peak."""
    import ctypes as C

    import torch

    import nnlib_jl_b200 as nb
    from nnlib_jl_b200 import _lib
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    lib = _lib.load()
    peaks = measured_peaks()
    rows = []
    dt = torch.bfloat16
    for (Lq, Lkv, H, B) in [(1, 32768, 32, 1), (1, 32768, 8, 1), (1, 8192, 32, 8), (8, 32768, 16, 1), (16, 131072, 8, 1)]:
        d = 128
        q = nb.jl_empty((H * d, Lq, B), dt, dev); q.normal_()
        k = nb.jl_empty((H * d, Lkv, B), dt, dev); k.normal_()
        v = nb.jl_empty((H * d, Lkv, B), dt, dev); v.normal_()
        pr = nb.attention._Problem(q, k, v, None, nb.CausalMask(Lkv - Lq), H, None, need_v=True)
        pr.alloc_x(); pr.alloc_lse()
        need = lib.nnlib_b200_attn_decode_workspace_bytes(C.byref(pr.p))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(max(5, args.steps)):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts)

        t_fwd = timed(lambda: lib.nnlib_b200_attn_fwd(C.byref(pr.p), st))
        t_dec = timed(lambda: lib.nnlib_b200_attn_decode(C.byref(pr.p), ws.data_ptr(), need, st))
        nbytes = 2.0 * (d + d) * Lkv * H * B
        rows.append({"Lq": Lq, "Lkv": Lkv, "H": H, "B": B, "workspace_bytes": int(need),
                     "attn_fwd_us": round(t_fwd * 1e3, 1), "attn_decode_us": round(t_dec * 1e3, 1),
                     "decode_GBps": round(nbytes / t_dec / 1e6, 1),
                     "decode_frac_of_hbm_peak": round(nbytes / t_dec / 1e6 / peaks["hbm"], 3)})
        del q, k, v, pr, ws
    nb.device_health(dev)
    emit({"note": "split-key forward for few queries (--decode): not a bench line; L2 flushed between launches",
          "dtype": "bf16", "hbm_peak_GBps": peaks["hbm"], "rows": rows})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler captures)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip strong_c5 / sharded_driver / host_copy_ceiling (default workload only)")
    ap.add_argument("--backward", action="store_true", help="time the pullback (dq, dk, dv) of the workload instead")
    ap.add_argument("--softmax", action="store_true", help="time the stand-alone softmax kernels instead")
    ap.add_argument("--batched-mul", action="store_true", help="time batched_mul on the product kernel instead")
    ap.add_argument("--decode", action="store_true", help="time the split-key forward for few queries instead")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (smaller profiler captures)")
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of CPU work for the cpu_baseline sample")
    args = ap.parse_args()
    claim_stdout()
    w = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["B"] = args.batch
        w["desc"] += f" [batch overridden to {args.batch}]"
    if args.softmax:
        run_softmax(args)
    elif args.batched_mul:
        run_batched_mul(args)
    elif args.decode:
        run_decode(args)
    elif args.impl == "reference":
        claim_host_threads()
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
