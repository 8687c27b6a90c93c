"""Benchmark of the state-space hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload lm_cfg3|scan_cfg2|scan_cfg4|...] [--impl reference]

Prints ONE JSON line.  A step is one pass of the hot path over one batch of seeded synthetic input
(inputs far larger than L2, so no flush between steps is needed).  `value` is whole-job tokens/s with
inputs resident in HBM; `e2e` is the same metric through the host-buffer C-ABI call, host<->device
copies inside the timed region.  With N > 1 (torchrun, one rank per GPU) the default workload, the byte-LM
prefill of one batch of 32 sequences, is sharded by batch rows (32 -> 16 / 8 / 4 rows per GPU, a weight replica per
rank, no collective on the path: strong scaling); `--scaling weak` gives every rank the whole batch instead.  The
time is the max over ranks.  `--impl reference` times the CPU oracle port of the same path on the host cores.
The `kernels_*`, `s4_cfg1`, `decode_cfg3` and `ref_benches` workloads time single kernels / calls of the path
(one JSON line per case); the ncu summaries under profiles/ were captured on them."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Mamba-block prefill tokens/s at 1/2/4/8 B200; scan HBM GB/s vs roofline"

WORKLOADS = {
    # benchmark configuration 2: standalone fused selective scan, bf16 I/O, fp32 state
    "scan_cfg2": dict(kind="scan", batch=16, seq_len=4096, d_inner=1536, d_state=16, d_conv=4, seed=2),
    # benchmark configuration 4 per-GPU shard at 8 GPUs is [64, 16384, 640]; the full tensor is 43 GB
    "scan_cfg4": dict(kind="scan", batch=64, seq_len=16384, d_inner=5120, d_state=16, d_conv=4, seed=4),
    # configuration 4 with fewer rows and steps, for trying the channel shard and its gather on two GPUs
    "scan_cfg4_small": dict(kind="scan", batch=8, seq_len=4096, d_inner=5120, d_state=16, d_conv=4, seed=4),
    # the per-GPU shard of configuration 4 at 8 GPUs (channel shard): [64, 16384, 640]
    "scan_cfg4_shard8": dict(kind="scan", batch=64, seq_len=16384, d_inner=640, d_state=16, d_conv=4, seed=4),
    # benchmark configuration 3: byte-level Mamba LM prefill, 24 blocks, d_model 768, batch 32 x seq 2048, bf16
    # a mid-size scan for profiling: enough chains for every kernel variant, 1.6 GB on the device
    "scan_mid": dict(kind="scan", batch=64, seq_len=2048, d_inner=1536, d_state=16, d_conv=4, seed=5),
    # the scan of one block of configuration 3 (batch 32 x 2048, d_inner 1536)
    "scan_cfg3": dict(kind="scan", batch=32, seq_len=2048, d_inner=1536, d_state=16, d_conv=4, seed=3),
    "lm_cfg3": dict(kind="lm", n_layer=24, d_model=768, d_state=16, d_conv=4, expand=2, batch=32, seq_len=2048, seed=3),
    # what one GPU of eight gets of configuration 3 (4 sequences): the few-chains case of the scan
    "lm_cfg3_rows4": dict(kind="lm", n_layer=24, d_model=768, d_state=16, d_conv=4, expand=2, batch=4, seq_len=2048, seed=3),
    "scan_cfg3_rows4": dict(kind="scan", batch=4, seq_len=2048, d_inner=1536, d_state=16, d_conv=4, seed=3),
    # single kernels / calls of the path at the shapes of configuration 3 (and 1): one JSON line per case
    "kernels_gemm": dict(kind="kernels"), "kernels_conv": dict(kind="kernels"), "kernels_norm": dict(kind="kernels"),
    "s4_cfg1": dict(kind="kernels"), "decode_cfg3": dict(kind="kernels"), "ref_benches": dict(kind="kernels"),
}

STAGE_NAMES = ["embedding", "rmsnorm", "in_proj", "conv_silu", "x_proj", "dt_proj", "scan", "out_proj", "lm_head"]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]),
                "bf16_tflops_sustained": float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the dominant kernel, from an ncu
# capture of this workload.  A figure is reported only while the kernel that ran is the kernel that was captured;
# otherwise `traffic` is null (a run cannot measure it: ncu is not part of a timed run).
NCU_TRAFFIC = {
    ("lm_cfg3", "scan_direct_kernel (chained segments), dt_proj kernel before it"):
        {"bytes": 816_670_720, "capture": "ncu --set full, one launch inside the 24-block step: 614.7 MB read + 201.9 MB written"},
    ("lm_cfg3", "scan_direct_kernel (chained segments, dt projection inside)"):
        {"bytes": 607_432_960, "capture": "ncu --set full, one launch inside the 24-block step: 413.5 MB read + 193.9 MB written"},
    ("scan_cfg2", "scan_direct_kernel (look-back: aggregate pass + output pass)"):
        {"bytes": 1_108_681_472, "capture": "ncu --set full, both launches of one call: 304.2 + 4.6 MB (aggregate pass) and "
                                            "617.2 + 182.7 MB (output pass)"},
    ("scan_cfg2", "scan_tiled_kernel"):
        {"bytes": 791_900_000, "capture": "ncu --set full, one launch: 608.9 MB read + 182.9 MB written"},
}


def ncu_traffic(workload, kernel):
    t = NCU_TRAFFIC.get((workload, kernel))
    return (t["bytes"], t["capture"]) if t else (None, "no ncu capture of this kernel on this workload")


def scan_kernel_name(variant, cfg, splits=0):
    """The kernel hx_selective_scan_fwd runs for this variant (HX_SCAN_AUTO: one lane per channel when there are at
    least 8 warps of chains per SM, the lane-split kernel otherwise)."""
    if variant == "auto":
        import torch
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        if cfg["batch"] * cfg["d_inner"] / 32.0 >= 8.0 * sms:
            variant = "direct"
        else:
            variant = "lookback" if splits > 1 else "tiled"
    return {"direct": "scan_direct_kernel", "simple": "scan_simple_kernel",
            "lookback": "scan_direct_kernel (look-back: aggregate pass + output pass)"}.get(variant, "scan_tiled_kernel")


def scan_algorithmic_bytes(batch, seq_len, d_inner, d_state, d_conv, es=2):
    """x, dt, z read + y written once; B and C read once; parameters once."""
    pts = batch * seq_len * d_inner
    return pts * 4 * es + 2 * batch * seq_len * d_state * es + d_inner * (d_state + d_conv + 1) * 4


def pipe_rates():
    """fp32 FMA and special-function (ex2) results per second of this GPU, measured with the library's probes."""
    from helixml_b200 import ops
    return {"fma_per_s": ops.probe_pipe("fma"), "fma2_lanes_per_s": ops.probe_pipe("fma2"), "ex2_per_s": ops.probe_pipe("ex2")}


def scan_compute_roof(points, d_state, d_conv, alg_bytes, hbm_gbs, rates, launch_ms):
    """The scan against the slowest of its three ceilings: bytes at the measured copy bandwidth, exponentials
    at the measured ex2 rate, fp32 operations at the measured FMA rate.

    `spec`: the operation as it is defined, one exponential per state for the decays plus softplus and the two
    SiLUs (N + 3 per point) and 3N + k + 8 fp32 operations per point.
    `kernel`: what the direct kernel issues when A[d][n] = (n+1) A[d][0]: one exponential gives all N decays
    as powers, so 7 special-function results per point (4 ex2, 2 rcp, 1 lg2) and about 86 fp32 pipe
    operations (15 for the powers, 48 for the recurrence and the C contraction, 23 point-wise)."""
    t_hbm = alg_bytes / (hbm_gbs * 1e9) * 1e6
    out = {"rates": {k: round(v / 1e12, 3) for k, v in rates.items()}, "rates_unit": "1e12 results/s", "t_hbm_us": t_hbm}
    conv = 1 if d_conv > 0 else 0  # without the conv (it ran in its own kernel) its taps and its SiLU are not this kernel's
    for name, sfu, fp in (("spec", d_state + 2 + conv, 3 * d_state + d_conv + 8), ("kernel", 5 + 2 * conv, 79 + 7 * conv)):
        t_sfu = points * sfu / rates["ex2_per_s"] * 1e6
        t_fma = points * fp / rates["fma_per_s"] * 1e6
        t_roof = max(t_hbm, t_sfu, t_fma)
        out[name] = {"sfu_per_point": sfu, "fp32_per_point": fp, "t_sfu_us": t_sfu, "t_fma_us": t_fma, "t_roof_us": t_roof,
                     "bound": "hbm" if t_roof == t_hbm else ("sfu" if t_roof == t_sfu else "fma"),
                     "frac_of_t_roof": t_roof / (launch_ms * 1e3)}
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.rows = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def gpu_inputs(torch, cfg, device, seed_offset=0):
    """Seeded synthetic inputs with the configuration's value distributions, generated on the device."""
    B, L, D, N, K = cfg["batch"], cfg["seq_len"], cfg["d_inner"], cfg["d_state"], cfg["d_conv"]
    import numpy as np
    from helixml_b200 import synth
    g = torch.Generator(device=device).manual_seed(cfg["seed"] + 1000 * seed_offset)
    bf = torch.bfloat16
    t = {
        "x": torch.randn((B, L, D), device=device, generator=g).to(bf),
        "z": torch.randn((B, L, D), device=device, generator=g).to(bf),
        "dt": (torch.rand((B, L, D), device=device, generator=g) * 3 - 4).to(bf),
        "B": torch.randn((B, L, N), device=device, generator=g).to(bf),
        "C": torch.randn((B, L, N), device=device, generator=g).to(bf),
        "A": torch.from_numpy((-np.exp(synth.a_log_s4d_real(D, N))).astype(np.float32)).to(device),
        "D": torch.ones(D, device=device),
        "conv_w": torch.from_numpy(synth.uniform(cfg["seed"], "conv_w", (D, K), -0.5, 0.5)).to(device),
    }
    return t


def _use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs use every core this process may run on."""
    from oracle import cbind
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    cbind.set_num_threads(max(1, n))
    return cbind.num_threads()


def cpu_baseline_scan(cfg, seconds_hint=12.0):
    """Times the CPU oracle (C port, OpenMP over batch x channel) on a bounded sample of the workload:
    a few whole batch rows at full d_inner and full L, so tokens/s needs no rescaling."""
    import numpy as np
    from helixml_b200 import synth
    from oracle import cbind
    D, N, K, L = cfg["d_inner"], cfg["d_state"], cfg["d_conv"], cfg["seq_len"]
    cores = _use_all_host_threads()
    rows = 1
    inp = synth.scan_inputs(cfg["seed"], rows, L, D, N, K, bf16=True)
    t0 = time.perf_counter()
    cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    dt1 = time.perf_counter() - t0
    reps = max(1, min(8, int(seconds_hint / max(dt1, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        cbind.selective_scan(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], D=inp["D"], z=inp["z"], conv_w=inp["conv_w"])
    dt = (time.perf_counter() - t0) / reps
    return {"value": rows * L / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{rows} batch row(s) x L {L} x d_inner {D} (f32 oracle, OpenMP over channels), {reps} repetition(s)"}


def run_reference(args, cfg, name):
    """The reference arm: the reference cannot be compiled here (Rust, no toolchain), so its CPU
    implementation of the path is the oracle port, run with every host thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline_scan(cfg, seconds_hint=2.0)
        if i >= args.warmup:
            vals.append(base["value"])
    v = sum(vals) / len(vals)
    tokens_per_step = cfg["seq_len"]
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * tokens_per_step / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, **{k: cfg[k] for k in ("batch", "seq_len", "d_inner", "d_state", "d_conv")}},
            "cpu_baseline": {**base, "value": v},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def run_scan(args, cfg, name):
    import torch
    import torch.distributed as dist
    from helixml_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _lib.lib()  # fail loudly here if the CUDA library is missing

    full_cfg = cfg
    # configuration 4 shards by channels as soon as there is more than one GPU; everything else runs whole on every rank
    by_channels = args.shard == "channels" or (args.shard == "auto" and world > 1 and name.startswith("scan_cfg4"))
    c0 = 0
    if by_channels:
        from helixml_b200 import shard as sh
        c0, c1 = sh.channel_shard(cfg["d_inner"], world, rank)
        cfg = dict(cfg, d_inner=c1 - c0)          # this rank's channels; B and C are replicated
    t = gpu_inputs(torch, cfg, device, seed_offset=rank)
    y = torch.empty_like(t["x"])
    variant = {"auto": _lib.SCAN_AUTO, "tiled": _lib.SCAN_TILED, "simple": _lib.SCAN_SIMPLE, "direct": _lib.SCAN_DIRECT,
               "lookback": _lib.SCAN_LOOKBACK}[args.variant]
    splits = args.splits
    if splits == 0 and args.variant == "auto":
        # ask the library how to cut the sequence for this shape (chained segments to even out the load when chains
        # are plentiful, parallel segments when they are few)
        splits = ops.suggest_splits(cfg["batch"], cfg["seq_len"], cfg["d_inner"], torch.bfloat16, a_geometric=True)
    ws = torch.empty(max(ops.scan_workspace_bytes(cfg["batch"], cfg["seq_len"], cfg["d_inner"], torch.bfloat16, splits), 256),
                     dtype=torch.uint8, device=device) if splits > 1 else None

    def scan_rows(r0, r1, out):
        ops.selective_scan(t["x"][r0:r1], t["dt"][r0:r1], t["A"], t["B"][r0:r1], t["C"][r0:r1], D=t["D"], z=t["z"][r0:r1],
                           conv_w=t["conv_w"], variant=variant, a_geometric=True, lanes_per_channel=args.lpc, out=out[r0:r1],
                           tune=args.tune, seq_splits=splits, workspace=ws)

    def step():
        scan_rows(0, cfg["batch"], y)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ranks(ms):
        if world > 1:
            tt = torch.tensor([ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())
        return ms

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.device_status()
    ms_step = max_ranks(ms) / args.steps
    if by_channels:
        tokens_step = cfg["batch"] * cfg["seq_len"]   # every rank works on the same tokens (strong scaling)
    else:
        tokens_step = cfg["batch"] * cfg["seq_len"] * world
    value = tokens_step / (ms_step * 1e-3)
    gather = None
    if by_channels and world > 1 and not args.no_gather:
        # the one exchange of the channel-sharded scan: every rank pushes its y shard into every rank's full
        # [B, L, D] buffer with peer stores (hx_allgather_y_push), rows in `gather_groups` groups so that a group's
        # push runs on a second stream under the scan of the next group
        from helixml_b200 import shard as sh
        pg = sh.PeerGather(cfg["batch"], cfg["seq_len"], full_cfg["d_inner"], torch.bfloat16, world, rank)
        side = torch.cuda.Stream(device=device)
        main = torch.cuda.current_stream()
        groups = max(1, min(args.gather_groups, cfg["batch"]))
        bounds = [cfg["batch"] * g // groups for g in range(groups + 1)]

        def step_gather():
            for g in range(groups):
                scan_rows(bounds[g], bounds[g + 1], y)
                e = torch.cuda.Event()
                e.record(main)
                side.wait_event(e)
                pg.push(y, c0, bounds[g], bounds[g + 1], side.cuda_stream)
            e = torch.cuda.Event()
            e.record(side)
            main.wait_event(e)

        def timed(fn, steps):
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(steps):
                fn()
            a1.record()
            barrier()
            return max_ranks(a0.elapsed_time(a1)) / steps

        for _ in range(2):
            step_gather()
        both_ms = timed(step_gather, args.steps)
        push_ms = timed(lambda: pg.push(y, c0, 0, cfg["batch"], main.cuda_stream), args.steps)
        # check: column sums of every rank's shard, exchanged on the host side, against the same columns of the result
        full = pg.tensor()
        mine = y.float().sum(dim=(0, 1)).double().cpu()
        sums = [None] * world
        dist.all_gather_object(sums, (c0, mine))
        ok = all(torch.allclose(full[:, :, cc:cc + sm.numel()].float().sum(dim=(0, 1)).double().cpu(), sm, rtol=1e-6, atol=1e-3)
                 for cc, sm in sums)
        okt = torch.tensor([1.0 if ok else 0.0], device=device)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        es = 2
        out_bytes = cfg["batch"] * cfg["seq_len"] * cfg["d_inner"] * es * (world - 1)
        gather = {"how": "peer stores (hx_allgather_y_push), one kernel per rank, result [B, L, D] on every rank",
                  "row_groups": groups, "scan_plus_gather_ms": both_ms, "push_alone_ms": push_ms,
                  "bytes_out_per_rank": out_bytes, "push_alone_gbs_out_per_rank": out_bytes / (push_ms * 1e-3) / 1e9,
                  "link_peak_gbs": 770.0, "checked": bool(okt.item() == 1.0),
                  "tokens_per_s_with_gather": tokens_step / (both_ms * 1e-3)}
        pg.close()

    # end to end through the host-buffer entry point (pinned host activations in, y back to the host)
    e2e = None
    if not args.no_e2e and not by_channels:
        hs = ops.HostScan(cfg["batch"], cfg["seq_len"], cfg["d_inner"], cfg["d_state"], torch.bfloat16, t["A"], D=t["D"],
                          conv_w=t["conv_w"], variant=variant, lanes_per_channel=args.lpc, device=device)
        for name_, src in (("x", t["x"]), ("dt", t["dt"]), ("z", t["z"]), ("Bm", t["B"]), ("Cm", t["C"])):
            getattr(hs, name_).copy_(src)
        torch.cuda.synchronize()
        e_steps = max(1, min(args.steps, 5))
        for _ in range(2):
            hs.run()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e_steps):
            hs.run()
        e1.record()
        barrier()
        ems = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([ems], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ems = float(tt.item())
        e2e = {"value": tokens_step / (ems / e_steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": hs.h2d_bytes,
               "d2h_bytes_per_step": hs.d2h_bytes, "steps": e_steps}
        del hs

    if rank == 0:
        peaks = measured_peaks()
        alg = scan_algorithmic_bytes(cfg["batch"], cfg["seq_len"], cfg["d_inner"], cfg["d_state"], cfg["d_conv"])
        achieved = alg / (ms_step * 1e-3) / 1e9
        cpu = None if (args.no_cpu or world > 1) else cpu_baseline_scan(cfg)  # the CPU leg is timed at N = 1 only
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if by_channels else "weak",
            "vs_baseline": None, "dtype": "f32", "io_dtype": "bf16", "data": "synthetic", "allgather_y": gather,
            "config": {"workload": name, **{k: full_cfg[k] for k in ("batch", "seq_len", "d_inner", "d_state", "d_conv")},
                       "per_gpu": ("channel shard of %d channels, B and C replicated" % cfg["d_inner"]) if by_channels
                       else "full workload on every rank", "l2": "inputs (0.8 GB+) exceed the 126 MB L2, no flush",
                       "variant": args.variant, "lanes_per_channel": args.lpc, "tune": args.tune, "seq_splits": splits},
            "roofline": {"bound": "hbm", "kernel": scan_kernel_name(args.variant, cfg, splits), "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "algorithmic_bytes_per_launch": alg,
                         "traffic": ncu_traffic(name, scan_kernel_name(args.variant, cfg, splits))[0] if world == 1 else None,
                         "traffic_source": ncu_traffic(name, scan_kernel_name(args.variant, cfg, splits))[1]},
            "compute_roof": scan_compute_roof(cfg["batch"] * cfg["seq_len"] * cfg["d_inner"], cfg["d_state"], cfg["d_conv"], alg,
                                              peaks["hbm_gbs"], pipe_rates(), ms_step),
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": args.steps * (2 if "look-back" in scan_kernel_name(args.variant, cfg, splits) else 1),
            "clocks": clocks, "device_status": status,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def lm_flops_per_token(cfg):
    M, E, N = cfg["d_model"], cfg["d_model"] * cfg["expand"], cfg["d_state"]
    R = (M + 15) // 16
    per_block = 2 * (M * 2 * E + E * (R + 2 * N) + R * E + E * M)
    return cfg["n_layer"] * per_block + 2 * M * 256


def _lm_oracle_weights(cfg):
    import numpy as np
    from helixml_b200 import synth
    M, nl = cfg["d_model"], cfg["n_layer"]
    layers = []
    for l in range(nl):
        w = synth.mamba_block_weights(cfg["seed"], M, cfg["d_state"], cfg["d_conv"], cfg["expand"], init="0.02", prefix=f"l{l}.")
        w["norm_w"] = np.ones(M, np.float32)
        layers.append(w)
    return synth.normal(cfg["seed"], "emb", (256, M), 0, 0.02), layers, np.ones(M, np.float32)


def cpu_baseline_lm(cfg, seconds_hint=15.0, threads=None):
    """Times the CPU oracle port of the byte LM (naive i-j-k GEMMs as the reference's, rows spread over the host
    threads with OpenMP) on a bounded sample: ONE sequence of a few hundred tokens through all layers.
    threads = 1 is the reference-faithful leg: the reference's CPU backend is single-threaded."""
    from helixml_b200 import synth
    from oracle import cbind
    if threads is None:
        _use_all_host_threads()
    else:
        cbind.set_num_threads(threads)
    nl = cfg["n_layer"]
    emb, layers, normf = _lm_oracle_weights(cfg)
    L = 32 if threads == 1 else 64
    tok = synth.random_bytes(cfg["seed"], "tok", (1, L))
    t0 = time.perf_counter()
    cbind.byte_lm(tok, emb, layers, normf, cfg["d_state"], cfg["d_conv"])
    dt1 = time.perf_counter() - t0
    # grow the sample until it is worth ~seconds_hint of CPU time (cost is linear in tokens)
    L2 = int(min(cfg["seq_len"], max(L, L * seconds_hint / max(dt1, 1e-3))))
    L2 = max(L, (L2 // L) * L)
    tok = synth.random_bytes(cfg["seed"], "tok", (1, L2))
    t0 = time.perf_counter()
    cbind.byte_lm(tok, emb, layers, normf, cfg["d_state"], cfg["d_conv"])
    dt = time.perf_counter() - t0
    how = "one thread, as the reference's single-threaded CPU backend" if threads == 1 else "OpenMP over rows"
    return {"value": L2 / dt, "unit": "tokens/s", "cores": cbind.num_threads(), "kind": "port",
            "sample": f"1 sequence x {L2} tokens through all {nl} blocks + head (f32 oracle, naive GEMMs, {how})"}


def lm_parity_check(lm, cfg, tok_row, logits_row):
    """The logits the timed path produced for one sequence against the CPU oracle of the whole model, with the
    model's own weights read back from the device: rel. L2 (gate 2e-2 for bf16) and the worst single position."""
    import numpy as np
    from oracle import cbind
    _use_all_host_threads()
    emb, layers, normf = lm.weights_numpy()
    t0 = time.perf_counter()
    ref = cbind.byte_lm(tok_row[None, :], emb, layers, normf, cfg["d_state"], cfg["d_conv"])[0].astype(np.float64)
    got = logits_row.astype(np.float64)
    rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
    pos = float(np.max(np.linalg.norm(got - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-30)))
    return {"against": "CPU oracle (f32) of the whole model on one sequence of this run's batch", "tokens": int(tok_row.shape[0]),
            "rel_l2": rel, "worst_position_rel_l2": pos, "gate_rel_l2": 2e-2, "ok": bool(rel <= 2e-2),
            "oracle_seconds": time.perf_counter() - t0}


def lm_config(cfg, name, world, strong):
    """The `config` object of an lm line: the same for this arm and for the reference arm."""
    GB, L = cfg["batch"], cfg["seq_len"]
    per_gpu = (f"{GB} / {world} rows of ONE batch of {GB} sequences per GPU (contiguous blocks, first ranks take the remainder), "
               "weight replica per rank") if strong else f"batch {GB} x {L} on every rank (independent replicas)"
    return {"workload": name, **{k: cfg[k] for k in ("n_layer", "d_model", "d_state", "d_conv", "expand", "batch", "seq_len")},
            "vocab": 256, "global_batch": GB if strong else GB * world, "per_gpu": per_gpu,
            "l2": "per-layer activations exceed the 126 MB L2 at 32 rows; at fewer rows the layers' weights and "
                  "activations rotate through it (24 layers x 0.1-0.4 GB per step), no flush"}


def run_lm(args, cfg, name):
    import numpy as np
    import torch
    import torch.distributed as dist
    from helixml_b200 import _lib, nn, shard, synth
    import ctypes as C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _lib.lib()

    GB, L = cfg["batch"], cfg["seq_len"]
    strong = args.scaling == "strong"
    nn.manual_seed(cfg["seed"])          # same weights on every rank: a replica per GPU
    lm = nn.ByteLM(cfg["n_layer"], cfg["d_model"], cfg["d_state"], cfg["d_conv"], cfg["expand"], nn.Device.cuda(local), nn.BF16)
    if args.no_graph:
        lm.forward_graph(False)
    if strong:
        # ONE batch of GB sequences, rank r prefills its contiguous block of rows (no collective on the path)
        r0, r1 = shard.batch_shard(GB, world, rank)
        tok_np = np.ascontiguousarray(synth.random_bytes(cfg["seed"], "tok", (GB, L))[r0:r1])
    else:
        tok_np = synth.random_bytes(cfg["seed"] + 1000 * rank, "tok", (GB, L))
    B = tok_np.shape[0]
    if B == 0:
        raise SystemExit(f"rank {rank} has no batch rows: more ranks than sequences")
    tok_host = torch.from_numpy(tok_np).pin_memory()
    tok_dev = tok_host.to(device)
    logits_dev = torch.empty((B, L, 256), dtype=torch.bfloat16, device=device)
    logits_host = torch.empty((B, L, 256), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        lm.forward_device(tok_dev.data_ptr(), logits_dev.data_ptr(), B, L, stream)

    def step_host():
        lm.forward_host(tok_host.data_ptr(), logits_host.data_ptr(), B, L, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([ms], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms / steps

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_step = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    tokens_step = GB * L if strong else GB * L * world
    value = tokens_step / (ms_step * 1e-3)

    for _ in range(2):
        step_host()
    e_steps = max(1, min(args.steps, 10))
    ems = timed(step_host, e_steps)
    e2e = {"value": tokens_step / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * L, "d2h_bytes_per_step": B * L * 256 * 2,
           "steps": e_steps, "bytes_are": "per rank"}

    # per-stage breakdown with CUDA events on the launching stream (a second pass over the same steps, so the
    # event records do not sit inside the region `value` is taken from)
    L_ = _lib.lib()
    _lib.check(L_.hx_byte_lm_profile(lm._h, 1))
    for _ in range(args.steps):
        step()
    ms9 = (C.c_float * 9)()
    nf = C.c_int32(0)
    _lib.check(L_.hx_byte_lm_profile_read(lm._h, ms9, C.byref(nf)))
    _lib.check(L_.hx_byte_lm_profile(lm._h, 0))
    stage_ms = {n: float(ms9[i]) / max(nf.value, 1) for i, n in enumerate(STAGE_NAMES)}
    status = _lib.device_status()
    launches = lm.launches_per_forward

    if rank == 0:
        peaks = measured_peaks()
        E, N = cfg["d_model"] * cfg["expand"], cfg["d_state"]
        # algorithmic bytes of one selective scan of this rank's shape: u, dt, z read, y written, B and C read once
        # (12 354 bytes per token at d_inner 1536).  The block's kernel computes dt from the low-rank x_proj
        # output instead of reading it, so its DRAM traffic is lower than this figure; the figure stays that of
        # the operation so that fused and unfused kernels are compared on the same basis.
        scan_bytes = scan_algorithmic_bytes(B, L, E, N, 0)
        scan_ms = stage_ms["scan"] / cfg["n_layer"]
        scan_gbs = scan_bytes / (scan_ms * 1e-3) / 1e9
        # the tensor-core (tcgen05) projections; dt_proj is counted with them only while it runs as one of them
        fused_dt = stage_ms["dt_proj"] < 0.008 * cfg["n_layer"]
        dt_is_tile_gemm = False  # K = dt_rank <= 64 goes to the store-shaped kernel, reported on its own below
        fused_cx = stage_ms["x_proj"] < 0.008 * cfg["n_layer"]   # only the event marks: conv and x_proj were one kernel
        gemm_keys = ("in_proj", "out_proj", "lm_head") + (() if fused_cx else ("x_proj",)) + (("dt_proj",) if dt_is_tile_gemm else ())
        gemm_ms = sum(stage_ms[k] for k in gemm_keys)
        M_, E_ = cfg["d_model"], cfg["d_model"] * cfg["expand"]
        dt_flops_tok = cfg["n_layer"] * 2 * ((M_ + 15) // 16) * E_
        xp_flops_tok = cfg["n_layer"] * 2 * E_ * ((M_ + 15) // 16 + 2 * cfg["d_state"]) if fused_cx else 0
        gemm_tflops = (lm_flops_per_token(cfg) - dt_flops_tok - xp_flops_tok) * B * L / (gemm_ms * 1e-3) / 1e12
        # launches per block beyond norm, in_proj, conv (+ x_proj in the same kernel, or a GEMM of its own) and
        # out_proj: 1 = one-pass scan with the dt projection inside; 2 = dt_proj kernel + one-pass scan, or look-back
        # scan (aggregate pass + output pass) with the dt projection inside; 3 = dt_proj kernel + look-back scan
        per_block = (launches - 3) // cfg["n_layer"]
        scan_launches = per_block - 4 - (0 if fused_cx else 1)
        fused = fused_dt   # only the event marks: no kernel ran in that stage
        if fused and scan_launches == 1:
            scan_kernel = "scan_direct_kernel (chained segments, dt projection inside)"
        elif fused:
            scan_kernel = "scan_direct_kernel (look-back: aggregate pass + output pass, dt projection inside)"
        elif scan_launches == 3:
            scan_kernel = "scan_direct_kernel (look-back: aggregate pass + output pass), dt_proj GEMM before it"
        else:
            scan_kernel = "scan_direct_kernel (chained segments), dt_proj kernel before it"
        traffic, traffic_src = ncu_traffic(name, scan_kernel) if world == 1 else (None, "single-GPU captures only")
        # the scan is the largest single stage (and the top entry of the ncu launch list); the GEMMs, five
        # shapes of one kernel, are reported beside it under "gemm"
        dominant_scan = stage_ms["scan"] >= max(stage_ms[k] for k in ("in_proj", "x_proj", "dt_proj", "out_proj", "lm_head"))
        dt_bytes = B * L * E_ * 2
        if dominant_scan:
            roof = {"bound": "hbm", "kernel": scan_kernel, "achieved": scan_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": scan_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                    "algorithmic_bytes_per_launch": scan_bytes, "launch_ms": scan_ms, "traffic": traffic, "traffic_source": traffic_src,
                    "note": "per call of the scan stage (all its launches; the dt projection is inside them when the kernel "
                            "name says so, otherwise the dt_proj kernel is not included); algorithmic bytes are those "
                            "of the selective scan: u, dt, z read, y written, B and C read once"}
        else:
            roof = {"bound": "tensor", "kernel": "gemm_tc_kernel (all projections)", "achieved": gemm_tflops,
                    "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": gemm_tflops / peaks["bf16_tflops_sustained"],
                    "peak_source": peaks["source"] + " (sustained)", "traffic": None}
        parity = None
        if not args.no_parity:
            parity = lm_parity_check(lm, cfg, tok_np[0], logits_dev[0].float().cpu().numpy())
        cpu = cpu1 = None
        if not (args.no_cpu or world > 1):  # the CPU legs are timed at N = 1 only
            cpu = cpu_baseline_lm(cfg)
            cpu1 = cpu_baseline_lm(cfg, seconds_hint=6.0, threads=1)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": lm_config(cfg, name, world, strong),
            "roofline": roof,
            "stages_ms": stage_ms,
            "scan": {"gbs": scan_gbs, "frac_of_hbm_peak": scan_gbs / peaks["hbm_gbs"], "ms_per_launch": scan_ms,
                     "compute_roof": scan_compute_roof(B * L * E, N, 0, scan_bytes, peaks["hbm_gbs"], pipe_rates(),
                                                       scan_ms)},
            "gemm": {"tflops": gemm_tflops, "frac_of_sustained_peak": gemm_tflops / peaks["bf16_tflops_sustained"], "ms_total": gemm_ms,
                     "covers": "in_proj, out_proj, tied head" + ("" if fused_cx else ", x_proj") + " (tcgen05 kernels)"},
            "dt_proj": None if fused_dt else {"kernel": "gemm_lowk_kernel (K = dt_rank: bound by writing its result)",
                                              "ms_total": stage_ms["dt_proj"],
                                              "store_gbs": dt_bytes * cfg["n_layer"] / (stage_ms["dt_proj"] * 1e-3) / 1e9,
                                              "frac_of_hbm_peak": dt_bytes * cfg["n_layer"] / (stage_ms["dt_proj"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "conv_x_proj": "one kernel (conv_xproj_kernel; its time is under conv_silu)" if fused_cx else "conv kernel + GEMM",
            "forward_as": "plain launches" if args.no_graph else "one CUDA graph replay per step (captured on the second call)",
            "parity_checked": parity,
            "cpu_baseline": cpu, "cpu_baseline_1core": cpu1, "e2e": e2e, "gpu_launches": args.steps * launches, "clocks": clocks,
            "device_status": status,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_reference_lm(args, cfg, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, base = [], None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline_lm(cfg, seconds_hint=3.0)
        if i >= args.warmup:
            vals.append(base["value"])
    v = sum(vals) / len(vals)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * cfg["batch"] * cfg["seq_len"] / v, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": lm_config(cfg, name, int(os.environ.get("WORLD_SIZE", "1")), args.scaling == "strong"),
            "cpu_baseline": {**base, "value": v},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
            "note": "the reference is Rust and cannot be built here (no toolchain): this arm is the CPU oracle port of the same path"}
    print(json.dumps(line))


GEMM_SHAPES = {"in_proj": (65536, 3072, 768), "out_proj": (65536, 768, 1536), "out_proj_acc": (65536, 768, 1536),
               "x_proj": (65536, 80, 1536), "dt_proj": (65536, 1536, 48), "lm_head": (65536, 256, 768),
               "in_proj_8k": (8192, 3072, 768), "out_proj_acc_8k": (8192, 768, 1536),   # _8k, _16k: one GPU's share
               "in_proj_16k": (16384, 3072, 768), "out_proj_acc_16k": (16384, 768, 1536)}  # of 8 and of 4


def run_kernels(args, name):
    """Single kernels / calls of the path, timed alone with CUDA events on torch's current stream: `warmup` untimed
    calls, then `steps` calls between two events, queued behind a ~2 ms spin so that the host's launch rate does not
    limit a kernel of a few tens of microseconds.  One JSON line per case."""
    import torch
    from helixml_b200 import _lib, nn, ops, synth
    torch.cuda.set_device(0)
    _lib.lib()
    reps, warm = max(1, args.steps), max(3, args.warmup)

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(4_000_000)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def emit(case, ms, **kw):
        print(json.dumps({"workload": name, "case": case, "us": ms * 1e3, "steps": reps, "warmup": warm, **kw}))

    peaks = measured_peaks()
    if name == "kernels_gemm":
        for case in args.cases or list(GEMM_SHAPES):
            M, N, K = GEMM_SHAPES[case]
            a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
            w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
            acc = "_acc" in case   # the block's out_proj: adds into an fp32 C
            c = torch.zeros(M, N, device="cuda", dtype=torch.float32 if acc else torch.bfloat16)
            call = (lambda: ops.gemm_acc(a, w, c)) if acc else (lambda: ops.gemm(a, w, out=c))
            ms = timed(call)
            if acc:
                c.zero_()
                call()
            err = (c[:256].float() - a[:256].float() @ w.float().t()).abs().max().item()
            tf = 2 * M * N * K / ms / 1e9
            extra = {}
            if args.compare:
                # the same shape with single CTAs only, with CTA pairs wherever allowed, and through the vendor library
                # (torch.matmul, bf16 result): yardsticks, not paths of this repository
                for label, mode in (("us_single_ctas", 0), ("us_cta_pairs", 2)):
                    ops.gemm_pair_mode(mode)
                    extra[label] = timed(call) * 1e3
                ops.gemm_pair_mode(1)
                cl, wt = torch.empty(M, N, device="cuda", dtype=torch.bfloat16), w.t()
                extra["us_vendor_library_bf16_out"] = timed(lambda: torch.matmul(a, wt, out=cl)) * 1e3
            emit(case, ms, M=M, N=N, K=K, tflops=tf, frac_of_burst_peak=tf / peaks["bf16_tflops"], max_abs_err_256_rows=err, **extra)
    elif name == "kernels_conv":
        B, L, E = 32, 2048, 1536
        xz = torch.randn(B, L, 2 * E, device="cuda").to(torch.bfloat16)
        w = torch.rand(E, 4, device="cuda") - 0.5
        b = torch.zeros(E, device="cuda")
        u = torch.empty(B, L, E, device="cuda", dtype=torch.bfloat16)
        ms = timed(lambda: ops.conv1d_silu(xz[:, :, :E], w, b, out=u))
        gbs = B * L * E * 2 * 2 / ms / 1e6
        emit("conv_silu [32, 2048, 1536] bf16, x a strided half of [B, L, 2E]", ms, gbs=gbs, frac_of_hbm_peak=gbs / peaks["hbm_gbs"])
    elif name == "kernels_norm":
        T, M = 65536, 768
        x = torch.randn(T, M, device="cuda").to(torch.bfloat16)
        r = torch.randn(T, M, device="cuda")
        w = torch.ones(M, device="cuda")
        ms = timed(lambda: ops.rmsnorm(x, w, 1e-5, residual=r, out_dtype=torch.bfloat16))
        gbs = T * M * (2 + 4 + 4 + 2) / ms / 1e6
        emit("rmsnorm + residual add [65536, 768]", ms, gbs=gbs, frac_of_hbm_peak=gbs / peaks["hbm_gbs"])
    elif name == "s4_cfg1":
        # benchmark configuration 1: diagonal S4, f32, batch 8, L 2048, d_model 256, d_state 64
        inp = synth.s4_inputs(1, 8, 2048, 256, 64)
        dev = {k: torch.from_numpy(v).cuda() for k, v in inp.items()}
        ms = timed(lambda: ops.s4_diag(dev["u"], dev["A"], dev["B"], dev["C"], dev["delta"], dev["D"]))
        emit("s4_diag [8, 2048, 256] N 64 f32", ms, gbs=2 * 8 * 2048 * 256 * 4 / ms / 1e6, g_state_updates_per_s=8 * 2048 * 256 * 64 / ms / 1e6)
        M, L, N = 256, 2048, 64
        r = {"u": torch.randn(M, L, device="cuda"), "Ar": -torch.rand(N, device="cuda"), "Ai": torch.randn(N, device="cuda"),
             "B": torch.randn(N, M, device="cuda") * 0.1, "C": torch.randn(M, N, device="cuda") * 0.1, "D": torch.randn(M, device="cuda")}
        ms = timed(lambda: ops.s4_ref_forward_ssm(r["u"], r["Ar"], r["Ai"], r["B"], r["C"], r["D"]))
        emit("reference-literal S4Block::forward_ssm [256, 2048] N 64 f32", ms)
    elif name == "decode_cfg3":
        # byte LM of configuration 3: prefill 32 x 2048, then single-token steps, plain launches and CUDA-graph replays
        B, L0 = 32, 2048
        nn.manual_seed(3)
        lm = nn.ByteLM(24, 768, dtype=nn.BF16)
        tok = torch.randint(0, 256, (B, L0), device="cuda", dtype=torch.uint8)
        pre = torch.empty(B, L0, 256, device="cuda", dtype=torch.bfloat16)
        nxt = torch.randint(0, 256, (B,), device="cuda", dtype=torch.uint8)
        lg = torch.empty(B, 256, device="cuda", dtype=torch.bfloat16)
        for graph in (False, True):
            lm.decode_graph(graph)
            lm.prefill_device(tok.data_ptr(), pre.data_ptr(), B, L0)
            for _ in range(4):  # the first step is plain, the second captures
                lm.decode_step_device(nxt.data_ptr(), lg.data_ptr(), B)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(64):
                lm.decode_step_device(nxt.data_ptr(), lg.data_ptr(), B)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 64
            emit(f"decode step, batch 32, 24 blocks, {'CUDA graph' if graph else 'plain launches'}", ms,
                 kernels=lm.launches_per_decode_step, tokens_per_s=B / ms * 1e3)
    elif name == "ref_benches":
        # the reference's own criterion shapes (benches/src/neural_networks.rs:11-51): S4Block::new(512, 64) and
        # MambaBlock::new(512, 64, 4, 2) forward on [seq, 512], seq 64 / 128 / 256, f32.  There the S4 forward is
        # input.clone() and the Mamba forward out_proj(silu(gate(x))); here they are the real recurrences.
        # Module::forward returns a finished tensor (it allocates its result and synchronises), so these are host
        # wall-clock times per call, as criterion measures them.
        def wall(fn):
            for _ in range(warm):
                fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) / reps * 1e3

        s4 = nn.S4Block(512, 64)
        mb = nn.MambaBlock(512, 64, 4, 2, nn.Device.cuda(0))
        for seq in (64, 128, 256):
            x = nn.Tensor.from_numpy(synth.normal(1, f"x{seq}", (seq, 512)))
            emit(f"S4Block(512, 64).forward [{seq}, 512]", wall(lambda: s4.forward(x)), timing="host wall clock per call")
            emit(f"MambaBlock(512, 64, 4, 2).forward [{seq}, 512]", wall(lambda: mb.forward(x)), timing="host wall clock per call")
    assert _lib.device_status() == 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="lm_cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", choices=["auto", "tiled", "simple", "direct", "lookback"])
    ap.add_argument("--lpc", type=int, default=0)
    ap.add_argument("--tune", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--shard", default="auto", choices=["auto", "none", "channels"],
                    help="auto: configuration 4 is sharded by channels when N > 1")
    ap.add_argument("--no-gather", action="store_true", help="channel shard: skip the all-gather of y")
    ap.add_argument("--gather-groups", type=int, default=1, help="row groups whose pushes overlap the next group's scan")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="lm workloads: plain launches instead of the replayed CUDA graph of the forward")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of one sequence of the timed path")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="lm workloads at N > 1: one batch sharded by rows (strong) or the whole batch on every rank (weak)")
    ap.add_argument("cases", nargs="*", help="kernels_gemm: shapes to time (default all)")
    ap.add_argument("--compare", action="store_true",
                    help="kernels_gemm: also time single CTAs, CTA pairs and the vendor library's GEMM on each shape")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (to look at one GPU's share of a sharded batch)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.batch > 0 and "batch" in cfg:
        cfg = dict(cfg, batch=args.batch)
    if args.impl == "reference":
        (run_reference_lm if cfg["kind"] == "lm" else run_reference)(args, cfg, args.workload)
        return
    if cfg["kind"] == "scan":
        run_scan(args, cfg, args.workload)
    elif cfg["kind"] == "kernels":
        run_kernels(args, args.workload)
    else:
        run_lm(args, cfg, args.workload)


if __name__ == "__main__":
    main()
