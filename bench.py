#!/usr/bin/env python
"""LUT-AMM benchmark: tokens/s through the LUT-NN approximate matrix multiply on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
                    [--impl ours|reference] [--shard m|n]

One "step" is one pass of the hot path (closest-centroid search + LUT gather-accumulate +
dequantise) over one batch of synthetic tokens for every linear of the workload.  Rank 0
prints ONE JSON line.  Three measurements go into it:

  value     device-resident: inputs and outputs already in HBM, calls queued on one stream,
            timed with CUDA events on that stream, L2 flushed before every timed step
  e2e       the same metric through the C ABI with pinned HOST buffers, so every step pays
            its host->device and device->host copies inside the timed region
  roofline  for the dominant kernel (the LUT gather/contraction kernel): its algorithmic
            bytes per step divided by its device time, taken live with CUDA-event pairs
            around each launch, against the measured HBM copy bandwidth

and, at one GPU, `cpu_baseline`: the CPU oracle timed on this machine's host cores on a
bounded sample.  `--impl reference` prints the CPU path's own line for the same workload.

Multi-GPU (launched by torchrun, one rank per GPU): tokens are sharded across ranks and the
weights replicated, so there is no data-path collective (weak scaling: every rank runs the
full per-GPU batch).  `--shard n` instead shards the output columns and all-gathers the
result with NCCL, for comparison.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "lut_amm_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--variant", default="auto", choices=["auto", "gather", "umma", "tune"])
    ap.add_argument("--shard", default="m", choices=["m", "n"])
    ap.add_argument("--v", type=int, default=None, help="override sub-vector length (c5 sweep)")
    ap.add_argument("--ct", type=int, default=None, help="override centroid count (c5 sweep)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def measured_bf16_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p)).get("bf16_tflops", 0.0)) or None
    return 1590.0  # the pool's earlier measurement, used when the file is absent


def recorded_traffic(workload: str):
    """DRAM bytes per step of the dominant kernel from the committed ncu capture, if any."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(p):
        return json.load(open(p)).get(workload)
    return None


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower() == "active":
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(reasons)}


def workload_spec(args):
    from pim_dl_asplos_b200 import synth
    w = dict(synth.WORKLOADS[args.workload])
    if args.v:
        w["v"] = args.v
    if args.ct:
        w["CT"] = args.ct
    return w


# --------------------------------------------------------------------------- reference arm
CPU_ARM_TEXT = {
    "reference": "the reference's own CPU AMM, amm_cpu() of inference-engine/test/test_amm.cpp compiled unmodified "
                 "(g++ -O3 OpenMP, no -march), all host threads",
    "port": "CPU restatement of the reference AMM (gcc -O3 OpenMP, no -march), bit-identical to the reference's "
            "amm_cpu() and index_calc_host.cpp where those were built",
}


class CpuArm:
    """The CPU oracle on `sample_tokens` tokens of the workload (weights built once)."""

    def __init__(self, w, sample_tokens: int, threads: int):
        import oracle
        from pim_dl_asplos_b200 import synth
        self.oracle, self.threads = oracle, threads
        self.cases = []
        for li, (_, K, N) in enumerate(w["linears"]):
            cen, lut, bias = synth.make_weights(K, N, w["v"], w["CT"], seed=0, stream=li)
            x = synth.make_input(sample_tokens, K, seed=0, stream=li)
            self.cases.append((x, cen, lut, bias))

        # the reference's own CPU AMM (amm_cpu of its test_amm.cpp, compiled unmodified into oracle/_ref)
        # when that object was built; else the restatement
        self.kind = "reference" if oracle.have_ref_amm_cpu() else "port"

    def step(self):
        for x, cen, lut, bias in self.cases:
            if self.kind == "reference":
                self.oracle.ref_amm_cpu(x, cen, lut, bias, 0.01, 0.0, nthreads=self.threads)
            else:
                self.oracle.amm(x, cen, lut, bias, 0.01, 0.0, nthreads=self.threads)

    def seconds_per_step(self, warmup: int, reps: int) -> float:
        for _ in range(warmup):
            self.step()
        t0 = time.perf_counter()
        for _ in range(reps):
            self.step()
        return (time.perf_counter() - t0) / reps


def pick_cpu_sample(w, budget_s: float, threads: int):
    """Tokens per CPU step so that a step costs about `budget_s` seconds (bounded sample)."""
    import oracle
    adds_per_token = sum((K // w["v"]) * N for _, K, N in w["linears"])
    # byte-adds per second and thread: the restatement measured about 2e9, the reference's amm_cpu about 2.5e8
    est_rate = (2.5e8 if oracle.have_ref_amm_cpu() else 2.0e9) * threads
    tok = int(budget_s * est_rate / adds_per_token)
    return max(16, min(w["M"], tok))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    w = workload_spec(args)
    threads = os.cpu_count() or 1
    # bounded sample: a step of about half a second of CPU work, so K steps end in minutes
    tok = pick_cpu_sample(w, min(0.5, 60.0 / max(args.steps + args.warmup, 1)), threads)
    arm = CpuArm(w, tok, threads)
    sec = arm.seconds_per_step(max(args.warmup, 1), max(args.steps, 1))
    val = tok / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3 * (w["M"] / tok), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 search / int8->int32 gather", "data": "synthetic",
        "config": config_dict(args, w),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": arm.kind,
                         "sample": f"{tok} of {w['M']} tokens per step, {args.steps} steps; " + CPU_ARM_TEXT[arm.kind]},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def config_dict(args, w):
    return {"workload": f"{args.workload}: {w['what']}", "tokens_per_gpu": w["M"],
            "linears": [{"name": n, "K": K, "N": N, "CB": K // w["v"]} for n, K, N in w["linears"]],
            "sub_vec_len": w["v"], "num_centroid": w["CT"], "sharding": "tokens" if args.shard == "m" else "columns+allgather",
            "l2_flush_between_steps": True, "variant": args.variant}


# --------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import pim_dl_asplos_b200 as P
    from pim_dl_asplos_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the CUDA path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at VERSION level
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    w = workload_spec(args)
    M, v, CT = w["M"], w["v"], w["CT"]
    if args.shard == "n" and world > 1:
        from pim_dl_asplos_b200 import shard as sh
    ctx = P.LutAmmContext(local)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)

    layers = []
    for li, (name, K, N) in enumerate(w["linears"]):
        cen, lut, bias = synth.make_weights(K, N, v, CT, seed=0, stream=li)
        n_lo, n_hi = 0, N
        if args.shard == "n" and world > 1:
            n_lo, n_hi = sh.column_range(N, rank, world)
            lut = np.ascontiguousarray(lut[:, :, n_lo:n_hi])
            bias = np.ascontiguousarray(bias[n_lo:n_hi])
        ctx.load_weights(li, cen, lut, bias, 0.01, 0.0)
        x = synth.make_input(M, K, seed=rank, stream=li)
        layers.append(dict(name=name, K=K, N=N, n_loc=n_hi - n_lo, x_host=x))
        del cen, lut, bias
    plan_variant = {"auto": P.VARIANT_AUTO, "gather": P.VARIANT_GATHER, "umma": P.VARIANT_UMMA}.get(args.variant)
    for li, L in enumerate(layers):
        if args.variant == "tune":
            L["plan"] = ctx.tune(li, M)
        else:
            ctx.set_plan(li, variant=plan_variant)
            L["plan"] = ctx.get_plan(li)

    with torch.cuda.stream(stream):
        for L in layers:
            L["x_dev"] = torch.from_numpy(L["x_host"]).cuda(non_blocking=False)
            L["y_dev"] = torch.empty(M, L["n_loc"], device="cuda", dtype=torch.float32)
            if args.shard == "n" and world > 1:
                L["y_all"] = torch.empty(world * M, L["n_loc"], device="cuda", dtype=torch.float32)
                L["y_full"] = torch.empty(M, L["N"], device="cuda", dtype=torch.float32)
        flush = torch.empty(256 * 1024 * 1024, device="cuda", dtype=torch.uint8)
    stream.synchronize()

    def step_device():
        for li, L in enumerate(layers):
            ctx.amm_host(li, L["x_dev"], L["y_dev"], n_tokens=M, flags=P.FLAG_ASYNC)
            if args.shard == "n" and world > 1:
                with torch.cuda.stream(stream):
                    dist.all_gather_into_tensor(L["y_all"], L["y_dev"])
                    # interleave the column slabs into row-major [M][N]
                    L["y_full"].view(M, world, L["n_loc"]).copy_(L["y_all"].view(world, M, L["n_loc"]).permute(1, 0, 2))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        barrier()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        with torch.cuda.stream(stream):
            for s, e in ev:
                flush.zero_()          # evict L2 (256 MiB > 126 MB); outside the timed interval
                s.record(stream)
                step_fn()
                e.record(stream)
        barrier()
        ms = sum(s.elapsed_time(e) for s, e in ev)
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count
    total_ms = timed(step_device, args.steps, max(args.warmup, 3))
    gpu_launches = ctx.launch_count - launches0 - 0
    # warm-up launches are inside that count; scale to the timed steps only
    per_step_launches = (ctx.launch_count - launches0) // (args.steps + max(args.warmup, 3))
    gpu_launches = per_step_launches * args.steps
    ctx.sync()
    ms_per_step = total_ms / args.steps
    value = world * M / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel: CUDA-event pairs around each launch
    ctx.enable_timing(True)
    lut_ms = ccs_ms = 0.0
    reps = min(args.steps, 20)
    for _ in range(reps):
        for li, L in enumerate(layers):
            with torch.cuda.stream(stream):
                flush.zero_()
            ctx.amm_host(li, L["x_dev"], L["y_dev"], n_tokens=M)
            t = ctx.timings()
            lut_ms += t["lut_kernel_ms"]
            ccs_ms += t["index_calc_ms"]
    ctx.enable_timing(False)
    lut_ms /= reps
    ccs_ms /= reps
    clocks = sampler.stop() if rank == 0 else None
    alg = [synth.algorithmic_bytes(M, L["K"], L["n_loc"], v, CT) for L in layers]
    lut_bytes = sum(a["lut"] for a in alg)
    peak, peak_kind = peaks()
    achieved = lut_bytes / (lut_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "lut gather-accumulate + dequantise (step 2+3), summed over the step's linears",
                "achieved": achieved, "peak": peak, "peak_source": f"{peak_kind} HBM copy bandwidth",
                "unit": "GB/s", "frac": achieved / peak, "traffic": recorded_traffic(args.workload),
                "algorithmic_bytes_per_step": lut_bytes, "kernel_ms_per_step": lut_ms,
                "search_kernel_ms_per_step": ccs_ms,
                "search_algorithmic_bytes_per_step": sum(a["ccs"] for a in alg),
                "whole_step_frac": (sum(a["total"] for a in alg) / (ms_per_step * 1e-3) / 1e9) / peak}
    # the same launches seen as what they are on the default plan, an int8 one-hot contraction on the
    # tensor pipe: 2*M*N*CB*CT operations; against twice the measured dense bf16 rate (the int8 rate is
    # not in MEASURED_PEAKS.json; nominally it is twice bf16's)
    ops = sum(2.0 * M * L["n_loc"] * (L["K"] // v) * CT for L in layers)
    bf16 = measured_bf16_tflops()
    roofline["tensor_view"] = {"int8_tops": ops / (lut_ms * 1e-3) / 1e12,
                               "assumed_int8_peak_tops": 2.0 * bf16 if bf16 else None,
                               "frac": (ops / (lut_ms * 1e-3) / 1e12) / (2.0 * bf16) if bf16 else None}

    # ---- end to end: pinned host buffers through the public call, copies inside the timing
    e2e = None
    if not args.no_e2e:
        for L in layers:
            L["x_pin"] = torch.from_numpy(L["x_host"]).pin_memory()
            L["y_pin"] = torch.empty(M, L["n_loc"], dtype=torch.float32).pin_memory()

        def step_host():
            # the public call with HOST buffers: every linear pays its H2D and D2H; the calls are
            # queued without waiting, so the library overlaps one linear's copy-out with the next
            # one's copy-in and kernels (both directions of the host link busy at once)
            for li, L in enumerate(layers):
                ctx.amm_host(li, L["x_pin"], L["y_pin"], n_tokens=M, flags=P.FLAG_ASYNC)

        for _ in range(3):
            step_host()
        ctx.sync()
        barrier()
        e_steps = max(3, min(args.steps, 30))
        t0 = time.perf_counter()
        for _ in range(e_steps):
            step_host()
        ctx.sync()   # one lutamm_sync after the last step, as a streaming caller would: the region starts
        wall_ms = (time.perf_counter() - t0) * 1e3   # and ends synchronised, so wall clock == device time
        barrier()
        tt = torch.tensor([wall_ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item()) / e_steps
        h2d_b = sum(M * L["K"] * 4 for L in layers)
        d2h_b = sum(M * L["n_loc"] * 4 for L in layers)
        e2e = {"value": world * M / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d_b, "d2h_bytes_per_step": d2h_b, "steps": e_steps,
               "sync": "calls queued with LUTAMM_FLAG_ASYNC, one lutamm_sync after the last step"}
        # what bounds it: the host link.  Measured here with plain copies of the step's own pinned
        # buffers (largest input, largest output), each direction alone, best of three; a step can
        # do no better than its slower direction at that rate.
        big_in = max(layers, key=lambda L: L["x_pin"].numel())["x_pin"]
        big_out = max(layers, key=lambda L: L["y_pin"].numel())["y_pin"]
        d_in, d_out = torch.empty_like(big_in, device="cuda"), torch.empty_like(big_out, device="cuda")
        rates = []
        for src, dst in ((big_in, d_in), (d_out, big_out)):
            nbytes, reps, best = src.numel() * 4, max(1, (64 << 20) // (src.numel() * 4)), 0.0
            for _ in range(4):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    dst.copy_(src, non_blocking=True)
                e1.record()
                torch.cuda.synchronize()
                best = max(best, reps * nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
            rates.append(best)
        # both directions at once (two streams): on some hosts of this pool the two directions add up
        # to little more than one (the link behaves half duplex), on others to almost twice
        s_a, s_b = torch.cuda.Stream(), torch.cuda.Stream()
        duplex = 0.0
        for _ in range(3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(4):
                with torch.cuda.stream(s_a):
                    d_in.copy_(big_in, non_blocking=True)
                with torch.cuda.stream(s_b):
                    big_out.copy_(d_out, non_blocking=True)
            torch.cuda.synchronize()
            duplex = max(duplex, 4 * (big_in.numel() + big_out.numel()) * 4 / (time.perf_counter() - t0) / 1e9)
        # a step can do no better than its slower direction at that direction's rate, nor than all its
        # bytes at the combined rate
        # (the probe's copies of small buffers have measured well under what the pipelined step itself
        # moved: a rate the step demonstrably reached is a lower bound of what the link can do)
        rates[0] = max(rates[0], h2d_b / (e2e_ms * 1e-3) / 1e9)
        rates[1] = max(rates[1], d2h_b / (e2e_ms * 1e-3) / 1e9)
        duplex = max(duplex, (h2d_b + d2h_b) / (e2e_ms * 1e-3) / 1e9)
        bound_ms = max(h2d_b / rates[0], d2h_b / rates[1], (h2d_b + d2h_b) / max(duplex, 1e-9)) / 1e6
        e2e.update({"host_link_h2d_gbs": rates[0], "host_link_d2h_gbs": rates[1], "host_link_both_gbs": duplex,
                    "host_link_bound_ms": bound_ms, "host_link_frac": bound_ms / e2e_ms})
        del d_in, d_out

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        threads = os.cpu_count() or 1
        tok = pick_cpu_sample(w, 2.0, threads)
        arm = CpuArm(w, tok, threads)
        sec = arm.seconds_per_step(1, 5)
        cpu = {"value": tok / sec, "unit": UNIT, "cores": threads, "kind": arm.kind,
               "sample": f"{tok} of {M} tokens per step, 1 warm-up + 5 timed steps; " + CPU_ARM_TEXT[arm.kind]}

    # ---- the same device-resident step replayed from a CUDA graph (launch overhead off the host):
    # informative only, measured last so that a capture the driver refuses cannot touch the rest
    graph_replay = None
    if world == 1 and args.shard == "m":
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step_device()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            g_steps = max(3, min(args.steps, 50))
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(g_steps)]
            for s0, e0 in ev:
                flush.zero_()
                s0.record()
                g.replay()
                e0.record()
            torch.cuda.synchronize()
            g_ms = sum(s0.elapsed_time(e0) for s0, e0 in ev) / g_steps
            graph_replay = {"ms_per_step": g_ms, "value": M / (g_ms * 1e-3), "unit": UNIT, "steps": g_steps}
            del g
        except Exception as ex:  # noqa: BLE001
            graph_replay = {"error": str(ex)[:200]}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp32 search / int8->int32 gather", "data": "synthetic",
                "config": config_dict(args, w), "plans": [L["plan"] for L in layers],
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches, "clocks": clocks,
                "graph_replay": graph_replay}
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    world_env = int(os.environ.get("WORLD_SIZE", "0"))
    if args.gpus > 1 and world_env == 0:
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
