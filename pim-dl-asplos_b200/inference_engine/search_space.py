"""Search-space illustration of the reference's artifact evaluation (asplos24-ae/search-space-illustration/
run_experiments.py:62-400) on the GPU path.

The reference takes ONE AMM - 32768 tokens, 1024 -> 4096, 256 codebooks, 16 centroids (its configs/*/*.yaml)
- and measures it under hand-picked points of its mapping space: coarse-grain / fine-grain / static LUT
loading x tile shapes, and loop order x sub-LUT tile for the "global optimal" plot, each normalised to a
baseline latency; it then marks the auto-tuner's pick against the measured best and worst.  On a GPU the
mapping space is the execution plan of the library (lutamm_plan), so the same experiment is a sweep of that:

  operand-tile   where the one-hot operand lives (tensor / shared memory) x tile width      (tcgen05 kernel)
  split-ring     split of the codebook axis x depth of the LUT ring                         (tcgen05 kernel)
  builders       one-hot builder groups x tile width                                        (tcgen05 kernel)
  epilogue       how finished tiles leave the SM (transposing stores / copy engine) x width (tcgen05 kernel)
  gather         tile configurations of the CUDA-core gather kernel
  global         all of the above in one table, with the tuner's pick, the measured best and the worst marked

    python search_space.py                                        # all explorations -> CSV
    python search_space.py --single_point --experiment_type operand-tile --exploration_value 2-192
    python search_space.py --plot_only                            # re-emit the summary from saved CSVs

Results are CSV (no matplotlib here): per point the device time of the whole operator (search + LUT kernel),
and the speed-up over the library's default plan.
"""
import argparse
import csv
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, os.path.dirname(PKG))

SHAPE = dict(n=32768, K=1024, N=4096, CB=256, CT=16)   # search-space-illustration/configs/*/*.yaml
EXPERIMENTS = ("operand-tile", "split-ring", "builders", "epilogue", "gather", "global")


def points(experiment: str):
    """(label, plan dict) per point."""
    U, G = 2, 1
    if experiment == "operand-tile":
        return [(f"{op}-{nt}", dict(variant=U, umma_operand=op, umma_n_tile=nt, umma_split=1))
                for op, tiles in ((2, (64, 128, 160, 192)), (1, (64, 128, 256))) for nt in tiles]
    if experiment == "split-ring":
        return [(f"{sp}-{st}", dict(variant=U, umma_operand=2, umma_n_tile=192, umma_split=sp, umma_stages=st))
                for sp in (1, 2, 4) for st in (2, 4, 6, 0)]
    if experiment == "builders":
        return [(f"{g}-{nt}", dict(variant=U, umma_operand=2, umma_n_tile=nt, umma_split=1, umma_groups=g))
                for nt in (128, 192) for g in (1, 2, 3, 4)]
    if experiment == "epilogue":   # 1 = transposing stores, 2 = tiled bulk stores by the copy engine
        return [(f"{ep}-{nt}", dict(variant=U, umma_operand=2, umma_n_tile=nt, umma_split=1, umma_epilogue=ep))
                for nt in (128, 192) for ep in (1, 2)]
    if experiment == "gather":
        return [(f"{cfg}", dict(variant=G, gather_cfg=cfg)) for cfg in range(5)]
    if experiment == "global":
        seen, out = set(), []
        for e in EXPERIMENTS[:-1]:
            for label, plan in points(e):
                key = tuple(sorted(plan.items()))
                if key not in seen:
                    seen.add(key)
                    out.append((f"{e}:{label}", plan))
        return out
    raise ValueError(experiment)


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument('--plot_only', action='store_true', default=False)
    p.add_argument('--single_point', action='store_true', default=False)
    p.add_argument('--experiment_type', type=str, default='operand-tile', choices=EXPERIMENTS)
    p.add_argument('--exploration_value', type=str, default="2-192")
    p.add_argument('--out_dir', type=str, default=os.path.join(os.getcwd(), "search_space_results"))
    p.add_argument('--tokens', type=int, default=SHAPE["n"])
    p.add_argument('--dry_run', action='store_true', help='list the points, run nothing')
    p.add_argument('--device', type=int, default=0)
    return p.parse_args(argv)


class Bench:
    def __init__(self, tokens: int, device: int):
        import torch
        import pim_dl_asplos_b200 as P
        from pim_dl_asplos_b200 import synth
        self.P, self.torch, self.M = P, torch, tokens
        torch.cuda.set_device(device)
        self.ctx = P.LutAmmContext(device)
        self.stream = torch.cuda.Stream()
        self.ctx.set_stream(self.stream.cuda_stream)
        K, N, CB, CT = SHAPE["K"], SHAPE["N"], SHAPE["CB"], SHAPE["CT"]
        cen, lut, bias = synth.make_weights(K, N, K // CB, CT, seed=0)
        self.ctx.load_weights(0, cen, lut, bias, 0.1, 0.2)     # the reference configs' scale / bias
        with torch.cuda.stream(self.stream):
            self.x = torch.from_numpy(synth.make_input(tokens, K, seed=0)).cuda()
            self.y = torch.empty(tokens, N, device="cuda", dtype=torch.float32)
        self.stream.synchronize()

    def seconds(self, plan: dict, reps: int = 10) -> float:
        P, torch = self.P, self.torch
        self.ctx.set_plan(0, **plan)
        for _ in range(3):
            self.ctx.amm_host(0, self.x, self.y, n_tokens=self.M, flags=P.FLAG_ASYNC)
        self.ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(self.stream):
            e0.record(self.stream)
            for _ in range(reps):
                self.ctx.amm_host(0, self.x, self.y, n_tokens=self.M, flags=P.FLAG_ASYNC)
            e1.record(self.stream)
        self.ctx.sync()
        return e0.elapsed_time(e1) * 1e-3 / reps

    def tuned(self) -> dict:
        return self.ctx.tune(0, self.M)


def run_experiment(bench, experiment: str, out_dir: str):
    base = bench.seconds(dict(variant=0))
    rows = []
    for label, plan in points(experiment):
        try:
            t = bench.seconds(plan)
            rows.append(dict(experiment=experiment, point=label, amm_time_s=t, speedup_over_default=base / t, **plan))
        except bench.P.LutAmmError as e:   # the reference's "illegal shapes": a plan the kernel does not admit
            rows.append(dict(experiment=experiment, point=label, amm_time_s="", speedup_over_default="", note=str(e)[:80], **plan))
        print(f"{experiment}, {len(rows)} of {len(points(experiment))} jobs finished")
    ok = [r for r in rows if r["amm_time_s"] != ""]
    if experiment == "global" and ok:
        pick = bench.tuned()
        t_pick = bench.seconds(pick)
        best, worst = min(ok, key=lambda r: r["amm_time_s"]), max(ok, key=lambda r: r["amm_time_s"])
        rows.append(dict(experiment=experiment, point="tuner pick", amm_time_s=t_pick, speedup_over_default=base / t_pick,
                         **{k: v for k, v in pick.items() if k in ("variant", "gather_cfg", "umma_n_tile", "umma_split", "umma_stages",
                                                                   "umma_groups", "umma_operand", "umma_epilogue")}))
        print(f"best mapping in the tuner: {t_pick:.6f} s; best in real performance: {best['point']} {best['amm_time_s']:.6f} s; "
              f"worst: {worst['point']} {worst['amm_time_s']:.6f} s; default plan {base:.6f} s")
    write_csv(os.path.join(out_dir, experiment + ".csv"), rows)
    return rows


def write_csv(path, rows):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    keys = []
    for r in rows:
        for k in r:
            if k not in keys:
                keys.append(k)
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys)
        w.writeheader()
        w.writerows(rows)


def main(argv=None):
    args = parse_args(argv)
    if args.dry_run:
        return {e: [label for label, _ in points(e)] for e in EXPERIMENTS}
    if args.plot_only:
        for e in EXPERIMENTS:
            p = os.path.join(args.out_dir, e + ".csv")
            if os.path.exists(p):
                print(open(p).read())
        return None
    bench = Bench(args.tokens, args.device)
    if args.single_point:
        plan = dict(points(args.experiment_type)).get(args.exploration_value)
        if plan is None:
            raise SystemExit(f"unknown point {args.exploration_value}; known: {[l for l, _ in points(args.experiment_type)]}")
        t = bench.seconds(plan)
        print(f"PIM AVG AMM time {t:.6f}")
        return t
    out = {e: run_experiment(bench, e, args.out_dir) for e in EXPERIMENTS}
    bench.ctx.close()
    return out


if __name__ == '__main__':
    main()
