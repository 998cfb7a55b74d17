"""Single-AMM launcher with the reference's command line (inference-engine/run_amm.py:7-13):

    python run_amm.py --amm_config_file configs/bert_base_ffn1_amm.yaml [--need_compile] [--tune]

The reference re-runs cmake with the kernel shape as -D macros and rebuilds the DPU binary for
every configuration (run_amm.py:15-53).  Shapes are run-time arguments here, so "compile"
only (re)builds the library when its sources are newer than the binary.  --tune runs the
measurement-driven tuner first and uses the YAML it writes.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, os.path.dirname(PKG))


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument('--amm_config_file', type=str, required=True)
    p.add_argument('--need_compile', action='store_true', default=True)
    p.add_argument('--need_breakdown', action='store_true', default=False)
    p.add_argument('--tune', action='store_true', default=False)
    return p.parse_args()


def compile_():
    import pim_dl_asplos_b200  # noqa: F401
    from pim_dl_asplos_b200 import build
    build.build_all()


def main():
    args = parse_args()
    if args.need_compile:
        compile_()
    cfg = args.amm_config_file
    bindir = os.path.join(PKG, "bin")
    if args.tune:
        tuned = os.path.splitext(cfg)[0] + ".tuned.yaml"
        rc = subprocess.call([os.path.join(bindir, "tuner"), "0", cfg, tuned])
        if rc != 0:
            sys.exit(rc)
        cfg = tuned
    cmd = [os.path.join(bindir, "test_amm"), cfg, "unused_dpu_binary"]
    if args.need_breakdown:
        cmd.append("--breakdown")
    sys.exit(subprocess.call(cmd))


if __name__ == '__main__':
    main()
