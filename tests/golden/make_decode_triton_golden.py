"""Generates tests/golden/decode_triton_<regime>.npz from the reference's OWN Triton decode kernels.

oracle/reference_triton.py cuts the kernels of the batch-1 MoE half-layer out of the reference checkout
(benchmarks/shape-lab/four_layer_mini_engine.py: triton_rmsnorm_kernel :844, triton_router_topk_stage1 / stage2 /
stage2_softmax kernels :391-473, raw_row_gate_up_activation_kernel :1152, raw_row_down_sum_kernel :1189,
triton_matvec_kernel :304, triton_fused_shared_down_kernel :360) and runs them on the CPU under Triton's
interpreter with the reference's launch parameters.  This script runs it once per regime, in a child process
(TRITON_INTERPRET must be set before Triton is imported), on seeded synthetic inputs that the tests rebuild.
It needs the reference checkout (its location: AIMA_REFERENCE_ROOT in the environment) and takes about a
minute and a half per regime:

    python tests/golden/make_decode_triton_golden.py            # regenerate (all, or the regimes named)
    python tests/golden/make_decode_triton_golden.py --check    # regenerate into a temporary folder and compare

Stored per regime (BF16 as uint16 bit patterns): h2 [2048], ids [8] int32, scores [8] FP32, weights [8],
act [8,512], routed [2048], shared_input [1025], shared_out [2048], out [2048]; for "chain" the input and every
layer's ids, weights and out.
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
HERE = Path(__file__).resolve().parent
SEED = 4321
REGIMES = ("normal", "ties8", "ties4", "chain")       # "chain": three half-layers free-running, input0/ids/weights/out per layer


CHAIN_LAYERS = 3


def generate(regime: str, out: Path, stages: str = "all") -> None:
    env = dict(os.environ, TRITON_INTERPRET="1")
    what = ["--chain", str(CHAIN_LAYERS)] if regime == "chain" else ["--regime", regime, "--stages", stages]
    subprocess.run([sys.executable, str(ROOT / "oracle" / "reference_triton.py"), *what,
                    "--seed", str(SEED), "--out", str(out)], check=True, env=env)


def main() -> int:
    check = "--check" in sys.argv[1:]
    failures = 0
    with tempfile.TemporaryDirectory() as scratch:
        only = [a for a in sys.argv[1:] if not a.startswith("--")]
        for regime in (only or REGIMES):
            target = HERE / f"decode_triton_{regime}.npz"
            if not check:
                generate(regime, target)
                continue
            fresh = Path(scratch) / target.name
            generate(regime, fresh)
            old, new = np.load(target), np.load(fresh)
            same = sorted(old.files) == sorted(new.files) and all(np.array_equal(old[k], new[k]) for k in old.files)
            print(f"{target.name}: {'reproduced' if same else 'DIFFERS'}")
            failures += 0 if same else 1
    return failures


if __name__ == "__main__":
    sys.exit(main())
