#!/usr/bin/env python3
"""Generate tests/golden/*.npz: outputs of the REFERENCE ITSELF (oracle/_ref/libTNN.so, DEVICE_X86 and DEVICE_NAIVE)
on seeded synthetic models.  Inputs and weights are not stored; they are regenerated from the recorded seed and shape
by tnn_b200.model_synth.  Run in a container where oracle/build_ref.py has built the reference:

    python oracle/make_golden.py

TEST INFRASTRUCTURE ONLY.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import tnn_ref  # noqa: E402
from tnn_b200 import model_synth as ms  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden")

# name -> keyword arguments of golden_workload()
CASES = {
    # config 1 of the benchmark: one BERT-base attention block + residual + LayerNorm, B=1, S=128, all-ones mask
    "c1_attention_block": dict(kind="config1"),
    # 2-layer BERT-base encoder, ragged lengths, non-trivial biases / gamma / beta
    "base_2layer_ragged": dict(kind="encoder", geometry="base", batch=2, seq=128, layers=2, seed=1,
                               length_range=(16, 128), randomize_affine=True),
    # 1-layer BERT-large geometry, sequence length not a multiple of the 128-row tiles
    "large_1layer_s96": dict(kind="encoder", geometry="large", batch=2, seq=96, layers=1, seed=2,
                             length_range=(1, 96), randomize_affine=True),
    # S = 200 spans two key tiles with a partial second tile
    "base_1layer_s200": dict(kind="encoder", geometry="base", batch=1, seq=200, layers=1, seed=3,
                             length_range=(130, 200), randomize_affine=False),
}


def golden_workload(kind, geometry=None, batch=None, seq=None, layers=None, seed=0, length_range=None,
                    randomize_affine=False):
    if kind == "config1":
        return ms.config_workload(1)
    cfg = ms.BERT_BASE if geometry == "base" else ms.BERT_LARGE
    return ms.make_workload(cfg, batch, seq, seed=seed, length_range=length_range,
                            randomize_affine=randomize_affine, num_layers=layers)


def main():
    os.makedirs(GOLDEN, exist_ok=True)
    for name, kw in CASES.items():
        wl = golden_workload(**kw)
        x86, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_X86)
        naive, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_NAIVE)
        path = os.path.join(GOLDEN, name + ".npz")
        # DEVICE_NAIVE (the reference's own unit-test oracle) is recorded as its distance from DEVICE_X86 only.
        np.savez(path, x86=x86.astype(np.float32), lengths=wl.lengths,
                 x86_vs_naive_max_abs=np.float32(np.abs(x86 - naive).max()))
        print(name, x86.shape, "x86-vs-naive max-abs", float(np.abs(x86 - naive).max()))


if __name__ == "__main__":
    main()
