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

# encoder + pooler head (MatMul -> Add -> Tanh on the last layer's output); same keyword arguments plus `pooler_seed`
POOLER_CASES = {
    "base_1layer_pooler": dict(kind="encoder", geometry="base", batch=2, seq=64, layers=1, seed=4,
                               length_range=(7, 64), randomize_affine=True, pooler_seed=9),
}


# encoder + span-extraction head (MatMul [H, 2] -> Add -> SplitV -> Squeeze x 2); plus `qa_seed`
QA_CASES = {
    "base_1layer_qa": dict(kind="encoder", geometry="base", batch=2, seq=64, layers=1, seed=6,
                           length_range=(9, 64), randomize_affine=True, qa_seed=3),
}


# name -> keyword arguments of model_synth.make_frontend_workload(): the embedding front-end + mask builder
FRONTEND_CASES = {
    "frontend_base_s48": dict(hidden=768, batch=3, seq=48, vocab=2000, type_vocab=2, max_pos=64, seed=5,
                              length_range=(5, 48)),
}


def run_frontend(fw, device):
    import tempfile
    d = tempfile.mkdtemp(prefix="tnnref_frontend_")
    proto, model = os.path.join(d, "f.tnnproto"), os.path.join(d, "f.tnnmodel")
    ms.write_tnn_frontend_model(fw, proto, model)
    inst = tnn_ref.TnnInstance(proto, model, device=device)
    inst.set_input_i32("input_ids", fw.input_ids)
    inst.set_input_i32("segment_ids", fw.segment_ids)
    inst.set_input_i32("input_mask", fw.input_mask)
    inst.forward()
    out = inst.get_output("emb_out"), inst.get_output("mask_add")
    inst.close()
    return out


def golden_workload(kind, geometry=None, batch=None, seq=None, layers=None, seed=0, length_range=None,
                    randomize_affine=False):
    if kind == "config1":
        return ms.config_workload(1)
    cfg = ms.BERT_BASE if geometry == "base" else ms.BERT_LARGE
    return ms.make_workload(cfg, batch, seq, seed=seed, length_range=length_range,
                            randomize_affine=randomize_affine, num_layers=layers)


def main():
    os.makedirs(GOLDEN, exist_ok=True)
    only = sys.argv[1:]      # optional: names of the cases to (re)generate
    for name, kw in CASES.items():
        if only and name not in only:
            continue
        wl = golden_workload(**kw)
        x86, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_X86)
        naive, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_NAIVE)
        path = os.path.join(GOLDEN, name + ".npz")
        # DEVICE_NAIVE (the reference's own unit-test oracle) is recorded as its distance from DEVICE_X86 only.
        np.savez(path, x86=x86.astype(np.float32), lengths=wl.lengths,
                 x86_vs_naive_max_abs=np.float32(np.abs(x86 - naive).max()))
        print(name, x86.shape, "x86-vs-naive max-abs", float(np.abs(x86 - naive).max()))
    for name, kw in POOLER_CASES.items():
        if only and name not in only:
            continue
        kw = dict(kw)
        pooler = ms.make_pooler(768 if kw["geometry"] == "base" else 1024, kw.pop("pooler_seed"))
        wl = golden_workload(**kw)
        x86, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_X86, pooler=pooler)
        naive, _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_NAIVE, pooler=pooler)
        np.savez(os.path.join(GOLDEN, name + ".npz"), x86=x86.astype(np.float32), lengths=wl.lengths,
                 x86_vs_naive_max_abs=np.float32(np.abs(x86 - naive).max()))
        print(name, x86.shape, "x86-vs-naive max-abs", float(np.abs(x86 - naive).max()))
    for name, kw in QA_CASES.items():
        if only and name not in only:
            continue
        kw = dict(kw)
        qa = ms.make_qa_head(768 if kw["geometry"] == "base" else 1024, kw.pop("qa_seed"))
        wl = golden_workload(**kw)
        (s86, e86), _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_X86, qa=qa)
        (sn, en), _ = tnn_ref.run_workload(wl, tnn_ref.DEVICE_NAIVE, qa=qa)
        dev = max(np.abs(s86 - sn).max(), np.abs(e86 - en).max())
        np.savez(os.path.join(GOLDEN, name + ".npz"), start_x86=s86.astype(np.float32), end_x86=e86.astype(np.float32),
                 lengths=wl.lengths, x86_vs_naive_max_abs=np.float32(dev))
        print(name, s86.shape, e86.shape, "x86-vs-naive max-abs", float(dev))
    for name, kw in FRONTEND_CASES.items():
        if only and name not in only:
            continue
        fw = ms.make_frontend_workload(**kw)
        e86, m86 = run_frontend(fw, tnn_ref.DEVICE_X86)
        en, mn = run_frontend(fw, tnn_ref.DEVICE_NAIVE)
        np.savez(os.path.join(GOLDEN, name + ".npz"), emb_x86=e86.astype(np.float32), mask_x86=m86.astype(np.float32),
                 x86_vs_naive_max_abs=np.float32(max(np.abs(e86 - en).max(), np.abs(m86 - mn).max())))
        print(name, e86.shape, m86.shape, "x86-vs-naive max-abs", float(np.abs(e86 - en).max()))


if __name__ == "__main__":
    main()
