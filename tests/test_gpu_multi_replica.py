"""GPU, two devices: the multi-GPU form of the path through the drop-in boundary — one host thread and one TNN instance
per GPU (NetworkConfig.device_id), a contiguous shard of the batch each, host-side scatter / gather, no collective —
against one instance running the whole batch on GPU 0.  Skipped on a single-GPU box."""
import os
import tempfile
import threading

import numpy as np
import pytest
import torch

from tnn_b200 import model_synth as ms
from tnn_b200 import sharding
from tnn_b200 import tnn_runtime as rt

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not rt.available(), reason="TNN host framework / plug-in missing"),
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _files(wl):
    d = tempfile.mkdtemp(prefix="replica_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    ms.write_tnn_model(wl, proto, model)
    return proto, model


def _sub(wl, rows):
    return ms.Workload(wl.cfg, wl.weights, wl.x[rows], wl.lengths[rows], wl.mask_add[rows], dict(wl.meta))


def test_two_replicas_equal_one_instance():
    world = 2
    wl = ms.make_workload(ms.BERT_BASE, 6, 128, seed=21, length_range=(20, 128), num_layers=2, randomize_affine=True)
    proto, model = _files(wl)
    inst = rt.Instance(proto, model, device=rt.DEVICE_CUDA, device_id=0)
    inst.set_input("x", wl.x)
    inst.set_input("mask", wl.mask_add)
    inst.forward()
    want = inst.get_output()
    inst.close()

    plan = sharding.balanced_shards(wl.lengths, world, wl.cfg.hidden, wl.cfg.ffn)
    parts, errors = [None] * world, []

    def replica(g):
        try:
            sub = _sub(wl, plan[g])
            p, m = _files(sub)
            r = rt.Instance(p, m, device=rt.DEVICE_CUDA, device_id=g)
            for _ in range(2):                      # a replica is reused Forward after Forward
                r.set_input("x", sub.x)
                r.set_input("mask", sub.mask_add)
                r.forward()
            parts[g] = r.get_output()
            r.close()
        except Exception as e:                      # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=replica, args=(g,)) for g in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    got = sharding.gather(parts, plan, wl.x.shape[0])
    assert np.array_equal(got, want)                # sequences are independent: bit-identical
