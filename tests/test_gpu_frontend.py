"""The step in front of the encoder path (embedding lookups + LayerNorm, key mask from the 0/1 input mask) through the
C ABI, against the numpy restatement and the reference's own DEVICE_X86 run of the unfused front-end graph."""
import os

import numpy as np
import pytest
import torch

from oracle import bert_oracle
from oracle.make_golden import FRONTEND_CASES, GOLDEN
from tnn_b200 import capi, model_synth, ops
from util import max_abs

pytestmark = pytest.mark.gpu


def _run(fw, table_dtype, out_dtype, with_segments=True):
    dev = "cuda"
    t = lambda a: torch.from_numpy(a).to(dev).to(table_dtype)   # noqa: E731
    ids = torch.from_numpy(fw.input_ids).to(dev)
    seg = torch.from_numpy(fw.segment_ids).to(dev) if with_segments else None
    out = ops.embedding_layernorm(ids, seg, t(fw.word_emb), t(fw.type_emb) if with_segments else None, t(fw.pos_emb),
                                  torch.from_numpy(fw.gamma).to(dev), torch.from_numpy(fw.beta).to(dev), fw.eps,
                                  out_dtype=out_dtype)
    mask_add, kv_len = ops.mask_from_input_mask(torch.from_numpy(fw.input_mask).to(dev))
    torch.cuda.synchronize()
    return out.float().cpu().numpy(), mask_add.cpu().numpy(), kv_len.cpu().numpy()


@pytest.mark.parametrize("name", sorted(FRONTEND_CASES))
def test_frontend_against_reference_x86_fixture(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    fw = model_synth.make_frontend_workload(**FRONTEND_CASES[name])
    emb, mask_add, kv_len = _run(fw, torch.float32, torch.float32)
    assert capi.device_status() == capi.OK
    assert max_abs(emb, g["emb_x86"]) < 1e-5                     # fp32 tables, fp32 out: summation order only
    assert np.array_equal(mask_add.reshape(g["mask_x86"].shape), g["mask_x86"])
    assert np.array_equal(kv_len, fw.lengths.astype(np.int32))
    # half-precision tables and output, as the fused region consumes them
    emb16, _, _ = _run(fw, torch.float16, torch.float16)
    assert max_abs(emb16, g["emb_x86"]) < 2e-2


@pytest.mark.parametrize("hidden,batch,seq", [(768, 64, 128), (1024, 3, 384), (256, 5, 7), (64, 1, 1)])
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_frontend_against_oracle(hidden, batch, seq, table_dtype):
    fw = model_synth.make_frontend_workload(hidden, batch, seq, vocab=3000, max_pos=512, seed=hidden + seq,
                                            length_range=(1, seq))
    if table_dtype != torch.float32:            # the oracle sees the same rounded tables
        r = lambda a: torch.from_numpy(a).to(table_dtype).float().numpy()   # noqa: E731
        fw.word_emb, fw.type_emb, fw.pos_emb = r(fw.word_emb), r(fw.type_emb), r(fw.pos_emb)
    want, want_mask = bert_oracle.embedding_frontend(fw)
    emb, mask_add, kv_len = _run(fw, table_dtype, torch.float32)
    assert capi.device_status() == capi.OK
    assert max_abs(emb, want) < 2e-5
    assert np.array_equal(mask_add, want_mask.reshape(batch, seq))
    assert np.array_equal(kv_len, fw.lengths.astype(np.int32))


def test_frontend_without_segments_and_out_of_range_index():
    fw = model_synth.make_frontend_workload(256, 2, 16, vocab=100, max_pos=32, seed=3)
    fw.type_emb = np.zeros_like(fw.type_emb)
    want, _ = bert_oracle.embedding_frontend(fw)
    emb, _, _ = _run(fw, torch.float32, torch.float32, with_segments=False)
    assert capi.device_status() == capi.OK
    assert max_abs(emb, want) < 2e-5
    # the reference's Gather refuses an index outside the table; the kernel flags it in the device status word
    fw.input_ids = fw.input_ids.copy()
    fw.input_ids[1, 3] = 100
    _run(fw, torch.float32, torch.float32, with_segments=False)
    assert capi.device_status() == capi.ERR_INDEX
    assert capi.device_status() == capi.OK       # reading clears it


def test_frontend_rejects_bad_arguments():
    d = capi.EmbeddingDesc()
    assert capi.lib().b200_embedding_layernorm_fwd(None, None) == capi.ERR_PARAM
    assert capi.lib().b200_embedding_layernorm_fwd(d, None) == capi.ERR_PARAM
    assert capi.lib().b200_mask_from_input_mask(None, 1, 1, -10000.0, -5000.0, None, None, None) == capi.ERR_PARAM
