#!/usr/bin/env python3
"""Benchmark of the transformer-encoder attention path: BERT-base, sequence length 128, sequences/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the benchmark's config 5 — a 12-layer BERT-base encoder over 1024 sequences x 128 tokens per step in total,
split evenly over the N GPUs (1024 / N sequences per GPU; strong scaling; one process per GPU, batch-sharded
replicas, no collective on the data path).  One step = one Forward of the fused encoder over a rank's batch through
TNN's own Instance API on DEVICE_CUDA served by the tnn_b200 plug-in (fp32 activations in, fp16 fused region,
fp32 out).

Keys of the JSON line beyond the base contract:
  value        inputs resident in the instance's blobs: K x Instance::ForwardAsync, CUDA events on the instance's
               stream, the K-step block repeated until >= --min-seconds are measured, max over ranks
  e2e          host to host through TNN's API: BlobConverter::ConvertFromMatAsync of the inputs (fp32 Mats in page-locked
               memory) -> ForwardAsync -> ConvertToMat of the fp32 output every step, three instances per GPU in turn
  e2e_pageable the same loop, one instance, pageable Mats;  e2e_half_io: half-precision Mats (half the bytes)
  roofline     the projection/FFN GEMM kernel (dominant): algorithmic FLOPs of its launches / their CUDA-event time
  cpu_baseline the reference's own DEVICE_X86 implementation timed on this host on a bounded sample (rank 0, N = 1)
  parity       the timed workload's first Forward against the CPU oracle (first 2 sequences)
`--impl reference` times the reference's CPU implementation of the same path with all host cores.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "bert_base_seq128_sequences_per_s"
UNIT = "sequences/s"
TOTAL_BATCH = 1024      # config 5: 1024 sequences per step in total, split evenly over the GPUs
SEQ = 128


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"tflops": float(p["bf16_tflops"]), "tflops_sustained": float(p.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------ clocks sampler
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": (statistics.median(self.samples) if self.samples else None),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------ CPU reference
def cpu_reference_seq_per_s(sequences_per_instance, instances, layers=12, warmup=1, iters=1):
    """Times the reference's DEVICE_X86 encoder (oracle/_ref/libTNN.so) on `instances` host threads, each running its
    own TNN instance over `sequences_per_instance` sequences.  Returns (seq/s, kind, description)."""
    from tnn_b200 import model_synth
    from oracle import tnn_ref
    wl = model_synth.make_workload(model_synth.BERT_BASE, sequences_per_instance, SEQ, seed=0, num_layers=layers)
    if not tnn_ref.available():
        # the numpy restatement of the same arithmetic (single process; numpy's BLAS threads)
        from oracle import bert_oracle
        bert_oracle.encoder_forward(wl)
        t0 = time.perf_counter()
        for _ in range(iters):
            bert_oracle.encoder_forward(wl)
        dt = (time.perf_counter() - t0) / iters
        return sequences_per_instance / dt, "port", "numpy restatement, %d sequences x %d layers" % (
            sequences_per_instance, layers)
    import tempfile
    d = tempfile.mkdtemp(prefix="tnnref_bench_")
    proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
    model_synth.write_tnn_model(wl, proto, model)
    insts = []
    for _ in range(instances):
        inst = tnn_ref.TnnInstance(proto, model, device=tnn_ref.DEVICE_X86, threads=1)
        inst.set_input("x", wl.x)
        inst.set_input("mask", wl.mask_add)
        insts.append(inst)
    results = [None] * instances

    def run(i):
        results[i] = insts[i].time_forward(warmup, iters)   # ctypes releases the GIL inside the call

    t0 = time.perf_counter()
    threads = [threading.Thread(target=run, args=(i,)) for i in range(instances)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ms = max(results)
    for inst in insts:
        inst.close()
    seq_per_s = instances * sequences_per_instance / (ms / 1e3)
    desc = ("reference DEVICE_X86 fp32, %d instance(s) x %d sequences x %d layers, S=%d, %d warm-up + %d timed "
            "Forward (%.1f s wall)" % (instances, sequences_per_instance, layers, SEQ, warmup, iters, wall))
    return seq_per_s, "reference", desc


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------------ reference arm
def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = host_cores()
    instances = max(1, min(cores, 32))
    t0 = time.perf_counter()
    steps = max(1, min(args.steps, 3))
    value, kind, desc = cpu_reference_seq_per_s(2, instances, layers=12, warmup=1, iters=steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": 1e3 * instances * 2 / value, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 5: BERT-base 12-layer encoder, S=128, fp32, reference DEVICE_X86 on the host "
                               "cores; each step = a bounded sample of the 1024-sequence batch: %d instances x 2 "
                               "sequences" % instances},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": instances, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))
    return 0


def reduce_max_over_ranks(t, world):
    """MAX-reduce a tensor of timings over all ranks (the step time of the job is the slowest rank's)."""
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t


# ------------------------------------------------------------------------------------------------ our arm
class PluginReplica:
    """A few TNN instances of the encoder on one GPU, DEVICE_CUDA served by the plug-in: the drop-in path an unchanged
    TNN application takes.  Several instances are the serving arrangement: while one computes, another's input is on
    its way to the device and a third's output on its way back."""

    def __init__(self, wl, device_id, instances, input_dtype=None):
        import shutil
        import tempfile
        from tnn_b200 import model_synth, tnn_runtime
        self.rt = tnn_runtime
        self.dir = tempfile.mkdtemp(prefix="tnnb200_bench_")
        try:
            proto, model = os.path.join(self.dir, "m.tnnproto"), os.path.join(self.dir, "m.tnnmodel")
            model_synth.write_tnn_model(wl, proto, model, input_dtype=input_dtype)
            self.insts = [tnn_runtime.Instance(proto, model, device=tnn_runtime.DEVICE_CUDA, device_id=device_id)
                          for _ in range(instances)]
        finally:
            shutil.rmtree(self.dir, ignore_errors=True)   # the files are read at Init; nothing refers to them later

    def close(self):
        for i in self.insts:
            i.close()
        self.insts = []


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from tnn_b200 import capi, model_synth, ops, tnn_runtime
    from tnn_b200.encoder import Encoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = _bind_to_gpu_cpus(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()  # fail loudly here if the CUDA library is missing
    if not tnn_runtime.available():
        raise SystemExit("bench.py needs the TNN host framework and the plug-in (tnn_b200/host, tnn_b200/lib): "
                         "the benchmark runs through TNN's own Instance API")

    # ---- the benchmark's standalone attention sweep (16 heads x d64, batch 16, S = 512/1024/2048, all-ones mask).
    # A kernel timed alone, so it runs first, before the long loops bring the GPU to its power cap (the measured
    # tensor peak it is compared with is a burst figure too).
    peaks = measured_peaks()
    attention_sweep = []
    if rank == 0 and not args.no_attention_sweep:
        for S_ in (512, 1024, 2048):
            qkv_ = torch.randn(16, S_, 3 * 16 * 64, device=dev).to(torch.float16)
            msk_ = torch.zeros(16, S_, device=dev)
            kvl_ = ops.mask_to_kv_len(msk_)
            out_ = torch.empty(16, S_, 16 * 64, device=dev, dtype=torch.float16)
            for _ in range(10):                             # also brings the clocks up from idle
                ops.attention(qkv_, 16, msk_, kvl_, out=out_)
            torch.cuda.synchronize()
            best_ = None
            for _ in range(3):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(10):
                    ops.attention(qkv_, 16, msk_, kvl_, out=out_)
                a1.record()
                torch.cuda.synchronize()
                t_ = a0.elapsed_time(a1) / 10
                best_ = t_ if best_ is None or t_ < best_ else best_
            ms_ = best_
            fl_ = 4.0 * S_ * S_ * 64 * 16 * 16
            attention_sweep.append({"S": S_, "ms": round(ms_, 4), "tflops": round(fl_ / ms_ / 1e9, 1),
                                    "frac_of_tensor_peak": round(fl_ / ms_ / 1e9 / peaks["tflops"], 4)})
            del qkv_, out_

    # ---- the workload: config 5 — BERT-base, 1024 sequences x 128 tokens in total, split evenly over the GPUs
    total = args.total_batch
    if total % world:
        raise SystemExit("--total-batch must be a multiple of the number of GPUs")
    B = total // world

    # The step's two memory-bound kernels timed alone at this GPU's share of the batch, also before the long loops:
    # the measured copy bandwidth they are compared with is a burst figure, and inside a power-capped step the SM
    # clock is 30-40 % lower (the figures from inside the step are `attention_kernel` and `layernorm_kernel`).
    alone = {}
    if rank == 0 and not args.no_attention_sweep:
        rows_ = B * SEQ
        x_ = torch.randn(rows_, 768, device=dev).to(torch.float16)
        y_ = torch.empty_like(x_)
        g_, b_ = torch.ones(768, device=dev), torch.zeros(768, device=dev)
        qkv_ = torch.randn(B, SEQ, 3 * 768, device=dev).to(torch.float16)
        msk_ = torch.zeros(B, SEQ, device=dev)
        kvl_ = ops.mask_to_kv_len(msk_)
        for name_, fn_, bytes_ in (
                ("layernorm", lambda: ops.add_layernorm(x_, g_, b_, 1e-12, out=y_), rows_ * 768 * 2 * 2),
                ("attention", lambda: ops.attention(qkv_, 12, msk_, kvl_, out=y_.view(B, SEQ, 768)), rows_ * 768 * 2 * 4)):
            for _ in range(3):
                fn_()
            torch.cuda.synchronize()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(10):
                fn_()
            a1.record()
            torch.cuda.synchronize()
            ms_ = a0.elapsed_time(a1) / 10
            alone[name_] = {"ms": round(ms_, 4), "gbs": round(bytes_ / ms_ / 1e6, 1),
                            "frac_of_hbm_peak": round(bytes_ / ms_ / 1e6 / peaks["hbm_gbs"], 4)}
        del x_, y_, qkv_
        # The four GEMM shapes of a layer, each timed alone the way the measured tensor peak was (a short burst from
        # a cool GPU: three launches between one event pair, best of five, a pause in between).
        gemm_alone = {}
        fl_sum = ms_sum = 0.0
        for name_, (n_, k_, epi_) in (("qkv", (2304, 768, ops.EPI_BIAS)), ("out_proj", (768, 768, ops.EPI_BIAS_RESIDUAL)),
                                      ("ffn1", (3072, 768, ops.EPI_BIAS_GELU)), ("ffn2", (768, 3072, ops.EPI_BIAS_RESIDUAL))):
            xa_ = torch.randn(rows_, k_, device=dev).to(torch.float16)
            wa_ = (torch.randn(n_, k_, device=dev) * 0.02).to(torch.float16)
            ba_ = torch.zeros(n_, device=dev)
            ra_ = torch.randn(rows_, n_, device=dev).to(torch.float16) if epi_ == ops.EPI_BIAS_RESIDUAL else None
            ya_ = torch.empty(rows_, n_, device=dev, dtype=torch.float16)
            best_ = None
            for _ in range(6):
                time.sleep(0.05)
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(3):
                    ops.linear(xa_, wa_, ba_, residual=ra_, epilogue=epi_, out=ya_)
                a1.record()
                torch.cuda.synchronize()
                t_ = a0.elapsed_time(a1) / 3
                best_ = t_ if best_ is None or t_ < best_ else best_     # the first round is the warm-up
            fl_ = 2.0 * rows_ * n_ * k_
            gemm_alone[name_] = {"ms": round(best_, 4), "tflops": round(fl_ / best_ / 1e9, 1)}
            fl_sum += fl_
            ms_sum += best_
            del xa_, wa_, ra_, ya_
        gemm_alone["all_four"] = {"tflops": round(fl_sum / ms_sum / 1e9, 1),
                                  "frac_of_burst_peak": round(fl_sum / ms_sum / 1e9 / peaks["tflops"], 4)}
        alone["gemm"] = gemm_alone
    wl = model_synth.make_workload(model_synth.BERT_BASE, B, SEQ, seed=0 + rank)
    cfg = wl.cfg
    H, F, L = cfg.hidden, cfg.ffn, len(wl.weights)
    tokens = B * SEQ
    mask4 = np.ascontiguousarray(wl.mask_add.reshape(B, 1, 1, SEQ))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Three instances: one instance's chain per step is H2D -> Forward -> D2H; with 403 MB each way the two copies
    # together can take longer than a Forward, and the third instance keeps the GPU fed meanwhile.
    replica = PluginReplica(wl, local, instances=args.pipeline_instances)
    insts = replica.insts
    streams = [torch.cuda.ExternalStream(i.command_queue(), device=dev) for i in insts]

    # ---- one-step parity check of the timed workload (first 2 sequences against the CPU oracle), which is also the
    # layer-by-layer warm-up Forward of every instance
    n0 = capi.launch_count()
    insts[0].set_input("x", wl.x)
    insts[0].set_input("mask", mask4)
    insts[0].forward()
    launches_per_step = capi.launch_count() - n0          # kernels of one Forward (conversions of the two Mats included)
    y_first = insts[0].get_output()
    parity = None
    if rank == 0:
        from oracle import bert_oracle
        sub = model_synth.Workload(wl.cfg, wl.weights, wl.x[:2], wl.lengths[:2], wl.mask_add[:2], wl.meta)
        want = bert_oracle.encoder_forward(sub)
        err = float(np.abs(y_first[:2] - want).max())
        parity = {"max_abs_vs_oracle_first_2_sequences": err, "bound": 2e-2, "ok": bool(err <= 2e-2)}
        if not parity["ok"]:
            raise SystemExit("parity check of the timed workload failed: %g" % err)
    for inst in insts[1:]:
        inst.set_input("x", wl.x)
        inst.set_input("mask", mask4)
        inst.forward()
    for _ in range(max(3, args.warmup)):                   # graph capture happens on the first of these
        for inst in insts:
            inst.forward()
    graph_state = insts[0].graph_counters()
    barrier()

    # ---- timed region: inputs resident in the instances' blobs, `steps` x ForwardAsync over the instances in turn (the
    # serving arrangement: one instance's wave tails are filled by the next one's kernels), CUDA events on the first
    # instance's stream, which waits for the others at the end of the block; the block is repeated until at least
    # `--min-seconds` of device time have been measured
    sampler = ClockSampler(local)
    sampler.start()
    block_ms = []
    st0 = streams[0]
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(st0)
        for k in range(args.steps):
            insts[k % len(insts)].forward_async()
        for st in streams[1:]:                              # the block ends when every instance's stream has drained
            done = torch.cuda.Event()
            done.record(st)
            st0.wait_event(done)
        e1.record(st0)
        barrier()
        block_ms.append(e0.elapsed_time(e1))
        stop = torch.tensor([1.0 if sum(block_ms) >= args.min_seconds * 1e3 or len(block_ms) >= 64 else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(stop, op=dist.ReduceOp.MIN)    # every rank runs the same number of blocks
        if float(stop[0]) > 0:
            break
    blocks = len(block_ms)
    ms_total = sum(block_ms)
    clocks = sampler.stop()
    if capi.device_status() != capi.OK:
        raise SystemExit("device status word set: a bounded wait ran out")

    # ---- e2e: the same metric host to host through TNN's API — per step ConvertFromMatAsync of the inputs (fp32 Mats
    # in page-locked host memory), ForwardAsync, ConvertToMat of the fp32 output; the instances in turn
    def pinned(a):
        p = tnn_runtime.PinnedArray(a.shape, a.dtype)
        p.array[...] = a
        return p

    def e2e_run(replica_insts, x_arr, out_dtype, pin, steps):
        keep, ins, outs = [], [], []
        for _ in replica_insts:
            if pin:
                px, pm, po = pinned(x_arr), pinned(mask4), pinned(np.zeros((B, SEQ, H), out_dtype))
                keep += [px, pm, po]
                ins.append([("x", px.array), ("mask", pm.array)])
                outs.append([("", po.array)])
            else:
                ins.append([("x", np.array(x_arr, copy=True)), ("mask", np.array(mask4, copy=True))])
                outs.append([("", np.zeros((B, SEQ, H), out_dtype))])
        barrier()
        secs = tnn_runtime.run_pipeline(replica_insts, ins, outs, warmup=min(4, steps), steps=steps)
        barrier()
        ok = bool(np.array_equal(outs[0][0][1].astype(np.float32), y_first.astype(out_dtype).astype(np.float32))) \
            if out_dtype == np.float32 else None
        h2d = x_arr.nbytes + mask4.nbytes
        d2h = outs[0][0][1].nbytes
        for p in keep:
            p.free()
        return secs, h2d, d2h, ok

    e2e_steps = max(args.steps, int(np.ceil(args.min_seconds * 1e3 / (ms_total / (blocks * args.steps)))))
    e2e_s, h2d, d2h, e2e_same = e2e_run(insts, wl.x, np.float32, True, e2e_steps)
    pageable_steps = max(4, min(e2e_steps, args.steps))
    pageable_s, _, _, _ = e2e_run(insts[:1], wl.x, np.float32, False, pageable_steps)
    replica.close()

    # the same with half-precision Mats (the model declares a half input; RESERVED_FP16_TEST Mats): half the bytes
    half_s = None
    if not args.no_half_io:
        rep16 = PluginReplica(wl, local, instances=args.pipeline_instances, input_dtype="half")
        x16 = wl.x.astype(np.float16)
        for inst in rep16.insts:
            inst.set_input_half("x", x16)
            inst.set_input("mask", mask4)
            inst.forward()
            inst.forward()
        half_s, h2d16, d2h16, _ = e2e_run(rep16.insts, x16, np.float16, True, e2e_steps)
        rep16.close()

    # ---- roofline of the dominant kernel (the GEMM): the step's GEMM launches alone, in their order, with every
    # layer's own weights (170 MB per pass, more than L2) and the step's activation buffers, through the C ABI, replayed
    # as a CUDA graph and timed with one event pair; plus an instrumented pass with an event pair around every launch
    enc = Encoder.from_workload(wl, torch.float16, dev, fold_layernorm=False)
    shapes = {"qkv": (tokens, 3 * H, H), "out_proj": (tokens, H, H), "ffn1": (tokens, F, H), "ffn2": (tokens, H, F)}
    qkv_b = torch.empty(tokens, 3 * H, device=dev, dtype=torch.float16)
    ctx_b = torch.randn(tokens, H, device=dev).to(torch.float16)
    t_b = torch.empty(tokens, H, device=dev, dtype=torch.float16)
    f_b = torch.empty(tokens, F, device=dev, dtype=torch.float16)
    h_b = torch.randn(tokens, H, device=dev).to(torch.float16)
    mask_dev = torch.zeros(B, SEQ, device=dev)
    kv_len = ops.mask_to_kv_len(mask_dev)

    def gemm_only_step():
        for Lw in enc.layers:
            ops.linear(h_b, Lw["w_qkv"], Lw["b_qkv"], out=qkv_b)
            ops.linear(ctx_b, Lw["w_o"], Lw["b_o"], residual=h_b, epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b)
            ops.linear(h_b, Lw["w_ffn1"], Lw["b_ffn1"], epilogue=ops.EPI_BIAS_GELU, out=f_b)
            ops.linear(f_b, Lw["w_ffn2"], Lw["b_ffn2"], residual=h_b, epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b)

    def capture(fn):
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g
        except Exception as e:   # pragma: no cover - depends on the driver
            sys.stderr.write("CUDA graph capture failed (%s); running eagerly\n" % e)
            torch.cuda.synchronize()
            return None

    for _ in range(2):
        gemm_only_step()
    torch.cuda.synchronize()
    gemm_graph = capture(gemm_only_step)
    run_gemms = gemm_graph.replay if gemm_graph is not None else gemm_only_step
    for _ in range(2):
        run_gemms()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, min(args.steps, 20))
    g0.record()
    for _ in range(reps):
        run_gemms()
    g1.record()
    torch.cuda.synchronize()
    gemm_launches_per_pass = 4 * L
    gemm_pass_ms = g0.elapsed_time(g1) / reps
    flops_per_pass = sum(2.0 * m * n * kk for (m, n, kk) in shapes.values()) * L
    achieved = flops_per_pass / gemm_pass_ms / 1e9

    # per-kernel times: one event pair per launch, the stream held by a spin kernel while the host enqueues, so that
    # every pair spans exactly one kernel on the device (plus 3-6 us of event handling)
    ev_pairs = {k: [] for k in list(shapes) + ["attention", "layernorm"]}

    def timed(name, fn):
        a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b2.record()
        ev_pairs[name].append((a, b2))
        return r

    def instrumented_layers(n_layers):
        for Lw in enc.layers[:n_layers]:
            timed("qkv", lambda: ops.linear(h_b, Lw["w_qkv"], Lw["b_qkv"], out=qkv_b))
            timed("attention", lambda: ops.attention(qkv_b.view(B, SEQ, 3 * H), cfg.heads, mask_dev, kv_len,
                                                     out=ctx_b.view(B, SEQ, H)))
            timed("out_proj", lambda: ops.linear(ctx_b, Lw["w_o"], Lw["b_o"], residual=h_b,
                                                 epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b))
            timed("layernorm", lambda: ops.add_layernorm(t_b, Lw["ln1_g"], Lw["ln1_b"], cfg.ln_eps, out=ctx_b))
            timed("ffn1", lambda: ops.linear(ctx_b, Lw["w_ffn1"], Lw["b_ffn1"], epilogue=ops.EPI_BIAS_GELU, out=f_b))
            timed("ffn2", lambda: ops.linear(f_b, Lw["w_ffn2"], Lw["b_ffn2"], residual=ctx_b,
                                             epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b))
            timed("layernorm", lambda: ops.add_layernorm(t_b, Lw["ln2_g"], Lw["ln2_b"], cfg.ln_eps, out=ctx_b))

    instrumented_layers(2)
    torch.cuda.synchronize()
    for k in ev_pairs:
        ev_pairs[k].clear()
    for _ in range(3):
        torch.cuda._sleep(int(12e6))          # ~6 ms of GPU clock cycles: holds the stream while the host enqueues
        instrumented_layers(L)
        torch.cuda.synchronize()
    kernel_ms = {k: [a.elapsed_time(b2) for a, b2 in v] for k, v in ev_pairs.items()}
    per_shape = {}
    gemm_flops = gemm_ms = 0.0
    for k, (m, n, kk) in shapes.items():
        fl = 2.0 * m * n * kk
        tms = statistics.mean(kernel_ms[k])
        per_shape[k] = {"M": m, "N": n, "K": kk, "ms": round(tms, 4), "tflops": round(fl / tms / 1e9, 1)}
        gemm_flops += fl * len(kernel_ms[k])
        gemm_ms += sum(kernel_ms[k])
    achieved_bracketed = gemm_flops / gemm_ms / 1e9
    attn_ms = statistics.mean(kernel_ms["attention"])
    attn_flops = 4.0 * SEQ * SEQ * 64 * cfg.heads * B
    ln_ms = statistics.mean(kernel_ms["layernorm"])

    # ---- reduce over ranks (the job's time is the slowest rank's)
    ms_t = torch.tensor([ms_total, e2e_s * 1e3, pageable_s * 1e3, (half_s or 0.0) * 1e3], dtype=torch.float64, device=dev)
    ms_t = reduce_max_over_ranks(ms_t, world)
    ms_total_max = float(ms_t[0])
    timed_steps = blocks * args.steps
    value = world * B * timed_steps / (ms_total_max / 1e3)
    e2e_value = world * B * e2e_steps / (float(ms_t[1]) / 1e3)
    pageable_value = world * B * pageable_steps / (float(ms_t[2]) / 1e3)
    half_value = (world * B * e2e_steps / (float(ms_t[3]) / 1e3)) if half_s else None

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, kind, desc = cpu_reference_seq_per_s(8, 1, layers=12, warmup=1, iters=2)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": 1, "kind": kind, "sample": desc}

    if rank == 0:
        flops_per_seq = model_synth.layer_flops(SEQ, H, F) * L
        limiter = ("none at this N: the copies of the fp32 route (%.0f MB in + %.0f MB out per step per GPU) are hidden "
                   "behind the other instances' Forwards" % (h2d / 1e6, d2h / 1e6))
        if e2e_value < 0.9 * value:
            limiter = ("host <-> device copies of the fp32 route: %.0f MB in + %.0f MB out per step per GPU = %.0f GB/s "
                       "over the host's DMA path at the device-resident rate, shared by %d GPU(s)"
                       % (h2d / 1e6, d2h / 1e6, (h2d + d2h) * world / (ms_total_max / timed_steps) / 1e6, world))
        fp32_route = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "steps": e2e_steps, "mat_type": "NCHW_FLOAT (fp32)", "output_equals_blocking_forward": e2e_same,
                      "note": "through TNN's API with the plug-in: per step BlobConverter::ConvertFromMatAsync of x and "
                              "the mask (Mats over page-locked host memory) -> Instance::ForwardAsync -> blocking "
                              "BlobConverter::ConvertToMat of the output (the reference benchmark's loop, "
                              "test/test.cc:125-152), %d instances per GPU in turn; wall clock" % args.pipeline_instances
                              + ("" if numa is None else "; rank bound to the %d CPUs local to its GPU" % numa)}
        half_route = None if half_value is None else {
            "value": half_value, "unit": UNIT, "h2d_bytes_per_step": h2d16, "d2h_bytes_per_step": d2h16,
            "steps": e2e_steps, "mat_type": "RESERVED_FP16_TEST (half)",
            "note": "the same loop with half-precision Mats (model input declared half): half the bytes, no conversion "
                    "launches"}
        # One GPU: the fp32 Mats of an unchanged caller.  Several GPUs share the host's DMA path (it levels off near
        # 135 GB/s on these boxes, i.e. below 8 x the fp32 traffic): there the half-precision Mats are the reported
        # route, and the fp32 figure is printed beside it.
        if world > 1 and half_route is not None:
            e2e_line, e2e_other = dict(half_route), ("e2e_fp32", fp32_route)
        else:
            e2e_line, e2e_other = dict(fp32_route), ("e2e_half_io", half_route)
        e2e_line["limiter"] = limiter
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_total_max / timed_steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "config 5: BERT-base 12-layer encoder, %d sequences x %d tokens in total split over "
                                   "%d GPU(s) (%d per GPU per step), fp16 weights, all sequences full length, fp32 "
                                   "activations in/out" % (total, SEQ, world, B),
                       "total_batch": total, "batch_per_gpu": B, "seq_len": SEQ, "layers": L,
                       "parallelism": "batch-sharded replicas (%d TNN instances per GPU), no collective" % args.pipeline_instances,
                       "path": "TNN Instance::ForwardAsync on DEVICE_CUDA served by the tnn_b200 plug-in, the GPU's "
                               "instances in turn; CUDA-graph replay inside the plug-in: " + json.dumps(graph_state),
                       "timed_steps": timed_steps, "blocks_of_steps": blocks,
                       "l2": "per-step working set (170 MB fp16 weights + activations) exceeds the 126 MB L2; "
                             "no explicit flush"},
            "clocks": clocks,
            "parity": parity,
            "e2e": e2e_line,
            e2e_other[0]: e2e_other[1],
            "e2e_limiter": limiter,
            "e2e_pageable": {"value": pageable_value, "unit": UNIT, "steps": pageable_steps,
                             "note": "the same loop with ONE instance and pageable fp32 host Mats (what an unchanged "
                                     "single-instance caller does): the converter stages through page-locked memory"},
            "gpu_launches": launches_per_step * timed_steps,
            "roofline": {"bound": "tensor", "kernel": "linear_pair_kernel (projection/FFN GEMM, tcgen05 cta_group::2)",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"], "peak_source": "of " + peaks["source"] + " (burst)",
                         "peak_sustained": peaks["tflops_sustained"],
                         "frac_of_sustained": (achieved / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
                         "thermal_note": "the replays follow the timed loops, i.e. they run at the sustained (power-capped) "
                                         "clocks the `clocks` key shows; `frac` nevertheless divides by the burst peak",
                         "flops_per_launch_avg": flops_per_pass / gemm_launches_per_pass,
                         "ms_per_launch_avg": gemm_pass_ms / gemm_launches_per_pass,
                         "launches_timed": gemm_launches_per_pass * reps,
                         "method": "CUDA-graph replay of the step's %d GEMM launches alone (each layer's own weights, "
                                   "170 MB per pass), one CUDA-event pair around %d replays" % (gemm_launches_per_pass, reps),
                         "per_shape": per_shape,
                         "per_shape_note": "one event pair around every single launch (stream held while the host "
                                           "enqueues): includes 3-6 us of event handling per launch",
                         "achieved_event_bracketed": achieved_bracketed,
                         "traffic": ncu_traffic_per_launch(tokens, per_shape),
                         "traffic_note": "DRAM read+write bytes per launch, averaged over the four GEMM shapes: from the "
                                         "ncu captures at 32 768 rows (profiles/linear_pair_kernel_config5_shapes_"
                                         "m32768.md) scaled by rows / 32768 (activations grow with the rows, the "
                                         "weights are 1-5 MB); below the algorithmic bytes because part of every "
                                         "output is still in L2 when its kernel ends"},
            "attention_sweep": attention_sweep,
            "attention_sweep_note": "each point: 10 launches between one CUDA-event pair, best of 3, timed before the long loops "
                                    "(burst clocks, as the measured tensor peak was)",
            "attention_kernel": {"ms": attn_ms, "tflops": attn_flops / attn_ms / 1e9,
                                 "frac_of_tensor_peak": attn_flops / attn_ms / 1e9 / peaks["tflops"],
                                 "gbs": tokens * H * 2 * 4 / attn_ms / 1e6,
                                 "frac_of_hbm_peak": tokens * H * 2 * 4 / attn_ms / 1e6 / peaks["hbm_gbs"],
                                 "bound": "hbm at S = 128: 64 flop per compulsory byte (QKV in, context out) against "
                                          "a ridge of 256"},
            "layernorm_kernel": {"ms": ln_ms, "gbs": tokens * H * 2 * 2 / ln_ms / 1e6,
                                 "frac_of_hbm_peak": tokens * H * 2 * 2 / ln_ms / 1e6 / peaks["hbm_gbs"]},
            "kernels_alone": alone,
            "kernels_alone_note": "timed before the long loops, from a cool GPU (burst clocks, as the measured peaks were): "
                                  "layernorm / attention 10 launches between one CUDA-event pair, compulsory bytes / time "
                                  "against the measured copy bandwidth; gemm: each of a layer's four shapes at this GPU's "
                                  "rows, 3 launches per event pair, best of 5, against the measured burst tensor peak",
            "model_tflops": value * flops_per_seq / 1e12,
            "model_frac_of_tensor_peak": value * flops_per_seq / 1e12 / peaks["tflops"] / world,
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of linear_pair_kernel, from ncu captures of the GEMM shapes
# (profiles/linear_pair_kernel_*.md), keyed by the row count M the capture ran at.  ncu's size rule keeps captures small,
# so the config-5 shares (131 072 ... 16 384 rows per GPU) are represented by the 32 768-row capture scaled by the row
# count: x, the residual and y grow with M, the weights (1-5 MB) do not.
NCU_DRAM_BYTES = {
    8192: {"qkv": 16.16e6 + 0.54e6, "ffn1": 17.35e6 + 2.26e6, "ffn2": 67.69e6 + 4.36e6},
    32768: {"qkv": 53.91e6 + 99.29e6, "ffn1": 55.09e6 + 148.87e6, "ffn2": 257.54e6 + 39.24e6,
            "out_proj": 101.89e6 + 24.31e6},
}


def ncu_traffic_per_launch(tokens, per_shape):
    """Average DRAM bytes per GEMM launch of the step (the four shapes launch equally often)."""
    if tokens in NCU_DRAM_BYTES:
        table, scale = NCU_DRAM_BYTES[tokens], 1.0
    elif tokens >= 16384:
        table, scale = NCU_DRAM_BYTES[32768], tokens / 32768.0
    else:
        return None
    vals = [table[k] * scale for k in per_shape if k in table]
    return sum(vals) / len(vals) if vals else None


def _bind_to_gpu_cpus(index):
    """One rank per GPU: run this process (and first-touch its pinned host buffers) on the CPUs NVML reports as local
    to its GPU, so that H2D / D2H copies do not cross the socket interconnect.  Host-side process affinity only; no
    setting of the GPU is touched.  Returns the number of CPUs bound to, or None when NVML or the cpuset refuses."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {w * 64 + b for w, m in enumerate(words) for b in range(64) if (int(m) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--total-batch", type=int, default=TOTAL_BATCH,
                    help="sequences per step over all GPUs (config 5: 1024, split evenly)")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="the block of --steps timed steps is repeated until this much device time has been measured")
    ap.add_argument("--no-half-io", action="store_true", help="skip the half-precision-Mat end-to-end figure")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-attention-sweep", action="store_true")
    ap.add_argument("--pipeline-instances", type=int, default=3,
                    help="TNN instances per GPU that the end-to-end loop alternates between")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
