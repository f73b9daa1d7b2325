#!/usr/bin/env python3
"""Benchmark of the transformer-encoder attention path: BERT-base, sequence length 128, sequences/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one Forward of the fused 12-layer encoder over one batch (fp32 activations in, fp16 fused region, fp32 out).
Per GPU the batch is the benchmark's config 2 (64 sequences x 128 tokens); with N GPUs every rank runs its own batch
(independent replicas, no collective on the data path), so `value` = N * 64 * K / max-over-ranks(device time).

Keys of the JSON line beyond the base contract:
  roofline     the projection/FFN GEMM kernel (dominant): algorithmic FLOPs of its launches / their CUDA-event time
  cpu_baseline the reference's own DEVICE_X86 implementation timed on this host on a bounded sample (rank 0, N = 1)
  e2e          the same metric with HOST buffers: pinned fp32 input -> H2D -> Forward -> D2H of the fp32 output per step
  e2e_half_io  the same with half-precision host buffers (half the bytes, no conversions): informational
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
BATCH_PER_GPU = 64
SEQ = 128


def tnn_plugin_seq_per_s(wl, warmup=5, iters=30):
    """The same workload through the drop-in path: the unmodified reference framework (oracle/_ref/libTNN.so) with the
    tnn_b200 plug-in serving DEVICE_CUDA — Instance::Forward over the fused graph, fp32 blobs at both ends.  Returns a
    dict (Forward-only and host-to-host figures) or None when the reference build is not present."""
    try:
        from tnn_b200 import model_synth, tnn_runtime
        if not tnn_runtime.available():
            return None
        import shutil
        import tempfile
        d = tempfile.mkdtemp(prefix="tnnb200_bench_")
        try:
            proto, model = os.path.join(d, "m.tnnproto"), os.path.join(d, "m.tnnmodel")
            model_synth.write_tnn_model(wl, proto, model)
            inst = tnn_runtime.Instance(proto, model, device=tnn_runtime.DEVICE_CUDA)
            inst.set_input("x", wl.x)
            inst.set_input("mask", wl.mask_add)
            ms = inst.time_forward(warmup, iters)               # Instance::Forward incl. its stream synchronise
            n = min(iters, 10)
            t0 = time.perf_counter()
            for _ in range(n):
                inst.set_input("x", wl.x)                       # host Mat -> device blob
                inst.forward()
                inst.get_output()                               # device blob -> host Mat
            host_ms = (time.perf_counter() - t0) / n * 1e3
            inst.close()
        finally:
            shutil.rmtree(d, ignore_errors=True)
        B = wl.x.shape[0]
        return {"forward_value": B / ms * 1e3, "forward_ms": ms, "host_to_host_value": B / host_ms * 1e3,
                "host_to_host_ms": host_ms, "unit": UNIT,
                "note": "TNN Instance::Forward on DEVICE_CUDA served by the plug-in (fused graph, eager launches, "
                        "blocking Forward); host_to_host adds SetInputMat/GetOutputMat with pageable fp32 host Mats"}
    except Exception as e:   # the drop-in measurement is supplementary: never fail the bench line over it
        return {"error": str(e)[:300]}


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
        "warmup": 1, "ms_per_step": 1e3 * instances * 2 / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BERT-base 12-layer encoder, S=128, fp32, reference DEVICE_X86 on host cores; "
                               "each step = %d instances x 2 sequences" % instances},
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
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from tnn_b200 import capi, model_synth, ops
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
            for _ in range(3):
                ops.attention(qkv_, 16, msk_, kvl_, out=out_)
            torch.cuda.synchronize()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(10):
                ops.attention(qkv_, 16, msk_, kvl_, out=out_)
            a1.record()
            torch.cuda.synchronize()
            ms_ = a0.elapsed_time(a1) / 10
            fl_ = 4.0 * S_ * S_ * 64 * 16 * 16
            attention_sweep.append({"S": S_, "ms": round(ms_, 4), "tflops": round(fl_ / ms_ / 1e9, 1),
                                    "frac_of_tensor_peak": round(fl_ / ms_ / 1e9 / peaks["tflops"], 4)})
            del qkv_, out_

    B = args.batch
    wl = model_synth.make_workload(model_synth.BERT_BASE, B, SEQ, seed=0 + rank)
    cfg = wl.cfg
    enc = Encoder.from_workload(wl, torch.float16, dev, fold_layernorm=args.fold_layernorm)
    x_dev = torch.from_numpy(wl.x).to(dev)
    mask_dev = torch.from_numpy(wl.mask_add.reshape(B, SEQ)).to(dev).contiguous()
    kv_len = ops.mask_to_kv_len(mask_dev)
    hidden = torch.empty((B, SEQ, cfg.hidden), dtype=torch.float16, device=dev)
    out_dev = torch.empty((B, SEQ, cfg.hidden), dtype=torch.float32, device=dev)

    def step_resident():
        ops.convert(x_dev, torch.float16, out=hidden)
        enc.forward_hidden(hidden, mask_dev, kv_len)
        ops.convert(hidden, torch.float32, out=out_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """One Forward as a CUDA graph (the launch sequence is fixed: same buffers, same kernels every step)."""
        if args.no_graph:
            return None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g
        except Exception as e:   # pragma: no cover - depends on the driver
            sys.stderr.write("CUDA graph capture failed (%s); running eagerly\n" % e)
            torch.cuda.synchronize()
            return None

    for _ in range(3):
        step_resident()
    torch.cuda.synchronize()
    n0 = capi.launch_count()
    step_resident()
    launches_per_step = capi.launch_count() - n0
    graph = capture(step_resident)
    run_step = graph.replay if graph is not None else step_resident
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()

    # ---- timed region: device-resident inputs
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = launches_per_step * args.steps      # kernels of this library executed in the timed region
    clocks = sampler.stop()
    if capi.device_status() != capi.OK:
        raise SystemExit("device status word set: a bounded wait ran out")

    # ---- e2e: host buffers, copies inside the timed region (double-buffered so copies overlap the previous step)
    x_host = torch.from_numpy(wl.x).pin_memory()
    out_host = [torch.empty((B, SEQ, cfg.hidden), dtype=torch.float32).pin_memory() for _ in range(2)]
    x_in = [torch.empty_like(x_dev) for _ in range(2)]
    o_out = [torch.empty_like(out_dev) for _ in range(2)]
    hid = [torch.empty_like(hidden) for _ in range(2)]
    s_copy_in, s_copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_main = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]

    def compute_on(b):
        ops.convert(x_in[b], torch.float16, out=hid[b])
        enc.forward_hidden(hid[b], mask_dev, kv_len)
        ops.convert(hid[b], torch.float32, out=o_out[b])

    e2e_graphs = [capture(lambda b=b: compute_on(b)) for b in range(2)]

    def e2e_loop(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_copy_in):
                s_copy_in.wait_event(ev_free[b])           # the compute that last read x_in[b] is done
                x_in[b].copy_(x_host, non_blocking=True)
                ev_in[b].record(s_copy_in)
            s_main.wait_event(ev_in[b])
            s_main.wait_event(ev_out[b])                    # o_out[b] has been drained to the host
            if e2e_graphs[b] is not None:
                e2e_graphs[b].replay()
            else:
                compute_on(b)
            ev_free[b].record(s_main)
            ev_done[b].record(s_main)
            with torch.cuda.stream(s_copy_out):
                s_copy_out.wait_event(ev_done[b])
                out_host[b].copy_(o_out[b], non_blocking=True)
                ev_out[b].record(s_copy_out)

    e2e_loop(4)
    barrier()
    t0 = time.perf_counter()
    e2e_loop(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    h2d = x_host.numel() * 4
    d2h = out_host[0].numel() * 4

    # ---- the same with half-precision host buffers (RESERVED_FP16_TEST Mats in the plug-in): half the bytes over PCIe,
    # no conversion launches; the copies go straight into / out of the encoder's hidden-state buffer
    x_host16 = torch.from_numpy(wl.x.astype(np.float16)).pin_memory()
    out_host16 = [torch.empty((B, SEQ, cfg.hidden), dtype=torch.float16).pin_memory() for _ in range(2)]
    half_graphs = [capture(lambda b=b: enc.forward_hidden(hid[b], mask_dev, kv_len)) for b in range(2)]

    def half_loop(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_copy_in):
                s_copy_in.wait_event(ev_out[b])            # hid[b]'s previous result has been drained to the host
                hid[b].view(B, SEQ, cfg.hidden).copy_(x_host16, non_blocking=True)
                ev_in[b].record(s_copy_in)
            s_main.wait_event(ev_in[b])
            if half_graphs[b] is not None:
                half_graphs[b].replay()
            else:
                enc.forward_hidden(hid[b], mask_dev, kv_len)
            ev_done[b].record(s_main)
            with torch.cuda.stream(s_copy_out):
                s_copy_out.wait_event(ev_done[b])
                out_host16[b].copy_(hid[b].view(B, SEQ, cfg.hidden), non_blocking=True)
                ev_out[b].record(s_copy_out)

    torch.cuda.synchronize()
    half_loop(4)
    barrier()
    t0 = time.perf_counter()
    half_loop(args.steps)
    torch.cuda.synchronize()
    e2e_half_s = time.perf_counter() - t0
    barrier()

    # ---- roofline of the dominant kernel (the GEMM): an instrumented pass with an event pair around every launch
    tokens = B * SEQ
    H, F = cfg.hidden, cfg.ffn
    shapes = {"qkv": (tokens, 3 * H, H), "out_proj": (tokens, H, H), "ffn1": (tokens, F, H), "ffn2": (tokens, H, F)}
    ev_pairs = {k: [] for k in list(shapes) + ["attention", "layernorm"]}

    def timed(name, fn):
        a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b2.record()
        ev_pairs[name].append((a, b2))
        return r

    def instrumented_step():
        h = ops.convert(x_dev, torch.float16, out=hidden)
        for L in enc.layers:
            qkv = timed("qkv", lambda: ops.linear(h, L["w_qkv"], L["b_qkv"]))
            ctx = timed("attention", lambda: ops.attention(qkv, cfg.heads, mask_dev, kv_len))
            t = timed("out_proj", lambda: ops.linear(ctx, L["w_o"], L["b_o"], residual=h,
                                                     epilogue=ops.EPI_BIAS_RESIDUAL))
            a = timed("layernorm", lambda: ops.add_layernorm(t, L["ln1_g"], L["ln1_b"], cfg.ln_eps))
            f1 = timed("ffn1", lambda: ops.linear(a, L["w_ffn1"], L["b_ffn1"], epilogue=ops.EPI_BIAS_GELU))
            t2 = timed("ffn2", lambda: ops.linear(f1, L["w_ffn2"], L["b_ffn2"], residual=a,
                                                  epilogue=ops.EPI_BIAS_RESIDUAL))
            h = timed("layernorm", lambda: ops.add_layernorm(t2, L["ln2_g"], L["ln2_b"], cfg.ln_eps))

    # The host needs ~20 us per launch-plus-two-events, the kernels 10-35 us: issued naively, the event pairs would time
    # the host.  Each instrumented step is therefore queued behind a spin kernel that holds the stream for a few
    # milliseconds, so that all its launches and events are already in the queue when the GPU reaches them and every
    # event pair spans exactly one kernel on the device (launch gap included).
    def hold_stream():
        torch.cuda._sleep(int(12e6))          # ~6 ms of GPU clock cycles

    for _ in range(2):
        instrumented_step()
    torch.cuda.synchronize()
    for k in ev_pairs:
        ev_pairs[k].clear()
    for _ in range(min(args.steps, 20)):
        hold_stream()
        instrumented_step()
        torch.cuda.synchronize()
    kernel_ms = {k: [a.elapsed_time(b2) for a, b2 in v] for k, v in ev_pairs.items()}
    gemm_flops = gemm_ms = 0.0
    per_shape = {}
    for k, (m, n, kk) in shapes.items():
        fl = 2.0 * m * n * kk
        tms = statistics.mean(kernel_ms[k])
        per_shape[k] = {"M": m, "N": n, "K": kk, "ms": round(tms, 4), "tflops": round(fl / tms / 1e9, 1)}
        gemm_flops += fl * len(kernel_ms[k])
        gemm_ms += sum(kernel_ms[k])
    peaks = measured_peaks()
    achieved_bracketed = gemm_flops / gemm_ms / 1e9
    n_gemm = sum(len(kernel_ms[k]) for k in shapes)

    # The roofline figure itself: the step's GEMM launches alone, in their order, with every layer's own weights (170 MB
    # per pass, more than L2) and the step's activation buffers, replayed as a CUDA graph and timed with one event
    # pair.  (An event pair around every single launch adds 3-6 us of event handling to each 15-40 us kernel and
    # switches off the overlap of consecutive launches; those bracketed figures are kept in `per_shape`.)
    qkv_b = torch.empty(tokens, 3 * H, device=dev, dtype=torch.float16)
    ctx_b = torch.randn(tokens, H, device=dev).to(torch.float16)
    t_b = torch.empty(tokens, H, device=dev, dtype=torch.float16)
    f_b = torch.empty(tokens, F, device=dev, dtype=torch.float16)
    h_b = torch.randn(tokens, H, device=dev).to(torch.float16)

    def gemm_only_step():
        for L in enc.layers:
            ops.linear(h_b, L["w_qkv"], L["b_qkv"], out=qkv_b)
            ops.linear(ctx_b, L["w_o"], L["b_o"], residual=h_b, epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b)
            ops.linear(h_b, L["w_ffn1"], L["b_ffn1"], epilogue=ops.EPI_BIAS_GELU, out=f_b)
            ops.linear(f_b, L["w_ffn2"], L["b_ffn2"], residual=h_b, epilogue=ops.EPI_BIAS_RESIDUAL, out=t_b)

    for _ in range(3):
        gemm_only_step()
    torch.cuda.synchronize()
    gemm_graph = capture(gemm_only_step)
    run_gemms = gemm_graph.replay if gemm_graph is not None else gemm_only_step
    for _ in range(3):
        run_gemms()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 50)
    g0.record()
    for _ in range(reps):
        run_gemms()
    g1.record()
    torch.cuda.synchronize()
    gemm_launches_per_pass = 4 * len(enc.layers)
    gemm_pass_ms = g0.elapsed_time(g1) / reps
    flops_per_pass = sum(2.0 * m * n * kk for (m, n, kk) in shapes.values()) * len(enc.layers)
    achieved = flops_per_pass / gemm_pass_ms / 1e9
    attn_ms = statistics.mean(kernel_ms["attention"])
    attn_flops = 4.0 * SEQ * SEQ * 64 * cfg.heads * B

    # ---- reduce over ranks
    ms_t = torch.tensor([ms_total, e2e_s * 1e3, e2e_half_s * 1e3], dtype=torch.float64, device=dev)
    ms_t = reduce_max_over_ranks(ms_t, world)
    ms_total_max, e2e_ms_max = float(ms_t[0]), float(ms_t[1])
    seqs = world * B * args.steps
    value = seqs / (ms_total_max / 1e3)
    e2e_value = seqs / (e2e_ms_max / 1e3)
    e2e_half_value = seqs / (float(ms_t[2]) / 1e3)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, kind, desc = cpu_reference_seq_per_s(8, 1, layers=12, warmup=1, iters=2)
        cpu_baseline = {"value": v, "unit": UNIT, "cores": 1, "kind": kind, "sample": desc}

    tnn_plugin = None
    if rank == 0 and world == 1 and not args.no_tnn_plugin:
        tnn_plugin = tnn_plugin_seq_per_s(wl)

    if rank == 0:
        flops_per_seq = model_synth.layer_flops(SEQ, H, F) * len(enc.layers)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_total_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "config 2: BERT-base 12-layer encoder, batch %d x seq %d per GPU, fp16 weights, "
                                   "all sequences full length, fp32 activations in/out" % (B, SEQ),
                       "batch_per_gpu": B, "seq_len": SEQ, "layers": len(enc.layers),
                       "parallelism": "independent replicas, batch-sharded, no collective",
                       "launch": "CUDA graph of one Forward" if graph is not None else "eager launches",
                       "layernorm": "folded into the GEMM epilogues" if enc.fold else "separate kernels",
                       "l2": "per-step working set (170 MB fp16 weights + activations) exceeds the 126 MB L2; "
                             "no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "pinned fp32 host buffers, copies double-buffered on side streams, wall clock"
                            + ("" if numa is None else "; rank bound to the %d CPUs local to its GPU" % numa)},
            "e2e_half_io": {"value": e2e_half_value, "unit": UNIT, "h2d_bytes_per_step": h2d // 2,
                            "d2h_bytes_per_step": d2h // 2,
                            "note": "the same with pinned fp16 host buffers (half-precision Mats): half the bytes, no "
                                    "conversion launches; informational, the fp32 line above is the e2e number"},
            "gpu_launches": launches,
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
                         "traffic": ncu_traffic_per_launch(B, per_shape),
                         "traffic_note": "DRAM read+write bytes per launch from one ncu capture per GEMM shape "
                                         "(profiles/linear_pair_kernel_config2_shapes.md), averaged over the shapes "
                                         "captured; equals the operand bytes, outputs stay in L2"},
            "attention_sweep": attention_sweep,
            "attention_sweep_note": "each point: 10 launches between one CUDA-event pair, timed before the long loops "
                                    "(burst clocks, as the measured tensor peak was)",
            "attention_kernel": {"ms": attn_ms, "tflops": attn_flops / attn_ms / 1e9,
                                 "frac_of_tensor_peak": attn_flops / attn_ms / 1e9 / peaks["tflops"]},
            "layernorm_kernel": {"ms": statistics.mean(kernel_ms["layernorm"]),
                                 "gbs": tokens * H * 2 * 2 / statistics.mean(kernel_ms["layernorm"]) / 1e6},
            "model_tflops": value * flops_per_seq / 1e12,
            "model_frac_of_tensor_peak": value * flops_per_seq / 1e12 / peaks["tflops"] / world,
            "cpu_baseline": cpu_baseline,
            "tnn_plugin": tnn_plugin,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of linear_pair_kernel, from ncu captures of the GEMM shapes
# of the default workload (batch 64 x seq 128: M = 8192).  The figures belong to that M only.
NCU_DRAM_BYTES_M8192 = {"qkv": 16.16e6 + 0.54e6, "ffn1": 17.35e6 + 2.26e6, "ffn2": 67.69e6 + 4.36e6}


def ncu_traffic_per_launch(batch, per_shape):
    if batch != BATCH_PER_GPU:
        return None
    vals = [NCU_DRAM_BYTES_M8192[k] for k in per_shape if k in NCU_DRAM_BYTES_M8192]
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="sequences per GPU per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-attention-sweep", action="store_true")
    ap.add_argument("--no-tnn-plugin", action="store_true", help="skip the measurement through TNN + plug-in")
    ap.add_argument("--fold-layernorm", action="store_true",
                    help="fold both LayerNorms of a layer into the neighbouring GEMM epilogues (5 launches per layer)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying "
                                                            "a captured CUDA graph of one Forward")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
