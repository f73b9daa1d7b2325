"""Run one kernel of the path a few times in isolation (for `ncu` captures and quick timing).

    python profile_case.py linear --M 8192 --N 2304 --K 768 [--epilogue gelu] [--block-n 256] [--iters 5]
    python profile_case.py attention --B 64 --S 128 --heads 12
    python profile_case.py layernorm --rows 8192 --H 768
    python profile_case.py encoder --B 64 --S 128 --layers 2
    python profile_case.py encoder --config 4 --iters 10          # BERT-large, 64 x 384, ragged, 24 layers
    python profile_case.py qa_head --rows 131072 --H 768
    python profile_case.py embedding --B 1024 --S 128 --H 768

Prints the mean CUDA-event time per launch.  Operands are seeded random device tensors; sizes default to the
benchmark's config 2 shapes.
"""
import argparse

import torch

from tnn_b200 import capi, ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["linear", "attention", "layernorm", "encoder", "qa_head", "embedding"])
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=2304)
    ap.add_argument("--K", type=int, default=768)
    ap.add_argument("--epilogue", default="bias", choices=["bias", "gelu", "residual"])
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--ln-in", action="store_true", help="linear: x is pre-LayerNorm, LayerNorm folded into the GEMM")
    ap.add_argument("--res-ln", action="store_true", help="linear: residual goes through a folded LayerNorm")
    ap.add_argument("--out-stats", action="store_true", help="linear: write row statistics of the output")
    ap.add_argument("--B", type=int, default=64)
    ap.add_argument("--S", type=int, default=128)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--H", type=int, default=768)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--fold", action="store_true", help="encoder: the five-launch layer with both LayerNorms folded")
    ap.add_argument("--config", type=int, default=0, help="encoder: run benchmark configuration 2..5 as specified")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--eager", action="store_true", help="time host-launched calls instead of a CUDA graph replay")
    a = ap.parse_args()
    dt = torch.float16 if a.dtype == "f16" else torch.bfloat16
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    capi.lib()

    if a.kernel == "linear":
        x = torch.randn(a.M, a.K, device=dev).to(dt)
        w = (torch.randn(a.N, a.K, device=dev) * 0.02).to(dt)
        b = torch.randn(a.N, device=dev)
        r = torch.randn(a.M, a.N, device=dev).to(dt) if a.epilogue == "residual" else None
        y = torch.empty(a.M, a.N, device=dev, dtype=dt)
        epi = {"bias": ops.EPI_BIAS, "gelu": ops.EPI_BIAS_GELU, "residual": ops.EPI_BIAS_RESIDUAL}[a.epilogue]
        kw = {}
        if a.ln_in:
            kw["ln_in"] = (torch.rand(ops.stats_buffer(a.M, a.K, dev).shape, device=dev) + 32.0,
                           torch.randn(a.N, device=dev), torch.randn(a.N, device=dev))
        if a.res_ln:
            kw["res_ln"] = (torch.rand(ops.stats_buffer(a.M, a.N, dev).shape, device=dev) + 32.0,
                            torch.ones(a.N, device=dev), torch.zeros(a.N, device=dev))
        if a.out_stats:
            kw["out_stats"] = ops.stats_buffer(a.M, a.N, dev)
        fn = lambda: ops.linear(x, w, b, residual=r, epilogue=epi, out=y, block_n=a.block_n, **kw)  # noqa: E731
        work = 2.0 * a.M * a.N * a.K
        unit = "TFLOP/s"
    elif a.kernel == "attention":
        H = a.heads * 64
        qkv = torch.randn(a.B, a.S, 3 * H, device=dev).to(dt)
        mask = torch.zeros(a.B, a.S, device=dev)
        kv = ops.mask_to_kv_len(mask)
        out = torch.empty(a.B, a.S, H, device=dev, dtype=dt)
        fn = lambda: ops.attention(qkv, a.heads, mask, kv, out=out)  # noqa: E731
        work = 4.0 * a.S * a.S * 64 * a.heads * a.B
        unit = "TFLOP/s"
    elif a.kernel == "layernorm":
        x = torch.randn(a.rows, a.H, device=dev).to(dt)
        g = torch.ones(a.H, device=dev)
        be = torch.zeros(a.H, device=dev)
        y = torch.empty_like(x)
        fn = lambda: ops.add_layernorm(x, g, be, 1e-12, out=y)  # noqa: E731
        work = 2.0 * a.rows * a.H * 2 * 1e3   # bytes, scaled so that the print below reads GB/s
        unit = "GB/s"
    elif a.kernel == "qa_head":
        x = torch.randn(a.rows, a.H, device=dev).to(dt)
        w = (torch.randn(a.H, 2, device=dev) * 0.05).contiguous()
        b = torch.randn(2, device=dev)
        out = torch.empty(2, a.rows, device=dev)
        fn = lambda: ops.qa_head(x, w, b, out=out)  # noqa: E731
        work = (a.rows * a.H * 2 + a.rows * 8) * 1e3   # bytes: x once, two fp32 logits per token
        unit = "GB/s"
    elif a.kernel == "embedding":
        vocab = 30522
        ids = torch.randint(0, vocab, (a.B, a.S), device=dev, dtype=torch.int32)
        seg = torch.randint(0, 2, (a.B, a.S), device=dev, dtype=torch.int32)
        word = torch.randn(vocab, a.H, device=dev).to(dt)
        typ = torch.randn(2, a.H, device=dev).to(dt)
        pos = torch.randn(512, a.H, device=dev).to(dt)
        g = torch.ones(a.H, device=dev)
        be = torch.zeros(a.H, device=dev)
        out = torch.empty(a.B, a.S, a.H, device=dev, dtype=dt)
        fn = lambda: ops.embedding_layernorm(ids, seg, word, typ, pos, g, be, 1e-12, out=out)  # noqa: E731
        work = a.B * a.S * a.H * 2 * 4 * 1e3   # bytes per token: three table rows in, one row out
        unit = "GB/s"
    else:
        from tnn_b200 import model_synth
        from tnn_b200.encoder import Encoder
        if a.config:
            # one of the benchmark's five configurations at its own batch, lengths and depth (3 and 4 are ragged:
            # the figure printed is on effective FLOPs, padding earns nothing)
            wl = model_synth.config_workload(a.config)
            a.B, a.S = wl.x.shape[0], wl.x.shape[1]
        else:
            wl = model_synth.make_workload(model_synth.BERT_BASE, a.B, a.S, seed=0, num_layers=a.layers)
        enc = Encoder.from_workload(wl, dt, dev, fold_layernorm=a.fold)
        hidden = torch.from_numpy(wl.x).to(dev).to(dt)
        mask = torch.from_numpy(wl.mask_add.reshape(a.B, a.S)).to(dev)
        kv = ops.mask_to_kv_len(mask)
        fn = lambda: enc.forward_hidden(hidden, mask, kv)  # noqa: E731
        work = float(model_synth.workload_flops(wl))
        unit = "TFLOP/s"

    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    # The `iters` launches are replayed from a CUDA graph so that host launch overhead (tens of microseconds per
    # call through ctypes) does not enter the measurement of short kernels.
    run = None
    if not a.eager:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(a.iters):
                    fn()
            run = graph.replay
            run()
            torch.cuda.synchronize()
        except Exception:
            run = None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if run is not None:
        run()
    else:
        for _ in range(a.iters):
            fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print("%s: %.4f ms per call, %.1f %s, device status %d" % (a.kernel, ms, work / ms / 1e9, unit,
                                                              capi.device_status()))
    if a.kernel == "encoder":
        print("encoder: %d sequences x %d tokens, %d layers: %.1f sequences/s" % (a.B, a.S, len(wl.weights),
                                                                                 a.B / ms * 1e3))


if __name__ == "__main__":
    main()
