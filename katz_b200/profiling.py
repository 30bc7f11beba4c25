"""Small, self-contained workloads for kernel profilers and calibration runs.

    python -m katz_b200.profiling gemm           # the step's dominant linear shapes, 3 launches each
    python -m katz_b200.profiling attention      # the step's two self-attention shapes, 2 launches each
    python -m katz_b200.profiling conv           # two of the step's 3x3 convolutions, 2 launches each
    python -m katz_b200.profiling merge          # one LoRA merge over a 102-layer subset (0.7 GB of weights)
    python -m katz_b200.profiling merge-fp32     # the same subset with fp32 weights and adapters
    python -m katz_b200.profiling step [--batch B] [--latent HW]   # ONE eager UNet step
    python -m katz_b200.profiling norms          # LayerNorm / GroupNorm launches of the step's shapes
    python -m katz_b200.profiling compare-cublas # katz_linear_f16 against torch.addmm on the step's shapes (no profiler)
    python -m katz_b200.profiling compare-cudnn  # katz_conv3x3_nhwc_f16 against F.conv2d (channels-last) on the step's shapes
    python -m katz_b200.profiling ablate [--batch B] [--latent HW]     # CUDA-graph replay of the step with one entry point's
                                                 # launches left out at a time: what each family costs INSIDE the graph
    python -m katz_b200.profiling families [--batch B] [--latent HW]   # time share per kernel family of one eager step, CUDA
                                                 # events around every op (also under torchrun: the row-split step, rank 0 reports)

Every mode but the last warms up, then brackets the launches of interest with cudaProfilerStart/Stop, so that
`ncu --profile-from-start off` captures exactly those; each holds well under a few GB on the device (the `step` mode
holds the 5.1 GB of UNet weights: capture it only with single-pass metrics). Each prints one JSON line.
"""
import argparse
import json

import torch


def _time_events(fn, iters):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _bracket(fn):
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    fn()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


STEP_LINEAR_SHAPES = [(2048, 10240, 1280), (2048, 1280, 1280), (2048, 3840, 1280), (2048, 1280, 5120), (8192, 640, 640),
                      (8192, 5120, 640), (8192, 640, 2560), (1024, 1280, 1280), (8192, 8192, 4096)]


def gemm(dev, args):
    from . import ops
    shapes = [(2048, 10240, 1280), (2048, 1280, 1280), (8192, 640, 2560)]
    sets = []
    for (M, N, K) in shapes:
        sets.append((torch.randn(M, K, device=dev).half(), (torch.randn(N, K, device=dev) * 0.03).half(),
                     torch.empty(M, N, dtype=torch.float16, device=dev)))
    for x, w, o in sets:
        ops.linear(x, w, out=o)

    def run():
        for x, w, o in sets:
            for _ in range(3):
                ops.linear(x, w, out=o)
    _bracket(run)
    return {"profiled": "linear GEMMs, 3 launches each", "shapes": shapes, "kernel": ops.gemm_kernel_name(),
            "tc05_status": ops.tc05_status()}


def attention(dev, args):
    from . import ops
    shapes = [(2, 20, 1024), (2, 10, 4096), (1, 20, 1024), (1, 10, 4096)]
    bufs = []
    for (B, H, S) in shapes:
        bufs.append((torch.randn(B, S, 3 * H * 64, device=dev).half(), H, torch.empty(B, S, H * 64, dtype=torch.float16, device=dev)))

    def run(n):
        for qkv, H, o in bufs:
            C = H * 64
            for _ in range(n):
                ops.attention(qkv[:, :, :C], qkv[:, :, C:2 * C], qkv[:, :, 2 * C:], H, out=o)
    run(1)
    _bracket(lambda: run(2))
    times = []
    for qkv, H, o in bufs:        # CUDA-graph time of 10 launches per shape (no profiler)
        C = H * 64
        times.append(round(_graph_time(lambda i: ops.attention(qkv[:, :, :C], qkv[:, :, C:2 * C], qkv[:, :, 2 * C:], H, out=o), n=10), 2))
    return {"profiled": "self-attention, 2 launches each", "shapes": shapes, "graph_us_per_launch": times, "tc05_status": ops.tc05_status()}


def conv(dev, args):
    from . import ops
    shapes = [(32, 1280, 1280), (64, 640, 640)]      # (H = W, Cin, Cout) at batch 2: 10 and 6 launches per step
    bufs = []
    for (H, Cin, Cout) in shapes:
        bufs.append((torch.randn(2, H, H, Cin, device=dev).half(), (torch.randn(Cout, 3, 3, Cin, device=dev) * 0.02).half(),
                     torch.randn(Cout, device=dev).half(), torch.empty(2, H, H, Cout, dtype=torch.float16, device=dev)))

    def run(n):
        for x, w, b, o in bufs:
            for _ in range(n):
                ops.conv2d(x, w, b, out=o)
    run(1)
    _bracket(lambda: run(2))
    times = [round(_graph_time(lambda i: ops.conv2d(x, w, b, out=o), n=10), 2) for x, w, b, o in bufs]
    return {"profiled": "3x3 convolutions, 2 launches each", "shapes": shapes, "graph_us_per_launch": times,
            "kernel": ops.gemm_kernel_name(), "tc05_status": ops.tc05_status()}


def _subset_merger(dev, dtype):
    from collections import OrderedDict
    from .lora import LoraMerger
    from .params import SDXL_UNET_CONFIG, lora_target_keys, unet_param_shapes
    shapes = unet_param_shapes(SDXL_UNET_CONFIG)
    keys = [k for k in lora_target_keys(SDXL_UNET_CONFIG, include_proj=True) if k.startswith("down_blocks.2.attentions.0.")]
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    W = OrderedDict((k, (torch.randn(shapes[k], generator=g, device=dev) * 0.02).to(dtype)) for k in keys)
    ad = OrderedDict((k, ((torch.randn(w.shape[0], 64, generator=g, device=dev) * 0.01).to(dtype),
                          (torch.randn(64, w.shape[1], generator=g, device=dev) / 64).to(dtype))) for k, w in W.items())
    return LoraMerger(W), ad, keys


def merge(dev, args, dtype=torch.float16):
    merger, ad, keys = _subset_merger(dev, dtype)
    for _ in range(2):
        merger.merge(ad, 1.0)
    _bracket(lambda: merger.merge(ad, 1.0))
    return {"profiled": "one LoRA merge", "dtype": str(dtype), "layers": len(keys), "bytes": merger.algorithmic_bytes([64])}


def merge_fp32(dev, args):
    return merge(dev, args, torch.float32)


def step(dev, args):
    from . import _lib, ops
    from .params import SDXL_UNET_CONFIG, init_state_dict, unet_param_shapes
    from .unet import KatzUNet
    cfg = SDXL_UNET_CONFIG
    unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev))
    B, HW = args.batch, args.latent
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, 4, HW, HW, generator=g).half().to(dev)
    ctx = torch.randn(B, 77, 2048, generator=g).half().to(dev)
    added = {"text_embeds": torch.randn(B, 1280, generator=g).half().to(dev),
             "time_ids": torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half().to(dev)}
    t = torch.tensor([500.0], device=dev)
    for _ in range(2):
        unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
    n0 = _lib.launch_count()
    _bracket(lambda: unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added))
    return {"profiled": "one eager UNet step", "batch": B, "latent": HW, "launches": _lib.launch_count() - n0,
            "tc05_status": ops.tc05_status()}


def norms(dev, args):
    from . import ops
    from .ops import ACT_SILU
    ln = [(2048, 1280), (8192, 640)]
    gn = [(2, 32 * 32, 1280), (2, 64 * 64, 640), (2, 128 * 128, 320), (2, 32 * 32, 2560)]
    lnb = [(torch.randn(r, c, device=dev).half(), torch.ones(c, device=dev).half(), torch.zeros(c, device=dev).half()) for r, c in ln]
    gnb = [(torch.randn(b, hw, c, device=dev).half(), torch.ones(c, device=dev).half(), torch.zeros(c, device=dev).half()) for b, hw, c in gn]

    def run():
        for x, g_, b_ in lnb:
            ops.layer_norm(x, g_, b_)
        for x, g_, b_ in gnb:
            ops.group_norm_nhwc(x, g_, b_, 32, 1e-5, ACT_SILU)
    run()
    _bracket(run)
    return {"profiled": "LayerNorm and GroupNorm launches", "layer_norm": ln, "group_norm": gn}


def compare_cublas(dev, args):
    """CUDA events around CUDA graphs of 20 launches, distinct weights per launch (they are cold in the step, too)."""
    from . import ops

    def graph_time(fn, n=20):
        for _ in range(3):
            fn(0)
        torch.cuda.synchronize()
        gr, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(st):
            fn(0)
            with torch.cuda.graph(gr, stream=st):
                for i in range(n):
                    fn(i)
        torch.cuda.synchronize()
        gr.replay()
        return _time_events(gr.replay, 5) * 1e3 / n
    rows = []
    for (M, N, K) in STEP_LINEAR_SHAPES:
        nw = 6 if N * K < 3e7 else 2
        if args.cold:      # as in the step: more distinct weights than the 126 MB L2 holds, every launch reads its weights from HBM
            nw = min(96, max(2, int(3e8 // (N * K * 2)) + 1))
        x = torch.randn(M, K, device=dev).half()
        ws = [(torch.randn(N, K, device=dev) * 0.03).half() for _ in range(nw)]
        b = torch.randn(N, device=dev).half()
        o = torch.empty(M, N, dtype=torch.float16, device=dev)
        n = max(20, nw) if args.cold else 20
        tk = graph_time(lambda i: ops.linear(x, ws[i % nw], b, out=o), n)
        tc = graph_time(lambda i: torch.addmm(b, x, ws[i % nw].t(), out=o), n)
        fl = 2.0 * M * N * K
        rows.append({"shape": [M, N, K], "katz_us": round(tk, 1), "katz_tflops": round(fl / tk / 1e6),
                     "cublas_us": round(tc, 1), "cublas_tflops": round(fl / tc / 1e6), "cublas_over_katz": round(tc / tk, 2)})
    return {"compared": "linear + bias, fp16, CUDA graph of 20 launches", "cold_weights": bool(args.cold), "rows": rows, "tc05_status": ops.tc05_status()}


# (H = W of the input, Cin, Cout, stride, launches per step) of the SDXL UNet's 3x3 convolutions at batch 2, latent 128 x 128
STEP_CONV_SHAPES = [(128, 320, 320, 1, 7), (128, 960, 320, 1, 1), (128, 640, 320, 1, 2), (128, 320, 320, 2, 1),
                    (64, 320, 640, 1, 1), (64, 640, 640, 1, 6), (64, 1920, 640, 1, 1), (64, 1280, 640, 1, 1), (64, 960, 640, 1, 1),
                    (64, 640, 640, 2, 1), (128, 640, 640, 1, 1),
                    (32, 640, 1280, 1, 1), (32, 1280, 1280, 1, 10), (32, 2560, 1280, 1, 2), (32, 1920, 1280, 1, 1), (64, 1280, 1280, 1, 1)]


def _graph_time(fn, n=20, reps=5):
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    gr, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(st):
        fn(0)
        with torch.cuda.graph(gr, stream=st):
            for i in range(n):
                fn(i)
    torch.cuda.synchronize()
    gr.replay()
    return _time_events(gr.replay, reps) * 1e3 / n


def compare_cudnn(dev, args):
    """The step's 3x3 convolutions (bias in the epilogue), CUDA graphs of 10 launches cycling through distinct weights."""
    import torch.nn.functional as F
    from . import ops
    rows, tot_k, tot_c = [], 0.0, 0.0
    B = args.batch
    for (H, Cin, Cout, stride, count) in STEP_CONV_SHAPES:
        nw = 4
        x = torch.randn(B, H, H, Cin, device=dev).half()
        ws = [(torch.randn(Cout, 3, 3, Cin, device=dev) * 0.02).half() for _ in range(nw)]
        b = torch.randn(Cout, device=dev).half()
        Ho = H // stride
        o = torch.empty(B, Ho, Ho, Cout, dtype=torch.float16, device=dev)
        tk = _graph_time(lambda i: ops.conv2d(x, ws[i % nw], b, stride=stride, out=o), n=10)
        xc = x.permute(0, 3, 1, 2)                      # NCHW view of channels-last memory
        wc = [w.permute(0, 3, 1, 2) for w in ws]
        tc = _graph_time(lambda i: F.conv2d(xc, wc[i % nw], b, stride=stride, padding=1), n=10)
        fl = 2.0 * B * Ho * Ho * Cout * 9 * Cin
        tot_k += tk * count
        tot_c += tc * count
        rows.append({"shape": [H, Cin, Cout, stride], "per_step": count, "katz_us": round(tk, 1), "katz_tflops": round(fl / tk / 1e6),
                     "cudnn_us": round(tc, 1), "cudnn_tflops": round(fl / tc / 1e6), "cudnn_over_katz": round(tc / tk, 2)})
    return {"compared": "3x3 conv + bias, fp16 NHWC, CUDA graph of 10 launches", "rows": rows, "katz_step_total_us": round(tot_k, 1),
            "cudnn_step_total_us": round(tot_c, 1), "tc05_status": ops.tc05_status()}


def ablate(dev, args):
    """What each kernel family costs inside the CUDA-graph replay of the step: the step is captured once whole and once per
    family with that family's entry points skipped (their outputs keep whatever the buffers held, so the results are
    meaningless; only the replay time is read). The difference includes the launch boundaries the family adds, which a list
    of isolated kernel times does not show."""
    from . import _lib, ops
    from .params import SDXL_UNET_CONFIG, init_state_dict, unet_param_shapes
    from .unet import KatzUNet
    cfg = SDXL_UNET_CONFIG
    unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev))
    B, HW = args.batch, args.latent
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, 4, HW, HW, generator=g).half().to(dev)
    ctx = torch.randn(B, 77, 2048, generator=g).half().to(dev)
    added = {"text_embeds": torch.randn(B, 1280, generator=g).half().to(dev),
             "time_ids": torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half().to(dev)}
    t = torch.tensor([500.0], device=dev)
    real_call = ops.call
    skipped = set()
    counts = {}

    def call(name, *a):
        if name in skipped:
            counts[name] = counts.get(name, 0) + 1
            return
        real_call(name, *a)
    ops.call = call

    def replay_ms():
        for _ in range(2):
            unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
        torch.cuda.synchronize()
        gr, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(st):
            with torch.cuda.graph(gr, stream=st):
                unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
        torch.cuda.synchronize()
        for _ in range(3):
            gr.replay()
        return _time_events(gr.replay, 10)
    families_ = [("nothing", ()), ("LayerNorm", ("katz_layer_norm_f16",)),
                 ("GroupNorm", ("katz_group_norm_nhwc_f16",)),
                 ("self- and cross-attention", ("katz_attention_f16", "katz_attention_split_f16", "katz_attention_f16_mma")),
                 ("self-attention (tcgen05)", ("katz_attention_f16", "katz_attention_split_f16")),
                 ("cross-attention (mma.sync)", ("katz_attention_f16_mma",)),
                 ("GEGLU GEMM", ("katz_linear_geglu_f16", "katz_linear_geglu_ex_f16")),
                 ("3x3 convolution (tcgen05)", ("katz_conv3x3_nhwc_f16",)),
                 ("linear GEMM", ("katz_linear_f16", "katz_linear_ex_f16")),
                 ("concat / upsample / layout", ("katz_concat_channels_f16", "katz_upsample_nearest2x_nhwc_f16"))]
    rows, base = [], None
    for name, eps in families_:
        skipped.clear()
        skipped.update(eps)
        counts.clear()
        ms = replay_ms()
        if base is None:
            base = ms
        rows.append({"skipped": name, "replay_ms": round(ms, 3), "family_ms": round(base - ms, 3),
                     "calls_skipped_per_step": sum(counts.values()) // 3 if counts else 0})
    ops.call = real_call
    return {"profiled": "CUDA-graph replay with one family skipped at a time", "batch": B, "latent": HW, "rows": rows}


def families(dev, args):
    """Time share per kernel family of ONE eager UNet step: CUDA events (with a synchronisation) around every call of the op
    layer, so launch gaps are excluded and absolute times are those of isolated kernels; the SHARES say where a step goes.
    Under torchrun every rank runs the row-split step (cfg x rows as bench.py splits it) and rank 0 prints."""
    import collections
    import os
    import torch.distributed as dist
    from . import latent_parallel, ops
    from .params import SDXL_UNET_CONFIG, init_state_dict, unet_param_shapes
    from .unet import KatzUNet
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    cfg = SDXL_UNET_CONFIG
    unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev))
    B, HW = args.batch, args.latent
    halves, rows_world, half, row_rank, lb = latent_parallel.cfg_rows_layout(B, world, rank)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, 4, HW, HW, generator=g).half().to(dev)[half * lb:(half + 1) * lb]
    ctx = torch.randn(B, 77, 2048, generator=g).half().to(dev)[half * lb:(half + 1) * lb]
    added = {"text_embeds": torch.randn(B, 1280, generator=g).half().to(dev)[half * lb:(half + 1) * lb],
             "time_ids": torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * lb).half().to(dev)}
    t = torch.tensor([500.0], device=dev)
    if rows_world > 1:
        grp = None
        if halves > 1:
            groups = [dist.new_group(list(range(h * rows_world, (h + 1) * rows_world))) for h in range(halves)]
            grp = groups[half]
        rp = latent_parallel.RowParallel(row_rank, rows_world, grp)
        if os.environ.get("KATZ_PEER", "1") != "0":
            from .peer import PeerArena
            rp.peer = PeerArena(row_rank, rows_world, group=grp, device=dev)
        unet.rp = rp
    for _ in range(2):
        unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
    torch.cuda.synchronize()
    rec = collections.OrderedDict()

    def wrap(mod, name, family):
        fn = getattr(mod, name)

        def f(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            r = fn(*a, **k)
            e1.record()
            torch.cuda.synchronize()
            ent = rec.setdefault(family, [0, 0.0])
            ent[0] += 1
            ent[1] += e0.elapsed_time(e1) * 1e3
            return r
        setattr(mod, name, f)
    for name, fam in (("linear", "linear GEMM"), ("feed_forward_geglu", "GEGLU GEMM"), ("conv2d", "convolution"), ("attention", "attention"),
                      ("layer_norm", "LayerNorm"), ("group_norm_nhwc", "GroupNorm"), ("group_norm_stats", "GroupNorm"),
                      ("group_norm_apply", "GroupNorm"), ("halo_assemble", "halo assemble"), ("concat_channels", "concat"),
                      ("upsample_nearest2x", "upsample")):
        wrap(ops, name, fam)
    if unet.rp is not None and unet.rp.peer is not None:
        wrap(unet.rp.peer, "allgather", "peer all-gather")
    if world > 1:
        dist.barrier()
    unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
    torch.cuda.synchronize()
    total = sum(v[1] for v in rec.values())
    out = {"profiled": "kernel families of one eager step (isolated launches, CUDA events)", "world": world, "split": "cfg%d x rows%d" % (halves, rows_world),
           "local_batch": lb, "latent": HW, "total_us": round(total, 1),
           "families": [{"family": k, "calls": v[0], "us": round(v[1], 1), "share": round(v[1] / total, 4)} for k, v in
                        sorted(rec.items(), key=lambda kv: -kv[1][1])]}
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        if rank != 0:
            os._exit(0)
        print(json.dumps(out), flush=True)
        os._exit(0)
    return out


MODES = {"families": families, "gemm": gemm, "attention": attention, "conv": conv, "merge": merge, "merge-fp32": merge_fp32, "step": step, "norms": norms,
         "compare-cublas": compare_cublas, "compare-cudnn": compare_cudnn, "ablate": ablate}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=sorted(MODES))
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--latent", type=int, default=128)
    ap.add_argument("--cold", action="store_true", help="compare-cublas: weights cycle through more memory than L2 holds")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("katz_b200.profiling needs a CUDA device")
    import os
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    print(json.dumps(MODES[args.mode](dev, args)), flush=True)


if __name__ == "__main__":
    main()
