"""Benchmark of the hot path: one SDXL UNet denoising step (fp16, batch 2 = CFG, latent 128x128, one rank-64 LoRA
merged), plus the LoRA merge itself, on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl katz|reference]

Prints ONE JSON line (rank 0). `value` is milliseconds per UNet step with inputs resident in HBM (CUDA-graph replay,
CUDA-event timing, max over ranks); `e2e` is the same step through the public `unet(...)` call with pinned HOST inputs
copied in and the prediction copied out every step. `roofline` describes the dominant kernel (the GEMM behind the
linears) timed alone; `step_roofline` the whole step against the sustained tensor peak; `lora_merge` the merge pass
against the HBM peak. `--impl reference` times the CPU restatement of the reference's torch path on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(int(float(r[1])) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [int(float(r[2])) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def time_events(fn, iters, stream=None):
    """Average milliseconds of fn() over `iters` calls, CUDA events on the current stream, sync on both sides."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def make_lora(unet, keys, rank, seed, device):
    from collections import OrderedDict
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    ad = OrderedDict()
    for k, w in unet.lora_targets(keys).items():
        o, n = w.shape
        down = (torch.randn(rank, n, generator=g, device=device) / rank).half()
        up = (torch.randn(o, rank, generator=g, device=device) * 0.01).half()
        ad[k] = (up, down)
    return ad


def cpu_reference_step(sample_hw, batch, threads):
    """The CPU restatement of the reference's torch path (oracle.unet_oracle, fp32) on the host cores, on a bounded
    sample of the workload: the full SDXL UNet at batch `batch`, latent `sample_hw`^2. Returns (seconds, flops)."""
    from collections import OrderedDict
    from katz_b200.params import SDXL_UNET_CONFIG, unet_param_shapes, unet_step_flops
    from oracle import unet_oracle
    torch.set_num_threads(threads)
    cfg = SDXL_UNET_CONFIG
    g = torch.Generator().manual_seed(0)
    sd = OrderedDict()
    for k, shp in unet_param_shapes(cfg).items():
        fan = 1
        for s in shp[1:]:
            fan *= s
        t = torch.empty(shp, dtype=torch.float32)
        if len(shp) == 1 and ("norm" in k):
            t.fill_(1.0 if k.endswith("weight") else 0.0)
        else:
            t.uniform_(-1.0 / max(fan, 1) ** 0.5, 1.0 / max(fan, 1) ** 0.5, generator=g)
        sd[k] = t
    x = torch.randn(batch, 4, sample_hw, sample_hw, generator=g)
    ctx = torch.randn(batch, 77, 2048, generator=g)
    te = torch.randn(batch, 1280, generator=g)
    ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * batch)
    with torch.no_grad():
        t0 = time.time()
        unet_oracle.unet_step(sd, cfg, x, 500.0, ctx, te, ti)
        dt = time.time() - t0
    return dt, unet_step_flops(cfg, batch, sample_hw, sample_hw)["total"]


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own implementation of the path is PyTorch on the host (its GPU path needs
    weights/a CUDA build of torch that are the same library calls this project replaces); what travels to the bench
    box is the CPU restatement of that torch path, pinned to the reference by tests/golden. Rank 0 only."""
    if rank != 0:
        return
    from katz_b200.params import SDXL_UNET_CONFIG, unet_step_flops
    threads = os.cpu_count() or 1
    full = unet_step_flops(SDXL_UNET_CONFIG, 2, 128, 128)["total"]
    hw, b = 32, 1
    times = []
    for i in range(args.warmup + args.steps):
        dt, fl = cpu_reference_step(hw, b, threads)
        if i >= args.warmup:
            times.append(dt)
        if sum(times) > 120:
            break
    per = sum(times) / len(times)
    ms_full = per * 1e3 * (full / fl)
    line = {
        "impl": "reference", "metric": "sdxl_unet_step_ms", "value": ms_full, "unit": "ms", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "SDXL UNet step, batch 2 (CFG), latent 128x128, 1 rank-64 LoRA merged (configs[1])",
                   "latent_parallel": args.gpus},
        "cpu_baseline": {"value": ms_full, "unit": "ms", "cores": threads, "kind": "port",
                         "sample": "full SDXL UNet, batch %d, latent %dx%d, fp32 torch on CPU (%.3f TFLOP, %.2f s), scaled by "
                                   "FLOPs to batch 2 latent 128x128 (%.3f TFLOP)" % (b, hw, hw, fl / 1e12, per, full / 1e12)},
        "e2e": {"value": ms_full, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="katz", choices=["katz", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-step", action="store_true",
                    help="run ONE eager UNet step between cudaProfilerStart/Stop and exit (for `ncu --profile-from-start off`)")
    ap.add_argument("--profile-gemm", action="store_true",
                    help="launch the dominant linear GEMM shapes between cudaProfilerStart/Stop and exit")
    ap.add_argument("--profile-attn", action="store_true",
                    help="run the two self-attention shapes of the step under cudaProfilerStart/Stop (for ncu) and exit")
    ap.add_argument("--compare-cublas", action="store_true",
                    help="time the step's linear shapes against torch.addmm (cuBLAS) in CUDA graphs of 20 launches and exit")
    ap.add_argument("--profile-merge", action="store_true",
                    help="run ONE LoRA merge over a reduced layer set between cudaProfilerStart/Stop and exit")
    ap.add_argument("--parallel", default="auto", choices=["auto", "rows"],
                    help="N > 1: 'auto' splits the CFG batch over two halves of the ranks and the latent rows inside a half; "
                         "'rows' splits latent rows only")
    ap.add_argument("--latent", type=int, default=128, help="latent height = width (128 = 1024^2 images)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "katz" else max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from katz_b200 import _lib
    from katz_b200.engine import GraphedStep
    from katz_b200.lora import LoraMerger
    from katz_b200.params import SDXL_UNET_CONFIG, init_state_dict, lora_target_keys, unet_param_shapes, unet_step_flops
    from katz_b200.unet import KatzUNet
    from katz_b200 import ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; katz_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    cfg = SDXL_UNET_CONFIG
    B, HW = 2, args.latent

    if args.profile_gemm:
        # the dominant GEMM shapes of the step, each launched 3 times under the profiler range
        shapes = [(2048, 10240, 1280), (2048, 1280, 1280), (8192, 640, 2560)]
        outs = []
        for (M, N, K) in shapes:
            xs = torch.randn(M, K, device=dev).half()
            ws = (torch.randn(N, K, device=dev) * 0.03).half()
            outs.append((xs, ws, torch.empty(M, N, dtype=torch.float16, device=dev)))
        for xs, ws, o in outs:
            ops.linear(xs, ws, out=o)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for xs, ws, o in outs:
            for _ in range(3):
                ops.linear(xs, ws, out=o)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "linear GEMMs", "shapes": shapes, "kernel": ops.gemm_kernel_name()}))
        return
    if args.compare_cublas:
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
            return time_events(gr.replay, 3) * 1e3 / n
        rows = []
        for (M, N, K) in [(2048, 10240, 1280), (2048, 1280, 1280), (2048, 3840, 1280), (2048, 1280, 5120), (8192, 640, 640),
                          (8192, 5120, 640), (1024, 1280, 1280), (8192, 8192, 4096)]:
            nw = 6 if N * K < 3e7 else 2          # distinct weights per launch: they are cold in the step, too
            x = torch.randn(M, K, device=dev).half()
            ws = [(torch.randn(N, K, device=dev) * 0.03).half() for _ in range(nw)]
            b = torch.randn(N, device=dev).half()
            o = torch.empty(M, N, dtype=torch.float16, device=dev)
            tk = graph_time(lambda i: ops.linear(x, ws[i % nw], b, out=o))
            tc = graph_time(lambda i: torch.addmm(b, x, ws[i % nw].t(), out=o))
            fl = 2.0 * M * N * K
            rows.append({"shape": [M, N, K], "katz_us": round(tk, 1), "katz_tflops": round(fl / tk / 1e6),
                         "cublas_us": round(tc, 1), "cublas_tflops": round(fl / tc / 1e6)})
        print(json.dumps({"compared": "linear + bias, fp16, CUDA graph of 20 launches", "rows": rows}))
        return
    if args.profile_attn:
        # self-attention of the 32x32 level (20 heads, 1024 tokens) and of the 64x64 level (10 heads, 4096 tokens)
        shapes = [(2, 20, 1024), (2, 10, 4096)]
        bufs = []
        for (Bq, Hh, S) in shapes:
            qkv = torch.randn(Bq, S, 3 * Hh * 64, device=dev).half()
            bufs.append((qkv, Hh, torch.empty(Bq, S, Hh * 64, dtype=torch.float16, device=dev)))
        for qkv, Hh, o in bufs:
            C = Hh * 64
            ops.attention(qkv[:, :, :C], qkv[:, :, C:2 * C], qkv[:, :, 2 * C:], Hh, out=o)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for qkv, Hh, o in bufs:
            C = Hh * 64
            for _ in range(2):
                ops.attention(qkv[:, :, :C], qkv[:, :, C:2 * C], qkv[:, :, 2 * C:], Hh, out=o)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "self-attention", "shapes": shapes}))
        return
    # ---- model: random-init SDXL UNet (seed 0), weights drawn on the device
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev)
    unet = KatzUNet(cfg, dev, sd)
    del sd
    keys = lora_target_keys(cfg, include_proj=True)     # the reference's 722-entry target set
    if args.profile_step:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(B, 4, HW, HW, generator=g).half().to(dev)
        ctx = torch.randn(B, 77, 2048, generator=g).half().to(dev)
        added = {"text_embeds": torch.randn(B, 1280, generator=g).half().to(dev),
                 "time_ids": torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half().to(dev)}
        t = torch.tensor([500.0], device=dev)
        for _ in range(2):
            unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        unet(x, t, encoder_hidden_states=ctx, added_cond_kwargs=added)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "one eager UNet step", "launches": _lib.launch_count() // 3}))
        return
    if args.profile_merge:
        keys = [k for k in keys if k.startswith("down_blocks.2.attentions.0.")]     # 102 layers, 0.7 GB of weights
        merger = LoraMerger(unet.lora_targets(keys))
        lora = make_lora(unet, keys, 64, 100, dev)
        for _ in range(2):
            merger.merge(lora, 1.0)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        merger.merge(lora, 1.0)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": "one LoRA merge", "layers": len(keys), "bytes": merger.algorithmic_bytes([64])}))
        return
    merger = LoraMerger(unet.lora_targets(keys))
    lora = make_lora(unet, keys, 64, 100, dev)

    # ---- LoRA merge: HBM-bound pass, timed alone (weights 4.4 GB >> L2)
    for _ in range(3):
        merger.merge(lora, 1.0)
    merge_request_ms = time_events(lambda: merger.merge(lora, 1.0), 10)     # host table build + upload + kernel
    merge_ms = time_events(lambda: merger.replay(), 10)                     # the kernel alone, table resident
    merger.restore()
    restore_ms = time_events(lambda: merger.replay(), 5)
    merger.merge(lora, 1.0)
    merge_bytes = merger.algorithmic_bytes([64])
    merge_gbs = merge_bytes / (merge_ms * 1e-3) / 1e9

    # ---- inputs (pinned host copies for the e2e leg)
    g = torch.Generator().manual_seed(0)
    h_sample = torch.randn(B, 4, HW, HW, generator=g).half().pin_memory()
    h_ctx = torch.randn(B, 77, 2048, generator=g).half().pin_memory()
    h_te = torch.randn(B, 1280, generator=g).half().pin_memory()
    h_ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half().pin_memory()
    h_t = torch.tensor([500.0]).pin_memory()
    h_out = torch.empty(B, 4, HW, HW, dtype=torch.float16).pin_memory()

    if world > 1:
        from katz_b200.latent_parallel import CfgRowParallelStep
        # batch halves first (the reference's own 2-GPU mode), latent rows inside a half; --parallel rows = rows only
        step = CfgRowParallelStep(unet, B, HW, HW, rank, world, split_cfg=(args.parallel == "auto"))
    else:
        step = GraphedStep(unet, B, HW, HW)
    step.run(sample=h_sample, timestep=h_t, encoder_hidden_states=h_ctx, text_embeds=h_te, time_ids=h_ti)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(args.warmup):
        step.replay()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public call: host inputs in, prediction out, every step
    unet.use_cuda_graph = True
    added = {"text_embeds": h_te, "time_ids": h_ti}

    def e2e_step():
        out = unet(h_sample, h_t, encoder_hidden_states=h_ctx, added_cond_kwargs=added, return_dict=False)[0]
        h_out.copy_(out, non_blocking=True)

    if world == 1:
        for _ in range(args.warmup):
            e2e_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.steps
    else:
        def e2e_step():  # noqa: F811
            out = step.run(sample=h_sample, timestep=h_t, encoder_hidden_states=h_ctx, text_embeds=h_te, time_ids=h_ti)
            h_out[:, :, :out.shape[2]].copy_(out, non_blocking=True)
        for _ in range(args.warmup):
            e2e_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.steps
    h2d = sum(t.numel() * t.element_size() for t in (h_sample, h_ctx, h_te, h_ti, h_t))
    d2h = h_out.numel() * h_out.element_size()

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    # ---- dominant kernel alone: the feed-forward projection GEMM (2048 x 10240 x 1280), burst conditions
    flops = unet_step_flops(cfg, B, HW, HW)
    roof = None
    if rank == 0:
        M, N, K = B * (HW // 4) * (HW // 4), 10240, 1280
        xs = [torch.randn(M, K, device=dev).half() for _ in range(8)]
        ws = [(torch.randn(N, K, device=dev) * 0.03).half() for _ in range(8)]   # 8 x 26 MB of weights: > L2
        o = torch.empty(M, N, dtype=torch.float16, device=dev)
        it = [0]

        def gemm():
            i = it[0] % 8
            it[0] += 1
            ops.linear(xs[i], ws[i], out=o)
        for _ in range(8):
            gemm()
        gemm_ms = time_events(gemm, 40)
        ach = 2.0 * M * N * K / (gemm_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": ops.gemm_kernel_name(), "shape": [M, N, K], "achieved": ach,
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                "peak_source": peaks["_source"] + " burst", "launch_ms": gemm_ms,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape, from the ncu capture summarised
                # in profiles/tc05_gemm_linear_2048x10240x1280.md (31.81 MB + 8.74 MB; algorithmic bytes 73.4 MB, the
                # output is still in L2 when the launch ends)
                "traffic": 40551168 if (M, N, K) == (2048, 10240, 1280) else None, "traffic_unit": "bytes"}

    if rank == 0:
        step_tflops = flops["total"] / world / (ms * 1e-3) / 1e12
        line = {
            "metric": "sdxl_unet_step_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "SDXL UNet step, batch 2 (CFG), latent %dx%d, 1 rank-64 LoRA merged (configs[1])" % (HW, HW),
                       "latent_parallel": world,
                       "parallelism": ("1 GPU" if world == 1 else "cfg%d x rows%d" % (step.halves, step.rows_world)),
                       "l2": "inputs larger than L2: 5.1 GB of weights streamed per step",
                       "timing": "CUDA-graph replay, CUDA events, max over ranks"},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": step.launches_per_step * args.steps,
            "launches_per_step": step.launches_per_step,
            "clocks": clocks,
            "roofline": roof,
            "step_roofline": {"bound": "tensor", "achieved": step_tflops, "peak": peaks["bf16_tflops_sustained"],
                              "unit": "TFLOP/s", "frac": step_tflops / peaks["bf16_tflops_sustained"],
                              "peak_source": peaks["_source"] + " sustained", "flop_per_step": flops["total"],
                              "note": "per-GPU algorithmic FLOPs of the whole step / step time"},
            "lora_merge": {"bound": "hbm", "ms": merge_ms, "restore_ms": restore_ms, "request_ms": merge_request_ms, "bytes": merge_bytes, "achieved": merge_gbs,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": merge_gbs / peaks["hbm_gbs"],
                           "layers": len(keys), "rank": 64, "peak_source": peaks["_source"],
                           # ncu capture of a 102-layer subset scaled by weight bytes (profiles/lora_merge_ws_*.md)
                           "traffic": int(0.965 * merge_bytes)},
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            dt, fl = cpu_reference_step(32, 1, threads)
            ms_full = dt * 1e3 * flops["total"] / fl
            line["cpu_baseline"] = {"value": ms_full, "unit": "ms", "cores": threads, "kind": "port",
                                    "sample": "full SDXL UNet, batch 1, latent 32x32, fp32 torch on CPU (%.3f TFLOP in %.2f s), "
                                              "scaled by FLOPs to the benchmark step (%.3f TFLOP)" % (fl / 1e12, dt, flops["total"] / 1e12)}
        print(json.dumps(line), flush=True)
    if world > 1:
        # Tearing the NCCL communicator down while CUDA graphs that captured its collectives are still alive blocks in
        # the process-group watchdog. The measurement is printed; leave without running destructors.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
