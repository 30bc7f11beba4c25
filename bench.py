"""Benchmark of the hot path: one SDXL UNet denoising step (fp16, batch 2 = CFG, latent 128x128, one rank-64 LoRA
merged), plus the LoRA merge itself, on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl katz|reference]

Prints ONE JSON line (rank 0). `value` is milliseconds per UNet step with inputs resident in HBM (CUDA-graph replay,
CUDA-event timing, max over ranks); `e2e` is the same step through the public `unet(...)` call with pinned HOST inputs
copied in and the prediction copied out every step. `checked` says that the timed step's output was compared (with the
eager step, with torch's fp16 path on the same GPU) and that no bounded device-side wait gave up; the run exits
non-zero otherwise. `roofline` describes the dominant kernel (the GEMM behind the linears) timed alone;
`step_roofline` the whole step against the sustained tensor peak; `lora_merge*` the merge passes against the HBM peak;
`torch_gpu_baseline` the same step through torch's own fp16 kernels (cuBLAS / cuDNN / SDPA) under a CUDA graph on the
same GPU; `cpu_baseline` the fp32 torch path on the host cores. `--impl reference` times that CPU path alone.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from collections import OrderedDict

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
WORKLOAD = "SDXL UNet step, batch 2 (CFG), latent %dx%d, 1 rank-64 LoRA merged (configs[1])"


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


def time_events(fn, iters):
    """Average milliseconds of fn() over `iters` calls, CUDA events on the current stream, sync on both sides."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def make_lora(targets, rank, seed, device, dtype=torch.float16):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    ad = OrderedDict()
    for k, w in targets.items():
        o, n = w.shape
        down = (torch.randn(rank, n, generator=g, device=device) / rank).to(dtype)
        up = (torch.randn(o, rank, generator=g, device=device) * 0.01).to(dtype)
        ad[k] = (up, down)
    return ad


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm())


# ---------------------------------------------------------------------------------------------- CPU baseline ------
def cpu_weights():
    """fp32 random weights of the SDXL UNet on the host, drawn once."""
    from katz_b200.params import SDXL_UNET_CONFIG, unet_param_shapes
    g = torch.Generator().manual_seed(0)
    sd = OrderedDict()
    for k, shp in unet_param_shapes(SDXL_UNET_CONFIG).items():
        fan = 1
        for s in shp[1:]:
            fan *= s
        t = torch.empty(shp, dtype=torch.float32)
        if len(shp) == 1 and ("norm" in k):
            t.fill_(1.0 if k.endswith("weight") else 0.0)
        else:
            t.uniform_(-1.0 / max(fan, 1) ** 0.5, 1.0 / max(fan, 1) ** 0.5, generator=g)
        sd[k] = t
    return sd


def cpu_reference_steps(latent, batch, threads, max_steps, budget_s, warmup=0):
    """The CPU restatement of the reference's torch path (oracle.unet_oracle, fp32) on the host cores, on the benchmark's
    own configuration; the weights are built once, then up to `max_steps` steps are timed while `budget_s` lasts (at
    least one). Returns (mean seconds per step, steps timed)."""
    from katz_b200.params import SDXL_UNET_CONFIG
    from oracle import unet_oracle
    torch.set_num_threads(threads)
    sd = cpu_weights()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(batch, 4, latent, latent, generator=g)
    ctx = torch.randn(batch, 77, 2048, generator=g)
    te = torch.randn(batch, 1280, generator=g)
    ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * batch)
    times = []
    with torch.no_grad():
        for i in range(warmup + max_steps):
            t0 = time.time()
            unet_oracle.unet_step(sd, SDXL_UNET_CONFIG, x, 500.0, ctx, te, ti)
            if i >= warmup:
                times.append(time.time() - t0)
            if sum(times) > budget_s:
                break
    return sum(times) / len(times), len(times)


def cpu_lora_merge_fp32(threads, stride=10):
    """`W += up @ down * scale` (lora_utils.py:29-33) in fp32 torch on the host cores over every `stride`-th layer of the
    700-layer set. Returns (GB/s of algorithmic bytes, layers timed)."""
    from katz_b200.params import SDXL_UNET_CONFIG, lora_target_keys, unet_param_shapes
    torch.set_num_threads(threads)
    shapes = unet_param_shapes(SDXL_UNET_CONFIG)
    keys = lora_target_keys(SDXL_UNET_CONFIG)[::stride]
    g = torch.Generator().manual_seed(0)
    layers = []
    for k in keys:
        o, n = shapes[k]
        layers.append((torch.randn(o, n, generator=g) * 0.02, torch.randn(o, 64, generator=g) * 0.01, torch.randn(64, n, generator=g) / 64))
    nbytes = sum(2 * w.numel() * 4 + (u.numel() + d.numel()) * 4 for w, u, d in layers)
    t0 = time.time()
    for w, u, d in layers:
        w += u @ d * 1.0
    dt = time.time() - t0
    return nbytes / dt / 1e9, len(layers)


def run_reference(args, rank, world):
    """`--impl reference`: the reference's implementation of this path is torch; its GPU route is the library calls this
    project replaces, so the arm times its CPU route — the fp32 restatement pinned to the reference's own classes by
    tests/golden — with all host threads, on the benchmark's own configuration. Rank 0 only."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    per, n = cpu_reference_steps(args.latent, 2, threads, max(1, args.steps), 150.0, warmup=1 if args.warmup > 0 else 0)
    ms = per * 1e3
    line = {
        "impl": "reference", "metric": "sdxl_unet_step_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": n, "warmup": 1 if args.warmup > 0 else 0, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD % (args.latent, args.latent), "latent_parallel": args.gpus},
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": threads, "kind": "port",
                         "sample": "the full benchmark step (batch 2, latent %dx%d, fp32 torch on the host cores), %d steps "
                                   "timed, nothing scaled" % (args.latent, args.latent, n)},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- GPU helpers -------
def capture(fn, warmup=2):
    """Capture fn() in a CUDA graph after `warmup` eager calls on a side stream. Returns (graph, fn's captured result)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g, out


def torch_gpu_baseline(unet, cfg, inputs, steps, warmup):
    """The same step through torch's own fp16 kernels (cuBLAS linears, cuDNN convolutions, SDPA, native GroupNorm /
    LayerNorm) on this GPU under a CUDA graph: the reference's GPU route, restated functionally by oracle.unet_oracle
    and run on the exported (LoRA-merged) weights. Both memory formats are timed; the faster one is reported."""
    from oracle import unet_oracle
    dev = unet.device
    sd = unet.state_dict()
    x, ctx, te, ti = (t.to(dev) for t in inputs)
    t = torch.tensor([500.0], device=dev)
    best = None
    for fmt in ("contiguous", "channels_last"):
        if fmt == "channels_last":
            sd = OrderedDict((k, v.contiguous(memory_format=torch.channels_last) if v.dim() == 4 else v) for k, v in sd.items())
            xin = x.contiguous(memory_format=torch.channels_last)
        else:
            xin = x
        with torch.no_grad():
            g, out = capture(lambda: unet_oracle.unet_step(sd, cfg, xin, t, ctx, te, ti))
            for _ in range(warmup):
                g.replay()
            ms = time_events(g.replay, steps)
        if best is None or ms < best[0]:
            best = (ms, fmt, out.clone())
        del g
    del sd
    torch.cuda.empty_cache()
    return {"ms": best[0], "kind": "torch %s fp16 (cuBLAS/cuDNN/SDPA) under a CUDA graph, same GPU, same weights and inputs; "
                                   "memory format %s (the faster of contiguous / channels_last)" % (torch.__version__, best[1])}, best[2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="katz", choices=["katz", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the legs that do not feed `value`/`e2e` (GEMM roofline, torch baseline, ControlNet, fp32 merge)")
    ap.add_argument("--parallel", default="auto", choices=["auto", "rows"],
                    help="N > 1: 'auto' splits the CFG batch over two halves of the ranks and the latent rows inside a half; "
                         "'rows' splits latent rows only")
    ap.add_argument("--latent", type=int, default=128, help="latent height = width (128 = 1024^2 images)")
    ap.add_argument("--stream", default=None, metavar="REQUESTS:STEPS",
                    help="also run a stream of requests (configs[4]: one ControlNet, one LoRA per request drawn from a pool of 16 "
                         "rank-64 adapters, so consecutive requests force a switch): e.g. 4:10 = four requests of ten Euler "
                         "steps. 1 GPU. Adds `request_stream` to the line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "katz" else max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from katz_b200 import _lib, ops
    from katz_b200.engine import GraphedStep
    from katz_b200.lora import LoraMerger
    from katz_b200.params import (SDXL_UNET_CONFIG, controlnet_param_shapes, init_state_dict, lora_target_keys,
                                  unet_param_shapes, unet_step_flops)
    from katz_b200.unet import KatzControlNet, KatzUNet

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; katz_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    cfg = SDXL_UNET_CONFIG
    B, HW = 2, args.latent

    # ---- model: random-init SDXL UNet (seed 0), weights drawn on the device
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev)
    unet = KatzUNet(cfg, dev, sd)
    del sd
    keys = lora_target_keys(cfg, include_proj=True)     # the reference's 722-entry target set
    targets = unet.lora_targets(keys)
    merger = LoraMerger(targets, on_change=unet.invalidate_caches)
    lora = make_lora(targets, 64, 100, dev)

    # ---- LoRA merge: HBM-bound pass, timed alone (weights 4.4 GB >> L2)
    def merge_leg(adapters, ranks):
        sc = [1.0] * len(adapters)
        for _ in range(3):
            merger.merge(adapters, sc)
        request_ms = time_events(lambda: merger.merge(adapters, sc), 10)     # host table build + upload + kernel
        ms_ = time_events(merger.replay, 10)                                 # the kernel alone, table resident
        nb = merger.algorithmic_bytes(ranks)
        gbs = nb / (ms_ * 1e-3) / 1e9
        return {"bound": "hbm", "ms": ms_, "request_ms": request_ms, "bytes": nb, "achieved": gbs, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "layers": len(keys), "ranks": ranks, "dtype": "f16",
                "peak_source": peaks["_source"]}
    merge2 = None
    if rank == 0 and not args.no_extras:
        lora32 = make_lora(targets, 32, 101, dev)
        merge2 = merge_leg([lora, lora32], [64, 32])
        del lora32
    merge1 = merge_leg([lora], [64])
    merger.restore()
    merge1["restore_ms"] = time_events(merger.replay, 5)
    merger.merge(lora, 1.0)
    # DRAM traffic of one merge launch: an ncu capture of a 102-layer subset, scaled by weight bytes (it grows in proportion)
    merge1["traffic"] = int(0.965 * merge1["bytes"])

    # ---- inputs (pinned host copies for the e2e leg)
    g = torch.Generator().manual_seed(0)
    h_sample = torch.randn(B, 4, HW, HW, generator=g).half().pin_memory()
    h_ctx = torch.randn(B, 77, 2048, generator=g).half().pin_memory()
    h_te = torch.randn(B, 1280, generator=g).half().pin_memory()
    h_ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half().pin_memory()
    h_t = torch.tensor([500.0]).pin_memory()
    h_out = torch.empty(B, 4, HW, HW, dtype=torch.float16).pin_memory()
    feed = dict(sample=h_sample, timestep=h_t, encoder_hidden_states=h_ctx, text_embeds=h_te, time_ids=h_ti)

    # ---- the eager single-GPU step on the same inputs: what the timed step's output is compared with
    added_dev = {"text_embeds": h_te.to(dev), "time_ids": h_ti.to(dev)}
    eager = unet(h_sample.to(dev), h_t.to(dev), encoder_hidden_states=h_ctx.to(dev), added_cond_kwargs=added_dev)[0].clone()

    if world > 1:
        from katz_b200.latent_parallel import CfgRowParallelStep
        # batch halves first (the reference's own 2-GPU mode), latent rows inside a half; --parallel rows = rows only
        step = CfgRowParallelStep(unet, B, HW, HW, rank, world, split_cfg=(args.parallel == "auto"))
    else:
        step = GraphedStep(unet, B, HW, HW)
    step.run(**feed)
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out_timed = step.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    out_timed = out_timed.clone()
    checks = {"timed_output_equals_eager_step": bool(torch.equal(out_timed, eager)),
              "timed_output_vs_eager_rel_l2": rel_l2(out_timed, eager),
              "timed_output_vs_eager_max_abs": float((out_timed.float() - eager.float()).abs().max())}

    # ---- end to end through the public call: host inputs in, prediction out, every step
    added = {"text_embeds": h_te, "time_ids": h_ti}
    if world == 1:
        unet.use_cuda_graph = True

        def e2e_step():
            out = unet(h_sample, h_t, encoder_hidden_states=h_ctx, added_cond_kwargs=added, return_dict=False)[0]
            h_out.copy_(out, non_blocking=True)
    else:
        def e2e_step():
            out = step.run(**feed)
            h_out.copy_(out, non_blocking=True)
    for _ in range(args.warmup):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    unet.use_cuda_graph = False
    h2d = sum(t.numel() * t.element_size() for t in (h_sample, h_ctx, h_te, h_ti, h_t))
    d2h = h_out.numel() * h_out.element_size()
    checks["e2e_output_equals_eager_step"] = bool(torch.equal(h_out, eager.cpu()))
    checks["e2e_output_vs_eager_rel_l2"] = rel_l2(h_out, eager.cpu())

    # ---- did any bounded device-side wait give up during the timed regions?
    tc05 = ops.tc05_status()
    peer = 0
    inner = getattr(step, "_inner", None)
    rp = getattr(inner, "rp", None)
    if rp is not None and rp.peer is not None:
        peer = rp.peer.status()
    ok_local = (tc05 == 0 and peer == 0 and checks["timed_output_vs_eager_rel_l2"] <= 2e-3 and checks["timed_output_vs_eager_max_abs"] <= 1e-2
                and checks["e2e_output_vs_eager_rel_l2"] <= 2e-3)
    if world > 1:
        t = torch.tensor([ms, e2e_ms, float(tc05), float(peer), 0.0 if ok_local else 1.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, tc05, peer, ok_all = float(t[0]), float(t[1]), int(t[2]), int(t[3]), float(t[4]) == 0.0
    else:
        ok_all = ok_local
    checks.update({"tc05_status": tc05, "peer_status": peer,
                   "against": "the eager single-GPU step of this build on the same inputs (itself checked against the fp32 "
                              "oracle at this size by tests/test_gpu_sdxl_size.py)"})

    flops = unet_step_flops(cfg, B, HW, HW)
    roof = tgb = cn_leg = merge32 = vae_leg = None
    if rank == 0 and not args.no_extras:
        # ---- dominant kernel alone: the feed-forward projection GEMM (2048 x 10240 x 1280), burst conditions
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
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape under ncu: 31.81 MB + 8.74 MB
                # (algorithmic bytes 73.4 MB; the output is still in L2 when the launch ends)
                "traffic": 40551168 if (M, N, K) == (2048, 10240, 1280) else None, "traffic_unit": "bytes"}
        del xs, ws, o
        if world == 1:
            # ---- torch's own fp16 path on this GPU: the bar to beat
            tgb, torch_out = torch_gpu_baseline(unet, cfg, (h_sample, h_ctx, h_te, h_ti), args.steps, args.warmup)
            tgb["katz_over_torch_time"] = ms / tgb["ms"]
            checks["timed_output_vs_torch_fp16_rel_l2"] = rel_l2(out_timed, torch_out)
            ok_all = ok_all and checks["timed_output_vs_torch_fp16_rel_l2"] <= 1e-2
            del torch_out
            # ---- configuration 3: one ControlNet (alone, and in one graph with the UNet)
            cn = KatzControlNet(cfg, dev, init_state_dict(controlnet_param_shapes(cfg), seed=1, dtype=torch.float16, device=dev,
                                                         generator_device=dev))
            cond = torch.rand(B, 3, 8 * HW, 8 * HW, device=dev).half()
            st = step.static
            kw = dict(encoder_hidden_states=st["encoder_hidden_states"], controlnet_cond=cond,
                      added_cond_kwargs={"text_embeds": st["text_embeds"], "time_ids": st["time_ids"]}, nhwc_out=True)
            n0 = _lib.launch_count()
            gcn, _ = capture(lambda: cn(st["sample"], st["timestep"], **kw))
            cn_launches = (_lib.launch_count() - n0) // 3
            for _ in range(args.warmup):
                gcn.replay()
            cn_ms = time_events(gcn.replay, args.steps)
            cn_fl = unet_step_flops(cfg, B, HW, HW, controlnet=True)["total"]
            both = GraphedStep(unet, B, HW, HW, controlnets=[cn], conditioning_scales=[0.5])
            both.static["controlnet_cond"].copy_(cond)
            for k in ("sample", "timestep", "encoder_hidden_states", "text_embeds", "time_ids"):
                both.static[k].copy_(st[k])
            for _ in range(args.warmup):
                both.replay()
            both_ms = time_events(both.replay, args.steps)
            ach = cn_fl / (cn_ms * 1e-3) / 1e12
            cn_leg = {"workload": "one SDXL ControlNet step, batch 2, latent %dx%d, conditioning image %dx%d (configs[2])" % (HW, HW, 8 * HW, 8 * HW),
                      "ms": cn_ms, "flop": cn_fl, "achieved": ach, "unit": "TFLOP/s", "peak": peaks["bf16_tflops_sustained"],
                      "frac": ach / peaks["bf16_tflops_sustained"], "launches": cn_launches,
                      "unet_plus_controlnet_ms": both_ms, "unet_plus_controlnet_launches": both.launches_per_step}
            tc05 = max(tc05, ops.tc05_status())
            del gcn, both, cn, cond
            torch.cuda.empty_cache()
            # ---- the VAE decode that follows the last step (one image): 10.47 TFLOP at 1024x1024 pixels
            if HW <= 128:
                from katz_b200.params import SDXL_VAE_CONFIG, vae_decode_flops, vae_decoder_param_shapes
                from katz_b200.vae import KatzVaeDecoder
                dec = KatzVaeDecoder(SDXL_VAE_CONFIG, dev, init_state_dict(vae_decoder_param_shapes(SDXL_VAE_CONFIG), seed=5,
                                                                           dtype=torch.float16, device=dev, generator_device=dev))
                zlat = (torch.randn(1, 4, HW, HW, generator=torch.Generator().manual_seed(6)) * SDXL_VAE_CONFIG["scaling_factor"]).half().to(dev)
                eager_img = dec.decode_latents(zlat).clone()
                dec.use_cuda_graph = True
                for _ in range(2):
                    img = dec.decode_latents(zlat)
                vae_ms = time_events(lambda: dec.decode_latents(zlat), max(3, args.steps // 4))
                vfl = vae_decode_flops(SDXL_VAE_CONFIG, 1, HW, HW)
                ach = vfl / (vae_ms * 1e-3) / 1e12
                vae_leg = {"workload": "SDXL VAE decode of one %dx%d latent to %dx%d pixels, fp16 (AutoencoderKL.decode)" % (HW, HW, 8 * HW, 8 * HW),
                           "ms": vae_ms, "flop": vfl, "achieved": ach, "unit": "TFLOP/s", "peak": peaks["bf16_tflops_sustained"],
                           "frac": ach / peaks["bf16_tflops_sustained"], "graph_equals_eager": bool(torch.equal(img, eager_img)),
                           "finite": bool(torch.isfinite(img).all())}
                tc05 = max(tc05, ops.tc05_status())
                del dec, zlat, img, eager_img
                torch.cuda.empty_cache()
            # ---- configuration 1: the 700-layer set with fp32 weights and fp32 adapters
            shapes = unet_param_shapes(cfg)
            keys32 = lora_target_keys(cfg)
            gg = torch.Generator(device=dev)
            gg.manual_seed(0)
            W32 = OrderedDict((k, torch.randn(shapes[k], generator=gg, device=dev) * 0.02) for k in keys32)
            m32 = LoraMerger(W32)
            l32 = make_lora(W32, 64, 0, dev, dtype=torch.float32)
            for _ in range(2):
                m32.merge(l32, 1.0)
            ms32 = time_events(m32.replay, 5)
            nb = m32.algorithmic_bytes([64])
            m32.restore()
            r32 = time_events(m32.replay, 3)
            gbs = nb / (ms32 * 1e-3) / 1e9
            merge32 = {"bound": "hbm", "ms": ms32, "restore_ms": r32, "bytes": nb, "achieved": gbs, "peak": peaks["hbm_gbs"],
                       "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "layers": len(keys32), "ranks": [64], "dtype": "f32",
                       "peak_source": peaks["_source"]}
            del W32, m32, l32
            torch.cuda.empty_cache()

    stream_leg = None
    if rank == 0 and world == 1 and args.stream:
        from katz_b200.pipeline import KatzDenoiser, LoraRequestStream
        n_req, n_steps = (int(v) for v in args.stream.split(":"))
        merger.restore()
        cn = KatzControlNet(cfg, dev, init_state_dict(controlnet_param_shapes(cfg), seed=1, dtype=torch.float16, device=dev,
                                                     generator_device=dev))
        den = KatzDenoiser(unet, HW, HW, controlnets=[cn], conditioning_scales=[0.5], guidance_scale=5.0)
        pool = [make_lora(targets, 64, 100 + i, dev) for i in range(16)]
        ids = torch.randint(0, 16, (n_req,), generator=torch.Generator().manual_seed(0)).tolist()
        rs = LoraRequestStream(den, merger, pool, scale=1.0)
        gi = torch.Generator().manual_seed(1)
        req = dict(prompt_embeds=torch.randn(2, 77, 2048, generator=gi).half().to(dev), text_embeds=torch.randn(2, 1280, generator=gi).half().to(dev),
                   time_ids=torch.tensor([[8.0 * HW, 8.0 * HW, 0., 0., 8.0 * HW, 8.0 * HW]] * 2).half().to(dev),
                   controlnet_cond=torch.rand(2, 3, 8 * HW, 8 * HW, generator=gi).half().to(dev))
        rs.run(ids[:1], lambda i: req, num_inference_steps=2)                   # warm-up
        t0 = time.time()
        res = rs.run(ids, lambda i: req, num_inference_steps=n_steps)
        wall = time.time() - t0
        lat = sorted(ms_ for _, ms_ in res)
        per_step = sum(lat) / len(lat) / n_steps
        stream_leg = {"workload": "stream of requests at %dx%d pixels: 1 ControlNet (scale 0.5), CFG 5.0, one rank-64 LoRA per request "
                                  "from a pool of 16 (switch = one merge pass from the pristine weights), Euler (configs[4])" % (8 * HW, 8 * HW),
                      "requests": n_req, "steps_per_request": n_steps, "lora_ids": ids, "ms_per_request_median": lat[len(lat) // 2],
                      "ms_per_request_max": lat[-1], "ms_per_step": per_step, "images_per_s": n_req / wall,
                      "ms_per_50_step_request_extrapolated": per_step * 50 if n_steps != 50 else None,
                      "images_per_s_50_steps_extrapolated": 1e3 / (per_step * 50) if n_steps != 50 else None,
                      "launches_per_step": den.step.launches_per_step + 2}
        tc05 = max(tc05, ops.tc05_status())
        ok_all = ok_all and tc05 == 0
        del den, rs, pool, cn
        merger.merge(lora, 1.0)
        torch.cuda.empty_cache()

    if rank == 0:
        step_tflops = flops["total"] / world / (ms * 1e-3) / 1e12
        line = {
            "metric": "sdxl_unet_step_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD % (HW, HW), "latent_parallel": world,
                       "parallelism": ("1 GPU" if world == 1 else "cfg%d x rows%d" % (step.halves, step.rows_world)),
                       "l2": "inputs larger than L2: 5.1 GB of weights streamed per step",
                       "timing": "CUDA-graph replay, CUDA events, max over ranks"},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": step.launches_per_step * args.steps,
            "launches_per_step": step.launches_per_step,
            "checked": bool(ok_all), "checks": checks,
            "clocks": clocks,
            "roofline": roof,
            "step_roofline": {"bound": "tensor", "achieved": step_tflops, "peak": peaks["bf16_tflops_sustained"],
                              "unit": "TFLOP/s", "frac": step_tflops / peaks["bf16_tflops_sustained"],
                              "frac_of_burst": step_tflops / peaks["bf16_tflops"],
                              "peak_source": peaks["_source"] + " sustained", "flop_per_step": flops["total"],
                              "note": "per-GPU algorithmic FLOPs of the whole step / step time"},
            "lora_merge": merge1, "lora_merge_2adapters": merge2, "lora_merge_fp32": merge32, "vae_decode": vae_leg,
            "controlnet_step": cn_leg, "torch_gpu_baseline": tgb, "request_stream": stream_leg,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            per, n = cpu_reference_steps(HW, B, threads, 2, 60.0)
            line["cpu_baseline"] = {"value": per * 1e3, "unit": "ms", "cores": threads, "kind": "port",
                                    "sample": "the full benchmark step (batch 2, latent %dx%d, fp32 torch on the host cores), "
                                              "%d steps timed, nothing scaled" % (HW, HW, n)}
            if merge32 is not None:
                gbs, nl = cpu_lora_merge_fp32(threads)
                merge32["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                           "sample": "W += up @ down * scale in fp32 torch on every 10th layer of the 700-layer set "
                                                     "(%d layers)" % nl}
        print(json.dumps(line), flush=True)
    code = 0 if ok_all else 3
    if world > 1:
        # Tearing the NCCL communicator down while CUDA graphs that captured its collectives are still alive blocks in
        # the process-group watchdog. The measurement is printed; leave without running destructors.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(code)
    if code:
        sys.stderr.write("bench.py: the timed step did not pass its checks: %s\n" % json.dumps(checks))
    sys.exit(code)


if __name__ == "__main__":
    main()
