"""Model-server loops of the reference's multi-process deployment, over katz_b200 models.

`unet_server_loop` mirrors sdxl_unet_server.py:96-220 (rank 1: the second UNet replica of the reference's 2-GPU
classifier-free-guidance split) and `controlnet_server_loop` mirrors sdxl_controlnet_server.py:60-115 (ranks 2..7: one
ControlNet per GPU). The torch.distributed message protocol is the reference's, message for message:

  per request   broadcast(src=0): int32[1] batch, int32[1] steps, fp16 [B,3,Hc,Wc] conditioning image
                recv(src=0 / dst_rank): prompt_embeds [B,77,D], text_embeds [B,E], time_ids [B,6]
                (the UNet server forwards those three to its ControlNet ranks, sdxl_unet_server.py:124-130)
  per step      [async LoRA mode: recv(src=0) int32 shm status; when it equals 10*n_loras the server gathers the
                adapters from shared memory and merges them, sdxl_unet_server.py:153-181]
                broadcast(src=0): fp16 latent [B,4,H,W], fp32 scalar t
                ControlNet server: send(dst) 9 down residuals then the mid residual (sdxl_controlnet_server.py:107-113)
                UNet server: recv per ControlNet rank 9 down then, per rank, the mid residual; sum; divide by the number
                of nets (unet_2d_condition.py:1418-1439); run; send(dst=0) the prediction (sdxl_unet_server.py:215)
  after         restore the pristine weights (sdxl_unet_server.py:217)

Differences: requests are bounded by `max_requests` (the reference loops forever and is killed with SIGTERM,
run_katz.py:227-233), the restore is one bit-exact copy pass instead of deepcopy + load_state_dict, and the per-rank
LoRA merge computes sum_i B_i A_i. Models are passed in as callables with the reference's call signatures, so the
loops are backend-agnostic (the tests drive them with gloo on CPU tensors and stand-in models).
"""
import argparse

import torch
import torch.distributed as dist


def residual_shapes(batch, block_out_channels, height, width, layers_per_block=2):
    """Shapes (NCHW) of the down residuals and of the mid residual a ControlNet sends: one per conv_in output, resnet
    output and downsampler output (sdxl_unet_server.py:136-147 lists the nine SDXL ones)."""
    shapes = [(batch, block_out_channels[0], height, width)]
    h, w = height, width
    for i, c in enumerate(block_out_channels):
        shapes += [(batch, c, h, w)] * layers_per_block
        if i != len(block_out_channels) - 1:
            h, w = h // 2, w // 2
            shapes.append((batch, c, h, w))
    return shapes, (batch, block_out_channels[-1], h, w)


def _recv_request_header(device, cond_hw):
    b = torch.empty((1,), dtype=torch.int32, device=device)
    dist.broadcast(b, src=0)
    steps = torch.empty((1,), dtype=torch.int32, device=device)
    dist.broadcast(steps, src=0)
    cond = torch.empty((int(b), 3, cond_hw[0], cond_hw[1]), dtype=torch.float16, device=device)
    dist.broadcast(cond, src=0)
    return int(b), int(steps), cond


def _recv_embeddings(device, batch, src, text_len, cross_dim, pooled_dim):
    pe = torch.empty((batch, text_len, cross_dim), dtype=torch.float16, device=device)
    te = torch.empty((batch, pooled_dim), dtype=torch.float16, device=device)
    ti = torch.empty((batch, 6), dtype=torch.float16, device=device)
    dist.recv(pe, src=src)
    dist.recv(te, src=src)
    dist.recv(ti, src=src)
    return pe, te, ti


def controlnet_server_loop(controlnet, device, dst_rank=0, latent_hw=(128, 128), cond_hw=(1024, 1024), text_len=77,
                           cross_dim=2048, pooled_dim=1280, max_requests=None, verbose=False):
    """sdxl_controlnet_server.py:60-115. `controlnet(sample, t, encoder_hidden_states=, controlnet_cond=,
    added_cond_kwargs=)` -> (list of down residuals, mid residual), NCHW."""
    served = 0
    while max_requests is None or served < max_requests:
        batch, steps, cond = _recv_request_header(device, cond_hw)
        begin = getattr(controlnet, "begin_request", None)
        if begin is not None:
            begin()       # per-request hoisting contract: what the net cached for the last prompt / image is dropped
        pe, te, ti = _recv_embeddings(device, batch, dst_rank, text_len, cross_dim, pooled_dim)
        added = {"text_embeds": te, "time_ids": ti}
        x = torch.empty((batch, 4, latent_hw[0], latent_hw[1]), dtype=torch.float16, device=device)
        t = torch.zeros((), dtype=torch.float32, device=device)
        for _ in range(steps):
            dist.broadcast(x, src=0)
            dist.broadcast(t, src=0)
            down, mid = controlnet(x, t, encoder_hidden_states=pe, controlnet_cond=cond, added_cond_kwargs=added)
            for d in down:
                dist.send(d.contiguous(), dst=dst_rank)
            dist.send(mid.contiguous(), dst=dst_rank)
        served += 1
        if verbose:
            print("ControlNet server: request %d done (%d steps)" % (served, steps))
    return served


def recv_controlnet_residuals(ranks, down_shapes, mid_shape, device):
    """unet_2d_condition.py:1418-1439: per ControlNet rank receive the down residuals, then per rank the mid residual.
    Returns (list over nets of lists of down residuals, list of mid residuals); the caller combines them."""
    downs = []
    for r in ranks:
        cur = []
        for shp in down_shapes:
            buf = torch.empty(shp, dtype=torch.float16, device=device)
            dist.recv(buf, src=r)
            cur.append(buf)
        downs.append(cur)
    mids = []
    for r in ranks:
        buf = torch.empty(mid_shape, dtype=torch.float16, device=device)
        dist.recv(buf, src=r)
        mids.append(buf)
    return downs, mids


def unet_server_loop(unet, device, controlnet_parallel_rank=(), local_controlnet=None, block_out_channels=(320, 640, 1280),
                     latent_hw=(128, 128), cond_hw=(1024, 1024), text_len=77, cross_dim=2048, pooled_dim=1280,
                     lora_hook=None, restore_hook=None, request_hook=None, check_hook=None, max_requests=None, verbose=False):
    """sdxl_unet_server.py:96-220. `unet(sample, t, encoder_hidden_states=, added_cond_kwargs=,
    down_block_additional_residuals=, mid_block_additional_residual=, combine_scales=)` -> (prediction,).
    request_hook() runs at the top of every request (`--lora-mode full`: patch_on_lora, sdxl_unet_server.py:99-100);
    lora_hook(status:int) -> bool is called every step until it returns True (async LoRA mode: `status` is the shm flag
    sum received from rank 0, sdxl_unet_server.py:153-181); restore_hook() runs after each request (:217); check_hook()
    after it (did a bounded device-side wait give up during the request?)."""
    ranks = list(controlnet_parallel_rank)
    served = 0
    while max_requests is None or served < max_requests:
        if request_hook is not None:
            request_hook()
        begin = getattr(unet, "begin_request", None)
        if begin is not None:
            begin()
        batch, steps, cond = _recv_request_header(device, cond_hw)
        pe, te, ti = _recv_embeddings(device, batch, 0, text_len, cross_dim, pooled_dim)
        added = {"text_embeds": te, "time_ids": ti}
        for r in ranks:
            dist.send(pe, dst=r)
        for r in ranks:
            dist.send(te, dst=r)
        for r in ranks:
            dist.send(ti, dst=r)
        x = torch.empty((batch, 4, latent_hw[0], latent_hw[1]), dtype=torch.float16, device=device)
        t = torch.zeros((), dtype=torch.float32, device=device)
        down_shapes, mid_shape = residual_shapes(batch, block_out_channels, latent_hw[0], latent_hw[1])
        patched = lora_hook is None
        for _ in range(steps):
            if not patched:
                status = torch.zeros((), dtype=torch.int32, device=device)
                dist.recv(status, src=0)
                patched = bool(lora_hook(int(status)))
            dist.broadcast(x, src=0)
            dist.broadcast(t, src=0)
            kw = {}
            if ranks:
                downs, mids = recv_controlnet_residuals(ranks, down_shapes, mid_shape, device)
                kw = dict(down_block_additional_residuals=downs, mid_block_additional_residual=mids,
                          combine_scales=[1.0 / len(ranks)] * len(ranks))
            elif local_controlnet is not None:
                d, m = local_controlnet(x, t, encoder_hidden_states=pe, controlnet_cond=cond, added_cond_kwargs=added)
                kw = dict(down_block_additional_residuals=d, mid_block_additional_residual=m)
            pred = unet(x, t, encoder_hidden_states=pe, added_cond_kwargs=added, return_dict=False, **kw)[0]
            dist.send(pred.contiguous(), dst=0)
        if restore_hook is not None:
            restore_hook()
        if check_hook is not None:
            check_hook()
        served += 1
        if verbose:
            print("UNet server: request %d done (%d steps)" % (served, steps))
    return served


REFERENCE_LORA_REPOS = {0: [], 1: ["TheLastBen/Papercut_SDXL"],
                        2: ["TheLastBen/William_Eggleston_Style_SDXL", "TheLastBen/Filmic"]}   # sdxl_unet_server.py:73-78


def make_lora_hooks(pipe, lora_mode, load_lora_mode, lora_model_repos, device, shm_prefix="", shm_client=None):
    """The three hooks of `unet_server_loop` for the reference's LoRA flags (sdxl_unet_server.py:24-38):

      --lora-mode full                        request_hook: lora_utils.patch_on_lora(pipe, repos) before every request
      --lora-mode sync --load-lora-mode async lora_hook: once the shm status equals 10 * len(repos) the adapters are
                                              gathered from shared memory, summed element-wise over the repos as the
                                              reference does (:169-173) and merged with pipe.patch_on_lora
      any mode                                restore_hook: the pristine weights come back after the request (:217)

    Returns (request_hook, lora_hook, restore_hook); a hook that the mode does not need is None."""
    import json
    import os
    from .lora_utils import patch_on_lora
    repos = list(lora_model_repos)
    request_hook = lora_hook = None
    if lora_mode == "full" and repos:
        def request_hook():
            patch_on_lora(pipe, repos)
    elif lora_mode == "sync" and load_lora_mode == "async" and repos:
        state = {"client": shm_client}

        def lora_hook(status):
            if status != 10 * len(repos):
                return False
            if state["client"] is None:
                from .lora_shm import LoraShmClient
                infos = []
                for r in repos:
                    with open(os.path.join(pipe.lora_info_dir, r.replace("/", "_") + ".json"), "r") as fr:
                        infos.append(json.load(fr))
                state["client"] = LoraShmClient(infos, prefix=shm_prefix)
            summed = {}
            for i in range(len(repos)):
                for k, t in state["client"].gather(i, device).items():
                    summed[k] = t if k not in summed else summed[k] + t
            pipe.patch_on_lora(summed, repos, None)
            return True
    return request_hook, lora_hook, pipe.restore_unet


def build_arg_parser(kind):
    """The reference's command-line flags (sdxl_unet_server.py:24-38, sdxl_controlnet_server.py:24-33)."""
    p = argparse.ArgumentParser()
    p.add_argument("--world-size", type=int, default=2)
    p.add_argument("--gpu-id", type=int, default=1)
    p.add_argument("--rank", type=int, default=1)
    p.add_argument("--controlnet-parallel-rank", type=int, nargs="+", default=[])
    p.add_argument("-v", "--verbose", action="store_true")
    if kind == "unet":
        p.add_argument("--controlnet-parallel", action="store_true")
        p.add_argument("--num-controlnets", type=int, default=0)
        p.add_argument("--lora-mode", type=str, default="without", choices=["without", "full", "sync"])
        p.add_argument("--load-lora-mode", type=str, default="default", choices=["default", "async"])
        p.add_argument("--max-lora-num", type=int, default=0, choices=[0, 1, 2])
    else:
        p.add_argument("--dst-rank", type=int, default=0)
    p.add_argument("--init-method", type=str, default="tcp://127.0.0.1:8000")
    p.add_argument("--state-dict", type=str, default=None, help="torch.save'd state dict with the reference's keys")
    p.add_argument("--max-requests", type=int, default=None)
    if kind == "unet":
        p.add_argument("--lora-info-dir", type=str, default="./lora_info_shm",
                       help="folder of the reference's <repo>.json / <repo>_key_match_unet.json files")
        p.add_argument("--lora-dir", type=str, default=None,
                       help="--lora-mode full: folder holding <repo with / as _>.safetensors (the hub is not reachable)")
        p.add_argument("--shm-prefix", type=str, default="", help="name prefix of the LoRA shared-memory segments")
    return p


def main(argv=None):
    """`python -m katz_b200.servers {unet,controlnet} <reference flags>`: one server process on one GPU."""
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("unet", "controlnet"):
        raise SystemExit("usage: python -m katz_b200.servers {unet,controlnet} [flags]")
    kind, args = argv[0], build_arg_parser(argv[0]).parse_args(argv[1:])
    from .params import SDXL_UNET_CONFIG, controlnet_param_shapes, init_state_dict, unet_param_shapes
    from .unet import KatzControlNet, KatzUNet
    torch.cuda.set_device(args.gpu_id)
    dev = torch.device("cuda", args.gpu_id)
    dist.init_process_group(backend="nccl", init_method=args.init_method, rank=args.rank, world_size=args.world_size)
    cfg = SDXL_UNET_CONFIG
    if kind == "controlnet":
        sd = torch.load(args.state_dict) if args.state_dict else init_state_dict(
            controlnet_param_shapes(cfg), seed=args.rank, dtype=torch.float16, device=dev, generator_device=dev)
        net = KatzControlNet(cfg, dev, sd)
        net.use_cuda_graph = False
        controlnet_server_loop(net, dev, dst_rank=args.dst_rank, max_requests=args.max_requests, verbose=args.verbose)
    else:
        sd = torch.load(args.state_dict) if args.state_dict else init_state_dict(
            unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev)
        net = KatzUNet(cfg, dev, sd)
        net.use_cuda_graph = True
        ranks = args.controlnet_parallel_rank if args.controlnet_parallel else []
        hooks = unet_lora_hooks_from_args(net, args, dev)
        from .engine import check_device_status
        unet_server_loop(net, dev, controlnet_parallel_rank=ranks, request_hook=hooks[0], lora_hook=hooks[1],
                         restore_hook=hooks[2], check_hook=lambda: check_device_status(net),
                         max_requests=args.max_requests, verbose=args.verbose)
    dist.destroy_process_group()


def unet_lora_hooks_from_args(unet, args, device, shm_client=None):
    """What `main` passes to `unet_server_loop` for the parsed reference flags. `--lora-mode full` reads the adapters
    from `--lora-dir` (safetensors files named after the repos)."""
    import os
    from .lora_utils import KatzPipe
    repos = REFERENCE_LORA_REPOS[args.max_lora_num]
    source = None
    if args.lora_mode == "full" and repos:
        if not args.lora_dir:
            raise SystemExit("--lora-mode full needs --lora-dir (the hub is not reachable)")
        from .lora_files import lora_state_dict

        def source(repo):
            return lora_state_dict(os.path.join(args.lora_dir, repo.replace("/", "_") + ".safetensors"))
    pipe = KatzPipe(unet, lora_source=source, lora_info_dir=args.lora_info_dir)
    return make_lora_hooks(pipe, args.lora_mode, args.load_lora_mode, repos, device, shm_prefix=args.shm_prefix,
                           shm_client=shm_client)


if __name__ == "__main__":
    main()
