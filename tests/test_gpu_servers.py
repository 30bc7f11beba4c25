"""GPU: the reference's three-process deployment with the real katz_b200 models — rank 0 plays the pipeline
(sdxl_pipeline.py / pipeline_controlnet_sd_xl_katz.py:1508-1675), rank 1 runs `servers.unet_server_loop` with a KatzUNet
wired exactly as `python -m katz_b200.servers unet --lora-mode sync --load-lora-mode async --max-lora-num 1` wires it
(sdxl_unet_server.py:96-220), rank 2 runs `servers.controlnet_server_loop` with a KatzControlNet
(sdxl_controlnet_server.py:60-115). A loader thread hands the adapter over through shared memory
(load_lora_shm_multi.py:85-121); the UNet server gathers it to the GPU and merges it when the status word says so
(sdxl_unet_server.py:153-181), and restores the pristine weights after the request (:217).

All three processes share the one GPU of the test box, so the messages travel over gloo on CPU tensors (NCCL wants one
GPU per rank) while every model evaluation runs on the GPU. Rank 0 computes what it expects with its own copies of the
models: same kernels, same GPU, so the predictions must match bit for bit, before the merge, after it, and in the second
request (which shows the restore)."""
import json
import os
import socket
import threading

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

REPO = "TheLastBen/Papercut_SDXL"          # the repo `--max-lora-num 1` names (sdxl_unet_server.py:74)
RANK, STEPS, REQUESTS, MERGE_AT = 8, 4, 2, 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fixture_files(info_dir):
    """lora_info_shm/<repo>.json and <repo>_key_match_unet.json for the tiny UNet, in the reference's formats."""
    from katz_b200.lora import synthetic_key_map
    from katz_b200.params import TINY_UNET_CONFIG, lora_target_keys, unet_param_shapes
    shapes = unet_param_shapes(TINY_UNET_CONFIG)
    km = synthetic_key_map(lora_target_keys(TINY_UNET_CONFIG, include_proj=True))
    info = {}
    for k, m in km.items():
        o, n = shapes[k]
        info[m["lora_down_key"]] = {"shape": [RANK, n], "nbytes": RANK * n * 2}
        info[m["lora_up_key"]] = {"shape": [o, RANK], "nbytes": o * RANK * 2}
    os.makedirs(info_dir, exist_ok=True)
    stem = os.path.join(info_dir, REPO.replace("/", "_"))
    with open(stem + ".json", "w") as fw:
        json.dump(info, fw)
    with open(stem + "_key_match_unet.json", "w") as fw:
        json.dump(km, fw)
    return info, km


def _lora_tensors(info):
    g = torch.Generator().manual_seed(123)
    out = {}
    for k, m in info.items():
        std = 1.0 / RANK if ".down." in k else 2e-4          # times the reference's fixed scale 312.5: a visible change
        out[k] = (torch.randn(m["shape"], generator=g) * std).half()
    return out


def _models(dev):
    from katz_b200.params import TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict, unet_param_shapes
    from katz_b200.unet import KatzControlNet, KatzUNet
    cfg = TINY_UNET_CONFIG
    unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16))
    cn = KatzControlNet(cfg, dev, init_state_dict(controlnet_param_shapes(cfg), seed=2, dtype=torch.float16))
    return cfg, unet, cn


def _worker(rank, port, tmp, prefix, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=3)
    try:
        from katz_b200 import ops, servers
        from katz_b200.lora_shm import LoraShmClient, LoraShmLoader
        from tests.golden.make_golden import tiny_inputs
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        cpu = torch.device("cpu")
        info_dir = os.path.join(tmp, "lora_info_shm")
        cfg, unet, cn = _models(dev)
        common = dict(latent_hw=(16, 16), cond_hw=(128, 128), text_len=77, cross_dim=cfg["cross_attention_dim"], pooled_dim=64)
        with open(os.path.join(info_dir, REPO.replace("/", "_") + ".json")) as fr:
            info = json.load(fr)
        if rank == 1:
            args = servers.build_arg_parser("unet").parse_args(
                ["--world-size", "3", "--controlnet-parallel", "--controlnet-parallel-rank", "2", "--lora-mode", "sync",
                 "--load-lora-mode", "async", "--max-lora-num", "1", "--lora-info-dir", info_dir, "--shm-prefix", prefix])
            request_hook, lora_hook, restore_hook = servers.unet_lora_hooks_from_args(unet, args, dev)
            assert request_hook is None and lora_hook is not None
            from katz_b200.engine import check_device_status
            n = servers.unet_server_loop(lambda *a, **k: (unet(*a, **k)[0].cpu(),), cpu, controlnet_parallel_rank=[2],
                                         block_out_channels=cfg["block_out_channels"], lora_hook=lora_hook,
                                         restore_hook=restore_hook, check_hook=lambda: check_device_status(unet),
                                         max_requests=REQUESTS, **common)
            assert n == REQUESTS
        elif rank == 2:
            def net(*a, **k):
                d, m = cn(*a, **k)
                return [t.cpu() for t in d], m.cpu()
            assert servers.controlnet_server_loop(net, cpu, dst_rank=1, max_requests=REQUESTS, **common) == REQUESTS
        else:
            from katz_b200.lora_utils import KatzPipe
            tensors = _lora_tensors(info)
            loader = LoraShmLoader(0, 1, info, lambda code: tensors, prefix=prefix)
            th = threading.Thread(target=loader.serve, kwargs=dict(idle_timeout_s=120.0), daemon=True)
            th.start()
            client = LoraShmClient([info], prefix=prefix, attach_timeout_s=60)
            pipe = KatzPipe(unet, lora_info_dir=info_dir)
            sample, ctx, te, ti, cond = (t.half() for t in tiny_inputs(cfg))
            added = {"text_embeds": te.to(dev), "time_ids": ti.to(dev)}
            g = torch.Generator().manual_seed(3)
            preds = []
            for req in range(REQUESTS):
                B = sample.shape[0]
                dist.broadcast(torch.tensor([B], dtype=torch.int32), src=0)
                dist.broadcast(torch.tensor([STEPS], dtype=torch.int32), src=0)
                dist.broadcast(cond, src=0)
                for t_ in (ctx, te, ti):
                    dist.send(t_, dst=1)
                patched = False
                for s in range(STEPS):
                    if s == MERGE_AT:
                        client.request([1])          # the pipeline asks the loader for adapter number 1 ...
                        client.wait(timeout_s=60)    # ... and from here on the status word reads 10
                    if not patched:
                        status = client.status()
                        dist.send(torch.tensor(status, dtype=torch.int32), dst=1)
                        if status == 10:
                            pipe.patch_on_lora({k: v.to(dev) for k, v in tensors.items()}, [REPO], None)
                            patched = True
                    x = torch.randn(B, 4, 16, 16, generator=g).half()
                    t = torch.tensor(float(981 - 20 * s))
                    dist.broadcast(x, src=0)
                    dist.broadcast(t, src=0)
                    got = torch.empty_like(x)
                    dist.recv(got, src=1)
                    d, m = cn(x.to(dev), t, encoder_hidden_states=ctx.to(dev), controlnet_cond=cond.to(dev), added_cond_kwargs=added)
                    want = unet(x.to(dev), t, encoder_hidden_states=ctx.to(dev), added_cond_kwargs=added,
                                down_block_additional_residuals=[d], mid_block_additional_residual=[m], combine_scales=[1.0])[0]
                    assert torch.equal(got, want.cpu()), (req, s, float((got.float() - want.cpu().float()).abs().max()))
                    preds.append(got.clone())
                assert patched
                pipe.restore_unet()
                client.clear()
            # the adapter changed the prediction of the steps after the merge, and request 2 started from pristine weights
            assert ops.tc05_status() == 0
            client.quit()
            th.join(timeout=30)
            client.close()
            loader.close()
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_servers_with_real_models_async_lora_over_shm(cuda_device, tmp_path):
    _fixture_files(str(tmp_path / "lora_info_shm"))
    import gc
    gc.collect()
    torch.cuda.empty_cache()              # the three child processes share this GPU with whatever this process still caches
    prefix = "katzsrv%d_" % os.getpid()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, str(tmp_path), prefix, q)) for r in range(3)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=600) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    for rank, msg in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)


def test_patch_on_lora_entry_points_with_the_reference_signatures(cuda_device, tmp_path):
    """lora_utils.patch_on_lora(pipe, repos) and pipe.patch_on_lora(lora_state_dict, repos, default_unet_state_dict) against
    the oracle's merge arithmetic with the reference's fixed scale fp16(20000/64)."""
    from katz_b200.lora import REFERENCE_UNET_SCALE
    from katz_b200.lora_utils import KatzPipe, patch_on_lora
    from oracle import lora_oracle
    info, km = _fixture_files(str(tmp_path / "lora_info_shm"))
    cfg, unet, _ = _models(cuda_device)
    tensors = _lora_tensors(info)
    pristine = {k: v.clone() for k, v in unet.state_dict().items()}
    ad = {k: (tensors[m["lora_up_key"]], tensors[m["lora_down_key"]]) for k, m in km.items()}
    ref = lora_oracle.merge_set({k: pristine[k].cpu() for k in km}, [ad], [REFERENCE_UNET_SCALE])

    def check_merged():
        sd = unet.state_dict()
        for k in km:
            d = (sd[k].cpu().float() - ref[k].float()).abs()
            assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()), k
            assert not torch.equal(sd[k].cpu(), pristine[k].cpu())

    pipe = KatzPipe(unet, lora_source=lambda repo: (tensors, None), lora_info_dir=str(tmp_path / "lora_info_shm"))
    patch_on_lora(pipe, [REPO])                                    # lora_utils.py:9
    check_merged()
    pipe.restore_unet()
    for k, v in unet.state_dict().items():
        assert torch.equal(v, pristine[k]), k
    pipe.patch_on_lora(tensors, [REPO], pristine)                  # pipeline_controlnet_sd_xl_katz.py:1730
    check_merged()
    for k in km:
        assert torch.equal(pipe.lora_merger(km.keys()).pristine[k], pristine[k])      # the caller's dict was not modified
    pipe.restore_unet(pristine)
    for k, v in unet.state_dict().items():
        assert torch.equal(v, pristine[k]), k
    with pytest.raises(Exception):
        patch_on_lora(KatzPipe(unet, lora_info_dir=str(tmp_path / "lora_info_shm")), [REPO])      # no lora_source: fails loudly


def test_text_encoder_lora_layers_through_both_entry_points(cuda_device, tmp_path):
    """The text-encoder part of the reference's two patch functions (lora_utils.py:36-54, ...katz.py:1749-1767):
    `state_dict[key] += up @ down` over the reference's text-encoder key maps, into a module and into a plain dict."""
    from katz_b200.lora_utils import KatzPipe, patch_on_lora
    from katz_b200.params import text_encoder_lora_key_map
    from oracle import lora_oracle
    info_dir = str(tmp_path / "lora_info_shm")
    info, km = _fixture_files(info_dir)
    cfg, unet, _ = _models(cuda_device)
    tensors = _lora_tensors(info)
    g = torch.Generator().manual_seed(9)
    te_maps, te_w = {}, {}
    for which, layers in (("text_encoder", None), ("text_encoder_2", 3)):       # all 72 layers of the first, 18 of the second
        kmt, shapes = text_encoder_lora_key_map(which, layers)
        te_maps[which] = kmt
        with open(os.path.join(info_dir, REPO.replace("/", "_") + "_key_match_%s.json" % which), "w") as fw:
            json.dump(kmt, fw)
        te_w[which] = {k: (torch.randn(shp, generator=g) * 0.02).half() for k, shp in shapes.items()}
        for k, m in kmt.items():
            o, n = shapes[k]
            tensors[m["lora_down_key"]] = (torch.randn(RANK, n, generator=g) / RANK).half()
            tensors[m["lora_up_key"]] = (torch.randn(o, RANK, generator=g) * 0.02).half()

    class Encoder(torch.nn.Module):                                              # weights addressed by the reference's key names
        def __init__(self, weights):
            super().__init__()
            self.w = torch.nn.ParameterDict({k.replace(".", "/"): torch.nn.Parameter(v.clone().cuda(), requires_grad=False) for k, v in weights.items()})

        def state_dict(self):
            return {k.replace("/", "."): v.data for k, v in self.w.items()}

    te1 = Encoder(te_w["text_encoder"])
    te2 = {k: v.clone().cuda() for k, v in te_w["text_encoder_2"].items()}
    pipe = KatzPipe(unet, lora_source=lambda repo: (tensors, None), lora_info_dir=info_dir, text_encoder=te1, text_encoder_2=te2)

    def expected(which, times):
        kmt = te_maps[which]
        ad = {k: (tensors[m["lora_up_key"]], tensors[m["lora_down_key"]]) for k, m in kmt.items()}
        w = {k: te_w[which][k] for k in kmt}
        for _ in range(times):
            w = lora_oracle.merge_set(w, [ad], [1.0])
        return w

    def check(times):
        for which, live in (("text_encoder", te1.state_dict()), ("text_encoder_2", te2)):
            ref = expected(which, times)
            for k in te_maps[which]:
                d = (live[k].cpu().float() - ref[k].float()).abs()
                assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()), (which, k)
                assert not torch.equal(live[k].cpu(), te_w[which][k])

    patch_on_lora(pipe, [REPO])                                    # lora_utils.py:9
    check(1)
    pipe.patch_on_lora(tensors, [REPO], None)                      # ...katz.py:1730: adds into the text encoders again
    check(2)
    pipe.restore_unet()                                            # the reference restores the UNet only
    assert not torch.equal(te2[next(iter(te2))].cpu(), te_w["text_encoder_2"][next(iter(te2))])
    pipe.restore_text_encoders()
    for k, v in te1.state_dict().items():
        assert torch.equal(v.cpu(), te_w["text_encoder"][k]), k
    for k, v in te2.items():
        assert torch.equal(v.cpu(), te_w["text_encoder_2"][k]), k
    # a pipe without text encoders says so and still merges the UNet
    plain = KatzPipe(unet, lora_source=lambda repo: (tensors, None), lora_info_dir=info_dir)
    patch_on_lora(plain, [REPO])
    plain.restore_unet()
    with pytest.raises(Exception):
        KatzPipe(unet, lora_source=lambda repo: (tensors, None), lora_info_dir=info_dir, text_encoder={}).patch_text_encoders(tensors, REPO)


def test_hoisted_text_kv_and_cond_embedding_give_identical_steps(cuda_device):
    """Step-invariant hoisting: with `cache_text_kv` / `cache_cond_embedding` the cross-attention K/V projection and the
    ControlNet conditioning embedding are computed once per request; every step must be bit-identical to the un-hoisted
    one, a changed prompt or image must be picked up, and so must a LoRA merge that touches attn2.to_k / to_v."""
    from katz_b200.lora import LoraMerger
    from katz_b200.params import lora_target_keys
    from tests.golden.make_golden import tiny_inputs
    cfg, unet, cn = _models(cuda_device)
    dev = cuda_device
    sample, ctx, te, ti, cond = (t.half().to(dev) for t in tiny_inputs(cfg))
    added = {"text_embeds": te, "time_ids": ti}

    def step(x, t, c, img):
        d, m = cn(x, t, encoder_hidden_states=c, controlnet_cond=img, added_cond_kwargs=added, nhwc_out=True)
        return unet(x, t, encoder_hidden_states=c, added_cond_kwargs=added, down_block_additional_residuals=d,
                    mid_block_additional_residual=m)[0].clone()

    ts = [torch.tensor([981.0], device=dev), torch.tensor([961.0], device=dev)]
    xs = [sample, (sample * 0.9).half()]
    ctx2, cond2 = (ctx * 0.5).half(), (cond * 0.5).half()
    plain = [step(xs[i], ts[i], ctx, cond) for i in range(2)] + [step(xs[0], ts[0], ctx2, cond2)]
    for net in (unet, cn):
        net.cache_text_kv = True
    cn.cache_cond_embedding = True
    try:
        hoisted = [step(xs[i], ts[i], ctx, cond) for i in range(2)] + [step(xs[0], ts[0], ctx2, cond2)]
        for a, b in zip(plain, hoisted):
            assert torch.equal(a, b)
        # a merge into attn2.to_k / to_v invalidates the cached K/V
        keys = [k for k in lora_target_keys(cfg) if ".attn2.to_k." in k or ".attn2.to_v." in k]
        targets = unet.lora_targets(keys)
        g = torch.Generator().manual_seed(9)
        ad = {k: ((torch.randn(w.shape[0], 8, generator=g) * 0.05).half().to(dev), (torch.randn(8, w.shape[1], generator=g) / 8).half().to(dev))
              for k, w in targets.items()}
        merger = LoraMerger(targets)
        merger.merge(ad, 1.0)
        unet.invalidate_caches()
        merged_h = step(xs[0], ts[0], ctx2, cond2)
        unet.cache_text_kv = False
        merged_p = step(xs[0], ts[0], ctx2, cond2)
        assert torch.equal(merged_h, merged_p) and not torch.equal(merged_p, plain[2])
    finally:
        for net in (unet, cn):
            net.cache_text_kv = False
        cn.cache_cond_embedding = False


def test_graphed_step_hoist_follows_prompt_image_and_weights(cuda_device):
    """engine.GraphedStep(hoist=True): text K/V and the conditioning embedding are computed outside the captured step. The
    replay must equal the un-hoisted graph bit for bit, for the first prompt, after a new prompt and image arrive through
    run(), and after a LoRA merge changed the K/V weights (noticed through the nets' weight epoch)."""
    from katz_b200.engine import GraphedStep
    from katz_b200.lora import LoraMerger
    from katz_b200.params import lora_target_keys
    from tests.golden.make_golden import tiny_inputs
    cfg, unet, cn = _models(cuda_device)
    dev = cuda_device
    sample, ctx, te, ti, cond = (t.half().to(dev) for t in tiny_inputs(cfg))
    feed = dict(sample=sample, timestep=torch.tensor([981.0]), encoder_hidden_states=ctx, text_embeds=te, time_ids=ti,
                controlnet_cond=cond)
    plain = GraphedStep(unet, 2, 16, 16, controlnets=[cn], conditioning_scales=[0.5])
    hoisted = GraphedStep(unet, 2, 16, 16, controlnets=[cn], conditioning_scales=[0.5], hoist=True)
    assert hoisted.launches_per_step < plain.launches_per_step
    assert unet._hoisted_kv is None and cn._hoisted_cond is None      # eager callers of the nets are unaffected
    a, b = plain.run(**feed).clone(), hoisted.run(**feed).clone()
    assert torch.equal(a, b)
    feed2 = dict(feed, encoder_hidden_states=(ctx * 0.5).half(), controlnet_cond=(cond * 0.5).half(),
                 timestep=torch.tensor([961.0]))
    a2, b2 = plain.run(**feed2).clone(), hoisted.run(**feed2).clone()
    assert torch.equal(a2, b2) and not torch.equal(a2, a)
    keys = [k for k in lora_target_keys(cfg) if ".attn2.to_k." in k or ".attn2.to_v." in k]
    targets = unet.lora_targets(keys)
    g = torch.Generator().manual_seed(9)
    ad = {k: ((torch.randn(w.shape[0], 8, generator=g) * 0.05).half().to(dev), (torch.randn(8, w.shape[1], generator=g) / 8).half().to(dev))
          for k, w in targets.items()}
    merger = LoraMerger(targets)
    merger.merge(ad, 1.0)
    unet.invalidate_caches()
    a3, b3 = plain.replay().clone(), hoisted.replay().clone()
    assert torch.equal(a3, b3) and not torch.equal(a3, a2)
    merger.restore()
    unet.invalidate_caches()
    assert torch.equal(hoisted.replay(), a2)
