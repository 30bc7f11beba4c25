"""CPU, gloo, world_size 3: the server message protocol (rank 0 = pipeline, rank 1 = UNet server, rank 2 = ControlNet
server) with stand-in models, message for message as the reference's scripts exchange them."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

BOC, LAT, COND, TL, CD, PD = (8, 16, 32), (8, 8), (64, 64), 7, 16, 12


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fake_controlnet(x, t, encoder_hidden_states, controlnet_cond, added_cond_kwargs):
    from katz_b200.servers import residual_shapes
    shapes, mid = residual_shapes(x.shape[0], BOC, *LAT)
    base = x.float().mean() + t + controlnet_cond.float().mean() + encoder_hidden_states.float().mean()
    return [torch.full(s, float(base) + i, dtype=torch.float16) for i, s in enumerate(shapes)], \
        torch.full(mid, float(base) - 1, dtype=torch.float16)


def _fake_unet(x, t, encoder_hidden_states, added_cond_kwargs, return_dict=False, down_block_additional_residuals=None,
               mid_block_additional_residual=None, combine_scales=None):
    acc = x.float() * 2 + t + added_cond_kwargs["time_ids"].float().sum()
    if down_block_additional_residuals is not None:
        for net, s in zip(down_block_additional_residuals, combine_scales):
            acc = acc + s * sum(float(d.float().mean()) for d in net)
        for m, s in zip(mid_block_additional_residual, combine_scales):
            acc = acc + s * float(m.float().mean())
    return (acc.half(),)


def _worker(rank, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=3)
    try:
        from katz_b200 import servers
        dev = torch.device("cpu")
        common = dict(latent_hw=LAT, cond_hw=COND, text_len=TL, cross_dim=CD, pooled_dim=PD)
        if rank == 1:
            restored = []
            n = servers.unet_server_loop(_fake_unet, dev, controlnet_parallel_rank=[2], block_out_channels=BOC,
                                         restore_hook=lambda: restored.append(1), max_requests=2, **common)
            assert n == 2 and len(restored) == 2
        elif rank == 2:
            assert servers.controlnet_server_loop(_fake_controlnet, dev, dst_rank=1, max_requests=2, **common) == 2
        else:
            g = torch.Generator().manual_seed(0)
            for req in range(2):
                B, steps = 1, 3
                dist.broadcast(torch.tensor([B], dtype=torch.int32), src=0)
                dist.broadcast(torch.tensor([steps], dtype=torch.int32), src=0)
                cond = torch.rand(B, 3, *COND, generator=g).half()
                dist.broadcast(cond, src=0)
                pe, te = torch.randn(B, TL, CD, generator=g).half(), torch.randn(B, PD, generator=g).half()
                ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half()
                for tns in (pe, te, ti):
                    dist.send(tns, dst=1)
                for s in range(steps):
                    x = torch.randn(B, 4, *LAT, generator=g).half()
                    t = torch.tensor(float(981 - 20 * s))
                    dist.broadcast(x, src=0)
                    dist.broadcast(t, src=0)
                    got = torch.empty_like(x)
                    dist.recv(got, src=1)
                    d, m = _fake_controlnet(x, t, pe, cond, None)
                    want = _fake_unet(x, t, pe, {"time_ids": ti}, down_block_additional_residuals=[d],
                                      mid_block_additional_residual=[m], combine_scales=[1.0])[0]
                    assert torch.equal(got, want), (req, s)
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_server_protocol_round_trip():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, msg in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)


def test_residual_shapes_match_the_sdxl_list():
    from katz_b200.servers import build_arg_parser, residual_shapes
    shapes, mid = residual_shapes(2, (320, 640, 1280), 128, 128)
    assert shapes == [(2, 320, 128, 128)] * 3 + [(2, 320, 64, 64), (2, 640, 64, 64), (2, 640, 64, 64), (2, 640, 32, 32),
                                                 (2, 1280, 32, 32), (2, 1280, 32, 32)]
    assert mid == (2, 1280, 32, 32)
    a = build_arg_parser("unet").parse_args(["--world-size", "8", "--controlnet-parallel", "--controlnet-parallel-rank", "3", "5", "7",
                                             "--lora-mode", "sync", "--load-lora-mode", "async", "--max-lora-num", "2"])
    assert a.controlnet_parallel_rank == [3, 5, 7] and a.lora_mode == "sync"


def test_reference_flags_select_the_lora_hooks():
    """What main() hands to unet_server_loop for each combination of the reference's LoRA flags (sdxl_unet_server.py:24-38)."""
    from katz_b200 import servers

    class FakePipe:
        lora_info_dir = "."

        def __init__(self):
            self.calls = []

        def patch_on_lora(self, sd, repos, default):
            self.calls.append((sorted(sd), list(repos), default))

        def restore_unet(self):
            self.calls.append("restore")

    class FakeClient:
        def gather(self, i, device):
            return {"a": torch.full((2,), float(i + 1)), "b": torch.ones(2)}

    def parse(*flags):
        return servers.build_arg_parser("unet").parse_args(list(flags))

    a = parse()
    assert a.lora_mode == "without" and a.load_lora_mode == "default" and a.max_lora_num == 0
    repos = servers.REFERENCE_LORA_REPOS
    assert repos[0] == [] and len(repos[1]) == 1 and len(repos[2]) == 2

    pipe = FakePipe()
    req, lora, restore = servers.make_lora_hooks(pipe, "without", "default", [], "cpu")
    assert req is None and lora is None and restore == pipe.restore_unet

    req, lora, restore = servers.make_lora_hooks(pipe, "full", "default", repos[1], "cpu")
    assert req is not None and lora is None

    # sync + async: nothing happens until the loader's status says every adapter is in shared memory; then the adapters
    # are summed element-wise and merged once through the pipeline entry point
    req, lora, restore = servers.make_lora_hooks(pipe, "sync", "async", repos[2], "cpu", shm_client=FakeClient())
    assert req is None and lora is not None
    assert lora(0) is False and lora(10) is False and pipe.calls == []
    assert lora(20) is True
    keys, got_repos, default = pipe.calls[0]
    assert keys == ["a", "b"] and got_repos == repos[2] and default is None
    restore()
    assert pipe.calls[-1] == "restore"
    # a mode that names adapters but has none to load needs no hook
    assert servers.make_lora_hooks(pipe, "sync", "async", [], "cpu")[:2] == (None, None)
