"""Run under torchrun on N GPUs (one process per GPU): the row-split UNet step must equal the single-GPU step.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 tests/row_parallel_check.py [--sdxl]

Without flags: the tiny configuration (latent 32x32) with a ControlNet's residuals. With `--sdxl`: the full SDXL UNet, batch
2, latent 128x128 (the benchmark's step). Each check compares with the single-GPU result of the same build computed on the
same rank: max-abs <= 1e-2 and relative L2 <= 2e-3 are required, bit identity is reported (the row split changes only the
order in which the GroupNorm partial sums are added). Prints one line per rank and check and exits non-zero on a mismatch
or when a bounded device-side wait gave up. tests/test_gpu_latent_parallel.py launches it when the box has at least two
GPUs."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from katz_b200.latent_parallel import RowParallel
    from katz_b200.params import TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict, unet_param_shapes
    from katz_b200.unet import KatzControlNet, KatzUNet
    from tests.golden.make_golden import tiny_inputs
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    from katz_b200 import ops
    sdxl = "--sdxl" in sys.argv
    if sdxl:
        from katz_b200.params import SDXL_UNET_CONFIG
        cfg = dict(SDXL_UNET_CONFIG)
        # the same seed on the same kind of GPU draws the same weights on every rank
        unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16, device=dev, generator_device=dev))
        g = torch.Generator().manual_seed(0)
        sample = torch.randn(2, 4, 128, 128, generator=g).half().to(dev)
        ctx = torch.randn(2, 77, 2048, generator=g).half().to(dev)
        te = torch.randn(2, 1280, generator=g).half().to(dev)
        ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * 2).half().to(dev)
        down = mid = None
    else:
        cfg = dict(TINY_UNET_CONFIG)
        cfg["sample_size"] = 32          # 32 rows: 8 per rank at world 4 on the finest level, 2 on the coarsest
        unet = KatzUNet(cfg, dev, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16))
        cn = KatzControlNet(cfg, dev, init_state_dict(controlnet_param_shapes(cfg), seed=2, dtype=torch.float16))
        sample, ctx, te, ti, cond = (t.half().to(dev) for t in tiny_inputs(cfg))
    kw = dict(encoder_hidden_states=ctx, added_cond_kwargs={"text_embeds": te, "time_ids": ti})
    t = torch.tensor([500.0], device=dev)
    if not sdxl:
        down, mid = cn(sample, t, controlnet_cond=cond, **kw)
    ref = unet(sample, t, down_block_additional_residuals=down, mid_block_additional_residual=mid, **kw)[0]
    unet.rp = RowParallel(rank, world)
    out = unet(sample, t, down_block_additional_residuals=down, mid_block_additional_residual=mid, **kw)[0]
    torch.cuda.synchronize()
    err = float((out.float() - ref.float()).abs().max())
    rel = float((out.float() - ref.float()).norm() / ref.float().norm())
    ok = err <= 1e-2 and rel <= 2e-3
    print("rank %d/%d %s row-split vs single-GPU: max-abs %.3e rel-l2 %.3e bit-identical %s %s"
          % (rank, world, "SDXL" if sdxl else "tiny", err, rel, bool(torch.equal(out, ref)), "OK" if ok else "MISMATCH"), flush=True)
    # the graphed step that splits the batch halves first and the rows inside a half
    from katz_b200.latent_parallel import CfgRowParallelStep
    unet.rp = None
    ref2 = unet(sample, t, **kw)[0]
    hw = sample.shape[-1]
    step = CfgRowParallelStep(unet, sample.shape[0], hw, hw, rank, world, text_len=ctx.shape[1])
    out2 = step.run(sample=sample, timestep=t, encoder_hidden_states=ctx, text_embeds=te, time_ids=ti)
    torch.cuda.synchronize()
    err2 = float((out2.float() - ref2.float()).abs().max())
    rel2 = float((out2.float() - ref2.float()).norm() / ref2.float().norm())
    ok2 = err2 <= 1e-2 and rel2 <= 2e-3
    try:
        step.check()
    except Exception as e:  # noqa: BLE001
        ok2 = False
        print("rank %d: %s" % (rank, e), flush=True)
    print("rank %d/%d cfg%d x rows%d graphed step vs single-GPU: max-abs %.3e rel-l2 %.3e bit-identical %s %s"
          % (rank, world, step.halves, step.rows_world, err2, rel2, bool(torch.equal(out2, ref2)), "OK" if ok2 else "MISMATCH"), flush=True)
    # the pure row split as a graphed step: its exchanges go over the peer-memory arena
    step3 = CfgRowParallelStep(unet, sample.shape[0], hw, hw, rank, world, text_len=ctx.shape[1], split_cfg=False)
    out3 = step3.run(sample=sample, timestep=t, encoder_hidden_states=ctx, text_embeds=te, time_ids=ti)
    torch.cuda.synchronize()
    unet.rp = None
    err3 = float((out3.float() - ref2.float()).abs().max())
    rel3 = float((out3.float() - ref2.float()).norm() / ref2.float().norm())
    peer = step3._inner.rp.peer
    ok3 = err3 <= 1e-2 and rel3 <= 2e-3 and (peer is None or peer.status() == 0) and ops.tc05_status() == 0
    print("rank %d/%d rows%d graphed step over %s vs single-GPU: max-abs %.3e rel-l2 %.3e bit-identical %s %s"
          % (rank, world, step3.rows_world, "peer memory" if peer is not None else "NCCL", err3, rel3,
             bool(torch.equal(out3, ref2)), "OK" if ok3 else "MISMATCH"), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    # NCCL communicators captured in live CUDA graphs do not tear down cleanly: leave without destroying the group
    os._exit(0 if (ok and ok2 and ok3) else 1)


if __name__ == "__main__":
    main()
