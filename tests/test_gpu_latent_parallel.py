"""GPU: the kernels behind latent-row parallelism — split GroupNorm, chunked K/V attention, halo-padded convolutions —
checked on one GPU by emulating the shards of several ranks, and the row-parallel UNet path at world size 1."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-12))


@pytest.mark.parametrize("C,HW,P", [(320, 4096, 2), (1280, 1024, 8), (64, 256, 4)])
def test_group_norm_split_equals_fused(cuda_device, C, HW, P):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(2, HW, C, generator=g) + 0.5).half().cuda()
    gamma, beta = torch.randn(C, generator=g).half().cuda(), torch.randn(C, generator=g).half().cuda()
    full = ops.group_norm_nhwc(x, gamma, beta, 32, 1e-5, ops.ACT_SILU)
    s = HW // P
    shards = [x[:, r * s:(r + 1) * s].contiguous() for r in range(P)]
    sums = sum(ops.group_norm_stats(sh, 32) for sh in shards)
    outs = [ops.group_norm_apply(sh, sums, gamma, beta, 32, float(HW) * (C // 32), 1e-5, ops.ACT_SILU) for sh in shards]
    assert _rel(torch.cat(outs, dim=1), full) < 2e-3


@pytest.mark.parametrize("B,H,s,P", [(2, 10, 512, 8), (2, 20, 128, 8), (1, 2, 64, 2)])
def test_attention_reads_gathered_kv_chunks(cuda_device, B, H, s, P):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(1)
    C = H * 64
    q = torch.randn(B, s, C, generator=g).half().cuda()
    kv = torch.randn(B, P * s, 2 * C, generator=g).half().cuda()
    ref = ops.attention(q, kv[:, :, :C], kv[:, :, C:], H)
    gathered = kv.view(B, P, s, 2 * C).permute(1, 0, 2, 3).contiguous()      # [P, B, s, 2C]: what the all-gather leaves
    out = ops.attention(q, gathered[0][:, :, :C], gathered[0][:, :, C:], H, kv_chunks=(P, s, B * s * 2 * C))
    # same kernel on both sides when the chunks are multiples of its 128-key tile (bit-equal); 64-row chunks go to the
    # mma.sync kernel, which differs from the tcgen05 one by accumulation order only
    if s % 128 == 0:
        assert torch.equal(out, ref)
    else:
        assert float((out.float() - ref.float()).abs().max()) < 4e-3


def test_attention_waits_for_pushed_kv_chunks(cuda_device):
    """The attention entry point for K/V chunks that peers push while the kernel already works on the local chunk, on one
    GPU: with every flag raised it must give the chunked result (the chunks are only walked in another order); with one
    flag missing its bounded wait must run out, leave a status word and return."""
    from katz_b200 import _lib, ops
    g = torch.Generator().manual_seed(3)
    B, H, s, P, me = 2, 10, 512, 4, 2
    C = H * 64
    q = torch.randn(B, s, C, generator=g).half().cuda()
    kv = torch.randn(B, P * s, 2 * C, generator=g).half().cuda()
    gathered = kv.view(B, P, s, 2 * C).permute(1, 0, 2, 3).contiguous()      # [P, B, s, 2C]
    chunks = (P, s, B * s * 2 * C)
    ref = ops.attention(q, gathered[0][:, :, :C], gathered[0][:, :, C:], H, kv_chunks=chunks)
    ctrl = torch.zeros(1024, dtype=torch.int32, device="cuda")      # control words as a peer arena holds them
    ctrl[0] = 7                                                      # the exchange that delivered the chunks
    ctrl[64:64 + P] = 7
    out = ops.attention(q, gathered[0][:, :, :C], gathered[0][:, :, C:], H, kv_chunks=chunks, peer=(ctrl.data_ptr(), me))
    assert ops.tc05_status() == 0
    assert float((out.float() - ref.float()).abs().max()) < 2e-3
    ctrl[64 + 1] = 6                                                 # rank 1's block of exchange 7 never arrives
    ops.attention(q, gathered[0][:, :, :C], gathered[0][:, :, C:], H, kv_chunks=chunks, peer=(ctrl.data_ptr(), me))
    assert ops.tc05_status() != 0
    _lib.check(_lib.load().katz_tc05_clear_status(), "katz_tc05_clear_status")
    ctrl[64 + 1] = 7
    out2 = ops.attention(q, gathered[0][:, :, :C], gathered[0][:, :, C:], H, kv_chunks=chunks, peer=(ctrl.data_ptr(), me))
    assert ops.tc05_status() == 0
    assert torch.equal(out2, out)


@pytest.mark.parametrize("gemm", ["tc05", "mma"])
def test_halo_padded_convolutions(cuda_device, gemm, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", gemm)
    from katz_b200 import ops
    g = torch.Generator().manual_seed(2)
    B, H, W, C, Co, P = 2, 16, 32, 64, 128, 4
    x = torch.randn(B, H, W, C, generator=g).half().cuda()
    w = (torch.randn(Co, 3, 3, C, generator=g) / 24).half().cuda()
    bias = torch.randn(Co, generator=g).half().cuda()
    h = H // P
    zero = torch.zeros(B, 1, W, C, dtype=torch.float16, device="cuda")
    xp = torch.cat([zero, x, zero], dim=1)
    full = ops.conv2d(x, w, bias)
    full_s2 = ops.conv2d(x, w, bias, stride=2)
    full_up = ops.conv2d(x, w, bias, upsample=True)
    for r in range(P):
        pad = xp[:, r * h:r * h + h + 2].contiguous()
        y = ops.conv2d(pad, w, bias, pad_h=0)
        assert _rel(y, full[:, r * h:(r + 1) * h]) < 1e-3
        y2 = ops.conv2d(pad[:, :h + 1].contiguous(), w, bias, stride=2, pad_h=0)
        assert _rel(y2, full_s2[:, r * h // 2:(r + 1) * h // 2]) < 1e-3
        up = ops.upsample_nearest2x(pad)[:, 1:2 * h + 3].contiguous()
        y3 = ops.conv2d(up, w, bias, pad_h=0)
        assert _rel(y3, full_up[:, 2 * r * h:2 * (r + 1) * h]) < 1e-3
    assert ops.tc05_status() == 0


def test_row_parallel_unet_world1_matches_plain(cuda_device):
    from katz_b200.latent_parallel import RowParallel
    from katz_b200.params import TINY_UNET_CONFIG, init_state_dict, unet_param_shapes
    from katz_b200.unet import KatzUNet
    from tests.golden.make_golden import tiny_inputs
    cfg = TINY_UNET_CONFIG
    unet = KatzUNet(cfg, cuda_device, init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16))
    sample, ctx, te, ti, _ = (t.half().cuda() for t in tiny_inputs(cfg))
    kw = dict(encoder_hidden_states=ctx, added_cond_kwargs={"text_embeds": te, "time_ids": ti})
    t = torch.tensor([500.0], device="cuda")
    plain = unet(sample, t, **kw)[0]
    unet.rp = RowParallel(rank=0, world=1)
    split = unet(sample, t, **kw)[0]
    unet.rp = None
    assert _rel(split, plain) < 2e-3


def test_row_split_equals_single_gpu_on_all_gpus(cuda_device):
    """One process per GPU under torchrun (NCCL): needs at least two GPUs on the box."""
    import os
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    n = 4 if n >= 4 else 2
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(root, "tests", "row_parallel_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 3 * n          # eager row split, batch halves x rows, graphed row split: every rank


@pytest.mark.parametrize("B,P", [(1, 4), (2, 2)])
def test_halo_assemble_equals_padded_slices(cuda_device, B, P):
    """The one-pass kernel that builds a shard's convolution input (neighbour rows, zeros at the image edge, optional
    nearest 2x upsample) against slicing the zero-padded whole tensor; the shards of P ranks are emulated on one GPU."""
    from katz_b200 import ops
    g = torch.Generator().manual_seed(3)
    H, W, C = 16, 8, 64
    x = torch.randn(B, H, W, C, generator=g).half().cuda()
    h = H // P
    shards = [x[:, r * h:(r + 1) * h].contiguous() for r in range(P)]
    edges = torch.stack([torch.stack([s[:, 0], s[:, -1]]) for s in shards]).contiguous()       # [P, 2, B, W, C]
    zero = torch.zeros(B, 1, W, C, dtype=torch.float16, device="cuda")
    xp = torch.cat([zero, x, zero], dim=1)
    up = xp.repeat_interleave(2, dim=1).repeat_interleave(2, dim=2)
    for r in range(P):
        both = ops.halo_assemble(shards[r], edges, r, P)
        assert torch.equal(both, xp[:, r * h:r * h + h + 2])
        top_only = ops.halo_assemble(shards[r], edges, r, P, bottom=False)
        assert torch.equal(top_only, xp[:, r * h:r * h + h + 1])
        ups = ops.halo_assemble(shards[r], edges, r, P, upsample=True)
        assert torch.equal(ups, up[:, 2 * r * h + 1:2 * r * h + 2 * h + 3])
    alone = ops.halo_assemble(x, None, 0, 1)
    assert torch.equal(alone, xp)
