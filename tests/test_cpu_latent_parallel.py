"""CPU, gloo, world_size 2 (and 4): the row-split communication logic — halo exchange, shard/gather, statistics
reduction, K/V gather order — checked by rebuilding full-tensor results from the shards with plain torch ops."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn_name, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from katz_b200.latent_parallel import RowParallel
        rp = RowParallel()
        globals()[fn_name](rp)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _run(world, fn_name):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, msg in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)


def _full(shape, seed=0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed))


def _nchw(x):
    return x.permute(0, 3, 1, 2)


def _nhwc(x):
    return x.permute(0, 2, 3, 1).contiguous()


def check_conv_split(rp):
    B, H, W, C, Co = 2, 16, 8, 4, 6
    x = _full((B, H, W, C))
    w = _full((Co, C, 3, 3), 1)
    loc = rp.shard_rows(x)
    r0, h = rp.rows_of(H)
    # stride 1: pad with both halos, no vertical padding left to the convolution
    pad = rp.pad_rows(loc)
    y = F.conv2d(_nchw(pad), w, padding=(0, 1))
    ref = F.conv2d(_nchw(x), w, padding=1)[:, :, r0:r0 + h]
    assert torch.allclose(y, ref, atol=1e-5)
    # stride 2: top halo only
    pad = rp.pad_rows(loc, bottom=False)
    y = F.conv2d(_nchw(pad), w, stride=2, padding=(0, 1))
    ref = F.conv2d(_nchw(x), w, stride=2, padding=1)[:, :, r0 // 2:(r0 + h) // 2]
    assert y.shape == ref.shape and torch.allclose(y, ref, atol=1e-5)
    # upsample then conv: exchange before the upsample, slice rows [1, 2h+3)
    pad = rp.pad_rows(loc)
    up = F.interpolate(_nchw(pad), scale_factor=2.0, mode="nearest")[:, :, 1:2 * h + 3]
    y = F.conv2d(up, w, padding=(0, 1))
    ref = F.conv2d(F.interpolate(_nchw(x), scale_factor=2.0, mode="nearest"), w, padding=1)[:, :, 2 * r0:2 * (r0 + h)]
    assert y.shape == ref.shape and torch.allclose(y, ref, atol=1e-5)
    # image edges are zero rows
    t, b = rp.exchange_halo(loc)
    if rp.rank == 0:
        assert float(t.abs().max()) == 0
    else:
        assert torch.equal(t, x[:, r0 - 1])
    if rp.rank == rp.world - 1:
        assert float(b.abs().max()) == 0
    else:
        assert torch.equal(b, x[:, r0 + h])


def check_stats_and_gather(rp):
    B, H, W, C, G = 2, 8, 4, 16, 4
    x = _full((B, H, W, C), 3)
    loc = rp.shard_rows(x)
    # GroupNorm statistics: fp64 sums over the shard, summed over ranks, equal the full-tensor sums
    v = loc.double().reshape(B, -1, G, C // G)
    sums = torch.stack([v.sum(dim=(1, 3)), (v * v).sum(dim=(1, 3))], dim=-1).contiguous()
    rp.reduce_stats(sums)
    vf = x.double().reshape(B, -1, G, C // G)
    ref = torch.stack([vf.sum(dim=(1, 3)), (vf * vf).sum(dim=(1, 3))], dim=-1)
    assert torch.allclose(sums, ref, rtol=1e-12)
    n = H * W * (C // G)
    mean = sums[..., 0] / n
    var = sums[..., 1] / n - mean * mean
    gn_ref = F.group_norm(_nchw(x), G, eps=1e-5)
    mine = (v - mean[:, None, :, None]) / torch.sqrt(var[:, None, :, None] + 1e-5)
    r0, h = rp.rows_of(H)
    assert torch.allclose(mine.reshape(B, h, W, C).float(), _nhwc(gn_ref)[:, r0:r0 + h], atol=1e-5)
    # row gather restores the original order; the K/V gather is rank-major = global token order
    assert torch.equal(rp.gather_rows(loc), x)
    kv = loc.reshape(B, h * W, C)
    g = rp.gather_shards(kv)
    assert tuple(g.shape) == (rp.world, B, h * W, C)
    assert torch.equal(g.permute(1, 0, 2, 3).reshape(B, H * W, C), x.reshape(B, H * W, C))


def check_bad_split(rp):
    from katz_b200 import KatzError
    with pytest.raises(KatzError):
        rp.rows_of(2 * rp.world + 1)


@pytest.mark.parametrize("world", [2, 4])
def test_row_split_convolutions(world):
    _run(world, "check_conv_split")


def test_row_split_stats_and_gathers():
    _run(2, "check_stats_and_gather")


def test_row_split_rejects_uneven_rows():
    _run(2, "check_bad_split")


def test_single_rank_is_identity():
    from katz_b200.latent_parallel import RowParallel
    rp = RowParallel(rank=0, world=1)
    x = _full((1, 4, 4, 8))
    t, b = rp.exchange_halo(x)
    assert float(t.abs().max()) == 0 and float(b.abs().max()) == 0
    assert torch.equal(rp.gather_rows(x), x) and torch.equal(rp.shard_rows(x), x)


def test_cfg_rows_layout_and_assembly():
    """Batch halves first, rows inside a half: the bookkeeping of the multi-GPU step, on CPU tensors."""
    from katz_b200.latent_parallel import assemble_halves, cfg_rows_layout
    assert cfg_rows_layout(2, 1, 0) == (1, 1, 0, 0, 2)
    assert cfg_rows_layout(2, 2, 1) == (2, 1, 1, 0, 1)
    assert cfg_rows_layout(2, 8, 5) == (2, 4, 1, 1, 1)
    assert cfg_rows_layout(2, 8, 5, split_cfg=False) == (1, 8, 0, 5, 2)
    assert cfg_rows_layout(3, 4, 2) == (1, 4, 0, 2, 3)          # odd batch: rows only
    assert cfg_rows_layout(2, 3, 2) == (1, 3, 0, 2, 2)          # odd world: rows only
    with pytest.raises(Exception):
        cfg_rows_layout(2, 2, 2)
    world, lb = 4, 1
    per_half = [torch.full((lb, 4, 8, 8), float(h + 1)) for h in range(2)]
    gathered = torch.stack([per_half[r // 2] for r in range(world)])       # every rank of a half holds that half, whole
    out = assemble_halves(gathered, 2, 2)
    assert out.shape == (2, 4, 8, 8) and float(out[0].mean()) == 1.0 and float(out[1].mean()) == 2.0
