"""GPU parity of the fused LoRA merge against the oracle (lora_utils.py:29-33 arithmetic) through the C ABI."""
import os
from collections import OrderedDict

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(shapes, rank, dtype, seed, a_std=None, b_std=0.01):
    g = torch.Generator().manual_seed(seed)
    W, ad = OrderedDict(), OrderedDict()
    for i, (o, n) in enumerate(shapes):
        k = "layer%d.weight" % i
        W[k] = (torch.randn(o, n, generator=g) * 0.02).to(dtype)
        down = (torch.randn(rank, n, generator=g) * (a_std if a_std else 1.0 / rank)).to(dtype)
        up = (torch.randn(o, rank, generator=g) * b_std).to(dtype)
        ad[k] = (up, down)
    return W, ad


def _cuda(d):
    return OrderedDict((k, tuple(t.cuda() for t in v) if isinstance(v, tuple) else v.cuda()) for k, v in d.items())


SHAPES = [(640, 640), (640, 2048), (5120, 640), (640, 2560), (1280, 1280), (200, 136)]


def test_merge_fp16_matches_oracle_and_restores(cuda_device):
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    W, ad = _make(SHAPES, 64, torch.float16, 0)
    Wg = _cuda(W)
    m = LoraMerger(Wg, keep_pristine=True)
    m.merge(_cuda(ad), 1.0)
    ref = lora_oracle.merge_set(W, [ad], [1.0])
    for k in W:
        d = (Wg[k].cpu().float() - ref[k].float()).abs()
        # identical rounding sequence; fp32 accumulation order may move the product by one half-ulp before rounding
        assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()) and float((d > 0).float().mean()) < 0.02, k
        assert not torch.equal(Wg[k].cpu(), W[k])
    m.restore()
    for k in W:
        assert torch.equal(Wg[k].cpu(), W[k]), k      # bit-exact restore (copy semantics)


def test_merge_reference_scale_and_golden(cuda_device, golden_dir):
    """The reference's hard-coded scale fp16(20000/64) on the golden layer produced by torch's own fp16 path."""
    from katz_b200.lora import REFERENCE_UNET_SCALE, LoraMerger
    g = np.load(os.path.join(golden_dir, "lora_small.npz"))
    W = OrderedDict(w=torch.from_numpy(g["W16"]).cuda())
    ad = OrderedDict(w=(torch.from_numpy(g["up16"]).cuda(), torch.from_numpy(g["down16"]).cuda()))
    m = LoraMerger(W)
    m.merge(ad, REFERENCE_UNET_SCALE)
    ref = torch.from_numpy(g["W16_merged"])
    d = (W["w"].cpu().float() - ref.float()).abs()
    assert float(d.max()) <= 2 ** -9 * float(ref.float().abs().max())
    m.restore()
    assert torch.equal(W["w"].cpu(), torch.from_numpy(g["W16"]))


def test_merge_two_adapters_ranks_64_32(cuda_device):
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    W, ad1 = _make(SHAPES[:4], 64, torch.float16, 1)
    _, ad2 = _make(SHAPES[:4], 32, torch.float16, 2)
    Wg = _cuda(W)
    m = LoraMerger(Wg)
    m.merge([_cuda(ad1), _cuda(ad2)], [1.0, 1.0])
    ref = lora_oracle.merge_set(W, [ad1, ad2], [1.0, 1.0])
    for k in W:
        d = (Wg[k].cpu().float() - ref[k].float()).abs()
        assert float(d.max()) <= 2 ** -8 * float(ref[k].float().abs().max()), k
    m.restore()
    for k in W:
        assert torch.equal(Wg[k].cpu(), W[k])


def test_merge_fp32_matches_oracle(cuda_device):
    """Configuration 1 of the baseline: fp32 W, fp32 A/B, rank 64, alpha 64 (scale 1)."""
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    W, ad = _make(SHAPES, 64, torch.float32, 3)
    Wg = _cuda(W)
    m = LoraMerger(Wg)
    m.merge(_cuda(ad), 1.0)
    ref = lora_oracle.merge_set(W, [ad], [1.0])
    for k in W:
        delta = (ref[k] - W[k]).abs().max()
        err = (Wg[k].cpu() - ref[k]).abs().max()
        assert float(err) <= 1e-5 * float(delta) + 4e-9, (k, float(err), float(delta))   # 3xTF32 ~ fp32 accuracy
    m.restore()
    for k in W:
        assert torch.equal(Wg[k].cpu(), W[k])
    # subtractive in-place unmerge: close, but not promised bit-exact (report the mismatch count)
    m.merge_in_place(_cuda(ad), 1.0)
    m.unmerge_in_place(_cuda(ad), 1.0)
    for k in W:
        assert float((Wg[k].cpu() - W[k]).abs().max()) < 1e-7


def test_merge_rejects_bad_adapters(cuda_device):
    from katz_b200 import KatzError
    from katz_b200.lora import LoraMerger
    W, ad = _make([(128, 128)], 8, torch.float16, 4)
    Wg = _cuda(W)
    m = LoraMerger(Wg)
    bad = OrderedDict((k, (u.cuda()[:, :7].contiguous(), d.cuda()[:7].contiguous())) for k, (u, d) in ad.items())
    with pytest.raises(KatzError):
        m.merge(bad, 1.0)       # rank 7 is not a multiple of 8
    with pytest.raises(KatzError):
        m.merge(OrderedDict((k, (u.cuda().float(), d.cuda().float())) for k, (u, d) in ad.items()), 1.0)


@pytest.mark.parametrize("rank", [8, 24, 48])
def test_merge_fast_path_odd_ranks_and_layers_without_adapter(cuda_device, rank):
    """One adapter of rank <= 64 per layer takes the bulk-copy staged kernel: ranks that are not multiples of 16, ragged
    edge tiles, and layers the adapter does not touch (restored from the pristine copy)."""
    from katz_b200 import ops
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    shapes = [(320, 320), (640, 320), (200, 136), (1280, 2048), (384, 1280)]
    W, ad = _make(shapes, rank, torch.float16, 5 + rank)
    skipped = "layer3.weight"
    del ad[skipped]
    Wg = _cuda(W)
    m = LoraMerger(Wg, keep_pristine=True)
    m.merge(_cuda(ad), 2.0)
    ref = lora_oracle.merge_set(W, [ad], [2.0])
    for k in W:
        if k == skipped:
            assert torch.equal(Wg[k].cpu(), W[k])
            continue
        d = (Wg[k].cpu().float() - ref[k].float()).abs()
        assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()) and float((d > 0).float().mean()) < 0.02, k
    m.merge(_cuda(ad), 2.0)                      # a second merge starts from the pristine weights again
    for k in ad:
        d = (Wg[k].cpu().float() - ref[k].float()).abs()
        assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()), k
    m.restore()
    for k in W:
        assert torch.equal(Wg[k].cpu(), W[k]), k
    assert ops.tc05_status() == 0


def test_two_adapters_fast_path_ragged_shapes_missing_second_adapter_and_registered_handles(cuda_device):
    """Two adapters per layer (ranks 64 and 32, one scale) run on the warp-specialised kernel with both products in one
    accumulator: ragged edge tiles, a layer the second adapter does not touch, a layer neither touches, a second merge
    from the pristine weights, and the pre-validated handles a serving loop uses."""
    from katz_b200 import ops
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    shapes = [(320, 320), (640, 2048), (200, 136), (1280, 1280), (384, 1280), (5120, 640)]
    W, ad1 = _make(shapes, 64, torch.float16, 21)
    _, ad2 = _make(shapes, 32, torch.float16, 22)
    del ad2["layer1.weight"]
    del ad1["layer4.weight"], ad2["layer4.weight"]
    Wg = _cuda(W)
    m = LoraMerger(Wg)
    h1, h2 = m.register_adapter(_cuda(ad1)), m.register_adapter(_cuda(ad2))
    ref = lora_oracle.merge_set(W, [ad1, ad2], [0.5, 0.5])
    for rep in range(2):
        m.merge([h1, h2], [0.5, 0.5])
        assert m._flags & 4                       # the two-adapter fast path was taken
        for k in W:
            d = (Wg[k].cpu().float() - ref[k].float()).abs()
            assert float(d.max()) <= 2 ** -8 * float(ref[k].float().abs().max()), (rep, k)
        assert torch.equal(Wg["layer4.weight"].cpu(), W["layer4.weight"])
    m.merge([h2], [2.0])                          # back to one adapter: whatever was merged is replaced
    ref1 = lora_oracle.merge_set(W, [ad2], [2.0])
    for k in W:
        d = (Wg[k].cpu().float() - ref1[k].float()).abs()
        assert float(d.max()) <= 2 ** -9 * float(ref1[k].float().abs().max()), k
    m.merge([h1, h2], [1.0, 0.5])                 # different scales: the general kernel
    assert not (m._flags & 5)
    ref2 = lora_oracle.merge_set(W, [ad1, ad2], [1.0, 0.5])
    for k in W:
        d = (Wg[k].cpu().float() - ref2[k].float()).abs()
        assert float(d.max()) <= 2 ** -8 * float(ref2[k].float().abs().max()), k
    m.restore()
    for k in W:
        assert torch.equal(Wg[k].cpu(), W[k]), k
    assert ops.tc05_status() == 0


def test_adapter_file_staged_and_copied_asynchronously_then_merged(cuda_device, tmp_path):
    """File -> pinned staging -> asynchronous copy on a side stream -> merge, the overlap the reference gets from loader
    processes (pipeline_controlnet_sd_xl_katz.py:1522-1558): the merge waits for the copy's event, nothing else does."""
    from katz_b200.lora import LoraMerger, adapter_from_lora_state_dict, synthetic_key_map
    from katz_b200.lora_files import lora_state_dict, stage_pinned, to_device_async, write_safetensors
    from oracle import lora_oracle
    shapes = [(640, 640), (5120, 640), (1280, 2048)]
    W, ad = _make(shapes, 16, torch.float16, 41)
    km = synthetic_key_map(list(W.keys()))
    sd = OrderedDict()
    for k, (up, down) in ad.items():
        sd[km[k]["lora_up_key"]], sd[km[k]["lora_down_key"]] = up, down
    path = str(tmp_path / "adapter.safetensors")
    write_safetensors(path, sd)
    staged = stage_pinned(lora_state_dict(path)[0])
    assert all(t.is_pinned() for t in staged.values())
    dev_sd, ev = to_device_async(staged, cuda_device)
    Wg = _cuda(W)
    m = LoraMerger(Wg)
    torch.cuda.current_stream().wait_event(ev)
    m.merge(adapter_from_lora_state_dict(dev_sd, km, cuda_device, torch.float16), 1.0)
    ref = lora_oracle.merge_set(W, [ad], [1.0])
    for k in W:
        d = (Wg[k].cpu().float() - ref[k].float()).abs()
        assert float(d.max()) <= 2 ** -9 * float(ref[k].float().abs().max()), k
