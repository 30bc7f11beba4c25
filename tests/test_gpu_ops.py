"""GPU parity of each kernel against the CPU oracle (torch fp32 / numpy half arithmetic), through the C ABI.
Tolerances: byte/layout ops bit-exact; fp16 GEMM-like ops 2e-3 relative to the output scale (fp32 accumulation, one
rounding); normalisations 2e-3 absolute on unit-scale outputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(256, 320, 640), (154, 640, 2048), (2, 1280, 320), (2048, 1280, 1280), (300, 72, 40)])
def test_linear_mma(cuda_device, M, N, K, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "mma")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    b = torch.randn(N, generator=g).half()
    r = torch.randn(M, N, generator=g).half()
    ref = F.linear(x.float(), w.float(), b.float()) + r.float()
    out = ops.linear(x.cuda(), w.cuda(), b.cuda(), residual=r.cuda())
    assert _rel(out, ref) < 2e-3
    ref2 = F.silu(F.linear(x.float(), w.float(), b.float())) * 0.5
    out2 = ops.linear(x.cuda(), w.cuda(), b.cuda(), act=ops.ACT_SILU, out_scale=0.5)
    assert _rel(out2, ref2) < 2e-3


def test_linear_rowvec_and_strided(cuda_device, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "mma")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(1)
    B, S, K, N = 2, 96, 64, 128
    x = torch.randn(B * S, 3 * K, generator=g).half().cuda()
    w = (torch.randn(N, K, generator=g) / 8).half().cuda()
    rv = torch.randn(B, 4 * N, generator=g).half().cuda()
    out = ops.linear(x[:, K:2 * K], w, rowvec=rv[:, N:2 * N], rows_per_batch=S)
    ref = F.linear(x[:, K:2 * K].float(), w.float()).view(B, S, N) + rv[:, N:2 * N].float()[:, None, :]
    assert _rel(out.view(B, S, N), ref) < 2e-3


@pytest.mark.parametrize("B,H,W,C1,C2,Cout,ks,stride,up", [
    (2, 16, 16, 64, 0, 128, 3, 1, False),
    (2, 16, 16, 64, 0, 64, 3, 2, False),
    (1, 8, 8, 128, 0, 128, 3, 1, True),
    (2, 12, 20, 64, 32, 96, 3, 1, False),
    (2, 32, 32, 8, 0, 64, 3, 1, False),
    (2, 16, 16, 320, 0, 4, 3, 1, False),
    (1, 16, 16, 64, 0, 64, 1, 1, False),
])
def test_conv2d_mma(cuda_device, B, H, W, C1, C2, Cout, ks, stride, up, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "mma")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(2)
    x = torch.randn(B, C1 + C2, H, W, generator=g).half()
    w = (torch.randn(Cout, C1 + C2, ks, ks, generator=g) / (ks * ks * (C1 + C2)) ** 0.5).half()
    bias = torch.randn(Cout, generator=g).half()
    xin = F.interpolate(x.float(), scale_factor=2.0, mode="nearest") if up else x.float()
    ref = F.conv2d(xin, w.float(), bias.float(), stride=stride, padding=ks // 2)
    temb = torch.randn(B, Cout, generator=g).half()
    res = torch.randn_like(ref).half()
    ref = ref + temb.float()[:, :, None, None] + res.float()
    xn = x.permute(0, 2, 3, 1).contiguous().cuda()
    x1 = xn[..., :C1].contiguous()
    x2 = xn[..., C1:].contiguous() if C2 else None
    wn = w.permute(0, 2, 3, 1).contiguous().cuda()
    out = ops.conv2d(x1, wn, bias.cuda(), ksize=ks, stride=stride, pad=ks // 2, upsample=up, x2=x2, rowvec=temb.cuda(),
                     residual=res.permute(0, 2, 3, 1).contiguous().cuda())
    assert _rel(out.permute(0, 3, 1, 2), ref) < 2e-3


@pytest.mark.parametrize("B,H,Sq,Sk", [(2, 2, 256, 256), (2, 5, 1024, 77), (1, 3, 200, 130), (2, 10, 4096, 4096)])
def test_attention_mma(cuda_device, B, H, Sq, Sk):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(3)
    C = H * 64
    qkv = torch.randn(B, Sq, 3 * C, generator=g).half()
    kv = torch.randn(B, Sk, 2 * C, generator=g).half()
    q = qkv[:, :, :C]
    k, v = (kv[:, :, :C], kv[:, :, C:]) if Sk != Sq else (qkv[:, :, C:2 * C], qkv[:, :, 2 * C:])

    def heads(t):
        return t.float().reshape(B, -1, H, 64).transpose(1, 2)
    dev = "cuda" if Sq * Sk > 1 << 22 else "cpu"   # the largest case takes the fp32 reference on the GPU
    ref = F.scaled_dot_product_attention(heads(q).to(dev), heads(k).to(dev), heads(v).to(dev)).transpose(1, 2).reshape(B, Sq, C)
    qg, kvg = qkv.cuda(), kv.cuda()
    if Sk != Sq:
        out = ops.attention(qg[:, :, :C], kvg[:, :, :C], kvg[:, :, C:], H)
    else:
        out = ops.attention(qg[:, :, :C], qg[:, :, C:2 * C], qg[:, :, 2 * C:], H)
    assert float((out.float().cpu() - ref.cpu()).abs().max()) < 4e-3


@pytest.mark.parametrize("B,HW,C,act,shift", [(2, 256, 64, 1, 0.0), (2, 4096, 320, 1, 3.0), (2, 1024, 1920, 0, 0.0), (1, 100, 2560, 1, -2.0)])
def test_group_norm_nhwc(cuda_device, B, HW, C, act, shift):
    from katz_b200 import ops
    from oracle import kernels_oracle
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(B, HW, C, generator=g) + shift).half()
    gamma = (1 + 0.1 * torch.randn(C, generator=g)).half()
    beta = (0.1 * torch.randn(C, generator=g)).half()
    ref = kernels_oracle.group_norm(x.permute(0, 2, 1).reshape(B, C, HW, 1), 32, gamma, beta, 1e-5, act == 1)
    out = ops.group_norm_nhwc(x.cuda(), gamma.cuda(), beta.cuda(), 32, 1e-5, act)
    assert float((out.cpu().float() - ref.reshape(B, C, HW).permute(0, 2, 1).float()).abs().max()) < 4e-3


def test_group_norm_fast_kernel_op(cuda_device):
    """The drop-in op with the reference's schema and calling convention (normalization.py:90-91)."""
    import fast_kernel  # noqa: F401
    from oracle import kernels_oracle
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 320, 32, 32, generator=g).half()
    w, b = torch.randn(320, generator=g).half(), torch.randn(320, generator=g).half()
    xc = x.cuda().contiguous(memory_format=torch.channels_last)
    y = torch.empty_like(xc)
    torch.ops.fast_kernel.group_norm_fp16(xc, y, 1e-5, 32, "silu", w.cuda(), b.cuda(), True, False)
    ref = kernels_oracle.group_norm(x, 32, w, b, 1e-5, True)
    assert float((y.cpu().float() - ref.float()).abs().max()) < 8e-3
    # channels-first branch
    y2 = torch.empty_like(x.cuda())
    torch.ops.fast_kernel.group_norm_fp16(x.cuda(), y2, 1e-5, 32, "none", w.cuda(), b.cuda(), True, True)
    ref2 = kernels_oracle.group_norm(x, 32, w, b, 1e-5, False)
    assert float((y2.cpu().float() - ref2.float()).abs().max()) < 8e-3
    # error behaviour: shape mismatch raises RuntimeError like TORCH_CHECK
    with pytest.raises(RuntimeError):
        torch.ops.fast_kernel.fast_gelu_mul_fp16(x.cuda(), x.cuda()[:1])


def test_fast_gelu_mul(cuda_device):
    import fast_kernel  # noqa: F401
    from oracle import kernels_oracle
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(2, 1024, 2560, generator=g) * 2).half()
    m = torch.randn(2, 1024, 2560, generator=g).half()
    out = torch.ops.fast_kernel.fast_gelu_mul_fp16(x.cuda(), m.cuda()).cpu()
    ref = torch.from_numpy(kernels_oracle.fast_gelu_mul(x.numpy(), m.numpy()))
    diff = (out.float() - ref.float()).abs()
    # same rounding sequence; the only freedom is tanh's last bit
    assert float(diff.max()) <= 4e-3 and float((diff > 0).float().mean()) < 0.02
    # 16-byte packs, the ragged tail after them and a start that is only 4-byte aligned give the same bits
    from katz_b200 import ops
    xs, ms = x.cuda().reshape(-1)[:4102], m.cuda().reshape(-1)[:4102]
    whole = out.cuda().reshape(-1)
    assert torch.equal(ops.fast_gelu_mul(xs.clone(), ms.clone()), whole[:4102])
    xo, mo = x.cuda().reshape(-1)[2:4100], m.cuda().reshape(-1)[2:4100]        # views: 4 bytes past a 16-byte boundary
    assert torch.equal(ops.fast_gelu_mul(xo, mo), whole[2:4100])


def test_layer_norm_and_geglu(cuda_device):
    from katz_b200 import ops
    from oracle import kernels_oracle
    g = torch.Generator().manual_seed(7)
    for C in (640, 1280, 64):
        x = (torch.randn(513, C, generator=g) * 2 + 0.5).half()
        w, b = torch.randn(C, generator=g).half(), torch.randn(C, generator=g).half()
        ref = F.layer_norm(x.float(), (C,), w.float(), b.float(), 1e-5)
        out = ops.layer_norm(x.cuda(), w.cuda(), b.cuda())
        assert float((out.cpu().float() - ref).abs().max()) < 8e-3
    hg = torch.randn(300, 2 * 2560, generator=g).half()
    out = ops.geglu_erf(hg.cuda()).cpu()
    ref = kernels_oracle.geglu_erf(hg)
    assert float((out.float() - ref.float()).abs().max()) <= 2e-3


def test_small_kernels(cuda_device, golden_dir):
    import os
    from katz_b200 import ops
    from oracle import unet_oracle
    g = torch.Generator().manual_seed(8)
    # layout moves are bit-exact
    x = torch.randn(2, 4, 16, 16, generator=g).half()
    n = ops.nchw_to_nhwc(x.cuda(), cpad=8)
    assert torch.equal(n[..., :4].cpu(), x.permute(0, 2, 3, 1)) and float(n[..., 4:].abs().max()) == 0
    assert torch.equal(ops.nhwc_to_nchw(n, c=4).cpu(), x)
    a, b = torch.randn(2, 8, 8, 64, generator=g).half(), torch.randn(2, 8, 8, 32, generator=g).half()
    assert torch.equal(ops.concat_channels(a.cuda(), b.cuda()).cpu(), torch.cat([a, b], dim=-1))
    # timestep embedding
    t = torch.tensor([500.0, 981.0, 1.0])
    ref = unet_oracle.timestep_embedding(t, 320)
    out = ops.timestep_embedding(t.cuda(), 320)
    assert float((out.cpu().float() - ref).abs().max()) < 2e-3
    # residual intake: sum and mean
    src = torch.randn(2, 8, 8, 64, generator=g).half()
    r1, r2 = torch.randn_like(src), torch.randn_like(src)
    out = ops.residual_intake(src.cuda(), [r1.cuda(), r2.cuda()], [0.5, 0.5]).cpu()
    ref = (src.float() + ((r1.float() + r2.float()) * 0.5).half().float()).half()
    assert float((out.float() - ref.float()).abs().max()) <= 2e-3
    # Euler / CFG arithmetic: bit-exact against what the reference scheduler produced
    gz = np.load(os.path.join(golden_dir, "euler_sdxl.npz"))
    sig = gz["sigmas"]
    lat = torch.from_numpy(gz["latent0"]).cuda()
    for i in range(4):
        inp = ops.euler_scale_input(lat, sig[i], copies=2, cpu_torch_rounding=True)
        assert torch.equal(inp[0].cpu(), torch.from_numpy(gz["scaled_%d" % i])[0])
        assert torch.equal(inp[1].cpu(), torch.from_numpy(gz["scaled_%d" % i])[0])
        ops.euler_cfg_step(lat, torch.from_numpy(gz["eps_u_%d" % i]).cuda(), torch.from_numpy(gz["eps_c_%d" % i]).cuda(),
                           5.0, sig[i], sig[i + 1], cpu_torch_rounding=True)
        assert torch.equal(lat.cpu(), torch.from_numpy(gz["latent_%d" % (i + 1)]))
    # default rounding = torch's CUDA kernels: the oracle's torch ops run on the device are the reference here
    lat = torch.from_numpy(gz["latent0"]).cuda()
    ref = lat.clone()
    for i in range(4):
        u, c = torch.from_numpy(gz["eps_u_%d" % i]).cuda(), torch.from_numpy(gz["eps_c_%d" % i]).cuda()
        assert torch.equal(ops.euler_scale_input(lat, sig[i]), unet_oracle.euler_scale_model_input(ref, float(sig[i])))
        ops.euler_cfg_step(lat, u, c, 5.0, sig[i], sig[i + 1])
        ref = unet_oracle.euler_step(ref, unet_oracle.cfg_combine(u, c, 5.0), float(sig[i]), float(sig[i + 1]))
        assert torch.equal(lat, ref)


@pytest.mark.parametrize("M,N,K", [(256, 320, 640), (154, 640, 2048), (2, 1280, 320), (2048, 1280, 1280),
                                   (8192, 5120, 640), (300, 72, 64), (4096, 640, 2560), (1024, 1280, 1280), (512, 640, 640)])
def test_linear_tcgen05(cuda_device, M, N, K, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "tc05")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(10)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    b = torch.randn(N, generator=g).half()
    r = torch.randn(M, N, generator=g).half()
    assert ops._tc05_linear_ok(x.cuda(), w.cuda(), b.cuda(), r.cuda(), None, torch.empty(M, N, dtype=torch.float16, device="cuda"))
    xg, wg, bg, rg = x.cuda(), w.cuda(), b.cuda(), r.cuda()
    ref = (xg.float() @ wg.float().t() + bg.float() + rg.float()).cpu()
    out = ops.linear(xg, wg, bg, residual=rg)
    assert ops.tc05_status() == 0
    assert _rel(out, ref) < 2e-3
    ref2 = (F.silu(xg.float() @ wg.float().t() + bg.float()) * 0.5).cpu()
    out2 = ops.linear(xg, wg, bg, act=ops.ACT_SILU, out_scale=0.5)
    assert _rel(out2, ref2) < 2e-3
    # same answer as the mma.sync kernel up to accumulation order
    monkeypatch.setenv("KATZ_GEMM", "mma")
    out3 = ops.linear(xg, wg, bg, residual=rg)
    assert _rel(out, out3.cpu()) < 1e-3


def test_linear_tcgen05_strided_views(cuda_device, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "tc05")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(11)
    B, S, K, N = 2, 160, 128, 256
    x = torch.randn(B * S, 3 * K, generator=g).half().cuda()
    w = (torch.randn(N, K, generator=g) / 11).half().cuda()
    rv = torch.randn(B, 4 * N, generator=g).half().cuda()
    big = torch.zeros(B * S, 2 * N, dtype=torch.float16, device="cuda")
    out = ops.linear(x[:, K:2 * K], w, rowvec=rv[:, N:2 * N], rows_per_batch=S, out=big[:, N:])
    ref = (x[:, K:2 * K].float() @ w.float().t()).view(B, S, N) + rv[:, N:2 * N].float()[:, None, :]
    assert ops.tc05_status() == 0
    assert _rel(out.reshape(B, S, N), ref) < 2e-3
    assert float(big[:, :N].abs().max()) == 0


@pytest.mark.parametrize("B,H,W,Cin,Cout,up,stride", [(2, 16, 16, 64, 128, False, 1), (2, 32, 32, 128, 320, False, 1),
                                                      (1, 128, 128, 64, 64, False, 1), (2, 64, 64, 320, 640, False, 1),
                                                      (1, 6, 16, 64, 64, False, 1), (1, 16, 16, 128, 128, True, 1),
                                                      (1, 8, 256, 64, 64, False, 1), (2, 32, 32, 64, 128, False, 2),
                                                      (2, 128, 128, 320, 320, False, 2), (1, 64, 64, 640, 640, False, 2),
                                                      (1, 10, 16, 64, 64, False, 2), (3, 16, 8, 64, 128, False, 1),
                                                      (3, 16, 16, 128, 320, False, 2)])
def test_conv3x3_tcgen05(cuda_device, B, H, W, Cin, Cout, up, stride, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "tc05")
    from katz_b200 import ops
    g = torch.Generator().manual_seed(12)
    x = torch.randn(B, Cin, H, W, generator=g).half().cuda()
    w = (torch.randn(Cout, Cin, 3, 3, generator=g) / (9 * Cin) ** 0.5).half().cuda()
    bias = torch.randn(Cout, generator=g).half().cuda()
    xin = F.interpolate(x.float(), scale_factor=2.0, mode="nearest") if up else x.float()
    ref = F.conv2d(xin, w.float(), bias.float(), padding=1, stride=stride)
    temb = torch.randn(B, Cout, generator=g).half().cuda()
    res = torch.randn(ref.shape, generator=g).half().cuda()
    ref = ref + temb.float()[:, :, None, None] + res.float()
    out = ops.conv2d(x.permute(0, 2, 3, 1).contiguous(), w.permute(0, 2, 3, 1).contiguous(), bias, upsample=up, stride=stride,
                     rowvec=temb, residual=res.permute(0, 2, 3, 1).contiguous())
    assert ops.tc05_status() == 0
    assert _rel(out.permute(0, 3, 1, 2), ref) < 2e-3


@pytest.mark.parametrize("B,H,W,Cin,Cout,stride,act", [(2, 64, 64, 8, 16, 1, 1), (1, 128, 96, 16, 16, 1, 1), (2, 64, 64, 16, 32, 2, 1),
                                                        (1, 70, 50, 32, 32, 1, 1), (2, 64, 64, 32, 96, 2, 1), (1, 40, 72, 32, 96, 1, 1),
                                                        (2, 64, 64, 16, 256, 2, 1), (1, 9, 33, 32, 72, 1, 0), (1, 11, 35, 16, 8, 2, 0),
                                                        (1, 1024, 1024, 8, 16, 1, 1)])      # the last: the embedding's first layer at size
def test_conv3x3_few_channels(cuda_device, B, H, W, Cin, Cout, stride, act, monkeypatch):
    """The direct convolution of the ControlNet conditioning embedding's layers (few channels, large images) against fp32
    F.conv2d (+ SiLU) and against the implicit-GEMM kernel it replaces for these shapes; ragged tile edges included."""
    from katz_b200 import ops
    g = torch.Generator().manual_seed(31)
    x = torch.randn(B, Cin, H, W, generator=g).half().cuda()
    w = (torch.randn(Cout, Cin, 3, 3, generator=g) / (9 * Cin) ** 0.5).half().cuda()
    bias = torch.randn(Cout, generator=g).half().cuda()
    ref = F.conv2d(x.float(), w.float(), bias.float(), padding=1, stride=stride)
    if act:
        ref = F.silu(ref)
    xn, wn = x.permute(0, 2, 3, 1).contiguous(), w.permute(0, 2, 3, 1).contiguous()
    n0 = ops._lib.launch_count()
    out = ops.conv2d(xn, wn, bias, stride=stride, act=ops.ACT_SILU if act else ops.ACT_NONE)
    assert ops._lib.launch_count() == n0 + 1
    assert _rel(out.permute(0, 3, 1, 2), ref) < 2e-3
    assert float((out.permute(0, 3, 1, 2).float() - ref).abs().max()) < 2e-2
    monkeypatch.setenv("KATZ_CONV_SMALL", "0")
    old = ops.conv2d(xn, wn, bias, stride=stride, act=ops.ACT_SILU if act else ops.ACT_NONE)
    assert _rel(out, old) < 1e-3
    # a row shard that carries its halo rows: no vertical padding
    monkeypatch.setenv("KATZ_CONV_SMALL", "1")
    if stride == 1 and H <= 128:
        xp = F.pad(xn, (0, 0, 0, 0, 1, 1))
        out2 = ops.conv2d(xp, wn, bias, stride=1, act=ops.ACT_SILU if act else ops.ACT_NONE, pad_h=0)
        assert torch.equal(out2, out)


@pytest.mark.parametrize("M,F,K", [(2048, 5120, 1280), (8192, 2560, 640), (300, 64, 64), (256, 80, 128)])
def test_feed_forward_geglu_fused(cuda_device, M, F, K, monkeypatch):
    monkeypatch.setenv("KATZ_GEMM", "tc05")
    from katz_b200 import ops
    from oracle import kernels_oracle
    g = torch.Generator().manual_seed(13)
    x = torch.randn(M, K, generator=g).half().cuda()
    w = (torch.randn(2 * F, K, generator=g) / K ** 0.5).half().cuda()
    b = torch.randn(2 * F, generator=g).half().cuda()
    hg = (x.float() @ w.float().t() + b.float()).half()
    ref = kernels_oracle.geglu_erf(hg.cpu())
    out = ops.feed_forward_geglu(x, w, b)
    assert ops.tc05_status() == 0
    d = (out.cpu().float() - ref.float()).abs()
    assert float(d.max()) <= 2e-2 and _rel(out, ref) < 4e-3
    monkeypatch.setenv("KATZ_FUSED_GEGLU", "0")
    out2 = ops.feed_forward_geglu(x, w, b)
    assert _rel(out, out2.cpu()) < 4e-3


@pytest.mark.parametrize("B,H,Sq,Sk", [(2, 2, 256, 256), (2, 5, 1024, 77), (1, 3, 200, 130), (2, 10, 4096, 4096),
                                       (2, 20, 1024, 1024), (1, 1, 128, 128),
                                       (1, 10, 16384, 16384)])      # the last: one image of the 2048x2048-pixel step
def test_attention_tcgen05(cuda_device, B, H, Sq, Sk, monkeypatch):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(14)
    C = H * 64
    qkv = (torch.randn(B, Sq, 3 * C, generator=g) * 1.5).half().cuda()
    kv = torch.randn(B, Sk, 2 * C, generator=g).half().cuda()
    q = qkv[:, :, :C]
    k, v = (kv[:, :, :C], kv[:, :, C:]) if Sk != Sq else (qkv[:, :, C:2 * C], qkv[:, :, 2 * C:])

    def heads(t):
        return t.float().reshape(B, -1, H, 64).transpose(1, 2)
    ref = F.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape(B, Sq, C)
    monkeypatch.setenv("KATZ_ATTN", "tc05")
    out = ops.attention(q, k, v, H)
    assert ops.tc05_status() == 0
    assert float((out.float() - ref).abs().max()) < 4e-3
    monkeypatch.setenv("KATZ_ATTN", "mma")
    out2 = ops.attention(q, k, v, H)
    assert float((out.float() - out2.float()).abs().max()) < 4e-3


@pytest.mark.parametrize("B,H,Sq,Sk", [(2, 20, 1024, 1024),      # 8 key tiles per query tile: too short to cut (same launch)
                                       (1, 2, 1024, 2048),       # 16 query tiles, less than one round: every tile cut into 4
                                       (1, 5, 1000, 2500),       # ragged query and key counts, every tile cut into 5
                                       (1, 37, 1024, 2048),      # exactly one round of 296 tiles: nothing is cut
                                       (2, 10, 4096, 4096),      # 640 tiles: 48 cut into 6 parts of 5 or 6 key tiles
                                       (1, 10, 4096, 4096)])     # 320 tiles: 24 cut into 8 parts of 4 key tiles
def test_attention_tcgen05_cut_wave_tail(cuda_device, B, H, Sq, Sk, monkeypatch):
    """The launch that cuts the query tiles of the last, partly filled dispatch round along the key axis against the launch
    that does not, and against fp32 SDPA; twice in a row, since the tickets in the scratch buffer must return to zero."""
    from katz_b200 import ops
    g = torch.Generator().manual_seed(21)
    C = H * 64
    q = (torch.randn(B, Sq, C, generator=g) * 1.5).half().cuda()
    kv = torch.randn(B, Sk, 2 * C, generator=g).half().cuda()
    k, v = kv[:, :, :C], kv[:, :, C:]

    def heads(t):
        return t.float().reshape(B, -1, H, 64).transpose(1, 2)
    ref = F.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape(B, Sq, C)
    monkeypatch.setenv("KATZ_ATTN", "tc05")
    monkeypatch.setenv("KATZ_ATTN_SPLIT", "0")
    whole = ops.attention(q, k, v, H)
    monkeypatch.setenv("KATZ_ATTN_SPLIT", "1")
    cut1 = ops.attention(q, k, v, H)
    cut2 = ops.attention(q, k, v, H)
    assert ops.tc05_status() == 0
    assert torch.equal(cut1, cut2)                       # parts are added in index order whichever arrives last
    assert float((cut1.float() - ref).abs().max()) < 4e-3
    assert float((cut1.float() - whole.float()).abs().max()) < 2e-3
    assert int(ops._attention_scratch(q.device)[:4096].view(torch.int32).abs().sum()) == 0


def test_attention_tcgen05_large_logits_rescale(cuda_device, monkeypatch):
    """Logits that grow along the key axis force the reference maximum (and the O accumulator) to be raised often."""
    from katz_b200 import ops
    monkeypatch.setenv("KATZ_ATTN", "tc05")
    g = torch.Generator().manual_seed(15)
    B, H, S = 1, 2, 1024
    q = (torch.randn(B, S, H * 64, generator=g) * 3).half().cuda()
    ramp = torch.linspace(0.2, 4.0, S)[None, :, None]
    k = (torch.randn(B, S, H * 64, generator=g) * ramp).half().cuda()
    v = torch.randn(B, S, H * 64, generator=g).half().cuda()

    def heads(t):
        return t.float().reshape(B, -1, H, 64).transpose(1, 2)
    ref = F.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape(B, S, H * 64)
    out = ops.attention(q, k, v, H)
    assert ops.tc05_status() == 0
    assert float((out.float() - ref).abs().max()) < 8e-3


@pytest.mark.parametrize("M,C,N,row_shift", [(2048, 1280, 3840, 0.0), (8192, 640, 1920, 3.0), (2048, 1280, 1280, -1.5), (300, 64, 192, 0.5)])
def test_layer_norm_folded_into_linear(cuda_device, M, C, N, row_shift):
    """nn.LayerNorm followed by nn.Linear as ONE GEMM on the raw rows (LN(x) W^T = rstd (x W'^T) - rstd mean c1 + c2): the
    producer GEMM leaves the rows' (sum, sum of squares) per 32-column chunk, the consumer applies them. Against fp32 torch
    on the same fp16 inputs, and against the unfused pair of kernels (whose extra fp16 rounding of the normalised rows the
    folded form does not have)."""
    from katz_b200 import ops
    g = torch.Generator().manual_seed(31)
    a = torch.randn(M, C, generator=g).half().cuda()
    wp = (torch.randn(C, C, generator=g) / C ** 0.5).half().cuda()
    bp = torch.randn(C, generator=g).half().cuda()
    res = (torch.randn(M, C, generator=g) * 2 + row_shift).half().cuda()      # rows with a mean that is not small
    gamma = (1 + 0.2 * torch.randn(C, generator=g)).half().cuda()
    beta = (0.2 * torch.randn(C, generator=g)).half().cuda()
    w = (torch.randn(N, C, generator=g) / C ** 0.5).half().cuda()
    bias = torch.randn(N, generator=g).half().cuda()
    # producer: x = a wp^T + bp + res, with the statistics of the fp16 x it stored
    x, st = ops.linear(a, wp, bp, residual=res, stats_out=True)
    assert torch.equal(x, ops.linear(a, wp, bp, residual=res))                # emitting statistics changes nothing else
    xf = x.float()
    s1 = st[:, :, 0].sum(0)
    s2 = st[:, :, 1].sum(0)
    # the statistics are taken from the fp32 values before their fp16 rounding: the sums agree with those of the stored rows up
    # to that rounding (2^-11 relative per element, random sign)
    assert torch.allclose(s1, xf.sum(1), rtol=1e-3, atol=0.25) and torch.allclose(s2, (xf * xf).sum(1), rtol=2e-3, atol=0.5)
    fold = ops.ln_fold(w, gamma, beta, bias)
    out = ops.linear(x, fold.wf, ln=fold, ln_stats=st)
    ref = F.linear(F.layer_norm(xf, (C,), gamma.float(), beta.float(), 1e-5), w.float(), bias.float())
    unfused = ops.linear(ops.layer_norm(x, gamma, beta), w, bias)
    e_fold = float((out.float() - ref).norm() / ref.norm())
    e_unf = float((unfused.float() - ref).norm() / ref.norm())
    assert e_fold <= 1e-3 and e_fold <= 2.0 * e_unf + 1e-4, (e_fold, e_unf)
    assert float((out.float() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert ops.tc05_status() == 0


@pytest.mark.parametrize("M,C,Fw", [(2048, 1280, 5120), (8192, 640, 2560), (256, 128, 512)])
def test_layer_norm_folded_into_geglu(cuda_device, M, C, Fw):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(32)
    a = torch.randn(M, C, generator=g).half().cuda()
    wp = (torch.randn(C, C, generator=g) / C ** 0.5).half().cuda()
    res = (torch.randn(M, C, generator=g) + 1.0).half().cuda()
    gamma = (1 + 0.2 * torch.randn(C, generator=g)).half().cuda()
    beta = (0.2 * torch.randn(C, generator=g)).half().cuda()
    w = (torch.randn(2 * Fw, C, generator=g) / C ** 0.5).half().cuda()
    bias = torch.randn(2 * Fw, generator=g).half().cuda()
    x, st = ops.linear(a, wp, None, residual=res, stats_out=True)
    fold = ops.ln_fold(w, gamma, beta, bias)
    out = ops.feed_forward_geglu(x, fold.wf, None, ln=fold, ln_stats=st)
    hg = F.linear(F.layer_norm(x.float(), (C,), gamma.float(), beta.float(), 1e-5), w.float(), bias.float())
    ref = hg[:, :Fw] * F.gelu(hg[:, Fw:])
    unfused = ops.feed_forward_geglu(ops.layer_norm(x, gamma, beta), w, bias)
    e_fold = float((out.float() - ref).norm() / ref.norm())
    e_unf = float((unfused.float() - ref).norm() / ref.norm())
    assert e_fold <= 1.5e-3 and e_fold <= 2.0 * e_unf + 1e-4, (e_fold, e_unf)
    assert ops.tc05_status() == 0
