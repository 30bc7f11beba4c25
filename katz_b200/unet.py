"""Host-side mirror of the reference's SDXL UNet / ControlNet step over the katz_b200 kernels.

Keeps the reference's call surface for this path — `unet(sample, timestep, encoder_hidden_states=...,
added_cond_kwargs={"text_embeds","time_ids"}, down_block_additional_residuals=..., mid_block_additional_residual=...,
return_dict=False)` as used by sdxl_unet_server.py:199-213, and `controlnet(sample, t, encoder_hidden_states=...,
controlnet_cond=..., added_cond_kwargs=..., conditioning_scale=0.5)` as used by sdxl_controlnet_server.py:94-100 — and
the state-dict key names of the reference fork, so weights, LoRA key maps and the pristine-state restore carry over.

The computation follows `_down_forward` -> ControlNet residual add -> `_up_forward`
(diffusers/models/unets/unet_2d_condition.py:1127-1341), i.e. the reference's CUDA-graph path that adds all nine down
residuals and the mid residual. Activations are NHWC fp16 end to end ([B, H, W, C] is also the [B, H*W, C] token
layout, so Transformer2DModel's permutes disappear); NCHW appears only at the model boundary.
"""
import os
from collections import OrderedDict

import torch

from . import ops
from .ops import ACT_NONE, ACT_SILU, KatzError
from .params import CONTROLNET_COND_CHANNELS, controlnet_param_shapes, unet_param_shapes

_ALT_NAMES = (
    (".norm1.", ".norm_silu1.0."),
    (".norm2.", ".norm_silu2.0."),
)


def _canonical_key(k):
    """Map upstream-diffusers key spellings onto the fork's (resnet.py:336-350, unet_2d_condition.py:521-529)."""
    if ".resnets." in k:
        for a, b in _ALT_NAMES:
            if a in k and ".transformer_blocks." not in k:
                k = k.replace(a, b)
    if k.startswith("conv_norm_out."):
        k = "conv_norm_silu.0." + k[len("conv_norm_out."):]
    return k


class _Weights:
    """Device-resident fp16 parameters in the layouts the kernels read, addressable by reference key.

    Linear weights are stored as-is ([N, K]); the three self-attention projections of a block live in one [3C, C]
    buffer, every block's cross-attention to_k/to_v in one [sum 2C, cross_dim] buffer, and every resnet's
    time_emb_proj in one [sum Cout, temb] buffer — each reference key is a row-range VIEW of those buffers, so a LoRA
    merge through the key writes the storage the fused GEMMs read. Convolution weights are stored [Cout, ky, kx, Cin].
    """

    def __init__(self, shapes, device):
        self.shapes = shapes
        self.device = device
        self.t = {}          # key -> tensor in kernel layout (views for fused groups)
        self.fused = {}      # name -> fused buffer
        self.conv_cin_pad = {}

    def alloc(self):
        dev = self.device
        shapes = self.shapes
        # --- fused groups
        qkv_blocks = sorted({k[: -len(".attn1.to_q.weight")] for k in shapes if k.endswith(".attn1.to_q.weight")})
        for b in qkv_blocks:
            c = shapes[b + ".attn1.to_q.weight"][0]
            buf = torch.zeros((3 * c, c), dtype=torch.float16, device=dev)
            self.fused[b + ".attn1.qkv"] = buf
            for i, n in enumerate(("to_q", "to_k", "to_v")):
                self.t["%s.attn1.%s.weight" % (b, n)] = buf[i * c:(i + 1) * c]
        kv_keys = [k for k in shapes if k.endswith(".attn2.to_k.weight")]
        if kv_keys:
            cross = shapes[kv_keys[0]][1]
            total = sum(2 * shapes[k][0] for k in kv_keys)
            buf = torch.zeros((total, cross), dtype=torch.float16, device=dev)
            self.fused["cross_kv"] = buf
            self.cross_kv_offset = {}
            off = 0
            for k in kv_keys:
                c = shapes[k][0]
                b = k[: -len(".attn2.to_k.weight")]
                self.t[b + ".attn2.to_k.weight"] = buf[off:off + c]
                self.t[b + ".attn2.to_v.weight"] = buf[off + c:off + 2 * c]
                self.cross_kv_offset[b] = off
                off += 2 * c
        te_keys = [k for k in shapes if k.endswith(".time_emb_proj.weight")]
        temb = shapes[te_keys[0]][1]
        total = sum(shapes[k][0] for k in te_keys)
        wbuf = torch.zeros((total, temb), dtype=torch.float16, device=dev)
        bbuf = torch.zeros((total,), dtype=torch.float16, device=dev)
        self.fused["temb_w"], self.fused["temb_b"] = wbuf, bbuf
        self.temb_offset = {}
        off = 0
        for k in te_keys:
            c = shapes[k][0]
            b = k[: -len(".time_emb_proj.weight")]
            self.t[k] = wbuf[off:off + c]
            self.t[b + ".time_emb_proj.bias"] = bbuf[off:off + c]
            self.temb_offset[b] = (off, c)
            off += c
        # --- everything else
        # The ControlNet conditioning embedding's 96-channel layers are stored with 128 channels (zero weights, zero bias:
        # the extra channels stay zero through SiLU), so that the convolutions that read them have a channel count the
        # tcgen05 implicit GEMM takes (a multiple of 64) instead of falling to the mma.sync kernel.
        # Likewise the UNet's last convolution (320 -> 4 channels) is stored with 8 output channels: the tcgen05 convolution
        # wants a multiple of 8, and the layout kernel that follows keeps the first 4.
        def widen(k, c):
            if c == 96 and k.startswith("controlnet_cond_embedding.blocks."):
                return 128
            if c == 4 and k in ("conv_out.weight", "conv_out.bias"):
                return 8
            return c
        for k, shp in shapes.items():
            if k in self.t:
                continue
            if len(shp) == 4:
                cout, cin, kh, kw = shp
                cin_pad = widen(k, (cin + 7) // 8 * 8)
                self.conv_cin_pad[k] = cin_pad
                self.t[k] = torch.zeros((widen(k, cout), kh, kw, cin_pad), dtype=torch.float16, device=dev)
            elif len(shp) == 1:
                self.t[k] = torch.zeros((widen(k, shp[0]),), dtype=torch.float16, device=dev)
            else:
                self.t[k] = torch.zeros(shp, dtype=torch.float16, device=dev)

    def load(self, sd, strict=True):
        missing = []
        seen = set()
        for k, v in sd.items():
            ck = _canonical_key(k)
            if ck.endswith(".proj_1.weight") or ck.endswith(".proj_2.weight") or ck.endswith(".proj_1.bias") or ck.endswith(".proj_2.bias"):
                # the fork's split GEGLU (activations.py:151-170): proj_1 = first half, proj_2 = second half
                base, which, kind = ck.rsplit(".", 2)[0], ck.rsplit(".", 2)[1], ck.rsplit(".", 2)[2]
                dst = self.t[base + ".proj." + kind]
                half = dst.shape[0] // 2
                sl = slice(0, half) if which == "proj_1" else slice(half, 2 * half)
                dst[sl].copy_(v.to(device=self.device, dtype=torch.float16))
                seen.add(base + ".proj." + kind)
                continue
            if ck not in self.t:
                if strict:
                    raise KatzError("unexpected key in state dict: %s" % k)
                continue
            dst = self.t[ck]
            src = v.to(device=self.device, dtype=torch.float16)
            if len(self.shapes[ck]) == 4:
                cin = self.shapes[ck][1]
                if tuple(src.shape) != tuple(self.shapes[ck]):
                    raise KatzError("shape mismatch for %s: %s vs %s" % (k, tuple(src.shape), self.shapes[ck]))
                dst[:src.shape[0], :, :, :cin].copy_(src.permute(0, 2, 3, 1))
            else:
                if tuple(src.shape) != tuple(self.shapes[ck]):
                    raise KatzError("shape mismatch for %s: %s vs %s" % (k, tuple(src.shape), tuple(self.shapes[ck])))
                if dst.shape == src.shape:
                    dst.copy_(src)
                else:
                    dst[:src.shape[0]].copy_(src)      # a widened bias vector: the padding stays zero
            seen.add(ck)
        if strict:
            missing = [k for k in self.shapes if k not in seen]
            if missing:
                raise KatzError("missing keys in state dict: %s ..." % missing[:5])
        return missing

    def export(self):
        """Reference-layout state dict (fresh tensors, torch conv layout)."""
        out = OrderedDict()
        for k, shp in self.shapes.items():
            t = self.t[k]
            if len(shp) == 4:
                out[k] = t[:shp[0], :, :, :shp[1]].permute(0, 3, 1, 2).contiguous()
            elif len(shp) == 1:
                out[k] = t[:shp[0]].clone()
            else:
                out[k] = t.clone()
        return out


class _Net:
    """Shared machinery of the UNet and the ControlNet: embeddings, down blocks, mid block."""

    def __init__(self, cfg, shapes, device):
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KatzError("katz_b200 models run on a CUDA device only (no CPU fallback)")
        self.w = _Weights(shapes, self.device)
        self.w.alloc()
        self.dtype = torch.float16
        self.rp = None                 # latent_parallel.RowParallel when the latent is row-split across GPUs
        # Step-invariant hoisting of the cross-attention K/V projection (it depends on the prompt only). Two forms:
        #  * eager calls: `cache_text_kv` keeps the projection of the last context tensor (off by default: the reference
        #    recomputes it every step). The key is the tensor's address, shape and version, so a caller that starts a new
        #    request calls begin_request() — a fresh tensor may reuse the old one's address. Never used during CUDA-graph
        #    capture: a graph that omitted the projection could not follow a new prompt.
        #  * CUDA graphs: engine.GraphedStep(hoist=True) computes the projection into a persistent buffer outside the graph
        #    (`_hoisted_kv`), refreshes it when the prompt or the weights change, and the captured step reads the buffer.
        self.cache_text_kv = False
        self._kv_cache_key = None
        self._kv_cache = None
        self._hoisted_kv = None
        self.weights_epoch = 0         # bumped whenever weights change (load_state_dict, LoRA merge / restore)
        # LayerNorms of the transformer blocks folded into the GEMMs that consume them (ops.LnFold per block: norm1 -> fused
        # q/k/v, norm2 -> attn2.to_q, norm3 -> GEGLU projection). The folded weights are DERIVED storage: the reference
        # keys keep addressing the plain weights (LoRA merges and state_dict() see those) and ensure_folds() re-derives
        # after every change. OFF by default: it removes 210 of the SDXL step's 957 launches but the step gets SLOWER
        # (19.2 -> 20.4 ms on a B200). With programmatic dependent launch a stand-alone LayerNorm runs in the shadow of the
        # next GEMM's set-up (a block of six GEMMs takes 146 us with or without the three LayerNorm launches between them),
        # while the statistics and the per-column correction lengthen the GEMM epilogues, which are on the critical path of
        # the single-wave launches (+12 us per block). It also costs 2.4 GB for the folded copies.
        self.fuse_ln = os.environ.get("KATZ_FUSED_LN", "0") == "1"
        self._folds = {}
        self._folds_epoch = -1

    # ---- state-dict surface (reference names)
    def load_state_dict(self, sd, strict=True):
        self.invalidate_caches()
        return self.w.load(sd, strict=strict)

    def state_dict(self):
        return self.w.export()

    def lora_targets(self, keys):
        """key -> live weight view [out, in] for LoRA merging."""
        out = OrderedDict()
        for k in keys:
            if k not in self.w.t or len(self.w.shapes[k]) != 2:
                raise KatzError("not a linear weight of this model: %s" % k)
            out[k] = self.w.t[k]
        return out

    def lora_merger(self, keys, keep_pristine=True):
        """A LoraMerger over this model's linears `keys` that tells the model whenever it rewrites them."""
        from .lora import LoraMerger
        return LoraMerger(self.lora_targets(keys), keep_pristine=keep_pristine, on_change=self.invalidate_caches)

    def invalidate_caches(self):
        """Call after anything that changes weights (a LoRA merge or restore writes the fused K/V weight buffer)."""
        self._kv_cache_key = None
        self.weights_epoch += 1

    def begin_request(self):
        """Start of a request in an eager serving loop: whatever was cached for the previous prompt / image is dropped."""
        self._kv_cache_key = None

    def ensure_folds(self):
        """Re-derive the LayerNorm-folded weights if any weight changed since they were built (a few GB of streaming, about a
        millisecond for SDXL). Called at the start of every eager step and before every graph replay; never inside a
        capture (the kernels would be baked into the graph)."""
        if not self.fuse_ln or self._folds_epoch == self.weights_epoch:
            return
        if torch.cuda.is_current_stream_capturing():
            raise KatzError("weights changed during CUDA-graph capture: call ensure_folds() before capturing")
        P = self._P
        blocks = sorted(k[: -len(".norm1.weight")] for k in self.w.shapes if k.endswith(".norm1.weight") and ".transformer_blocks." in k)
        for b in blocks:
            old = self._folds.get(b, (None, None, None))
            qkv = ops.ln_fold(self.w.fused[b + ".attn1.qkv"], P(b + ".norm1.weight"), P(b + ".norm1.bias"), None, 1e-5, out=old[0])
            q = ops.ln_fold(P(b + ".attn2.to_q.weight"), P(b + ".norm2.weight"), P(b + ".norm2.bias"), None, 1e-5, out=old[1])
            ff = ops.ln_fold(P(b + ".ff.net.0.proj.weight"), P(b + ".norm3.weight"), P(b + ".norm3.bias"),
                             P(b + ".ff.net.0.proj.bias"), 1e-5, out=old[2])
            self._folds[b] = (qkv, q, ff)
        self._folds_epoch = self.weights_epoch

    # ---- pieces
    def _P(self, k):
        return self.w.t[k]

    def _embeddings(self, timestep, text_embeds, time_ids, B):
        cfg, P = self.cfg, self._P
        if not torch.is_tensor(timestep):
            timestep = torch.tensor([float(timestep)], dtype=torch.float32, device=self.device)
        t = timestep.to(device=self.device, dtype=torch.float32).reshape(-1)
        if t.numel() == 1:
            t = t.expand(B)
        t = t.contiguous()
        c0 = cfg["block_out_channels"][0]
        t_emb = ops.timestep_embedding(t, c0)
        h = ops.linear(t_emb, P("time_embedding.linear_1.weight"), P("time_embedding.linear_1.bias"), act=ACT_SILU)
        emb = ops.linear(h, P("time_embedding.linear_2.weight"), P("time_embedding.linear_2.bias"))
        ad = cfg["addition_time_embed_dim"]
        n_ids = time_ids.shape[1]
        add_in = torch.empty((B, text_embeds.shape[1] + n_ids * ad), dtype=torch.float16, device=self.device)
        add_in[:, :text_embeds.shape[1]].copy_(text_embeds)
        tid = ops.timestep_embedding(time_ids.to(device=self.device, dtype=torch.float32).reshape(-1).contiguous(), ad)
        add_in[:, text_embeds.shape[1]:].copy_(tid.reshape(B, n_ids * ad))
        h = ops.linear(add_in, P("add_embedding.linear_1.weight"), P("add_embedding.linear_1.bias"), act=ACT_SILU)
        # emb = time_emb + aug_emb: the second MLP's output lands on emb through the residual epilogue
        emb = ops.linear(h, P("add_embedding.linear_2.weight"), P("add_embedding.linear_2.bias"), residual=emb)
        # every resnet's time_emb_proj(silu(emb)) in one GEMM
        semb = ops.silu(emb)
        temb_all = ops.linear(semb, self.w.fused["temb_w"], self.w.fused["temb_b"])
        return emb, temb_all

    def _cross_kv(self, ctx, out=None):
        """K/V projections of the text context for every transformer block at once: [B, S, sum 2C]."""
        if "cross_kv" not in self.w.fused:
            return None
        if out is None and self._hoisted_kv is not None:
            return self._hoisted_kv
        use_cache = self.cache_text_kv and out is None and not torch.cuda.is_current_stream_capturing()
        if use_cache:
            key = (ctx.data_ptr(), tuple(ctx.shape), ctx._version, self.weights_epoch)
            if self._kv_cache_key == key:
                return self._kv_cache
        B, S, D = ctx.shape
        kv = ops.linear(ctx.reshape(B * S, D), self.w.fused["cross_kv"], out=None if out is None else out.view(B * S, -1))
        kv = kv.view(B, S, -1)
        if use_cache:
            self._kv_cache_key, self._kv_cache = key, kv
        return kv

    # ---- the three operator classes that need an exchange when the latent is row-split (self.rp set)
    def _conv3x3(self, x, w, bias, stride=1, upsample=False, **epi):
        if self.rp is None:
            return ops.conv2d(x, w, bias, stride=stride, pad=1, upsample=upsample, **epi)
        return self.rp.conv3x3(x, w, bias, stride=stride, upsample=upsample, **epi)

    def _gn(self, x, gamma, beta, eps, act):
        if self.rp is None:
            return ops.group_norm_nhwc(x, gamma, beta, self.cfg["norm_num_groups"], eps, act)
        return self.rp.group_norm(x, gamma, beta, self.cfg["norm_num_groups"], eps, act)

    def _self_attention(self, qkv, C, heads):
        if self.rp is None:
            return ops.attention(qkv[:, :, :C], qkv[:, :, C:2 * C], qkv[:, :, 2 * C:], heads)
        return self.rp.self_attention(qkv, C, heads)

    def _resnet(self, p, x, temb_all):
        cfg, P = self.cfg, self._P
        eps = cfg["norm_eps"]
        B, H, W, Cin = x.shape
        off, cout = self.w.temb_offset[p]
        h = self._gn(x, P(p + ".norm_silu1.0.weight"), P(p + ".norm_silu1.0.bias"), eps, ACT_SILU)
        h = self._conv3x3(h, P(p + ".conv1.weight"), P(p + ".conv1.bias"), rowvec=temb_all[:, off:off + cout])
        h = self._gn(h, P(p + ".norm_silu2.0.weight"), P(p + ".norm_silu2.0.bias"), eps, ACT_SILU)
        if (p + ".conv_shortcut.weight") in self.w.t:
            sc = ops.linear(x.view(B * H * W, Cin), P(p + ".conv_shortcut.weight").view(cout, Cin),
                            P(p + ".conv_shortcut.bias")).view(B, H, W, cout)
        else:
            sc = x
        return self._conv3x3(h, P(p + ".conv2.weight"), P(p + ".conv2.bias"), residual=sc)

    def _transformer(self, p, x, kv, heads, n_layers):
        cfg, P = self.cfg, self._P
        B, H, W, C = x.shape
        M = B * H * W
        h = self._gn(x, P(p + ".norm.weight"), P(p + ".norm.bias"), 1e-6, ACT_NONE)
        # LayerNorm folded into its consumer: every GEMM whose output a LayerNorm reads also leaves that output's row
        # statistics, and the consumer applies them in its epilogue (no LayerNorm kernel, no normalised copy of the rows)
        fused = self.fuse_ln and self._folds_epoch == self.weights_epoch and ops.ln_fusable(M, C, C)
        if not fused:
            return self._transformer_unfused(p, x, h, kv, heads, n_layers)
        h, st = ops.linear(h.view(M, C), P(p + ".proj_in.weight"), P(p + ".proj_in.bias"), stats_out=True)
        for i in range(n_layers):
            b = "%s.transformer_blocks.%d" % (p, i)
            f_qkv, f_q, f_ff = self._folds[b]
            qkv = ops.linear(h, f_qkv.wf, ln=f_qkv, ln_stats=st).view(B, H * W, 3 * C)
            a = self._self_attention(qkv, C, heads)
            h, st = ops.linear(a.view(M, C), P(b + ".attn1.to_out.0.weight"), P(b + ".attn1.to_out.0.bias"), residual=h, stats_out=True)
            q = ops.linear(h, f_q.wf, ln=f_q, ln_stats=st).view(B, H * W, C)
            off = self.w.cross_kv_offset[b]
            a = ops.attention(q, kv[:, :, off:off + C], kv[:, :, off + C:off + 2 * C], heads)
            h, st = ops.linear(a.view(M, C), P(b + ".attn2.to_out.0.weight"), P(b + ".attn2.to_out.0.bias"), residual=h, stats_out=True)
            f = ops.feed_forward_geglu(h, f_ff.wf, None, ln=f_ff, ln_stats=st)
            if i + 1 < n_layers:
                h, st = ops.linear(f, P(b + ".ff.net.2.weight"), P(b + ".ff.net.2.bias"), residual=h, stats_out=True)
            else:
                h = ops.linear(f, P(b + ".ff.net.2.weight"), P(b + ".ff.net.2.bias"), residual=h)
        out = ops.linear(h, P(p + ".proj_out.weight"), P(p + ".proj_out.bias"), residual=x.view(M, C))
        return out.view(B, H, W, C)

    def _transformer_unfused(self, p, x, h, kv, heads, n_layers):
        """The same blocks with stand-alone LayerNorm kernels (shapes the folded path declines, KATZ_FUSED_LN=0)."""
        P = self._P
        B, H, W, C = x.shape
        M = B * H * W
        h = ops.linear(h.view(M, C), P(p + ".proj_in.weight"), P(p + ".proj_in.bias"))
        for i in range(n_layers):
            b = "%s.transformer_blocks.%d" % (p, i)
            n = ops.layer_norm(h, P(b + ".norm1.weight"), P(b + ".norm1.bias"))
            qkv = ops.linear(n, self.w.fused[b + ".attn1.qkv"]).view(B, H * W, 3 * C)
            a = self._self_attention(qkv, C, heads)
            h = ops.linear(a.view(M, C), P(b + ".attn1.to_out.0.weight"), P(b + ".attn1.to_out.0.bias"), residual=h)
            n = ops.layer_norm(h, P(b + ".norm2.weight"), P(b + ".norm2.bias"))
            q = ops.linear(n, P(b + ".attn2.to_q.weight")).view(B, H * W, C)
            off = self.w.cross_kv_offset[b]
            a = ops.attention(q, kv[:, :, off:off + C], kv[:, :, off + C:off + 2 * C], heads)
            h = ops.linear(a.view(M, C), P(b + ".attn2.to_out.0.weight"), P(b + ".attn2.to_out.0.bias"), residual=h)
            n = ops.layer_norm(h, P(b + ".norm3.weight"), P(b + ".norm3.bias"))
            f = ops.feed_forward_geglu(n, P(b + ".ff.net.0.proj.weight"), P(b + ".ff.net.0.proj.bias"))
            h = ops.linear(f, P(b + ".ff.net.2.weight"), P(b + ".ff.net.2.bias"), residual=h)
        out = ops.linear(h, P(p + ".proj_out.weight"), P(p + ".proj_out.bias"), residual=x.view(M, C))
        return out.view(B, H, W, C)

    def _down_and_mid(self, sample, temb_all, kv):
        cfg, P = self.cfg, self._P
        res = [sample]
        nb = len(cfg["block_out_channels"])
        for bi, btype in enumerate(cfg["down_block_types"]):
            heads = cfg["attention_head_dim"][bi]
            for li in range(cfg["layers_per_block"]):
                sample = self._resnet("down_blocks.%d.resnets.%d" % (bi, li), sample, temb_all)
                if btype == "CrossAttnDownBlock2D":
                    sample = self._transformer("down_blocks.%d.attentions.%d" % (bi, li), sample, kv, heads,
                                               cfg["transformer_layers_per_block"][bi])
                res.append(sample)
            if bi != nb - 1:
                p = "down_blocks.%d.downsamplers.0.conv" % bi
                sample = self._conv3x3(sample, P(p + ".weight"), P(p + ".bias"), stride=2)
                res.append(sample)
        heads = cfg["attention_head_dim"][-1]
        sample = self._resnet("mid_block.resnets.0", sample, temb_all)
        sample = self._transformer("mid_block.attentions.0", sample, kv, heads, cfg["transformer_layers_per_block"][-1])
        sample = self._resnet("mid_block.resnets.1", sample, temb_all)
        return sample, res

    def _prep_inputs(self, sample, encoder_hidden_states, added_cond_kwargs):
        if added_cond_kwargs is None or "text_embeds" not in added_cond_kwargs or "time_ids" not in added_cond_kwargs:
            raise ValueError("addition_embed_type 'text_time' requires `text_embeds` and `time_ids` in added_cond_kwargs")
        x = sample.to(device=self.device, dtype=torch.float16)
        ctx = encoder_hidden_states.to(device=self.device, dtype=torch.float16).contiguous()
        te = added_cond_kwargs["text_embeds"].to(device=self.device, dtype=torch.float16)
        ti = added_cond_kwargs["time_ids"].to(device=self.device)
        return x, ctx, te, ti


def _to_nhwc_residual(r, device):
    """ControlNet residuals arrive NCHW (reference layout) or NHWC-tagged; return a contiguous NHWC fp16 tensor."""
    if isinstance(r, NHWC):
        return r.t
    r = r.to(device=device, dtype=torch.float16)
    return ops.nchw_to_nhwc(r)


class NHWC:
    """Marks a tensor that is already [B, H, W, C]; lets an in-process ControlNet hand residuals to the UNet without
    two layout moves."""

    def __init__(self, t):
        self.t = t


class KatzUNet(_Net):
    """UNet2DConditionModel of the reference, SDXL structure."""

    def __init__(self, cfg, device="cuda", state_dict=None):
        super().__init__(cfg, unet_param_shapes(cfg), device)
        self.use_cuda_graph = False
        self._graphs = {}
        if state_dict is not None:
            self.load_state_dict(state_dict)

    def down_forward(self, x, timestep, ctx, te, ti):
        """`_down_forward` (unet_2d_condition.py:1127-1252) on NHWC tensors."""
        if not torch.cuda.is_current_stream_capturing():
            self.ensure_folds()
        B = x.shape[0]
        emb, temb_all = self._embeddings(timestep, te, ti, B)
        kv = self._cross_kv(ctx)
        h = ops.nchw_to_nhwc(x, cpad=self.w.conv_cin_pad["conv_in.weight"])
        if self.rp is not None:
            self.rp.begin_step()
            h = self.rp.shard_rows(h)          # every rank holds the whole latent; keep this rank's rows
        h = self._conv3x3(h, self._P("conv_in.weight"), self._P("conv_in.bias"))
        mid, res = self._down_and_mid(h, temb_all, kv)
        return mid, temb_all, res, kv

    def up_forward(self, sample, temb_all, res, kv, down_residuals=None, mid_residual=None, combine_scales=None):
        """`_up_forward` (unet_2d_condition.py:1254-1341). `down_residuals` is a list of 9 tensors, or a list of such
        lists (one per ControlNet) combined with `combine_scales` (sum: 1.0 each; the service path's mean: 1/N each,
        unet_2d_condition.py:1418-1439)."""
        cfg, P = self.cfg, self._P
        if down_residuals is not None:
            nets = down_residuals if isinstance(down_residuals[0], (list, tuple)) else [down_residuals]
            mids = mid_residual if isinstance(mid_residual, (list, tuple)) else [mid_residual]
            scales = combine_scales or [1.0] * len(nets)
            if any(len(n) != len(res) for n in nets):
                raise KatzError("expected %d down residuals per ControlNet" % len(res))
            def fit(t, like):
                t = _to_nhwc_residual(t, self.device)
                if self.rp is not None and t.shape[1] != like.shape[1]:
                    t = self.rp.shard_rows(t)     # a full-height residual from a ControlNet that is not row-split
                return t
            res = [ops.residual_intake(r, [fit(n[j], r) for n in nets], scales) for j, r in enumerate(res)]
            sample = ops.residual_intake(sample, [fit(m, sample) for m in mids], scales)
        nb = len(cfg["block_out_channels"])
        rev_heads = tuple(reversed(cfg["attention_head_dim"]))
        rev_layers = tuple(reversed(cfg["transformer_layers_per_block"]))
        res = list(res)
        for bi, btype in enumerate(cfg["up_block_types"]):
            n_res = cfg["layers_per_block"] + 1
            for li in range(n_res):
                skip = res.pop()
                sample = ops.concat_channels(sample, skip)
                sample = self._resnet("up_blocks.%d.resnets.%d" % (bi, li), sample, temb_all)
                if btype == "CrossAttnUpBlock2D":
                    sample = self._transformer("up_blocks.%d.attentions.%d" % (bi, li), sample, kv, rev_heads[bi],
                                               rev_layers[bi])
            if bi != nb - 1:
                p = "up_blocks.%d.upsamplers.0.conv" % bi
                sample = self._conv3x3(sample, P(p + ".weight"), P(p + ".bias"), upsample=True)
        h = self._gn(sample, P("conv_norm_silu.0.weight"), P("conv_norm_silu.0.bias"), cfg["norm_eps"], ACT_SILU)
        out = self._conv3x3(h, P("conv_out.weight"), P("conv_out.bias"))
        if self.rp is not None:
            out = self.rp.gather_rows(out)     # [B, H, W, c]: every rank returns the whole prediction
        return ops.nhwc_to_nchw(out, c=cfg["out_channels"])

    def __call__(self, sample, timestep, encoder_hidden_states, timestep_cond=None, cross_attention_kwargs=None,
                 added_cond_kwargs=None, down_block_additional_residuals=None, mid_block_additional_residual=None,
                 return_dict=False, combine_scales=None, **_ignored):
        """One denoising step; returns `(noise_pred,)` (NCHW fp16) like the reference with return_dict=False.
        With `use_cuda_graph` (the reference's ENABLE_CUDA_GRAPH=1) the step is captured once per input signature and
        replayed with the inputs copied into static buffers, as `_forward_w_separate_cuda_graph` does."""
        if self.use_cuda_graph and not torch.cuda.is_current_stream_capturing():
            from .engine import graphed_unet_call
            return (graphed_unet_call(self, sample, timestep, encoder_hidden_states, added_cond_kwargs,
                                      down_block_additional_residuals, mid_block_additional_residual, combine_scales),)
        x, ctx, te, ti = self._prep_inputs(sample, encoder_hidden_states, added_cond_kwargs)
        mid, temb_all, res, kv = self.down_forward(x, timestep, ctx, te, ti)
        out = self.up_forward(mid, temb_all, res, kv, down_block_additional_residuals, mid_block_additional_residual,
                              combine_scales)
        return (out,)

    forward = __call__


class KatzControlNet(_Net):
    """ControlNetModel of the reference (encoder + mid copy of the UNet, conditioning embedding, zero-convs)."""

    def __init__(self, cfg, device="cuda", state_dict=None, conditioning_channels=3):
        super().__init__(cfg, controlnet_param_shapes(cfg, conditioning_channels), device)
        # the conditioning embedding depends on the image only: same two forms of hoisting as the text K/V (see _Net)
        self.cache_cond_embedding = False
        self._cond_key = None
        self._cond_emb = None
        self._hoisted_cond = None
        if state_dict is not None:
            self.load_state_dict(state_dict)

    def begin_request(self):
        super().begin_request()
        self._cond_key = None

    def _cond_embedding(self, cond, out=None):
        """ControlNetConditioningEmbedding.forward (controlnet.py:113-127) up to, not including, its conv_out."""
        if out is None and self._hoisted_cond is not None:
            return self._hoisted_cond
        use_cache = self.cache_cond_embedding and out is None and not torch.cuda.is_current_stream_capturing()
        if use_cache:
            key = (cond.data_ptr(), tuple(cond.shape), cond._version, self.weights_epoch)
            if key == self._cond_key:
                return self._cond_emb
        P = self._P
        p = "controlnet_cond_embedding"
        h = ops.nchw_to_nhwc(cond.to(device=self.device, dtype=torch.float16), cpad=self.w.conv_cin_pad[p + ".conv_in.weight"])
        h = ops.conv2d(h, P(p + ".conv_in.weight"), P(p + ".conv_in.bias"), act=ACT_SILU)
        n = 2 * (len(CONTROLNET_COND_CHANNELS) - 1)
        for i in range(n):
            h = ops.conv2d(h, P("%s.blocks.%d.weight" % (p, i)), P("%s.blocks.%d.bias" % (p, i)),
                           stride=2 if i % 2 == 1 else 1, act=ACT_SILU, out=out if i == n - 1 else None)
        if use_cache:
            self._cond_key, self._cond_emb = key, h
        return h

    def __call__(self, sample, timestep, encoder_hidden_states, controlnet_cond, conditioning_scale=0.5,
                 added_cond_kwargs=None, return_dict=False, nhwc_out=False, **_ignored):
        """`_controlnet_forward` (controlnet.py:687-847): returns (list of 9 down residuals, mid residual), each already
        multiplied by `conditioning_scale`; NCHW like the reference unless `nhwc_out`."""
        P = self._P
        if not torch.cuda.is_current_stream_capturing():
            self.ensure_folds()
        x, ctx, te, ti = self._prep_inputs(sample, encoder_hidden_states, added_cond_kwargs)
        B = x.shape[0]
        emb, temb_all = self._embeddings(timestep, te, ti, B)
        kv = self._cross_kv(ctx)
        p = "controlnet_cond_embedding"
        ce = self._cond_embedding(controlnet_cond)
        h = ops.nchw_to_nhwc(x, cpad=self.w.conv_cin_pad["conv_in.weight"])
        h = ops.conv2d(h, P("conv_in.weight"), P("conv_in.bias"))
        # sample = conv_in(sample) + cond_embedding.conv_out(...): the add rides on the second conv's residual epilogue
        h = ops.conv2d(ce, P(p + ".conv_out.weight"), P(p + ".conv_out.bias"), residual=h)
        mid, res = self._down_and_mid(h, temb_all, kv)
        outs = []
        s = float(conditioning_scale)
        for i, r in enumerate(res):
            Bq, H, W, C = r.shape
            o = ops.linear(r.view(Bq * H * W, C), P("controlnet_down_blocks.%d.weight" % i).view(C, C),
                           P("controlnet_down_blocks.%d.bias" % i), out_scale=s).view(Bq, H, W, C)
            outs.append(o)
        Bq, H, W, C = mid.shape
        m = ops.linear(mid.view(Bq * H * W, C), P("controlnet_mid_block.weight").view(C, C), P("controlnet_mid_block.bias"),
                       out_scale=s).view(Bq, H, W, C)
        if nhwc_out:
            return [NHWC(o) for o in outs], NHWC(m)
        return [ops.nhwc_to_nchw(o) for o in outs], ops.nhwc_to_nchw(m)

    forward = __call__
