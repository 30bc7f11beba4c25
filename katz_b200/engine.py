"""CUDA-graph execution of the UNet (and ControlNet) step.

The reference runs its UNet as two CUDA graphs (`_down_forward`, `_up_forward`) with the ControlNet intake between
them and copies inputs into static tensors before each replay (unet_2d_condition.py:64-78,1344-1526); the ControlNet
is one graph (controlnet.py:903-929). Here the whole step — ControlNets, intake, UNet — is ONE graph of katz_b200
kernel launches: there is no process boundary between the graphs to wait on, and LoRA merges write the same weight
storage the graph reads, so a merge never forces a re-capture.
"""
import torch

from .ops import KatzError
from .unet import NHWC


def check_device_status(unet):
    """The status words the kernels leave behind instead of hanging: tcgen05 pipeline waits (ops.tc05_status) and, when
    the latent is row-split over peer memory, the all-gather's wait for a peer (PeerArena.status)."""
    from . import ops
    st = ops.tc05_status()
    if st != 0:
        raise KatzError("a bounded wait inside a tcgen05 kernel gave up (status %d): the step's result is not valid" % st)
    rp = getattr(unet, "rp", None)
    peer = getattr(rp, "peer", None) if rp is not None else None
    if peer is not None:
        ps = peer.status()
        if ps != 0:
            raise KatzError("a peer exchange timed out waiting for rank %d (status %d): the step's result is not valid"
                            % (ps - 100, ps))


class GraphedStep:
    """Static-input wrapper around `unet(...)` (+ optional in-process ControlNets).

    inputs: sample [B,4,H,W] fp16, timestep fp32 [1], encoder_hidden_states [B,77,D], text_embeds [B,E], time_ids [B,6],
    controlnet_cond [B,3,8H,8W] (when ControlNets are given). `run(**tensors)` copies the given tensors into the static
    buffers (host or device sources) and replays; the result is a static device tensor [B,4,H,W] fp16.
    """

    def __init__(self, unet, batch, height, width, text_len=77, controlnets=(), conditioning_scales=None,
                 combine="sum", warmup=2, hoist=False):
        if combine not in ("sum", "mean"):
            raise KatzError("combine must be 'sum' or 'mean'")
        dev = unet.device
        cfg = unet.cfg
        self.unet, self.controlnets = unet, list(controlnets)
        self.scales = list(conditioning_scales) if conditioning_scales else [0.5] * len(self.controlnets)
        n = len(self.controlnets)
        self.combine_scales = [1.0 / n if combine == "mean" else 1.0] * n if n else None
        n_text = cfg["projection_class_embeddings_input_dim"] - 6 * cfg["addition_time_embed_dim"]
        f16 = dict(dtype=torch.float16, device=dev)
        self.static = {
            "sample": torch.zeros((batch, cfg["in_channels"], height, width), **f16),
            "timestep": torch.zeros((1,), dtype=torch.float32, device=dev),
            "encoder_hidden_states": torch.zeros((batch, text_len, cfg["cross_attention_dim"]), **f16),
            "text_embeds": torch.zeros((batch, n_text), **f16),
            "time_ids": torch.zeros((batch, 6), **f16),
        }
        if n:
            self.static["controlnet_cond"] = torch.zeros((batch, 3, 8 * height, 8 * width), **f16)
        self.out = None
        self.graph = None
        self.launches_per_step = 0
        # hoist: the step-invariant parts (text K/V projection of every net, conditioning embedding of every ControlNet;
        # the reference recomputes both every step, sdxl_controlnet_server.py:87-100) live in persistent buffers that
        # `refresh_hoisted` fills outside the graph; the captured step reads them.
        self.hoist = bool(hoist)
        self._hoisted = []          # (net, kv buffer or None, conditioning-embedding buffer or None)
        self._hoist_epochs = None
        if self.hoist:
            s = self.static
            for net in [unet] + self.controlnets:
                kv = net._cross_kv(s["encoder_hidden_states"])
                ce = net._cond_embedding(s["controlnet_cond"]) if net is not unet else None
                self._hoisted.append((net, kv, ce))
            self._hoist_epochs = [n.weights_epoch for n, _, _ in self._hoisted]
        self._capture(warmup)

    def _step(self):
        s = self.static
        added = {"text_embeds": s["text_embeds"], "time_ids": s["time_ids"]}
        down = mid = None
        if self.controlnets:
            down, mid = [], []
            for cn, sc in zip(self.controlnets, self.scales):
                d, m = cn(s["sample"], s["timestep"], encoder_hidden_states=s["encoder_hidden_states"],
                          controlnet_cond=s["controlnet_cond"], conditioning_scale=sc, added_cond_kwargs=added,
                          nhwc_out=True)
                down.append(d)
                mid.append(m)
        return self.unet(s["sample"], s["timestep"], encoder_hidden_states=s["encoder_hidden_states"],
                         added_cond_kwargs=added, down_block_additional_residuals=down,
                         mid_block_additional_residual=mid, combine_scales=self.combine_scales)[0]

    def _set_hoisted(self, on):
        for net, kv, ce in self._hoisted:
            net._hoisted_kv = kv if on else None
            if ce is not None:
                net._hoisted_cond = ce if on else None

    def refresh_hoisted(self):
        """Recompute the hoisted buffers from the static inputs (new prompt, new conditioning image, changed weights), and
        whatever the nets derive from their weights. Callers that replay `self.graph` directly call this once per request."""
        for net in [self.unet] + self.controlnets:
            net.ensure_folds()
        if not self.hoist:
            return
        s = self.static
        for net, kv, ce in self._hoisted:
            if kv is not None:
                net._cross_kv(s["encoder_hidden_states"], out=kv)
            if ce is not None:
                net._cond_embedding(s["controlnet_cond"], out=ce)
        self._hoist_epochs = [n.weights_epoch for n, _, _ in self._hoisted]

    def _capture(self, warmup):
        from . import _lib
        self._set_hoisted(True)
        try:
            self._capture_inner(warmup, _lib)
        finally:
            self._set_hoisted(False)      # other callers of these nets keep the reference's per-step semantics

    def _capture_inner(self, warmup, _lib):
        for net in [self.unet] + self.controlnets:
            net.ensure_folds()
        side = torch.cuda.Stream(device=self.unet.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = _lib.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.out = self._step()
        self.launches_per_step = _lib.launch_count() - before
        self.graph = g

    def replay(self):
        """Run the step on whatever the static input buffers hold (a caller that wrote a new prompt or conditioning image
        into them directly calls refresh_hoisted() first; changed weights are noticed here)."""
        if self.hoist and self._hoist_epochs != [n.weights_epoch for n, _, _ in self._hoisted]:
            self.refresh_hoisted()
        for net in [self.unet] + self.controlnets:
            net.ensure_folds()        # LayerNorm-folded weights follow LoRA merges / restores (a no-op otherwise)
        self.graph.replay()
        return self.out

    def run(self, **tensors):
        for k, v in tensors.items():
            if k not in self.static:
                raise KatzError("unknown input %s" % k)
            self.static[k].copy_(v, non_blocking=True)
        if self.hoist and ("encoder_hidden_states" in tensors or "controlnet_cond" in tensors):
            self.refresh_hoisted()
        return self.replay()

    def check(self):
        """Raise if a bounded device-side wait of the tcgen05 kernels (or, row-split, of a peer exchange) ever gave up:
        the step then ran on incomplete data. Synchronises the device; call it once per request, not per step."""
        check_device_status(self.unet)


class _GraphedCall:
    """One captured `unet(...)` signature: static copies of every tensor argument, residuals included."""

    def __init__(self, unet, sample, timestep, ctx, added, down, mid, combine_scales):
        dev = unet.device

        def st(t, dtype=torch.float16):
            return torch.zeros(tuple(t.shape), dtype=dtype, device=dev)
        self.unet = unet
        self.sample, self.ctx = st(sample), st(ctx)
        self.timestep = torch.zeros((1,), dtype=torch.float32, device=dev)
        self.te, self.ti = st(added["text_embeds"]), st(added["time_ids"])
        self.down = self.mid = None
        if down is not None:
            nets = down if isinstance(down[0], (list, tuple)) else [down]
            mids = mid if isinstance(mid, (list, tuple)) else [mid]
            self.down = [[st(r) for r in n] for n in nets]
            self.mid = [st(m) for m in mids]
        self.combine_scales = combine_scales
        self.copy_in(sample, timestep, ctx, added, down, mid)
        unet.ensure_folds()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self._step()

    def _step(self):
        u = self.unet
        x, ctx, te, ti = u._prep_inputs(self.sample, self.ctx, {"text_embeds": self.te, "time_ids": self.ti})
        midt, temb_all, res, kv = u.down_forward(x, self.timestep, ctx, te, ti)
        return u.up_forward(midt, temb_all, res, kv, self.down, self.mid, self.combine_scales)

    def copy_in(self, sample, timestep, ctx, added, down, mid):
        self.sample.copy_(sample, non_blocking=True)
        self.ctx.copy_(ctx, non_blocking=True)
        if torch.is_tensor(timestep):
            self.timestep.copy_(timestep.reshape(-1)[:1], non_blocking=True)
        else:
            self.timestep.fill_(float(timestep))
        self.te.copy_(added["text_embeds"], non_blocking=True)
        self.ti.copy_(added["time_ids"], non_blocking=True)
        if self.down is not None:
            nets = down if isinstance(down[0], (list, tuple)) else [down]
            mids = mid if isinstance(mid, (list, tuple)) else [mid]
            for sn, n in zip(self.down, nets):
                for a, b in zip(sn, n):
                    a.copy_(b.t.permute(0, 3, 1, 2) if isinstance(b, NHWC) else b, non_blocking=True)
            for a, b in zip(self.mid, mids):
                a.copy_(b.t.permute(0, 3, 1, 2) if isinstance(b, NHWC) else b, non_blocking=True)


def graphed_unet_call(unet, sample, timestep, ctx, added, down, mid, combine_scales):
    """Dispatch of `KatzUNet.__call__` when `use_cuda_graph` is set: capture once per signature, then replay."""
    if added is None or "text_embeds" not in added or "time_ids" not in added:
        raise ValueError("addition_embed_type 'text_time' requires `text_embeds` and `time_ids` in added_cond_kwargs")
    n_nets = 0 if down is None else (len(down) if isinstance(down[0], (list, tuple)) else 1)
    key = (tuple(sample.shape), tuple(ctx.shape), n_nets, tuple(combine_scales) if combine_scales else None)
    gc = unet._graphs.get(key)
    if gc is None:
        gc = _GraphedCall(unet, sample, timestep, ctx, added, down, mid, combine_scales)
        unet._graphs[key] = gc
    else:
        gc.copy_in(sample, timestep, ctx, added, down, mid)
    unet.ensure_folds()
    gc.graph.replay()
    return gc.out
