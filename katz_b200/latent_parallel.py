"""Latent-row parallelism: the latent (and every activation derived from it) is split by rows across the GPUs of one
node, one process per GPU, and only three operator classes exchange data:

  * 3x3 convolutions need one halo row from each neighbour (stride 2: the upper neighbour only; the upsampling
    convolution exchanges the rows BEFORE the 2x upsample);
  * GroupNorm statistics are summed over all shards (fp64 (sum, sum of squares) per (batch, group));
  * self-attention keeps its query rows local and all-gathers the K/V shards.

Everything else (linears, LayerNorm, GEGLU, cross-attention, residual and ControlNet adds, 1x1 convolutions) is local.
The reference has no such split (its "latent_parallel" flag is a 2-GPU classifier-free-guidance split,
sdxl_unet_server.py:41,199-215); parity is therefore against the single-GPU result, to which a synchronous row split
is equal up to the order of the GroupNorm reduction.

Collectives go through torch.distributed (NCCL on GPUs). The communication primitives at the top of `RowParallel`
are backend-agnostic and are exercised with gloo on CPU tensors in the tests.
"""
import os

import torch
import torch.distributed as dist

from .ops import KatzError


class RowParallel:
    def __init__(self, rank=None, world=None, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        if self.world < 1 or not (0 <= self.rank < self.world):
            raise KatzError("bad rank/world for RowParallel: %s/%s" % (self.rank, self.world))
        self.peer = None          # peer.PeerArena: exchanges go over peer memory instead of torch.distributed
        self._exchange = 0        # index of the next exchange within the step

    def begin_step(self):
        """Called at the start of every step: the exchanges of a step are numbered from zero (each has its own buffer in
        the peer arena)."""
        self._exchange = 0

    # ---- sharding -------------------------------------------------------------------------------------------------
    def rows_of(self, H):
        """(first row, row count) this rank owns of an H-row tensor. H must split evenly into an even row count
        (the stride-2 convolutions halve it)."""
        if H % self.world:
            raise KatzError("%d rows do not split over %d ranks" % (H, self.world))
        h = H // self.world
        return self.rank * h, h

    def shard_rows(self, x_full):
        """[B, H, W, C] -> this rank's [B, H/P, W, C] (contiguous copy)."""
        r0, h = self.rows_of(x_full.shape[1])
        return x_full[:, r0:r0 + h].contiguous()

    # ---- communication primitives (any backend, any device) --------------------------------------------------------
    def exchange_halo(self, x):
        """x: [B, h, W, C] local rows. Returns (top, bottom): the neighbouring ranks' adjacent rows as [B, W, C]
        tensors, zeros at the image edge. One all-gather of every rank's first and last row."""
        if self.world == 1:
            z = torch.zeros_like(x[:, 0])
            return z, z.clone()
        edges = torch.stack([x[:, 0], x[:, -1]]).contiguous()              # [2, B, W, C]
        allg = self.gather_shards(edges)                                    # [P, 2, B, W, C]
        top = allg[self.rank - 1, 1] if self.rank > 0 else torch.zeros_like(edges[0])
        bottom = allg[self.rank + 1, 0] if self.rank < self.world - 1 else torch.zeros_like(edges[0])
        return top, bottom

    def gather_shards(self, t):
        """t: contiguous local shard -> [P, *t.shape], rank-major (the K/V all-gather and the final row gather)."""
        if self.world == 1:
            return t.unsqueeze(0)
        if self.peer is not None and t.is_cuda and (t.shape[-1] * t.element_size()) % 16 == 0:
            k = self._exchange
            self._exchange += 1
            return self.peer.allgather(t, k)        # takes a column slice as it is
        t = t.contiguous()
        # the concatenated form (dim 0 = P * t.shape[0]) is the one every backend accepts
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out.view((self.world,) + tuple(t.shape))

    def reduce_stats(self, sums):
        """In-place sum over ranks of the fp64 GroupNorm sums [B, G, 2]."""
        if self.world > 1 and self.peer is not None and sums.is_cuda:
            sums.copy_(self.gather_shards(sums).sum(0))      # rank order: the same bits on every rank
        elif self.world > 1:
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=self.group)
        return sums

    def gather_rows(self, x_local):
        """[B, h, W, C] shards -> the whole [B, H, W, C] on every rank."""
        g = self.gather_shards(x_local)                                     # [P, B, h, W, C]
        P, B, h, W, C = g.shape
        return g.permute(1, 0, 2, 3, 4).reshape(B, P * h, W, C).contiguous()

    def gather_edges(self, x):
        """[P, 2, B, W, C]: every rank's first and last row (None on a single rank)."""
        if self.world == 1:
            return None
        B, h = x.shape[0], x.shape[1]
        if B == 1 and h > 1 and self.peer is not None and x.is_cuda:
            # rows 0 and h-1 of the single image: two rows at a constant pitch, pushed without packing them first
            edges = x.as_strided((2, 1, x.shape[2], x.shape[3]), ((h - 1) * x.stride(1), x.stride(0), x.stride(2), x.stride(3)))
            k = self._exchange
            self._exchange += 1
            return self.peer.allgather(edges.view(2, -1), k).view(self.world, 2, 1, x.shape[2], x.shape[3])
        return self.gather_shards(torch.stack([x[:, 0], x[:, -1]]).contiguous())

    def assemble(self, x, top=True, bottom=True, upsample=False):
        """The input a 3x3 convolution of this shard reads: one kernel on the GPU (ops.halo_assemble)."""
        if x.is_cuda and x.dtype == torch.float16:
            from . import ops
            return ops.halo_assemble(x.contiguous(), self.gather_edges(x), self.rank, self.world, top, bottom, upsample)
        if upsample:
            up = self.pad_rows(x).repeat_interleave(2, dim=1).repeat_interleave(2, dim=2)
            return up[:, 1:2 * x.shape[1] + 3].contiguous()
        return self.pad_rows(x, top, bottom)

    def pad_rows(self, x, top=True, bottom=True):
        """x [B, h, W, C] -> [B, h + top + bottom, W, C] with the neighbours' rows (zeros at image edges) attached."""
        B, h, W, C = x.shape
        t, b = self.exchange_halo(x)
        out = torch.empty((B, h + int(top) + int(bottom), W, C), dtype=x.dtype, device=x.device)
        o = 0
        if top:
            out[:, 0].copy_(t)
            o = 1
        out[:, o:o + h].copy_(x)
        if bottom:
            out[:, o + h].copy_(b)
        return out

    # ---- operators on the CUDA kernels ----------------------------------------------------------------------------
    def conv3x3(self, x, w, bias, stride=1, upsample=False, **epi):
        from . import ops
        B, h, W, C = x.shape
        if upsample:
            # exchange the rows before the upsample, upsample the padded shard, drop the outermost upsampled rows:
            # rows [1, 2h+3) of the upsampled padded shard are exactly the 2h+2 input rows the 2h output rows read
            return ops.conv2d(self.assemble(x, upsample=True), w, bias, stride=1, pad=1, pad_h=0, **epi)
        if stride == 2:
            if h % 2:
                raise KatzError("a stride-2 convolution needs an even number of rows per rank (got %d)" % h)
            return ops.conv2d(self.assemble(x, bottom=False), w, bias, stride=2, pad=1, pad_h=0, **epi)
        return ops.conv2d(self.assemble(x), w, bias, stride=1, pad=1, pad_h=0, **epi)

    def group_norm(self, x, gamma, beta, groups, eps, act):
        from . import ops
        B, C = x.shape[0], x.shape[-1]
        rows_local = x.numel() // (B * C)
        sums = ops.group_norm_stats(x, groups)
        if self.peer is not None and self.world > 1:
            sums = self.gather_shards(sums)          # [P, B, G, 2]: the normalising kernel adds the shards' sums itself
        else:
            self.reduce_stats(sums)
        return ops.group_norm_apply(x, sums, gamma, beta, groups, float(rows_local) * self.world * (C // groups), eps, act)

    def self_attention(self, qkv, C, heads):
        """qkv: [B, s, 3C] local tokens. Queries stay local; K/V shards are all-gathered ([P, B, s, 2C]) and read in
        place by the attention kernel as P chunks."""
        from . import ops
        B, s, _ = qkv.shape
        kv_local = qkv[:, :, C:]
        if (self.peer is not None and self.world > 1 and s % 128 == 0 and (2 * C * qkv.element_size()) % 16 == 0
                and os.environ.get("KATZ_PEER_OVERLAP", "1") != "0"):
            # The shards are pushed without waiting for the peers: the attention kernel starts on this rank's own shard and
            # waits for each peer's flag only before it first touches that peer's chunk, so the NVLink transfer of the
            # remote shards overlaps the work on the local one.
            k = self._exchange
            self._exchange += 1
            g = self.peer.allgather(kv_local, k, wait=False)                # [P, B, s, 2C], chunks still arriving
            return ops.attention(qkv[:, :, :C], g[0][:, :, :C], g[0][:, :, C:], heads, kv_chunks=(self.world, s, B * s * 2 * C),
                                 peer=(self.peer.ctrl_address(), self.rank))
        g = self.gather_shards(kv_local)                                    # [P, B, s, 2C]
        if s % 64 == 0:
            return ops.attention(qkv[:, :, :C], g[0][:, :, :C], g[0][:, :, C:], heads,
                                 kv_chunks=(self.world, s, B * s * 2 * C))
        kv = g.permute(1, 0, 2, 3).reshape(B, self.world * s, 2 * C)        # small shards: make the keys contiguous
        return ops.attention(qkv[:, :, :C], kv[:, :, :C], kv[:, :, C:], heads)


def peer_arena_bytes(cfg, batch, height, width):
    """Arena size for one step's exchanges: every exchange has its own buffer (so none is acknowledged), and the
    self-attention K/V gathers dominate: per transformer layer 2 (K, V) x batch x tokens x channels fp16, whatever the number
    of ranks. 25% and 64 MiB on top for halo rows, GroupNorm sums and alignment; KATZ_PEER_ARENA_BYTES overrides."""
    if os.environ.get("KATZ_PEER_ARENA_BYTES"):
        return int(os.environ["KATZ_PEER_ARENA_BYTES"])
    total = 0
    boc = cfg["block_out_channels"]
    layers = cfg["transformer_layers_per_block"]
    h, w = height, width
    per_level = []
    for bi, btype in enumerate(cfg["down_block_types"]):
        per_level.append((boc[bi], h * w, layers[bi] if btype == "CrossAttnDownBlock2D" else 0))
        if bi != len(boc) - 1:
            h, w = h // 2, w // 2
    n_res = cfg["layers_per_block"]
    for bi, (c, tokens, n) in enumerate(per_level):
        blocks = n_res + (n_res + 1)                       # the down block's and the mirrored up block's attentions
        if bi == len(per_level) - 1:
            blocks += 1                                    # the mid block
        total += blocks * n * 2 * batch * tokens * c * 2
    return int(total * 1.25) + (64 << 20)


def _lib_clear_tc05_status():
    from . import _lib
    _lib.check(_lib.load().katz_tc05_clear_status(), "katz_tc05_clear_status")


class RowParallelStep:
    """CUDA-graph step of a row-split UNet: same interface as engine.GraphedStep. Every rank passes the same inputs
    and receives the whole prediction."""

    def __init__(self, unet, batch, height, width, rank, world, text_len=77, group=None, warmup=2):
        from .engine import GraphedStep
        rp = RowParallel(rank, world, group)
        rp.rows_of(height)
        for lvl in range(len(unet.cfg["block_out_channels"])):
            if (height >> lvl) % world or ((height >> lvl) // world) % (2 if lvl < len(unet.cfg["block_out_channels"]) - 1 else 1):
                raise KatzError("latent height %d cannot be row-split over %d ranks at every UNet level" % (height, world))
        if world > 1 and unet.device.type == "cuda" and os.environ.get("KATZ_PEER", "1") != "0":
            from .peer import PeerArena
            try:
                rp.peer = PeerArena(rank, world, group=group, device=unet.device,
                                    nbytes=peer_arena_bytes(unet.cfg, batch, height, width))
            except KatzError:
                rp.peer = None          # every rank reached the same verdict: the exchanges go through torch.distributed
        unet.rp = rp
        self.rp = rp
        if world > 1 and dist.is_initialized():
            dist.barrier(group=group)      # start the warm-up steps together: an exchange waits only a second or two for a peer
        self._inner = GraphedStep(unet, batch, height, width, text_len=text_len, warmup=warmup)
        if rp.peer is not None:
            # whatever skew the ranks had while they warmed up and captured is not the step's: from here on a time-out counts
            torch.cuda.synchronize()
            dist.barrier(group=group)
            rp.peer.clear_status()
            _lib_clear_tc05_status()      # the attention kernel's own wait for a peer's K/V reports through the tcgen05 status word
            dist.barrier(group=group)
        self.graph = self._inner.graph
        self.launches_per_step = self._inner.launches_per_step
        self.static = self._inner.static

    def replay(self):
        return self._inner.replay()

    def run(self, **tensors):
        return self._inner.run(**tensors)

    def check(self):
        """Raise KatzError if a tcgen05 wait or a peer exchange of this rank ever timed out (see engine.check_device_status).
        The unet's `rp` may have been replaced since this step was built, so the step's own RowParallel is checked."""
        from .engine import check_device_status

        class _U:
            rp = self.rp
        check_device_status(_U)


def cfg_rows_layout(batch, world, rank, split_cfg=True):
    """How `world` ranks share a step of `batch` samples: (halves, rows_world, half, row_rank, local_batch).

    With an even batch (classifier-free guidance: unconditional and conditional halves) and an even world the batch is
    split first — each half of the ranks runs one half of the batch, the reference's own 2-GPU mode
    (sdxl_unet_server.py:41,199-215), with no exchange inside the step — and only the ranks of one half row-split the
    latent among themselves. An odd batch or an odd world falls back to the pure row split."""
    if world < 1 or not (0 <= rank < world):
        raise KatzError("bad rank/world: %s/%s" % (rank, world))
    halves = 2 if (split_cfg and batch % 2 == 0 and world % 2 == 0) else 1
    rows_world = world // halves
    return halves, rows_world, rank // rows_world, rank % rows_world, batch // halves


def assemble_halves(gathered, halves, rows_world, out=None):
    """gathered: [world, local_batch, ...] (an all-gather of every rank's result, each already whole in rows) ->
    [batch, ...]: half h of the batch is what the first rank of half h holds."""
    world, lb = gathered.shape[0], gathered.shape[1]
    if out is None:
        out = torch.empty((halves * lb,) + tuple(gathered.shape[2:]), dtype=gathered.dtype, device=gathered.device)
    for h in range(halves):
        out[h * lb:(h + 1) * lb].copy_(gathered[h * rows_world])
    return out


class CfgRowParallelStep:
    """CUDA-graph step shared by `world` ranks: batch halves first, latent rows inside a half (cfg_rows_layout). Same
    interface as engine.GraphedStep; every rank passes the same full-batch inputs and receives the whole prediction."""

    def __init__(self, unet, batch, height, width, rank, world, text_len=77, warmup=2, split_cfg=True):
        from .engine import GraphedStep
        self.rank, self.world = rank, world
        self.halves, self.rows_world, self.half, self.row_rank, self.local_batch = cfg_rows_layout(batch, world, rank, split_cfg)
        row_group = None
        if self.halves > 1 and self.rows_world > 1:
            # every rank creates every group, in the same order
            groups = [dist.new_group(list(range(h * self.rows_world, (h + 1) * self.rows_world))) for h in range(self.halves)]
            row_group = groups[self.half]
        if self.rows_world > 1:
            self._inner = RowParallelStep(unet, self.local_batch, height, width, self.row_rank, self.rows_world,
                                          text_len=text_len, group=row_group, warmup=warmup)
        else:
            unet.rp = None
            self._inner = GraphedStep(unet, self.local_batch, height, width, text_len=text_len, warmup=warmup)
        self.graph = self._inner.graph
        self.launches_per_step = self._inner.launches_per_step
        self.static = self._inner.static
        self.out = None
        self._gathered = None
        if self.halves > 1:
            c = unet.cfg["out_channels"]
            self._gathered = torch.empty((world, self.local_batch, c, height, width), dtype=torch.float16, device=unet.device)
            self.out = torch.empty((batch, c, height, width), dtype=torch.float16, device=unet.device)

    def replay(self):
        """Run the step on whatever the static input buffers hold, then assemble the batch halves."""
        return self._finish(self._inner.replay())

    def run(self, **tensors):
        lb, h = self.local_batch, self.half
        local = {k: (v if (k == "timestep" or self.halves == 1) else v[h * lb:(h + 1) * lb]) for k, v in tensors.items()}
        return self._finish(self._inner.run(**local))

    def check(self):
        """Raise KatzError if a bounded device-side wait of this rank's step ever gave up."""
        self._inner.check()

    def _finish(self, o):
        lb = self.local_batch
        if self.halves == 1:
            return o
        dist.all_gather_into_tensor(self._gathered.view((self.world * lb,) + tuple(self._gathered.shape[2:])), o.contiguous())
        return assemble_halves(self._gathered, self.halves, self.rows_world, out=self.out)
