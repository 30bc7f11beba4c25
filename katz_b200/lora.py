"""LoRA merge / restore / unmerge over a set of device-resident linears, one kernel launch per operation.

The reference's own entry points (`patch_on_lora(pipe, repos)` of lora_utils.py:9-33 and the pipeline method
`patch_on_lora(lora_state_dict, repos, default_unet_state_dict)` of pipeline_controlnet_sd_xl_katz.py:1730-1747) live
in katz_b200/lora_utils.py with the reference's argument lists; they delegate to the `LoraMerger` of this file, whose
`restore()` is `unet.load_state_dict(deepcopy(default_unet_state_dict))` (sdxl_unet_server.py:217).

The merger keeps the pristine weights W0 resident in HBM next to the live weights, so `merge` is a single streaming
pass W_live = W0 + sum_i s_i * B_i A_i and `restore` is a bit-exact copy — the reference's copy semantics, without its
three full-model copies per request. `merge_in_place` / `unmerge_in_place` give the +/- arithmetic of
LoRACompatibleLinear._fuse_lora/_unfuse_lora (diffusers/models/lora.py:403-449), which floating point does not undo
exactly.
"""
import ctypes
import json
from collections import OrderedDict

import numpy as np
import torch

from . import _lib
from ._lib import KATZ_DTYPE_F16, KATZ_DTYPE_F32, KatzError, LoraLayer, LORA_MAX_ADAPTERS

# numpy view of `struct katz_lora_layer` (128 bytes): the host table is filled column by column
_LAYER_DTYPE = np.dtype([("W", "<u8"), ("W0", "<u8"), ("B", "<u8", (LORA_MAX_ADAPTERS,)), ("A", "<u8", (LORA_MAX_ADAPTERS,)),
                         ("rank", "<i4", (LORA_MAX_ADAPTERS,)), ("scale", "<f4", (LORA_MAX_ADAPTERS,)), ("out_features", "<i4"),
                         ("in_features", "<i4"), ("n_lora", "<i4"), ("reserved_", "<i4")])
assert _LAYER_DTYPE.itemsize == ctypes.sizeof(LoraLayer)


class RegisteredAdapter:
    """An adapter validated once against a LoraMerger's target set (LoraMerger.register_adapter)."""

    def __init__(self, merger, adapter, up_ptr, down_ptr, rank):
        self.merger, self.adapter, self.up_ptr, self.down_ptr, self.rank = merger, adapter, up_ptr, down_ptr, rank

REFERENCE_UNET_SCALE = float(torch.tensor(20000.0 / 64.0, dtype=torch.float16))  # lora_utils.py:22


def _dtype_code(dt):
    if dt == torch.float16:
        return KATZ_DTYPE_F16
    if dt == torch.float32:
        return KATZ_DTYPE_F32
    raise KatzError("LoRA merge supports fp16 or fp32 weights, not %s" % dt)


class LoraMerger:
    """Owns the layer table for a fixed set of target weights.

    weights: OrderedDict key -> CUDA tensor [out, in] (contiguous rows; views into fused buffers are fine).
    keep_pristine: clone every target weight once (W0) so restore is a copy and merge never accumulates error.
    on_change: callable run after every merge / restore launch; pass the model's `invalidate_caches` (KatzUNet.lora_merger
    does) so that whatever the model derives from its weights follows them.
    """

    def __init__(self, weights, keep_pristine=True, on_change=None):
        self.on_change = on_change      # called after every launch that rewrites the weights (a model passes its
        #                                 invalidate_caches, so storage derived from the weights is rebuilt before the next step)
        if not weights:
            raise KatzError("no target weights")
        self.keys = list(weights.keys())
        self.weights = OrderedDict(weights)
        first = next(iter(weights.values()))
        self.device = first.device
        self.dtype = first.dtype
        self.code = _dtype_code(self.dtype)
        for k, w in weights.items():
            if w.dim() != 2 or not w.is_contiguous() or w.dtype != self.dtype or w.device != self.device:
                raise KatzError("target %s must be a contiguous 2-D %s tensor on %s" % (k, self.dtype, self.device))
        lib = _lib.load()
        self.tile_rows = lib.katz_lora_tile_rows(self.code)
        self.tile_cols = lib.katz_lora_tile_cols()
        starts, total, self.max_tiles_per_layer = [], 0, 0
        for w in self.weights.values():
            starts.append(total)
            n = -(-w.shape[0] // self.tile_rows) * -(-w.shape[1] // self.tile_cols)
            self.max_tiles_per_layer = max(self.max_tiles_per_layer, n)
            total += n
        self.total_tiles = total
        self.d_tile_start = torch.tensor(starts, dtype=torch.int32, device=self.device)
        # the TMA-tiled fast paths count tiles in their own geometry (the same as above for fp16, 128 x 64 for fp32)
        fr, fc = lib.katz_lora_fast_tile_rows(self.code), lib.katz_lora_fast_tile_cols(self.code)
        fstarts, ftotal, self.max_tiles_per_layer_fast = [], 0, 0
        for w in self.weights.values():
            fstarts.append(ftotal)
            n = -(-w.shape[0] // fr) * -(-w.shape[1] // fc)
            self.max_tiles_per_layer_fast = max(self.max_tiles_per_layer_fast, n)
            ftotal += n
        self.total_tiles_fast = ftotal
        self.d_tile_start_fast = self.d_tile_start if (fr, fc) == (self.tile_rows, self.tile_cols) else \
            torch.tensor(fstarts, dtype=torch.int32, device=self.device)
        self.pristine = None
        if keep_pristine:
            self.snapshot_pristine()
        n = len(self.keys)
        # the host table lives in the pinned staging buffer itself, so an upload is one asynchronous copy
        self._h_pinned = torch.empty(ctypes.sizeof(LoraLayer) * n, dtype=torch.uint8).pin_memory()
        self._h_table = (LoraLayer * n).from_address(self._h_pinned.data_ptr())
        self._np_table = np.frombuffer((ctypes.c_char * (ctypes.sizeof(LoraLayer) * n)).from_address(self._h_pinned.data_ptr()),
                                       dtype=_LAYER_DTYPE, count=n)
        self._shapes = [tuple(w.shape) for w in self.weights.values()]
        self._np_table["W"] = np.array([w.data_ptr() for w in self.weights.values()], np.uint64)
        self._np_table["out_features"] = [sh[0] for sh in self._shapes]
        self._np_table["in_features"] = [sh[1] for sh in self._shapes]
        self._np_table["reserved_"] = 0
        self._w0_ptr = np.zeros(n, np.uint64)
        if self.pristine is not None:
            self._w0_ptr = np.array([self.pristine[k].data_ptr() for k in self.keys], np.uint64)
        self._d_table = torch.empty(ctypes.sizeof(self._h_table), dtype=torch.uint8, device=self.device)
        self._keepalive = []
        self._d_maps = None        # TMA tensor maps of the fp16 fast path (two per layer), encoded on first use
        self._flags = 0
        self._upload_done = None   # event after the last table upload: the pinned staging buffer is reused
        self.merged = []   # description of what is currently merged

    # -- pristine copy ------------------------------------------------------------------------------------------
    def snapshot_pristine(self):
        """Record the current live weights as W0 (gen_unet_state_dict.py:54-58 plays this role in the reference)."""
        self.pristine = OrderedDict((k, w.clone()) for k, w in self.weights.items())
        self._d_maps = None
        self._w0_ptr = np.array([self.pristine[k].data_ptr() for k in self.keys], np.uint64)

    def algorithmic_bytes(self, ranks):
        """Bytes one merge pass must move: read + write of every W, plus each adapter's A and B once."""
        es = 2 if self.dtype == torch.float16 else 4
        wb = sum(w.numel() for w in self.weights.values()) * es
        ab = sum(r * (w.shape[0] + w.shape[1]) for w in self.weights.values() for r in ranks) * es
        return 2 * wb + ab

    # -- table --------------------------------------------------------------------------------------------------
    def _adapter_arrays(self, ad):
        """Per-layer arrays (up pointers, down pointers, ranks) of one adapter, validated against the target set. A
        `RegisteredAdapter` carries them ready-made."""
        if isinstance(ad, RegisteredAdapter):
            if ad.merger is not self:
                raise KatzError("this adapter was registered with another LoraMerger")
            return ad.up_ptr, ad.down_ptr, ad.rank
        n = len(self.keys)
        up_ptr, down_ptr, rank = np.zeros(n, np.uint64), np.zeros(n, np.uint64), np.zeros(n, np.int32)
        dt, dev = self.dtype, self.device
        get = ad.get
        for i, k in enumerate(self.keys):
            pair = get(k)
            if pair is None:
                continue
            up, down = pair
            if up.dtype != dt or down.dtype != dt or up.device != dev or down.device != dev:
                raise KatzError("adapter tensors for %s must be %s on %s" % (k, dt, dev))
            if not up.is_contiguous() or not down.is_contiguous():
                raise KatzError("adapter tensors for %s must be contiguous" % k)
            r = down.shape[0]
            o, c = self._shapes[i]
            if up.shape != (o, r) or down.shape != (r, c):
                raise KatzError("adapter shapes for %s do not match W%s: up%s down%s" % (k, (o, c), tuple(up.shape), tuple(down.shape)))
            up_ptr[i], down_ptr[i], rank[i] = up.data_ptr(), down.data_ptr(), r
        return up_ptr, down_ptr, rank

    def register_adapter(self, ad):
        """Validate an adapter once and keep its table columns: a serving loop that switches between a fixed pool of
        adapters passes the returned handle to merge() and pays no per-layer host work per switch. The handle keeps
        the tensors alive; do not replace tensors inside `ad` afterwards."""
        up_ptr, down_ptr, rank = self._adapter_arrays(ad)
        return RegisteredAdapter(self, ad, up_ptr, down_ptr, rank)

    def _fill(self, adapters, scales, use_pristine):
        """adapters: list of dict key -> (up [out,r], down [r,in]) on this device, same dtype as W (or handles from
        register_adapter). The table is written as whole numpy columns into the pinned staging buffer."""
        if len(adapters) > LORA_MAX_ADAPTERS:
            raise KatzError("at most %d adapters per merge" % LORA_MAX_ADAPTERS)
        if use_pristine and self.pristine is None:
            raise KatzError("no pristine copy: construct with keep_pristine=True or call snapshot_pristine()")
        lib = _lib.load()
        if self._upload_done is not None:
            self._upload_done.synchronize()
        n = len(self.keys)
        tab = self._np_table
        tab["W0"] = self._w0_ptr if use_pristine else 0
        slot = np.zeros(n, np.int64)             # next free adapter slot of every layer
        cols = {f: np.zeros((n, LORA_MAX_ADAPTERS), tab[f].dtype) for f in ("B", "A", "rank", "scale")}
        rows = np.arange(n)
        for ad, s in zip(adapters, scales):
            up_ptr, down_ptr, rank = self._adapter_arrays(ad)
            has = rank > 0
            if isinstance(s, dict):
                sc = np.array([float(s.get(k, 0.0)) for k in self.keys], np.float32)
            else:
                sc = np.full(n, float(s), np.float32)
            r, c = rows[has], slot[has]
            cols["B"][r, c], cols["A"][r, c], cols["rank"][r, c], cols["scale"][r, c] = up_ptr[has], down_ptr[has], rank[has], sc[has]
            slot[has] += 1
        for f, v in cols.items():
            tab[f] = v
        tab["n_lora"] = slot
        bad = ctypes.c_int(-1)
        rc = lib.katz_lora_table_check(self._h_table, n, self.code, ctypes.byref(bad))
        if rc != 0:
            _lib.check(rc, "katz_lora_table_check(%s)" % self.keys[bad.value])
        self._keepalive = list(adapters)
        rk, sc, nl = cols["rank"], cols["scale"], slot
        any_adapter = bool((nl > 0).any())
        uniform = bool((nl <= 1).all() and (rk[:, 0] <= 64).all())                 # at most one adapter of rank <= 64 per layer
        uniform2 = bool((nl <= 2).all() and (rk[:, :2] <= 64).all() and ((nl < 2) | (sc[:, 0] == sc[:, 1])).all())
        # flags: bit 0 promises at most one adapter per layer of rank <= 64 (the fast path), bit 1 no adapter at all, bit 2
        # at most two adapters of rank <= 64 with one scale per layer (the same kernel, both products in one accumulator)
        self._flags = (1 if uniform else (4 if uniform2 else 0)) | (2 if not any_adapter else 0)
        self._d_table.copy_(self._h_pinned, non_blocking=True)
        self._upload_done = torch.cuda.Event()
        self._upload_done.record(torch.cuda.current_stream(self.device))

    def _tile_maps(self):
        """Device copy of the per-layer tensor maps (they depend only on the weight and pristine pointers)."""
        if self._d_maps is None:
            n = len(self.keys)
            table = (LoraLayer * n)()
            for i, k in enumerate(self.keys):
                w = self.weights[k]
                table[i].W = w.data_ptr()
                table[i].W0 = self.pristine[k].data_ptr() if self.pristine is not None else None
                table[i].out_features, table[i].in_features = w.shape
            host = torch.empty(n * 256, dtype=torch.uint8)
            _lib.check(_lib.load().katz_lora_encode_tile_maps_dtype(table, n, self.code, ctypes.c_void_p(host.data_ptr())),
                       "katz_lora_encode_tile_maps_dtype")
            self._d_maps = host.to(self.device)
        return self._d_maps

    def _launch(self, sign):
        lib = _lib.load()
        # fast paths: fp16 with at most two adapters of rank <= 64 per layer, fp32 with at most one
        fast = bool(self._flags & 1) or (self.dtype == torch.float16 and bool(self._flags & 4))
        maps = self._tile_maps() if fast else None
        flags = self._flags if fast else (self._flags & 2)
        starts, total, mx = ((self.d_tile_start_fast, self.total_tiles_fast, self.max_tiles_per_layer_fast) if fast else
                             (self.d_tile_start, self.total_tiles, self.max_tiles_per_layer))
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(lib.katz_lora_merge(ctypes.c_void_p(self._d_table.data_ptr()), ctypes.c_void_p(starts.data_ptr()),
                                       len(self.keys), total, self.code, float(sign), mx,
                                       flags, ctypes.c_void_p(maps.data_ptr() if maps is not None else None), st),
                   "katz_lora_merge")
        _lib.note_launches(1)
        if self.on_change is not None:
            self.on_change()

    # -- operations ---------------------------------------------------------------------------------------------
    def replay(self):
        """Launch the last merge or restore again from the table already on the device (no host work): what a caller that
        applies the same adapters repeatedly would do, and what the kernel-only timing measures."""
        self._launch(1.0)

    def merge(self, adapters, scales):
        """W_live = W0 + sum_i scale_i * up_i @ down_i (one pass; whatever was merged before is replaced)."""
        adapters = adapters if isinstance(adapters, (list, tuple)) else [adapters]
        scales = scales if isinstance(scales, (list, tuple)) else [scales] * len(adapters)
        self._fill(adapters, scales, use_pristine=True)
        self._launch(1.0)
        self.merged = list(zip(adapters, scales))

    def restore(self):
        """W_live = W0, bit-exact."""
        self._fill([], [], use_pristine=True)
        self._launch(1.0)
        self.merged = []

    def merge_in_place(self, adapters, scales):
        """W_live += sum_i scale_i * up_i @ down_i (no pristine copy involved)."""
        adapters = adapters if isinstance(adapters, (list, tuple)) else [adapters]
        scales = scales if isinstance(scales, (list, tuple)) else [scales] * len(adapters)
        self._fill(adapters, scales, use_pristine=False)
        self._launch(1.0)
        self.merged = self.merged + list(zip(adapters, scales))

    def unmerge_in_place(self, adapters, scales):
        """W_live -= sum_i scale_i * up_i @ down_i: the subtractive unmerge; NOT guaranteed to restore W bit-exactly."""
        adapters = adapters if isinstance(adapters, (list, tuple)) else [adapters]
        scales = scales if isinstance(scales, (list, tuple)) else [scales] * len(adapters)
        self._fill(adapters, scales, use_pristine=False)
        self._launch(-1.0)


def adapter_from_lora_state_dict(lora_state_dict, key_map, device, dtype):
    """Gather (up, down) per UNet key from a LoRA state dict using the reference's key-map format
    (lora_info_shm/*_key_match_unet.json: {unet_key: {"lora_down_key", "lora_up_key"}})."""
    out = OrderedDict()
    for k, m in key_map.items():
        down = lora_state_dict[m["lora_down_key"]].to(device=device, dtype=dtype, non_blocking=True).contiguous()
        up = lora_state_dict[m["lora_up_key"]].to(device=device, dtype=dtype, non_blocking=True).contiguous()
        out[k] = (up, down)
    return out


def synthetic_key_map(keys):
    """A key map in the reference's JSON format for a list of UNet weight keys."""
    km = OrderedDict()
    for k in keys:
        stem = "unet." + k[: -len(".weight")]
        km[k] = {"lora_down_key": stem + ".lora.down.weight", "lora_up_key": stem + ".lora.up.weight"}
    return km


def load_key_map(path):
    with open(path, "r") as fr:
        return json.load(fr, object_pairs_hook=OrderedDict)


def merge_lora_state_dicts(unet, merger, lora_state_dicts, key_maps, scale=REFERENCE_UNET_SCALE):
    """Merge LoRA state dicts (reference key names, gathered through reference-format key maps) into `unet` from the
    pristine weights: the arithmetic of lora_utils.py:29-33 with the dicts and maps passed in instead of read from the
    hub and from ./lora_info_shm. `lora_state_dicts` / `key_maps` may be per-adapter lists. Returns the adapters
    gathered on the device."""
    if not isinstance(lora_state_dicts, (list, tuple)):
        lora_state_dicts, key_maps = [lora_state_dicts], [key_maps]
    adapters = [adapter_from_lora_state_dict(sd, km, merger.device, merger.dtype) for sd, km in zip(lora_state_dicts, key_maps)]
    merger.merge(adapters, [scale] * len(adapters))
    unet.invalidate_caches()
    return adapters
