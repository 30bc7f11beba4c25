"""The reference's LoRA entry points, with the reference's argument lists, over `LoraMerger`.

  * `patch_on_lora(pipe, lora_model_repos)` — lora_utils.patch_on_lora (lora_utils.py:9-33): for every repo, for every
    key of `./lora_info_shm/<repo>_key_match_unet.json`, `unet.state_dict()[key] += up @ down * fp16(20000/64)`, then
    `load_state_dict`: an ADDITIVE merge into whatever the UNet currently holds.
  * `KatzLoraPipelineMixin.patch_on_lora(lora_state_dict, lora_model_repos, default_unet_state_dict)` —
    StableDiffusionXLControlNetPipelineKatz.patch_on_lora (pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1730-1747):
    the key map of `lora_model_repos[0]` only, applied to the PRISTINE dict the caller passes (the adapters of several
    repos arrive pre-summed element-wise in `lora_state_dict`, sdxl_unet_server.py:169-173), then `load_state_dict`.
  * `KatzLoraPipelineMixin.restore_unet()` — `unet.load_state_dict(deepcopy(default_unet_state_dict), strict=False)`
    (sdxl_unet_server.py:217).

What differs, and why: hub files are not reachable, so where the reference calls
`LoraLoaderMixin.lora_state_dict(repo)` the pipe supplies `lora_source(repo) -> (lora_state_dict, network_alphas)`;
the pristine weights stay resident on the device inside the merger, so a `default_unet_state_dict` argument is only
copied in when it is a different dict from the one seen last (and it is never modified, where the reference adds into
it).

The text-encoder part of both reference functions (lora_utils.py:36-54, ...katz.py:1749-1767) is here too:
`state_dict[key] += up @ down` (no scale) over `<repo>_key_match_text_encoder.json` and `..._text_encoder_2.json`, into
whatever `pipe.text_encoder` / `pipe.text_encoder_2` hold — an `nn.Module` whose `state_dict()` tensors are its live
parameters, or a plain dict of CUDA tensors. The reference hard-codes the one repo that ships text-encoder layers; here a
repo takes part when its key-map file exists. As in the reference the text encoders are ADDED into and never restored
by `restore_unet`; `restore_text_encoders()` is there for a caller that wants them back. A pipe without text encoders
skips the part with a note.
"""
import os
from collections import OrderedDict

from .lora import REFERENCE_UNET_SCALE, LoraMerger, adapter_from_lora_state_dict, load_key_map
from .ops import KatzError


def _repo_file(info_dir, repo, suffix):
    return os.path.join(info_dir, "%s%s" % (repo.replace("/", "_"), suffix))


class KatzLoraPipelineMixin:
    """For an object with a `unet` attribute (KatzUNet). `lora_info_dir` holds the reference's key-map files."""

    lora_info_dir = "./lora_info_shm"
    lora_source = None          # callable(repo) -> (lora_state_dict, network_alphas); stands in for the hub download
    _lora_merger = None
    _lora_keys = None
    _pristine_src = None
    _te_mergers = None

    def _text_encoder_weights(self, which, keys):
        te = getattr(self, which, None)
        if te is None:
            return None
        sd = te if isinstance(te, dict) else te.state_dict()
        missing = [k for k in keys if k not in sd]
        if missing:
            raise KatzError("%s has no weight %s (%d of %d keys missing)" % (which, missing[0], len(missing), len(keys)))
        return OrderedDict((k, sd[k]) for k in keys)

    def patch_text_encoders(self, lora_state_dict, repo):
        """`text_encoder[_2].state_dict()[key] += up @ down` for every key of the repo's two text-encoder key maps
        (lora_utils.py:36-54): an additive merge into the live weights, scale 1. Returns the number of layers merged."""
        merged = 0
        for which in ("text_encoder", "text_encoder_2"):
            path = _repo_file(self.lora_info_dir, repo, "_key_match_%s.json" % which)
            if not os.path.exists(path):
                continue
            km = load_key_map(path)
            weights = self._text_encoder_weights(which, list(km))
            if weights is None:
                print("patch_on_lora: no %s on this pipe; its LoRA layers of %s are not applied" % (which, repo))
                continue
            if self._te_mergers is None:
                self._te_mergers = {}
            m = self._te_mergers.get(which)
            if m is None or m.keys != list(km):
                m = self._te_mergers[which] = LoraMerger(weights)
            adapter = adapter_from_lora_state_dict(lora_state_dict, km, m.device, m.dtype)
            if m.merged:
                m.merge_in_place(adapter, 1.0)
            else:
                m.merge(adapter, 1.0)
            merged += len(km)
        return merged

    def restore_text_encoders(self):
        """The text encoders return to the weights they had before the first patch, bit-exactly."""
        for m in (self._te_mergers or {}).values():
            m.restore()

    def lora_key_map(self, repo):
        path = _repo_file(self.lora_info_dir, repo, "_key_match_unet.json")
        if not os.path.exists(path):
            raise KatzError("LoRA key map %s not found (set pipe.lora_info_dir)" % path)
        return load_key_map(path)

    def lora_merger(self, keys):
        """The merger over the UNet linears `keys` (built on first use; it snapshots the pristine weights then)."""
        keys = list(keys)
        if self._lora_merger is None or self._lora_keys != keys:
            if self._lora_merger is not None and self._lora_merger.merged:
                raise KatzError("the LoRA target set changed while adapters are merged; restore first")
            self._lora_merger = LoraMerger(self.unet.lora_targets(keys), on_change=self.unet.invalidate_caches)
            self._lora_keys = keys
            self._pristine_src = None
        return self._lora_merger

    def _adopt_pristine(self, merger, default_unet_state_dict):
        if default_unet_state_dict is None:
            return
        probe = next(iter(merger.keys))
        ident = (id(default_unet_state_dict), default_unet_state_dict[probe].data_ptr())
        if ident == self._pristine_src:
            return
        for k in merger.keys:
            src = default_unet_state_dict[k]
            if tuple(src.shape) != tuple(merger.pristine[k].shape):
                raise KatzError("default_unet_state_dict[%s] has shape %s, the UNet has %s" % (k, tuple(src.shape), tuple(merger.pristine[k].shape)))
            merger.pristine[k].copy_(src, non_blocking=True)
        self._pristine_src = ident

    def patch_on_lora(self, lora_state_dict, lora_model_repos, default_unet_state_dict=None):
        """W = default[key] + up @ down * fp16(20000/64) for every key of the first repo's key map, in one pass."""
        if not isinstance(lora_model_repos, (list, tuple)):
            lora_model_repos = [lora_model_repos]
        km = self.lora_key_map(lora_model_repos[0])
        merger = self.lora_merger(km.keys())
        self._adopt_pristine(merger, default_unet_state_dict)
        adapter = adapter_from_lora_state_dict(lora_state_dict, km, merger.device, merger.dtype)
        merger.merge(adapter, REFERENCE_UNET_SCALE)
        self.unet.invalidate_caches()
        for repo in lora_model_repos:
            self.patch_text_encoders(lora_state_dict, repo)

    def restore_unet(self, default_unet_state_dict=None):
        """The UNet returns to the pristine weights, bit-exactly (one copy pass)."""
        if self._lora_merger is None:
            return
        self._adopt_pristine(self._lora_merger, default_unet_state_dict)
        self._lora_merger.restore()
        self.unet.invalidate_caches()


class KatzPipe(KatzLoraPipelineMixin):
    """The slice of the reference pipeline object this path touches: `pipe.unet`, optional `pipe.controlnet` and
    `pipe.text_encoder` / `pipe.text_encoder_2` (modules or dicts of CUDA weights) for the text-encoder LoRA layers."""

    def __init__(self, unet, controlnet=None, lora_source=None, lora_info_dir=None, text_encoder=None, text_encoder_2=None):
        self.unet, self.controlnet = unet, controlnet
        self.text_encoder, self.text_encoder_2 = text_encoder, text_encoder_2
        self.lora_source = lora_source
        if lora_info_dir is not None:
            self.lora_info_dir = lora_info_dir


def patch_on_lora(pipe, lora_model_repos):
    """lora_utils.patch_on_lora (lora_utils.py:9-33): every repo's `up @ down * scale` is ADDED to the UNet's current
    weights. When nothing is merged yet the sum over the repos is one pass from the pristine copy; otherwise the pass
    adds in place, as the reference's `unet_state_dict[key] += ...` does."""
    if not isinstance(lora_model_repos, list):
        lora_model_repos = [lora_model_repos]
    if not lora_model_repos:
        return
    if getattr(pipe, "lora_source", None) is None:
        raise KatzError("patch_on_lora needs pipe.lora_source(repo) -> (lora_state_dict, network_alphas): the hub is not "
                        "reachable from here")
    key_maps = [pipe.lora_key_map(r) for r in lora_model_repos]
    keys = list(OrderedDict((k, None) for km in key_maps for k in km))
    merger = pipe.lora_merger(keys)
    adapters, dicts = [], []
    for repo, km in zip(lora_model_repos, key_maps):
        lora_state_dict, _network_alphas = pipe.lora_source(repo)
        dicts.append(lora_state_dict)
        adapters.append(adapter_from_lora_state_dict(lora_state_dict, km, merger.device, merger.dtype))
    scales = [REFERENCE_UNET_SCALE] * len(adapters)
    if merger.merged:
        merger.merge_in_place(adapters, scales)
    else:
        merger.merge(adapters, scales)
    pipe.unet.invalidate_caches()
    for repo, lora_state_dict in zip(lora_model_repos, dicts):
        pipe.patch_text_encoders(lora_state_dict, repo)
