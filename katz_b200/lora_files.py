"""LoRA files -> the (up, down) tensors the merge consumes: the ingestion side of the LoRA path.

Stands where the reference calls `LoraLoaderMixin.lora_state_dict(repo, unet_config=...)`
(diffusers/loaders/lora.py:146-307; callers lora_utils.py:16, load_lora_shm_multi.py:115) and its kohya/SGM key
conversion (diffusers/loaders/lora_conversion_utils.py:23-287):

  * `read_safetensors` — the safetensors container read directly (8-byte little-endian header length, JSON header with
    dtype / shape / byte offsets per tensor, raw little-endian data) through a memory map, so nothing is copied until a
    tensor is staged;
  * `lora_state_dict(path_or_dict, layers_per_block)` — returns `(state_dict, network_alphas)` with the key names the
    reference's key-map files (lora_info_shm/<repo>_key_match_unet.json) refer to: kohya names (`lora_unet_...`,
    `lora_te1_...`, `lora_te2_...`, SGM block numbering included) are renamed, alphas are collected;
  * `stage_pinned` / `to_device_async` — one pinned host buffer per adapter and one asynchronous copy per tensor on a
    side stream, so the 340 MB of an adapter cross PCIe while the first denoise steps run (the reference overlaps the
    same way with loader processes and shared memory, pipeline_controlnet_sd_xl_katz.py:1522-1558);
  * `shm_source(paths, infos)` — the `source(code)` callable of lora_shm.LoraShmLoader: request code n loads file n.

Hub download, `.bin` pickles and DoRA checkpoints are not handled (a DoRA file raises).
"""
import json
import re
import struct
from collections import OrderedDict

import numpy as np
import torch

from ._lib import KatzError

_ST_DTYPES = {"F16": (np.float16, torch.float16), "F32": (np.float32, torch.float32), "F64": (np.float64, torch.float64),
              "BF16": (np.int16, torch.bfloat16), "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
              "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8), "BOOL": (np.bool_, torch.bool)}
_ST_NAMES = {torch.float16: "F16", torch.float32: "F32", torch.float64: "F64", torch.bfloat16: "BF16", torch.int64: "I64",
             torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}


def read_safetensors(path):
    """OrderedDict name -> CPU tensor viewing the memory-mapped file (read-only storage: clone or stage before writing)."""
    with open(path, "rb") as fr:
        head = fr.read(8)
        if len(head) != 8:
            raise KatzError("%s is not a safetensors file (too short)" % path)
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or n > (1 << 30):
            raise KatzError("%s: implausible safetensors header length %d" % (path, n))
        try:
            header = json.loads(fr.read(n).decode("utf-8"), object_pairs_hook=OrderedDict)
        except (UnicodeDecodeError, ValueError) as e:
            raise KatzError("%s: bad safetensors header (%s)" % (path, e))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + n)
    out = OrderedDict()
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _ST_DTYPES:
            raise KatzError("%s: tensor %s has unsupported dtype %s" % (path, name, meta["dtype"]))
        npdt, tdt = _ST_DTYPES[meta["dtype"]]
        b0, b1 = meta["data_offsets"]
        shape = tuple(int(s) for s in meta["shape"])
        count = int(np.prod(shape)) if shape else 1
        if b1 - b0 != count * np.dtype(npdt).itemsize or b1 > data.shape[0]:
            raise KatzError("%s: tensor %s has inconsistent offsets" % (path, name))
        arr = np.frombuffer(data, dtype=npdt, count=count, offset=b0).reshape(shape)
        with _quiet_non_writable():
            t = torch.from_numpy(arr)
        out[name] = t.view(tdt) if meta["dtype"] == "BF16" else t
    return out


class _quiet_non_writable:
    """torch warns that a read-only numpy array becomes a writable-looking tensor; the tensors are documented read-only."""

    def __enter__(self):
        import warnings
        self._cm = warnings.catch_warnings()
        self._cm.__enter__()
        warnings.simplefilter("ignore")

    def __exit__(self, *a):
        return self._cm.__exit__(*a)


def write_safetensors(path, tensors, metadata=None):
    """The inverse of read_safetensors (fixtures, tests, converted adapters)."""
    header, blobs, off = OrderedDict(), [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _ST_NAMES:
            raise KatzError("cannot store dtype %s" % t.dtype)
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as fw:
        fw.write(struct.pack("<Q", len(hb)))
        fw.write(hb)
        for b in blobs:
            fw.write(b)


# ------------------------------------------------------------------------------------------- kohya -> diffusers ----
_KOHYA_PREFIXES = ("lora_unet_", "lora_te_", "lora_te1_", "lora_te2_")

# compound words of the module paths whose inner underscores survive the underscore -> dot split, longest first
_UNET_WORDS = ("transformer_blocks", "down_blocks", "up_blocks", "mid_block", "time_emb_proj", "conv_shortcut", "proj_in",
               "proj_out", "to_q", "to_k", "to_v", "to_out", "time_embedding", "add_embedding", "linear_1", "linear_2",
               "conv_in", "conv_out", "conv_norm_out")
_TE_WORDS = ("text_model", "self_attn", "q_proj", "k_proj", "v_proj", "out_proj", "layer_norm1", "layer_norm2",
             "final_layer_norm", "token_embedding", "position_embedding")


def _split_words(name, words):
    """'a_b_c' -> ['a', 'b', 'c'] with the listed compounds kept whole."""
    toks = name.split("_")
    out, i = [], 0
    while i < len(toks):
        for w in words:
            parts = w.split("_")
            if toks[i:i + len(parts)] == parts:
                out.append(w)
                i += len(parts)
                break
        else:
            out.append(toks[i])
            i += 1
    return out


def _sgm_to_diffusers_blocks(toks, layers_per_block):
    """SGM numbering (input_blocks.N.M / middle_block.M / output_blocks.N.M) -> diffusers block paths, as
    lora_conversion_utils.py:23-121 derives them: input block N sits in down block (N-1) // (layers+1) at position
    (N-1) % (layers+1); M selects resnets / attentions (or the downsampler `op`); output block N sits in up block
    N // (layers+1); the middle block is resnet 0, attention 0, resnet 1."""
    per = layers_per_block + 1
    kinds = ("resnets", "attentions", "upsamplers")
    if toks[:2] == ["input", "blocks"]:
        n, m = int(toks[2]), int(toks[3])
        rest = toks[4:]
        if rest and rest[0] == "op":
            return ["down_blocks", str((n - 1) // per), "downsamplers", "0", "conv"] + rest[1:]
        return ["down_blocks", str((n - 1) // per), kinds[m], str((n - 1) % per)] + rest
    if toks[:2] == ["middle", "block"]:
        m = int(toks[2])
        if m > 2:
            raise KatzError("invalid middle block index %d" % m)
        return ["mid_block"] + [["resnets", "0"], ["attentions", "0"], ["resnets", "1"]][m] + toks[3:]
    if toks[:2] == ["output", "blocks"]:
        n, m = int(toks[2]), int(toks[3])
        rest = toks[4:]
        if m >= 2 or (rest and rest[0] == "conv"):
            return ["up_blocks", str(n // per), "upsamplers", "0"] + rest
        return ["up_blocks", str(n // per), kinds[m], str(n % per)] + rest
    return toks


_SGM_RESNET = (("in_layers_2", "conv1"), ("out_layers_3", "conv2"), ("emb_layers_1", "time_emb_proj"), ("skip_connection", "conv_shortcut"))


def _unet_module_path(lora_name, layers_per_block):
    """'lora_unet_input_blocks_4_1_transformer_blocks_0_attn1_to_q' -> 'down_blocks.1.attentions.0.transformer_blocks.0.attn1.to_q'."""
    body = lora_name[len("lora_unet_"):]
    for sgm, dif in _SGM_RESNET:
        body = re.sub(r"(?<=_)%s$" % sgm, dif.replace("_", "\0"), body)
    toks = _split_words(body, _UNET_WORDS)
    toks = _sgm_to_diffusers_blocks(toks, layers_per_block)
    return ".".join(t.replace("\0", "_") for t in toks)


def _lora_leaf(path):
    """The reference's leaf spelling: attention projections carry the processor form (`attn1.processor.to_q_lora`, `to_out.0`
    becomes `to_out_lora`), everything else is `<module>.lora`."""
    m = re.match(r"^(.*\.attn[12])\.(to_q|to_k|to_v)$", path)
    if m:
        return "%s.processor.%s_lora" % (m.group(1), m.group(2))
    m = re.match(r"^(.*\.attn[12])\.to_out\.0$", path)
    if m:
        return "%s.processor.to_out_lora" % m.group(1)
    return path + ".lora"


def _te_module_path(body):
    toks = _split_words(body, _TE_WORDS)
    path = ".".join(toks)
    m = re.match(r"^(.*\.self_attn)\.(q|k|v|out)_proj$", path)
    if m:
        return "%s.to_%s_lora" % (m.group(1), m.group(2))
    if ".mlp." in path:
        return path + ".lora_linear_layer"
    return path + ".lora"


def kohya_to_diffusers(state_dict, layers_per_block=2):
    """kohya-ss LoRA names -> the names `LoraLoaderMixin.lora_state_dict` returns (lora_conversion_utils.py:124-287), plus
    the alphas as {"<prefix>.<module>.alpha": float}. Tensors are passed through untouched."""
    if any("dora_scale" in k for k in state_dict):
        raise KatzError("DoRA checkpoints are not supported")
    out, alphas = OrderedDict(), OrderedDict()
    names = OrderedDict((k.split(".")[0], None) for k in state_dict if k.endswith(".lora_down.weight"))
    used = set()
    for lora_name in names:
        down_k, up_k, alpha_k = lora_name + ".lora_down.weight", lora_name + ".lora_up.weight", lora_name + ".alpha"
        if up_k not in state_dict:
            raise KatzError("%s has no matching lora_up weight" % down_k)
        if lora_name.startswith("lora_unet_"):
            prefix, leaf = "unet", _lora_leaf(_unet_module_path(lora_name, layers_per_block))
        elif lora_name.startswith(("lora_te_", "lora_te1_")):
            cut = len("lora_te_") if lora_name.startswith("lora_te_") else len("lora_te1_")
            prefix, leaf = "text_encoder", _te_module_path(lora_name[cut:])
        elif lora_name.startswith("lora_te2_"):
            prefix, leaf = "text_encoder_2", _te_module_path(lora_name[len("lora_te2_"):])
        else:
            raise KatzError("unknown kohya prefix in %s" % lora_name)
        out["%s.%s.down.weight" % (prefix, leaf)] = state_dict[down_k]
        out["%s.%s.up.weight" % (prefix, leaf)] = state_dict[up_k]
        used.update((down_k, up_k))
        if alpha_k in state_dict:
            a = state_dict[alpha_k]
            # the reference names the alpha after the text before ".lora." of the leaf (processor leaves have none: the
            # whole down-weight name is kept)
            full = "%s.down.weight" % leaf
            alphas["%s.%s.alpha" % (prefix, full.split(".lora.")[0])] = float(a.item() if torch.is_tensor(a) else a)
            used.add(alpha_k)
    left = [k for k in state_dict if k not in used]
    if left:
        raise KatzError("keys that are not kohya LoRA entries: %s ..." % left[:3])
    return out, alphas


def is_kohya(state_dict):
    return len(state_dict) > 0 and all(k.startswith(_KOHYA_PREFIXES) for k in state_dict)


def lora_state_dict(path_or_dict, layers_per_block=2):
    """`LoraLoaderMixin.lora_state_dict` for a local safetensors file or an in-memory dict: returns
    (state_dict in diffusers naming, network_alphas or None)."""
    sd = read_safetensors(path_or_dict) if isinstance(path_or_dict, (str, bytes)) or hasattr(path_or_dict, "__fspath__") else path_or_dict
    if is_kohya(sd):
        return kohya_to_diffusers(sd, layers_per_block)
    return sd, None


# ------------------------------------------------------------------------------------------------- staging ----------
def stage_pinned(state_dict, dtype=torch.float16, keys=None):
    """Copy the tensors (all, or `keys`) into ONE pinned host buffer, converted to `dtype`, 256-byte aligned each.
    Returns OrderedDict name -> pinned tensor view. This is the only host copy of the adapter's bytes."""
    keys = list(state_dict.keys() if keys is None else keys)
    es = torch.empty((), dtype=dtype).element_size()
    offs, total = [], 0
    for k in keys:
        offs.append(total)
        total += (state_dict[k].numel() * es + 255) // 256 * 256
    buf = torch.empty(max(total, 256), dtype=torch.uint8)
    if torch.cuda.is_available():
        buf = buf.pin_memory()
    out = OrderedDict()
    for k, o in zip(keys, offs):
        src = state_dict[k]
        dst = buf[o:o + src.numel() * es].view(dtype).view(src.shape)
        dst.copy_(src)
        out[k] = dst
    out_buf = buf          # keep the backing buffer alive with the views
    for v in out.values():
        v._katz_backing = out_buf
    return out


def to_device_async(staged, device, stream=None):
    """Asynchronous host -> device copies of a staged adapter on `stream` (a side stream by default). Returns
    (OrderedDict name -> device tensor, event): make the consuming stream wait for the event before the merge."""
    device = torch.device(device)
    stream = stream or torch.cuda.Stream(device=device)
    out = OrderedDict()
    with torch.cuda.stream(stream):
        for k, v in staged.items():
            out[k] = v.to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(stream)
    return out, ev


def shm_source(paths, info, layers_per_block=2):
    """`source(code)` for lora_shm.LoraShmLoader: request code n (1..9) loads paths[n-1] and returns {key: fp16 array} for the
    keys of the loader's info file (lora_info_shm/<repo>.json), as load_lora_shm_multi.py:115-118 fills its segments."""
    def source(code):
        if not 1 <= int(code) <= len(paths):
            raise KatzError("no LoRA file for request code %d" % code)
        sd, _ = lora_state_dict(paths[int(code) - 1], layers_per_block)
        out = OrderedDict()
        for k, meta in info.items():
            if k not in sd:
                raise KatzError("%s has no tensor %s" % (paths[int(code) - 1], k))
            t = sd[k]
            if tuple(t.shape) != tuple(meta["shape"]):
                raise KatzError("%s: %s has shape %s, the info file says %s" % (paths[int(code) - 1], k, tuple(t.shape), meta["shape"]))
            out[k] = t.to(torch.float16).numpy()
        return out
    return source
