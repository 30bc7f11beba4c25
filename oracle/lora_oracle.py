"""TEST INFRASTRUCTURE — CPU oracle of the LoRA merge / restore / unmerge arithmetic.

Restates lora_utils.patch_on_lora's update (lora_utils.py:29-33; same loop in
pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1741-1746), the copy restore (sdxl_unet_server.py:217) and the
vendored subtractive form LoRACompatibleLinear._fuse_lora/_unfuse_lora (diffusers/models/lora.py:403-449).
Pinned by tests/golden/lora_small.npz (outputs of the reference's LoRACompatibleLinear and of the merge formula run
under torch). Only tests/, smoke() and bench.py's CPU baseline import this file.
"""
import torch


def merge_katz(W, up, down, scale):
    """`W += up @ down * scale` in W's dtype (fp16 on the reference's GPU path, fp32 in the CPU configuration):
    product rounded to W.dtype, scaled (rounded), then added (rounded)."""
    scale = torch.as_tensor(scale, dtype=W.dtype)
    out = W.clone()
    out += up @ down * scale
    return out


def merge_set(weights, adapters, scales):
    """Apply adapters in order over a dict of weights: key -> W, adapters: list of {key: (up, down)}."""
    out = {}
    for k, W in weights.items():
        w = W.clone()
        for ad, s in zip(adapters, scales):
            if k in ad:
                up, down = ad[k]
                w = merge_katz(w, up, down, s)
        out[k] = w
    return out


def restore(pristine):
    """load_state_dict(deepcopy(pristine)): a copy."""
    return {k: v.clone() for k, v in pristine.items()}


def fuse_lora_vendored(W, up, down, network_alpha, rank, lora_scale=1.0):
    """LoRACompatibleLinear._fuse_lora (models/lora.py:403-425): fp32 math, result cast back to W's dtype."""
    w_up, w_down = up.float(), down.float()
    if network_alpha is not None:
        w_up = w_up * network_alpha / rank
    fused = W.float() + (lora_scale * torch.bmm(w_up[None, :], w_down[None, :])[0])
    return fused.to(W.dtype)


def unfuse_lora_vendored(Wf, up, down, network_alpha, rank, lora_scale=1.0):
    """LoRACompatibleLinear._unfuse_lora (models/lora.py:427-449)."""
    w_up, w_down = up.float(), down.float()
    if network_alpha is not None:
        w_up = w_up * network_alpha / rank
    un = Wf.float() - (lora_scale * torch.bmm(w_up[None, :], w_down[None, :])[0])
    return un.to(Wf.dtype)
