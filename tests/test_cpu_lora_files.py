"""CPU: LoRA file ingestion — the safetensors container, the kohya/SGM -> diffusers renaming against what the reference's own
conversion produced (tests/golden/kohya_keys.json, written by tests/golden/make_golden.py from
diffusers/loaders/lora_conversion_utils.py), the key-map gather, pinned staging and the shared-memory loader source."""
import json
import os
from collections import OrderedDict

import pytest
import torch

from tests.golden.make_golden import kohya_names, kohya_state_dict


def test_safetensors_round_trip(tmp_path):
    from katz_b200.lora_files import read_safetensors, write_safetensors
    g = torch.Generator().manual_seed(0)
    t = OrderedDict(a=torch.randn(7, 64, generator=g).half(), b=torch.randn(3, generator=g), c=torch.randn(2, 5, generator=g).bfloat16(),
                    d=torch.tensor(8.0), e=torch.arange(6).reshape(2, 3))
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"ss_network_dim": 64})
    back = read_safetensors(p)
    assert list(back) == list(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k]), k
    # the same bytes are readable by the safetensors package where it is installed (the format, not a look-alike)
    try:
        from safetensors.torch import load_file
    except ImportError:
        load_file = None
    if load_file is not None:
        ref = load_file(p)
        for k in t:
            assert torch.equal(ref[k], t[k]), k
    with open(str(tmp_path / "bad.safetensors"), "wb") as fw:
        fw.write(b"\x05\x00\x00\x00\x00\x00\x00\x00nope!")
    from katz_b200 import KatzError
    with pytest.raises(KatzError):
        read_safetensors(str(tmp_path / "bad.safetensors"))


def test_kohya_conversion_matches_the_reference(golden_dir):
    from katz_b200.lora_files import is_kohya, kohya_to_diffusers, lora_state_dict
    with open(os.path.join(golden_dir, "kohya_keys.json")) as fr:
        gold = json.load(fr)
    sd = kohya_state_dict(kohya_names())
    assert is_kohya(sd)
    new_sd, alphas = kohya_to_diffusers(dict(sd), layers_per_block=2)
    by_value = {float(v): k for k, v in sd.items() if not k.endswith(".alpha")}
    mine = {by_value[float(v)]: k for k, v in new_sd.items()}
    assert mine == gold["keys"]
    assert alphas == gold["alphas"]
    # a dict that is already in diffusers naming passes through, with no alphas
    same, none = lora_state_dict(new_sd)
    assert same is new_sd and none is None
    from katz_b200 import KatzError
    bad = dict(sd)
    bad["lora_unet_x.dora_scale"] = torch.ones(1)
    with pytest.raises(KatzError):
        kohya_to_diffusers(bad)


def test_file_to_adapter_through_the_key_map_and_the_shm_source(tmp_path):
    """A kohya-named safetensors file -> diffusers names -> (up, down) per UNet key through a key map in the reference's format
    -> pinned staging; and the same file as the source of a shared-memory loader."""
    from katz_b200.lora import adapter_from_lora_state_dict
    from katz_b200.lora_files import lora_state_dict, shm_source, stage_pinned, write_safetensors
    g = torch.Generator().manual_seed(1)
    mods = {"lora_unet_input_blocks_4_1_transformer_blocks_0_attn1_to_q": (640, 640),
            "lora_unet_input_blocks_4_1_transformer_blocks_0_ff_net_0_proj": (5120, 640),
            "lora_unet_middle_block_1_proj_in": (1280, 1280)}
    sd = OrderedDict()
    for m, (o, n) in mods.items():
        sd[m + ".lora_down.weight"] = torch.randn(8, n, generator=g).half()
        sd[m + ".lora_up.weight"] = torch.randn(o, 8, generator=g).half()
        sd[m + ".alpha"] = torch.tensor(4.0)
    path = str(tmp_path / "adapter.safetensors")
    write_safetensors(path, sd)
    new_sd, alphas = lora_state_dict(path)
    km = {"down_blocks.1.attentions.0.transformer_blocks.0.attn1.to_q.weight":
          {"lora_down_key": "unet.down_blocks.1.attentions.0.transformer_blocks.0.attn1.processor.to_q_lora.down.weight",
           "lora_up_key": "unet.down_blocks.1.attentions.0.transformer_blocks.0.attn1.processor.to_q_lora.up.weight"},
          "down_blocks.1.attentions.0.transformer_blocks.0.ff.net.0.proj.weight":
          {"lora_down_key": "unet.down_blocks.1.attentions.0.transformer_blocks.0.ff.net.0.proj.lora.down.weight",
           "lora_up_key": "unet.down_blocks.1.attentions.0.transformer_blocks.0.ff.net.0.proj.lora.up.weight"},
          "mid_block.attentions.0.proj_in.weight":
          {"lora_down_key": "unet.mid_block.attentions.0.proj_in.lora.down.weight",
           "lora_up_key": "unet.mid_block.attentions.0.proj_in.lora.up.weight"}}
    assert set(alphas.values()) == {4.0} and len(alphas) == 3
    staged = stage_pinned(new_sd)
    ad = adapter_from_lora_state_dict(staged, km, "cpu", torch.float16)
    for (k, (up, down)), (m, (o, n)) in zip(ad.items(), mods.items()):
        assert torch.equal(up, sd[m + ".lora_up.weight"]) and torch.equal(down, sd[m + ".lora_down.weight"]), k
    info = {k: {"shape": list(v.shape), "nbytes": v.numel() * 2} for k, v in new_sd.items()}
    src = shm_source([path], info)
    got = src(1)
    assert set(got) == set(info) and all(got[k].dtype.name == "float16" for k in got)
    from katz_b200 import KatzError
    with pytest.raises(KatzError):
        src(2)


def test_text_encoder_key_maps_equal_the_reference(golden_dir):
    """The text encoders' LoRA key maps (names, order, adapter shapes) against the digest of the reference's own files."""
    import json
    import os
    from katz_b200.params import key_map_digest, text_encoder_lora_key_map
    with open(os.path.join(golden_dir, "text_encoder_key_maps.json")) as fr:
        gold = json.load(fr)
    for which in ("text_encoder", "text_encoder_2"):
        km, shapes = text_encoder_lora_key_map(which)
        assert len(km) == gold[which]["entries"] and list(km)[:6] == gold[which]["order"]
        assert key_map_digest(km, shapes, 64) == gold[which]["digest"]
    assert len(text_encoder_lora_key_map("text_encoder_2", layers=3)[0]) == 18
