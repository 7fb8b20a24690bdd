"""Gopunex: a hybrid decoder whose layers mix tokens by softmax attention with a distance-bucket bias and a sink, by
lightning (decayed linear) attention, or by a channel-wise gated delta rule, in any order; every sublayer's OUTPUT is
RMS-normalised with zero-centred weights (the norm multiplies by 1 + w), scaled and added to an fp32 residual stream;
dense feed-forwards use the squared ReLU.

The model is the generic backbone (`transformer.py`) configured by `ModelConfig.layer_specs`; this module only reads the
family's `config.json` / tensor names.  A checkpoint is `config.json` + `model.safetensors` with

    embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mlp.{up,down}, l<i>.mix.<name>

Sizes that the config does not spell out (rows of the distance table, the bottleneck ranks of the delta-rule layer) are
taken from the tensors' shapes.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Optional, Tuple

import torch

from .config import LayerSpec, MixerSpec, ModelConfig
from .transformer import TransformerLMHeadModel

__all__ = ["GopunexForCausalLM", "gopunex_config", "convert_gopunex_state_dict", "read_safetensors_shapes"]


class GopunexForCausalLM(TransformerLMHeadModel):
    pass


def read_safetensors_shapes(path: str) -> Dict[str, Tuple[int, ...]]:
    """name -> shape from the header of a safetensors file (8-byte little-endian length, then JSON)."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        hdr = json.loads(f.read(n))
    return {k: tuple(v["shape"]) for k, v in hdr.items() if k != "__metadata__"}


def gopunex_config(hf: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelConfig:
    shapes = shapes or {}
    specs = []
    for i, ly in enumerate(hf["layers"]):
        m, kind = ly["mixer"], ly["type"]
        pre = f"l{i}.mix."
        if kind == "attention":
            mixer = MixerSpec(kind="attention", heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), dim=m["dim"],
                              vdim=m.get("vdim", m["dim"]), bias=True, scale=m["scale"],
                              bias_buckets=shapes.get(pre + "rel", (m.get("bias_buckets", 0),))[0],
                              bias_max=float(m.get("bias_max", 0)), sink=True, proj_norm=True,
                              v_mix=bool(m.get("v_mix", False)))
        elif kind == "lightning":
            mixer = MixerSpec(kind="lightning", heads=m["heads"], dim=m["dim"], vdim=m.get("vdim", m["dim"]),
                              decay=[float(d) for d in m["decay"]])
        elif kind == "channel_delta":
            mixer = MixerSpec(kind="channel_delta", heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]),
                              dim=m["dim"], vdim=m.get("vdim", m["dim"]), conv=m["conv"],
                              decay_rank=shapes.get(pre + "a1", (m.get("decay_rank", 0),))[0],
                              gate_rank=shapes.get(pre + "g1", (m.get("gate_rank", 0),))[0])
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = ly.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        specs.append(LayerSpec(mixer=mixer, ff=None if mlp is None else mlp["ff"]))
    ffs = [s.ff for s in specs if s.ff is not None]
    return ModelConfig(model_type="gopunex", vocab_size=hf["vocab"], hidden_size=hf["width"],
                       intermediate_size=max(ffs) if ffs else hf["width"], layer_specs=specs,
                       norm_eps=hf["norm"]["eps"], norm_type="rms", hidden_act="relu2", glu=False, pos_type="none",
                       embed_scale=hf.get("embedding", {}).get("scale", 1.0), norm_placement="sublayer_out",
                       residual_mult=hf.get("residual_mult", 1.0), norm_weight_offset=1.0, fp32_residual=True,
                       tie_word_embeddings=False, max_position_embeddings=1 << 20)


def convert_gopunex_state_dict(sd: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names -> backbone parameter names; projections that read the same input are stacked into one GEMM."""
    out = {"model.embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "model.norm.weight": sd["final.norm"]}
    for i, spec in enumerate(cfg.layer_specs):
        src, dst = f"l{i}.", f"model.layers.{i}."
        out[dst + "input_layernorm.weight"] = sd[src + "norm1"]
        if spec.ff is not None:
            out[dst + "post_attention_layernorm.weight"] = sd[src + "norm2"]
            out[dst + "mlp.up_proj.weight"] = sd[src + "mlp.up"]
            out[dst + "mlp.down_proj.weight"] = sd[src + "mlp.down"]
        m, a = src + "mix.", dst + "self_attn."
        kind = spec.mixer.kind
        if kind == "attention":
            out[a + "qkv_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"]], 0)
            out[a + "qkv_proj.bias"] = torch.cat([sd[m + "q.b"], sd[m + "k.b"], sd[m + "v.b"]], 0)
            out[a + "q_norm_weight"] = sd[m + "q.norm"]
            out[a + "k_norm_weight"] = sd[m + "k.norm"]
            out[a + "rel_bias"] = sd[m + "rel"]
            if spec.mixer.v_mix:
                out[a + "v_mix"] = sd[m + "vmix"]
        elif kind == "lightning":
            out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"]], 0)
            out[a + "norm_weight"] = sd[m + "norm"]
        else:
            out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "b"], sd[m + "a1"],
                                                   sd[m + "g1"]], 0)
            out[a + "conv_weight"] = torch.cat([sd[m + "q.conv"], sd[m + "k.conv"], sd[m + "v.conv"]], 0)
            out[a + "decay_up.weight"] = sd[m + "a2"]
            out[a + "gate_up.weight"] = sd[m + "g2"]
            out[a + "A_log"] = sd[m + "A_log"]
            out[a + "dt_bias"] = sd[m + "dt_bias"]
            out[a + "norm_weight"] = sd[m + "norm"]
        out[a + "o_proj.weight"] = sd[m + "o"]
    return out


def load_gopunex(path: str, hf_cfg: dict, dtype: torch.dtype, device: str = "cpu") -> GopunexForCausalLM:
    from safetensors.torch import load_file

    st = os.path.join(path, "model.safetensors")
    cfg = gopunex_config(hf_cfg, read_safetensors_shapes(st))
    model = GopunexForCausalLM(cfg)
    sd = convert_gopunex_state_dict(load_file(st), cfg)
    missing, unexpected = model.load_state_dict({k: v.to(torch.float32) for k, v in sd.items()}, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"gopunex checkpoint does not fit the model: missing={missing[:6]} unexpected={unexpected[:6]}")
    model._pretrained_path = path
    return model.to(dtype).to(device)
