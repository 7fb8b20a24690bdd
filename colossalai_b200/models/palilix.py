"""Palilix: a decoder of PARALLEL layers - one layer norm (weight, no bias) in front of a token mixer and a feed-forward
that both read its output, their sum added to an fp32 residual stream - whose mixers are latent attention (keys / values
rebuilt from a small cached latent plus one rotated key part shared by all heads) or retention (decayed outer-product
memory with rotary positions), in any order; feed-forwards are dense (tanh-GELU) or routed (clamped gated experts, softmax
router, optional shared expert) or absent.  A span of layers may run several times in a row with the same weights; every
pass has caches / states of its own and starts by adding the embedding output (not the first pass) and a learned vector.
Logits are scaled and soft-capped with a tanh.

The model is the generic backbone (`transformer.py`) configured by `ModelConfig.layer_specs`; this module only reads the
family's `config.json` / tensor names.  A checkpoint is `config.json` + `model.safetensors` with

    embed, head, final.norm, loop.step, l<i>.norm1, l<i>.mix.<name>, l<i>.mlp.{up,down} or
    l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down}}
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .config import ExpertFFSpec, LayerSpec, MixerSpec, ModelConfig
from .transformer import TransformerLMHeadModel

__all__ = ["PalilixForCausalLM", "palilix_config", "convert_palilix_state_dict", "load_palilix"]


class PalilixForCausalLM(TransformerLMHeadModel):
    pass


def palilix_config(hf: dict) -> ModelConfig:
    specs = []
    for i, ly in enumerate(hf["layers"]):
        m, kind = ly["mixer"], ly["type"]
        rot = m.get("rot") or {}
        if kind == "latent_attention":
            mixer = MixerSpec(kind="latent", heads=m["heads"], kv_heads=1, dim=m["dim"], vdim=m["vdim"],
                              kv_rank=m["kv_rank"], rot_dim=m["rot_dim"], rot_dims=rot.get("dims", m["rot_dim"]),
                              rot_base=float(rot.get("base", 10000.0)), scale=m.get("scale"))
        elif kind == "retention":
            mixer = MixerSpec(kind="retention", heads=m["heads"], dim=m["dim"], vdim=m.get("vdim", m["dim"]),
                              decay=[float(d) for d in m["decay"]], rot_dims=rot.get("dims", 0),
                              rot_base=float(rot.get("base", 10000.0)))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = ly.get("mlp")
        if mlp is None:
            specs.append(LayerSpec(mixer=mixer))
        elif mlp.get("kind", "dense") == "dense":
            specs.append(LayerSpec(mixer=mixer, ff=mlp["ff"]))
        elif mlp["kind"] == "moe":
            sh = mlp.get("shared") or {}
            specs.append(LayerSpec(mixer=mixer, moe=ExpertFFSpec(
                experts=mlp["router"]["experts"], top=mlp["router"]["top"], ff=mlp["expert"]["ff"],
                limit=float(mlp["expert"]["limit"]), shared_ff=sh.get("ff", 0),
                shared_limit=float(sh.get("limit", mlp["expert"]["limit"])))))
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    ffs = [s.ff for s in specs if s.ff is not None]
    loop = hf.get("loop") or {}
    return ModelConfig(model_type="palilix", vocab_size=hf["vocab"], hidden_size=hf["width"],
                       intermediate_size=max(ffs) if ffs else hf["width"], layer_specs=specs,
                       norm_eps=hf["norm"]["eps"], norm_type="layer", norm_bias=False, hidden_act="gelu_tanh", glu=False,
                       pos_type="none", parallel_block=True, fp32_residual=True,
                       embed_scale=hf.get("embedding", {}).get("scale", 1.0), logit_scale=hf.get("logit_scale", 1.0),
                       logit_softcap=hf.get("logit_softcap"), loop_start=loop.get("start", 0),
                       loop_stop=loop.get("stop", 0), loop_times=loop.get("times", 1),
                       tie_word_embeddings=False, max_position_embeddings=1 << 20)


def _gated(sd: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return torch.cat([sd[prefix + "gate"], sd[prefix + "up"]], 0)


def convert_palilix_state_dict(sd: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names -> backbone parameter names; projections that read the same input are stacked into one GEMM,
    the experts of a layer into batched tensors, the per-head up-projections of latent attention into [heads, ., rank]."""
    out = {"model.embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "model.norm.weight": sd["final.norm"]}
    if cfg.looped:
        out["model.loop_step"] = sd["loop.step"]
    for i, spec in enumerate(cfg.layer_specs):
        src, dst = f"l{i}.", f"model.layers.{i}."
        out[dst + "input_layernorm.weight"] = sd[src + "norm1"]
        if spec.ff is not None:
            out[dst + "mlp.up_proj.weight"] = sd[src + "mlp.up"]
            out[dst + "mlp.down_proj.weight"] = sd[src + "mlp.down"]
        elif spec.moe is not None:
            p = src + "mlp."
            out[dst + "mlp.router.weight"] = sd[p + "router"]
            out[dst + "mlp.experts.w_up"] = torch.stack([_gated(sd, f"{p}e{e}.") for e in range(spec.moe.experts)])
            out[dst + "mlp.experts.w_down"] = torch.stack([sd[f"{p}e{e}.down"] for e in range(spec.moe.experts)])
            if spec.moe.shared_ff:
                out[dst + "mlp.shared.gate_up_proj.weight"] = _gated(sd, p + "shared.")
                out[dst + "mlp.shared.down_proj.weight"] = sd[p + "shared.down"]
        m, a, mx = src + "mix.", dst + "self_attn.", spec.mixer
        if mx.kind == "latent":
            out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "dkv"]], 0)
            out[a + "dkv_norm_weight"] = sd[m + "dkv.norm"]
            out[a + "uk"] = sd[m + "uk"].reshape(mx.heads, mx.dim, mx.kv_rank)
            out[a + "uv"] = sd[m + "uv"].reshape(mx.heads, mx.vdim, mx.kv_rank)
        else:
            out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"]], 0)
        out[a + "o_proj.weight"] = sd[m + "o"]
    return out


def load_palilix(path: str, hf_cfg: dict, dtype: torch.dtype, device: str = "cpu") -> PalilixForCausalLM:
    from safetensors.torch import load_file

    cfg = palilix_config(hf_cfg)
    model = PalilixForCausalLM(cfg)
    sd = convert_palilix_state_dict(load_file(os.path.join(path, "model.safetensors")), cfg)
    missing, unexpected = model.load_state_dict({k: v.to(torch.float32) for k, v in sd.items()}, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"palilix checkpoint does not fit the model: missing={missing[:6]} unexpected={unexpected[:6]}")
    model._pretrained_path = path
    return model.to(dtype).to(device)
