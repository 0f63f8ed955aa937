"""Zesapel as a ``ModelSpec`` of parts.

Scaled token embedding plus a learned position vector; S residual streams joined
to every sublayer by hyper-connections; per layer one of three mixers (a
state-space scan, attention through a cached latent with a sliding window and a
sink, a delta-rule recurrence) behind a causal convolution over the mixer's
input, and a mixture of experts chosen by a table of token ids; an RMS norm and
an output matrix of its own.  Tensor names are the checkpoint's own: ``embed``,
``pos``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc<q>.*``,
``l<i>.canon1``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zesapel import ZesapelConfig
from ..parts.base import PartSpec
from ..parts.model import ModelSpec
from ..registry import register_architecture

_NAMES = {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp.", "hc1": "hc1.", "hc2": "hc2.",
          "input_conv": "canon1"}


def _mixer(cfg: ZesapelConfig, layer: dict) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "mamba2":
        return PartSpec("mamba2", {"hidden_size": cfg.width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                                   "groups": m["groups"], "conv_taps": m["conv"], "norm_groups": m["norm_groups"],
                                   "eps": cfg.norm_eps})
    if kind == "latent_attention":
        rot = m["rot"]
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "eps": cfg.norm_eps, "rope_base": rot["base"],
            "rope_dims": rot.get("dims", m["rot_dim"]), "window": (m.get("mask") or {}).get("size"),
            "scale": m.get("scale")})
    return PartSpec("general_delta", {"hidden_size": cfg.width, "heads": m["heads"], "dim": m["dim"],
                                      "eps": cfg.norm_eps})


def build_spec(cfg: ZesapelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "param": ""})
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            ffn = PartSpec("table_experts", {"hidden_size": cfg.width, "num_experts": mlp["router"]["experts"],
                                             "top": mlp["router"]["top"], "expert_size": mlp["expert"]["ff"],
                                             "vocab_size": cfg.vocab, "activation": "gelu"})
        layers.append(PartSpec("hyper_connections", {
            "hidden_size": cfg.width, "streams": cfg.streams, "norm1": norm, "mixer": _mixer(cfg, layer),
            "norm2": norm if ffn is not None else None, "ffn": ffn, "input_taps": cfg.canon_taps, "names": _NAMES}))
        prefixes.append(f"l{i}.")
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, layer_prefixes=prefixes,
                     final_norm=norm, final_norm_prefix="final.norm", embed_name="embed", lm_head_name="head",
                     embed_position=PartSpec("learned", {"max_positions": cfg.max_positions, "hidden_size": cfg.width,
                                                         "param": "pos"}),
                     embed_scale=cfg.embedding_scale, residual_streams=cfg.streams)


register_architecture(ZesapelConfig.architecture, ZesapelConfig, build_spec, model_type=ZesapelConfig.model_type)
