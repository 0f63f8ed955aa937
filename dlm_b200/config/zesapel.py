"""Typed configuration of the Zesapel decoder.

``config.json`` of this design is nested: ``layers`` is a list with one entry per
layer, each naming its mixer (``type``), the mixer's sizes (``mixer``) and its
feed-forward (``mlp``, or null for none); the model-wide sizes and constants are
``vocab``, ``width``, ``streams``, ``max_positions``, ``embedding.scale``,
``norm.eps`` and ``canon.taps``.  Every size and constant is read from here (or
from a tensor's shape); the class checks what each mixer kind needs and keeps the
layer entries as they were written, so that ``to_dict`` gives the file back.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, as_float, as_int

MIXER_KEYS = {
    "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"),
    "general_delta": ("heads", "dim"),
}


def _section(raw: dict, key: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json lacks the section {key!r}")
    return v


@dataclass
class ZesapelConfig:
    vocab: int
    width: int
    layers: list[dict[str, Any]]
    streams: int = 1
    max_positions: int = 2048
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    canon_taps: int | None = None
    eos_token_ids: list[int] = field(default_factory=list)

    architecture = "Zesapel"
    model_type = "zesapel"

    # what the engine and the command line ask of any config
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, raw: dict) -> "ZesapelConfig":
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("config.json lacks 'layers' (a list with one entry per layer)")
        for key in ("vocab", "width"):
            if key not in raw:
                raise ConfigError(f"config.json lacks required key {key!r}")
        cfg = cls(vocab=as_int(raw["vocab"], "vocab", minimum=1), width=as_int(raw["width"], "width", minimum=1),
                  layers=copy.deepcopy(raw["layers"]),
                  streams=as_int(raw.get("streams", 1), "streams", minimum=1),
                  max_positions=as_int(raw.get("max_positions", 2048), "max_positions", minimum=1),
                  embedding_scale=as_float(raw.get("embedding", {}).get("scale", 1.0), "embedding.scale"),
                  norm_eps=as_float(_section(raw, "norm").get("eps", 1e-5), "norm.eps"),
                  canon_taps=(as_int(raw["canon"]["taps"], "canon.taps", minimum=1)
                              if isinstance(raw.get("canon"), dict) and raw["canon"].get("taps") else None))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.streams > 16:
            raise ConfigError("at most 16 residual streams")
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_KEYS:
                raise ConfigError(f"layer {i}: 'type' must be one of {sorted(MIXER_KEYS)}, got {layer.get('type')!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"layer {i}: lacks 'mixer'")
            for key in MIXER_KEYS[layer["type"]]:
                as_int(m.get(key), f"layers[{i}].mixer.{key}", minimum=1)
            if layer["type"] == "mamba2" and m["heads"] % m["groups"]:
                raise ConfigError(f"layer {i}: heads must be a multiple of groups")
            if layer["type"] == "latent_attention":
                rot = m.get("rot")
                if not isinstance(rot, dict) or "base" not in rot:
                    raise ConfigError(f"layer {i}: latent_attention needs 'rot' with 'base'")
                dims = as_int(rot.get("dims", m["rot_dim"]), f"layers[{i}].mixer.rot.dims", minimum=0)
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"layer {i}: rot.dims must be even and at most rot_dim")
                if m.get("mask") is not None:
                    as_int(_section(m, "mask").get("size"), f"layers[{i}].mixer.mask.size", minimum=1)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"layer {i}: 'mlp' must be null or of kind 'moe'")
                E = as_int(_section(mlp, "router").get("experts"), f"layers[{i}].mlp.router.experts", minimum=1)
                top = as_int(mlp["router"].get("top"), f"layers[{i}].mlp.router.top", minimum=1)
                if top > E:
                    raise ConfigError(f"layer {i}: top {top} exceeds experts {E}")
                as_int(_section(mlp, "expert").get("ff"), f"layers[{i}].mlp.expert.ff", minimum=1)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
               "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        return out
