"""Typed configuration of the Zasazen decoder.

``config.json`` of this design is nested: ``layers`` is a list with one entry per layer, each naming its mixer
(``type``: ``mamba1`` or ``parallel``), the mixer's sizes (``mixer``; a ``parallel`` mixer has the sections ``left``,
softmax attention, and ``right``, retention) and its feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for
none).  ``loop`` (optional) names a run of layers ``start .. stop - 1`` that is repeated ``times`` times with the same
weights.  Model-wide: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``.  Every size and constant is read from
here (or from a tensor's shape); the class checks what each kind needs and keeps the layer entries as they were
written, so that ``to_dict`` gives the file back.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, as_float, as_int

MAMBA1_KEYS = ("inner", "state", "dt_rank", "conv")
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim")
RIGHT_KEYS = ("heads", "dim", "vdim")


def _section(raw: dict, key: str, where: str = "config.json") -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where} lacks the section {key!r}")
    return v


@dataclass
class ZasazenConfig:
    vocab: int
    width: int
    layers: list[dict[str, Any]]
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    loop: dict[str, int] | None = None       # {"start", "stop", "times"}
    max_positions: int = 32768               # the design has no table of positions; this is the context an engine is
                                             # made for when its caller names none (the key `max_positions` overrides it)
    eos_token_ids: list[int] = field(default_factory=list)

    architecture = "Zasazen"
    model_type = "zasazen"

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
    def from_dict(cls, raw: dict) -> "ZasazenConfig":
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError("config.json lacks 'layers' (a list with one entry per layer)")
        for key in ("vocab", "width"):
            if key not in raw:
                raise ConfigError(f"config.json lacks required key {key!r}")
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("'loop' must be a section with start, stop and times")
            loop = {k: as_int(loop.get(k), f"loop.{k}", minimum=(1 if k == "times" else 0))
                    for k in ("start", "stop", "times")}
        cfg = cls(vocab=as_int(raw["vocab"], "vocab", minimum=1), width=as_int(raw["width"], "width", minimum=1),
                  layers=copy.deepcopy(raw["layers"]),
                  embedding_scale=as_float((raw.get("embedding") or {}).get("scale", 1.0), "embedding.scale"),
                  norm_eps=as_float(_section(raw, "norm").get("eps", 1e-5), "norm.eps"), loop=loop,
                  max_positions=as_int(raw.get("max_positions", 32768), "max_positions", minimum=1))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        n = len(self.layers)
        if self.loop is not None and not (0 <= self.loop["start"] < self.loop["stop"] <= n):
            raise ConfigError(f"loop: start < stop <= {n} layers is needed, got {self.loop['start']} .. {self.loop['stop']}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in ("mamba1", "parallel"):
                raise ConfigError(f"{where}: 'type' must be 'mamba1' or 'parallel', got {layer.get('type')!r}")
            m = _section(layer, "mixer", where)
            if layer["type"] == "mamba1":
                for key in MAMBA1_KEYS:
                    as_int(m.get(key), f"{where}.mixer.{key}", minimum=1)
            else:
                left, right = _section(m, "left", where + ".mixer"), _section(m, "right", where + ".mixer")
                for key in LEFT_KEYS:
                    as_int(left.get(key), f"{where}.mixer.left.{key}", minimum=1)
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}: left.heads must be a multiple of left.kv_heads")
                as_float(left.get("scale"), f"{where}.mixer.left.scale")
                qt = left.get("q_temp")
                if qt is not None:
                    as_float(_section(left, "q_temp", where).get("coef"), f"{where}.mixer.left.q_temp.coef")
                    as_int(qt.get("every"), f"{where}.mixer.left.q_temp.every", minimum=1)
                for key in RIGHT_KEYS:
                    as_int(right.get(key), f"{where}.mixer.right.{key}", minimum=1)
                decay = right.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"]:
                    raise ConfigError(f"{where}: right.decay must list one decay per head")
                for j, v in enumerate(decay):
                    as_float(v, f"{where}.mixer.right.decay[{j}]")
                rot = right.get("rot")
                if rot is not None:
                    as_float(_section(right, "rot", where).get("base"), f"{where}.mixer.right.rot.base")
                    dims = as_int(rot.get("dims", right["dim"]), f"{where}.mixer.right.rot.dims", minimum=0)
                    if dims % 2 or dims > right["dim"]:
                        raise ConfigError(f"{where}: right.rot.dims must be even and at most right.dim")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"{where}: 'mlp' must be null or of kind 'dense' or 'moe'")
            if mlp["kind"] == "dense":
                as_int(mlp.get("ff"), f"{where}.mlp.ff", minimum=1)
            else:
                E = as_int(_section(mlp, "router", where).get("experts"), f"{where}.mlp.router.experts", minimum=1)
                top = as_int(mlp["router"].get("top"), f"{where}.mlp.router.top", minimum=1)
                if top > E:
                    raise ConfigError(f"{where}: top {top} exceeds experts {E}")
                as_int(_section(mlp, "expert", where).get("ff"), f"{where}.mlp.expert.ff", minimum=1)
                if mlp.get("shared") is not None:
                    as_int(_section(mlp, "shared", where).get("ff"), f"{where}.mlp.shared.ff", minimum=1)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_positions != 32768:
            out["max_positions"] = self.max_positions
        return out
