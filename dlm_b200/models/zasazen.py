"""Zasazen as a ``ModelSpec`` of parts.

Scaled token embedding; layers that add a mixer and a feed-forward of the same input (each through its own RMS norm)
to the residual; per layer either a selective state-space mixer or two mixers side by side (softmax attention with
whole-projection query/key norms, a query temperature and a distance penalty; retention with constant decays); a
dense gelu feed-forward or routed gated experts with a shared one; optionally a run of layers repeated several times,
each pass with a cache and state of its own, opened by a product over the residual and the embedded tokens; an RMS
norm and an output matrix.  Tensor names are the checkpoint's own: ``embed``, ``loop.in``, ``loop.step``,
``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zasazen import ZasazenConfig
from ..parts.base import PartSpec
from ..parts.model import LayerCall, ModelSpec
from ..registry import register_architecture

_NAMES = {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp."}
_MOE_NAMES = {"router": "router", "router_bias": "router.b", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
              "shared_gate_proj": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down",
              "shared_gate": "shared.sg"}


def _mixer(cfg: ZasazenConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "mamba1":
        return PartSpec("mamba1", {"hidden_size": cfg.width, "inner": m["inner"], "state": m["state"],
                                   "dt_rank": m["dt_rank"], "conv_taps": m["conv"]})
    left, right = m["left"], m["right"]
    qt = left.get("q_temp") or {}
    rot = right.get("rot")
    return PartSpec("parallel_mixers", {
        "hidden_size": cfg.width, "eps": cfg.norm_eps, "coef": 0.5, "names": ("left", "right"),
        "left": PartSpec("normed_biased_attention", {
            "hidden_size": cfg.width, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"],
            "vdim": left["vdim"], "scale": left["scale"], "eps": cfg.norm_eps, "qkv_bias": True, "qk_norm": True,
            "temp_coef": qt.get("coef", 0.0), "temp_every": qt.get("every"), "slope_bits": 8.0}),
        "right": PartSpec("retention", {
            "hidden_size": cfg.width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
            "decay": list(right["decay"]), "eps": cfg.norm_eps,
            "rope_base": rot["base"] if rot else None,
            "rope_dims": rot.get("dims", right["dim"]) if rot else 0})})


def _ffn(cfg: ZasazenConfig, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("dense_act", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"],
                                      "activation": "gelu_tanh"})
    shared = mlp.get("shared")
    return PartSpec("moe_softmax_topk", {
        "hidden_size": cfg.width, "num_experts": mlp["router"]["experts"], "top_k": mlp["router"]["top"],
        "expert_intermediate_size": mlp["expert"]["ff"], "norm_topk_prob": True,
        "shared_intermediate_size": shared["ff"] if shared else None, "shared_gate": bool(shared),
        "router_bias": True, "names": _MOE_NAMES})


def layer_order(n_layers: int, loop: dict | None) -> list[LayerCall]:
    """Every layer once, in order; the layers of ``loop`` ``times`` times in a row, each pass opened at its first
    layer."""
    if not loop:
        return [LayerCall(i) for i in range(n_layers)]
    out = [LayerCall(i) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [LayerCall(i, enters_pass=t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return out + [LayerCall(i) for i in range(loop["stop"], n_layers)]


def build_spec(cfg: ZasazenConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "param": ""})
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn(cfg, layer.get("mlp"))
        layers.append(PartSpec("parallel", {"norm1": norm, "mixer": _mixer(cfg, layer),
                                            "norm2": norm if ffn is not None else None, "ffn": ffn, "names": _NAMES}))
        prefixes.append(f"l{i}.")
    entry = None
    if cfg.loop:
        entry = PartSpec("input_injection", {"hidden_size": cfg.width, "passes": cfg.loop["times"], "weight": "in",
                                             "step": "step"})
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, layer_prefixes=prefixes,
                     final_norm=norm, final_norm_prefix="final.norm", embed_name="embed", lm_head_name="head",
                     embed_scale=cfg.embedding_scale, order=layer_order(len(cfg.layers), cfg.loop),
                     pass_entry=entry, pass_entry_prefix="loop.")


register_architecture(ZasazenConfig.architecture, ZasazenConfig, build_spec, model_type=ZasazenConfig.model_type)
