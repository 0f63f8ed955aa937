"""Small Zesapel configurations and random weights for the tests.

The weights are drawn so that every mechanism matters to the logits: stream mixing away from the
identity, convolution taps of the size of the direct path, decays between slow and fast, sinks of the
size of the scores.  Matrices are stored in bfloat16 (so that a bfloat16 engine and the 64-bit plain
implementation read the same numbers), tables in int32.

X, Y, Z and W differ in every size and option (W: sizes that are multiples of neither 4 nor 8, so that no 16-byte
path applies; a window of 3; a last layer without feed-forward); none of the sizes is a power of two unless a kernel's
fast path needs it, and sizes that a config could make equal by accident (dim, rot_dim, vdim; heads
of the three mixers; state and vdim) are unequal.  Y has one stream, a layer without feed-forward, a
window equal to a page and a single expert choice; Z has larger heads (128-wide delta heads, 64-wide
state) and a latent of 128 for the wide paths (in bfloat16 its attention runs on the tensor-core kernel).
"""
from __future__ import annotations

import json
import math
import os

import torch


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _delta(heads, dim):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base, dims=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if scale is not None:
        m["scale"] = scale
    return {"type": "latent_attention", "mixer": m}


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    "X": {"architecture": "Zesapel", "vocab": 131, "width": 96, "streams": 3, "max_positions": 700,
          "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
          "layers": [_with(_latent(3, 24, 16, 40, 48, 40, 7, 10000.0, dims=8, scale=0.17), _moe(3, 1, 40)),
                     _with(_mamba(4, 24, 16, 2, 2, 2), _moe(5, 2, 56)),
                     _with(_delta(3, 24), _moe(3, 1, 40)),
                     _with(_latent(2, 40, 8, 24, 72, 56, 19, 500.0, scale=0.11), _moe(5, 2, 56))]},
    "Y": {"architecture": "Zesapel", "vocab": 77, "width": 64, "streams": 1, "max_positions": 600,
          "embedding": {"scale": 1.0}, "norm": {"eps": 3e-6}, "canon": {"taps": 4},
          "layers": [_with(_mamba(2, 40, 24, 1, 3, 1), None),
                     _with(_delta(1, 48), _moe(4, 3, 24)),
                     _with(_latent(5, 16, 24, 16, 36, 20, 64, 250000.0, scale=0.2), _moe(4, 3, 24)),
                     _with(_mamba(6, 8, 40, 3, 1, 6), _moe(2, 2, 72))]},
    "W": {"architecture": "Zesapel", "vocab": 97, "width": 90, "streams": 2, "max_positions": 500,
          "embedding": {"scale": 0.7}, "norm": {"eps": 2e-5}, "canon": {"taps": 5},
          "layers": [_with(_delta(5, 18), _moe(2, 2, 34)),
                     _with(_mamba(3, 30, 10, 3, 2, 3), _moe(2, 2, 34)),
                     _with(_latent(7, 10, 4, 14, 26, 22, 3, 777.0, dims=2, scale=0.3), None)]},
    "Z": {"architecture": "Zesapel", "vocab": 260, "width": 128, "streams": 2, "max_positions": 1200,
          "embedding": {"scale": 11.3}, "norm": {"eps": 1e-6}, "canon": {"taps": 3},
          "layers": [_with(_delta(2, 128), _moe(6, 2, 64)),
                     _with(_mamba(2, 136, 64, 1, 4, 1), _moe(6, 2, 64)),
                     _with(_latent(4, 64, 32, 64, 128, 96, 130, 10000.0, scale=0.09), _moe(6, 2, 64))]},
}


def one_layer(layer, width=64, vocab=53, streams=2, taps=3, mlp=None):
    """A model of a single layer (for a mechanism alone)."""
    return {"architecture": "Zesapel", "vocab": vocab, "width": width, "streams": streams, "max_positions": 400,
            "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "canon": {"taps": taps},
            "layers": [_with(layer, mlp)]}


def make_weights(cfg, seed=0, decay_rank=5):
    """name -> tensor (bfloat16, tables int32) for a config dict."""
    g = torch.Generator().manual_seed(seed)
    W, V, S = cfg["width"], cfg["vocab"], cfg["streams"]
    out = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    out["embed"] = rnd(V, W, std=0.5)
    out["pos"] = rnd(cfg["max_positions"], W, std=0.5)
    out["final.norm"] = rnd(W, std=0.1, mean=1.0)
    out["head"] = lin(V, W)
    taps = cfg["canon"]["taps"]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = rnd(W, std=0.1, mean=1.0)
        out[p + "canon1"] = rnd(W, taps, std=0.4)
        for q in ("hc1", "hc2") if L["mlp"] is not None else ("hc1",):
            out[p + q + ".in"] = rnd(S, std=0.2, mean=1.0 / S)
            out[p + q + ".out"] = rnd(S, std=0.2, mean=1.0)
            out[p + q + ".mix"] = (torch.eye(S) + 0.2 * torch.randn(S, S, generator=g)).to(torch.bfloat16)
        if L["type"] == "mamba2":
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "mix.in"] = lin(2 * inner + 2 * GN + m["heads"], W)
            out[p + "mix.conv"] = rnd(inner + 2 * GN, m["conv"], std=0.5)
            out[p + "mix.conv.b"] = rnd(inner + 2 * GN, std=0.2)
            out[p + "mix.dt_bias"] = rnd(m["heads"], std=0.7)
            out[p + "mix.A_log"] = (2.0 * torch.rand(m["heads"], generator=g) - 1.5).to(torch.bfloat16)
            out[p + "mix.D"] = rnd(m["heads"], std=0.3, mean=1.0)
            out[p + "mix.norm"] = rnd(inner, std=0.1, mean=1.0)
            out[p + "mix.o"] = lin(W, inner)
        elif L["type"] == "latent_attention":
            H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            out[p + "mix.dq"] = lin(m["q_rank"], W)
            out[p + "mix.dq.norm"] = rnd(m["q_rank"], std=0.1, mean=1.0)
            out[p + "mix.uq"] = lin(H * (dn + dr), m["q_rank"], gain=2.0)
            out[p + "mix.dkv"] = lin(m["kv_rank"] + dr, W)
            out[p + "mix.dkv.norm"] = rnd(m["kv_rank"], std=0.1, mean=1.0)
            out[p + "mix.uk"] = lin(H * dn, m["kv_rank"], gain=2.0)
            out[p + "mix.uv"] = lin(H * dv, m["kv_rank"])
            out[p + "mix.sink"] = rnd(H, std=1.5)
            out[p + "mix.g"] = lin(H, W)
            out[p + "mix.o"] = lin(W, H * dv)
        else:
            HD = m["heads"] * m["dim"]
            for n in ("r", "k", "v", "a", "g"):
                out[p + "mix." + n] = lin(HD, W)
            out[p + "mix.a.b"] = rnd(HD, std=1.0)
            out[p + "mix.w1"] = lin(decay_rank, W)
            out[p + "mix.w2"] = lin(HD, decay_rank, gain=2.0)
            out[p + "mix.w0"] = rnd(HD, std=1.0, mean=-1.0)
            out[p + "mix.norm"] = rnd(HD, std=0.1, mean=1.0)
            out[p + "mix.o"] = lin(W, HD)
        if L["mlp"] is not None:
            E, top, ff = L["mlp"]["router"]["experts"], L["mlp"]["router"]["top"], L["mlp"]["expert"]["ff"]
            out[p + "norm2"] = rnd(W, std=0.1, mean=1.0)
            keys = torch.rand(V, E, generator=g)
            out[p + "mlp.table"] = torch.argsort(keys, dim=1)[:, :top].to(torch.int32).contiguous()
            for e in range(E):
                out[p + f"mlp.e{e}.up"] = lin(ff, W, gain=1.5)
                out[p + f"mlp.e{e}.down"] = lin(W, ff, gain=1.5)
    return out


def write_model(cfg, folder, seed=0, tensors=None):
    from dlm_b200.weights.safetensors_io import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = make_weights(cfg, seed) if tensors is None else tensors
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return tensors


def tokens(seed, length, vocab):
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def row_error(got, ref):
    """Per row: root mean square of the difference (its mean taken off) over that of the reference."""
    got, ref = got.double(), ref.double()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((r * r).mean(-1))


# what a correct engine stays within (rounding of the format; measured values are printed by the tests)
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def references(oracle, reqs, dtype):
    """Per request the exact logits and a limit for every position: TOL, or in bfloat16 three times the error that
    rounding alone causes at that position where that is more (a norm over a few channels that happen to be
    small, or a decay near a tie, can magnify one rounding step a hundredfold at single positions; the plain
    model with rounding switched on shows where)."""
    import plain_zesapel as plain
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    lim = {rid: torch.full((len(t),), TOL[dtype], dtype=torch.float64) for rid, t in reqs.items()}
    if dtype == "bfloat16":
        rounded = plain.PlainZesapel(oracle.cfg, oracle.t, rounded=True)
        for rid, t in reqs.items():
            lim[rid] = torch.maximum(lim[rid], 3.0 * row_error(rounded.forward(t), ref[rid]))
    return ref, lim


def worst_ratio(got, ref, lim):
    """Largest error / limit over the rows ``{(request, position): logits}``."""
    return max(float(row_error(row, ref[rid][p]) / lim[rid][p]) for (rid, p), row in got.items())
