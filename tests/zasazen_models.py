"""Small Zasazen configurations and random weights for the tests.

The weights are drawn so that every mechanism matters to the logits: norm weights away from 1, biases of the size of
the projections, router biases of the size of the logits, step sizes between slow and fast, branch weights that
differ.  Matrices are stored in bfloat16 (so that a bfloat16 engine and the 64-bit plain implementation read the same
numbers).

A, B, C and D differ in every size and option; sizes that a config could make equal by accident (dim and vdim of
either half, the heads of the two halves, state and dt_rank) are unequal, and none is a power of two unless a
kernel's fast path needs it.  A: keys narrower than values, a temperature period of 16, a loop over the middle, a
layer without feed-forward.  B: no loop, a convolution of a single tap, one key/value head, one retention head,
values narrower than keys, experts without a shared one and as many choices as experts, sizes that are multiples of
neither 4 nor 8.  C: sizes of the tensor-core paths (64- and 128-wide heads), a loop that starts at the first layer.
D: a loop of one pass over all layers, a rotation over part of the head.
"""
from __future__ import annotations

import json
import math
import os

import torch


def _left(heads, kv, dim, vdim, scale, temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _right(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _parallel(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _mamba(inner, state, dt_rank, conv, mlp):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    "A": {"architecture": "Zasazen", "vocab": 131, "width": 96, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [_parallel(_left(6, 2, 24, 40, 0.21, (0.3, 16)), _right(3, 32, 16, [0.9, 0.97, 0.995], (10000.0, 16)),
                               _dense(200)),
                     _mamba(160, 12, 7, 4, _moe(5, 2, 56, 72)),
                     _parallel(_left(4, 4, 16, 8, 0.3), _right(2, 40, 24, [0.99, 0.8]), None),
                     _mamba(120, 20, 5, 2, _dense(72))]},
    "B": {"architecture": "Zasazen", "vocab": 77, "width": 62, "embedding": {"scale": 1.0}, "norm": {"eps": 3e-6},
          "layers": [_mamba(70, 5, 3, 1, _dense(50)),
                     _parallel(_left(8, 1, 10, 6, 0.37, (1.1, 5)), _right(1, 46, 38, [0.96], (300.0, 46)), _moe(3, 3, 22)),
                     _parallel(_left(3, 3, 18, 26, 0.2, (0.2, 7)), _right(5, 6, 10, [0.5, 0.9, 0.99, 0.999, 1.0], (50.0, 2)),
                               _moe(4, 1, 30, 14))]},
    "C": {"architecture": "Zasazen", "vocab": 260, "width": 128, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
          "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [_parallel(_left(4, 2, 64, 64, 0.1, (0.5, 64)), _right(2, 64, 128, [0.98, 0.999], (1e6, 64)),
                               _moe(8, 2, 64, 128)),
                     _mamba(256, 16, 8, 3, _dense(256)),
                     _parallel(_left(8, 1, 128, 96, 0.07, (0.25, 32)), _right(4, 32, 64, [0.9, 0.95, 0.99, 0.995], (1e4, 32)),
                               _dense(192))]},
    "D": {"architecture": "Zasazen", "vocab": 53, "width": 48, "embedding": {"scale": 0.6}, "norm": {"eps": 2e-5},
          "loop": {"start": 0, "stop": 2, "times": 1},
          "layers": [_parallel(_left(2, 1, 12, 20, 0.25), _right(3, 8, 12, [0.7, 0.9, 0.97], (100.0, 4)), _moe(6, 2, 20, 24)),
                     _mamba(60, 9, 4, 3, None)]},
}


def one_layer(layer, width=64, vocab=53, loop=None):
    """A model of a single layer (for a mechanism alone)."""
    cfg = {"architecture": "Zasazen", "vocab": vocab, "width": width, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
           "layers": [layer]}
    if loop:
        cfg["loop"] = loop
    return cfg


def make_weights(cfg, seed=0):
    """name -> tensor (bfloat16) for a config dict."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    def expert(p, ff):
        out[p + ".gate"], out[p + ".up"], out[p + ".down"] = lin(ff, W, 1.5), lin(ff, W, 1.5), lin(W, ff, 1.5)

    out["embed"] = rnd(V, W, std=0.5)
    out["final.norm"] = rnd(W, std=0.1, mean=1.0)
    out["head"] = lin(V, W)
    if cfg.get("loop"):
        out["loop.in"] = torch.cat([torch.eye(W) + 0.3 * torch.randn(W, W, generator=g) / math.sqrt(W),
                                    0.5 * torch.randn(W, W, generator=g) / math.sqrt(W)], dim=1).to(torch.bfloat16)
        out["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.3)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = rnd(W, std=0.1, mean=1.0)
        if L["type"] == "mamba1":
            inner, N, R = m["inner"], m["state"], m["dt_rank"]
            out[p + "mix.in"] = lin(2 * inner, W)
            out[p + "mix.conv"] = rnd(inner, m["conv"], std=0.6)
            out[p + "mix.conv.b"] = rnd(inner, std=0.2)
            out[p + "mix.x"] = lin(R + 2 * N, inner, gain=2.0)
            out[p + "mix.dt"] = lin(inner, R, gain=1.5)
            out[p + "mix.dt.b"] = rnd(inner, std=1.0, mean=-2.0)
            out[p + "mix.A_log"] = (3.0 * torch.rand(inner, N, generator=g) - 2.0).to(torch.bfloat16)
            out[p + "mix.D"] = rnd(inner, std=0.3, mean=1.0)
            out[p + "mix.o"] = lin(W, inner)
        else:
            lf, rt = m["left"], m["right"]
            H, G, d, dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                out[p + f"mix.left.{n}"] = lin(rows, W, gain=1.5)
                out[p + f"mix.left.{n}.b"] = rnd(rows, std=0.3)
            out[p + "mix.left.q.norm"] = rnd(H * d, std=0.3, mean=2.0)
            out[p + "mix.left.k.norm"] = rnd(G * d, std=0.3, mean=2.0)
            out[p + "mix.left.o"] = lin(W, H * dv)
            H2, d2, dv2 = rt["heads"], rt["dim"], rt["vdim"]
            out[p + "mix.right.q"], out[p + "mix.right.k"] = lin(H2 * d2, W, 1.5), lin(H2 * d2, W, 1.5)
            out[p + "mix.right.v"], out[p + "mix.right.g"] = lin(H2 * dv2, W), lin(H2 * dv2, W, 2.0)
            out[p + "mix.right.o"] = lin(W, H2 * dv2)
            out[p + "mix.left.out"] = rnd(W, std=0.2, mean=1.3)
            out[p + "mix.right.out"] = rnd(W, std=0.2, mean=0.7)
        mlp = L["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = rnd(W, std=0.1, mean=1.0)
        if mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.down"] = lin(mlp["ff"], W, 1.5), lin(W, mlp["ff"], 1.5)
        else:
            E = mlp["router"]["experts"]
            out[p + "mlp.router"] = lin(E, W, gain=3.0)
            out[p + "mlp.router.b"] = rnd(E, std=1.0)
            for e in range(E):
                expert(p + f"mlp.e{e}", mlp["expert"]["ff"])
            if mlp.get("shared"):
                expert(p + "mlp.shared", mlp["shared"]["ff"])
                out[p + "mlp.shared.sg"] = lin(1, W, gain=3.0)
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
    g = torch.Generator().manual_seed(9000 + seed)
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
# router gaps (in logit units) below which rounding may choose another expert: such positions are not compared
GAP = {"float32": 1e-3, "bfloat16": 0.15}


def references(oracle, reqs, dtype):
    """Per request the exact logits, a limit for every position (TOL, or in bfloat16 three times the error that
    rounding alone causes there where that is more) and which positions are compared at all (those whose routing is
    not a close call, here and in the rounded model; in bfloat16 also not within three positions after one)."""
    import plain_zasazen as plain
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    gap = {rid: oracle.smallest_gap(t) for rid, t in reqs.items()}
    lim = {rid: torch.full((len(t),), TOL[dtype], dtype=torch.float64) for rid, t in reqs.items()}
    if dtype == "bfloat16":
        rounded = plain.PlainZasazen(oracle.cfg, oracle.t, rounded=True)
        for rid, t in reqs.items():
            lim[rid] = torch.maximum(lim[rid], 3.0 * row_error(rounded.forward(t), ref[rid]))
            gap[rid] = torch.minimum(gap[rid], rounded.smallest_gap(t))
    clear = {rid: gap[rid] > GAP[dtype] for rid in reqs}
    if dtype == "bfloat16":
        # another expert at one position reaches the next few through the recurrences: those are left out as well
        for rid, c in clear.items():
            near = c.clone()
            for back in (1, 2, 3):
                near[back:] &= c[:-back]
            clear[rid] = near
    return ref, lim, clear


def worst_ratio(got, ref, lim, clear=None):
    """Largest error / limit over the compared rows ``{(request, position): logits}``, and the share compared."""
    rows = [(rid, p) for (rid, p) in got if clear is None or bool(clear[rid][p])]
    worst = max(float(row_error(got[k], ref[k[0]][k[1]]) / lim[k[0]][k[1]]) for k in rows)
    return worst, len(rows) / max(len(got), 1)
