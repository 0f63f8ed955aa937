"""A plain, slow statement of the Zesapel design in PyTorch, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dict and the
tensors by their stored names, runs whole sequences token by token where there is
a recurrence, and keeps nothing between calls.  Everything is computed in
``dtype`` (float64 by default) from the weights as they are stored.

Notation: ``h`` is a sublayer's input ``[T, width]``; ``p(name)`` gives a tensor of
the current layer; positions count from 0.
"""
from __future__ import annotations

import json
import math
import os

import torch


# ------------------------------------------------------------------ small pieces
def as_stored(x, rounded):
    """What a 16-bit engine hands to a matrix product or keeps in its cache: x rounded to bfloat16 (when
    ``rounded``), else x itself."""
    return x.to(torch.bfloat16).to(x.dtype) if rounded else x


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def causal_conv(x, w, bias=None):
    """``out[t, c] = sum_j w[c, j] * x[t - taps + 1 + j, c]`` (+ bias), zeros before the start.
    x: [T, C]; w: [C, taps] (the last column meets the current token)."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def rotate_half_pairs(x, positions, base, dims):
    """Rotates the first ``dims`` entries of the last dimension: entry i is paired with i + dims/2,
    angle = position * base^(-2i/dims).  x: [T, ..., D]; positions: [T]."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]            # [T, half]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------ mixers
def mamba2(h, p, m, eps, rounded=False):
    """State-space mixer.  m: the layer's 'mixer' dict."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ p("mix.in").T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, p("mix.conv"), p("mix.conv.b")))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + p("mix.dt_bias"))                         # [T, H]
    A = -torch.exp(p("mix.A_log"))                               # [H]
    D = p("mix.D")
    y = torch.zeros(T, H, P, dtype=h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = torch.exp(A[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + D[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = unit_rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * p("mix.norm")
    return as_stored(y, rounded) @ p("mix.o").T


def latent_attention(h, p, m, eps, positions, rounded=False):
    """Attention through a cached latent, sliding window, a sink in the softmax, an output gate."""
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = as_stored(rms_norm(h @ p("mix.dq").T, p("mix.dq.norm"), eps), rounded)
    q = (cq @ p("mix.uq").T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    kv = h @ p("mix.dkv").T
    c = as_stored(rms_norm(kv[:, :rank], p("mix.dkv.norm"), eps), rounded)
    k_rot = kv[:, rank:]
    rot = m["rot"]
    q_rot = rotate_half_pairs(q_rot, positions, rot["base"], rot["dims"])
    k_rot = as_stored(rotate_half_pairs(k_rot, positions, rot["base"], rot["dims"]), rounded)
    k_plain = (c @ p("mix.uk").T).reshape(T, H, dn)
    v = (c @ p("mix.uv").T).reshape(T, H, dv)
    window = m["mask"]["size"]
    sink = p("mix.sink")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - window + 1)
        for hd in range(H):
            s = (k_plain[lo:t + 1, hd] @ q_plain[t, hd] + k_rot[lo:t + 1] @ q_rot[t, hd]) * m["scale"]
            mx = torch.maximum(s.max(), sink[hd])
            e = torch.exp(s - mx)
            w = e / (e.sum() + torch.exp(sink[hd] - mx))
            out[t, hd] = w @ v[lo:t + 1, hd]
    gate = torch.sigmoid(h @ p("mix.g").T)                       # [T, H]
    out = out * gate[:, :, None]
    return as_stored(out.reshape(T, H * dv), rounded) @ p("mix.o").T


def general_delta(h, p, m, eps, rounded=False):
    """Delta-rule recurrence with per-channel decay and removal rate."""
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    r = (h @ p("mix.r").T).reshape(T, H, d)
    k = (h @ p("mix.k").T).reshape(T, H, d)
    v = (h @ p("mix.v").T).reshape(T, H, d)
    lw = as_stored(torch.tanh(h @ p("mix.w1").T), rounded) @ p("mix.w2").T + p("mix.w0")
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(lw)).reshape(T, H, d)
    a = torch.sigmoid(h @ p("mix.a").T + p("mix.a.b")).reshape(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    o = torch.zeros(T, H, d, dtype=h.dtype)
    S = torch.zeros(H, d, d, dtype=h.dtype)                      # [key channel, value channel]
    for t in range(T):
        for hd in range(H):
            old = S[hd]
            S[hd] = w[t, hd][:, None] * old - torch.outer(a[t, hd] * u[t, hd], u[t, hd] @ old) \
                + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ r[t, hd]
    o = unit_rms(o, eps).reshape(T, H * d) * p("mix.norm")
    o = o * torch.sigmoid(h @ p("mix.g").T)
    return as_stored(o, rounded) @ p("mix.o").T


# ------------------------------------------------------------------ feed-forward
def table_experts(h, p, mlp, tokens, rounded=False):
    """Experts chosen by a table row of the token id, each weighted 1/top."""
    top = mlp["router"]["top"]
    table = p("mlp.table")
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            up = p(f"mlp.e{int(e)}.up") @ h[t]
            out[t] += (p(f"mlp.e{int(e)}.down") @ as_stored(gelu_erf(up), rounded)) / top
    return out


# ------------------------------------------------------------------------- model
class PlainZesapel:
    def __init__(self, folder_or_config, tensors=None, dtype=torch.float64, rounded=False):
        """``rounded``: round to bfloat16 wherever an engine that computes in bfloat16 must (what enters a matrix
        product, what the cache keeps); everything else stays exact.  The difference to the exact result is what
        rounding alone causes at a position."""
        self.rounded = rounded
        if tensors is None:
            with open(os.path.join(folder_or_config, "config.json")) as f:
                self.cfg = json.load(f)
            tensors = read_safetensors(os.path.join(folder_or_config, "model.safetensors"))
        else:
            self.cfg = folder_or_config
        self.dtype = dtype
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v.to(torch.int64)) for k, v in tensors.items()}

    def layer(self, i, xs, tokens, positions):
        """xs: [streams, T, width] -> the same after layer i."""
        cfg, t = self.cfg, self.t
        eps = cfg["norm"]["eps"]
        L = cfg["layers"][i]

        def p(name):
            return t[f"l{i}.{name}"]

        def sub(q, xs, fn):
            u = torch.einsum("s,stw->tw", p(f"hc{q}.in"), xs)
            y = fn(rms_norm(u, p(f"norm{q}"), eps))
            return torch.einsum("sr,stw->rtw", p(f"hc{q}.mix"), xs) + p(f"hc{q}.out")[:, None, None] * y[None]

        rd = self.rounded

        def mixer(h):
            h = as_stored(h + causal_conv(h, p("canon1")), rd)
            kind, m = L["type"], L["mixer"]
            if kind == "mamba2":
                return mamba2(h, p, m, eps, rd)
            if kind == "latent_attention":
                return latent_attention(h, p, m, eps, positions, rd)
            if kind == "general_delta":
                return general_delta(h, p, m, eps, rd)
            raise ValueError(kind)

        xs = sub(1, xs, mixer)
        if L.get("mlp") is not None:
            xs = sub(2, xs, lambda h: table_experts(as_stored(h, rd), p, L["mlp"], tokens, rd))
        return xs

    def forward(self, tokens, return_layers=False):
        """Logits [T, vocab] of one sequence from its start (and the summed streams after every layer)."""
        cfg, t = self.cfg, self.t
        tokens = torch.as_tensor(tokens, dtype=torch.int64)
        T = tokens.shape[0]
        positions = torch.arange(T)
        x = t["embed"][tokens] * cfg["embedding"]["scale"] + t["pos"][positions]
        xs = x[None].repeat(cfg["streams"], 1, 1)
        after = []
        for i in range(len(cfg["layers"])):
            xs = self.layer(i, xs, tokens, positions)
            after.append(xs.sum(0))
        x = as_stored(rms_norm(xs.sum(0), t["final.norm"], cfg["norm"]["eps"]), self.rounded)
        logits = x @ t["head"].T
        return (logits, torch.stack(after)) if return_layers else logits


def read_safetensors(path):
    """name -> tensor, read with nothing but the file format: 8 bytes of length, a JSON header, raw data."""
    import struct
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64,
             "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[b:e]), dtype=kinds[info["dtype"]]).reshape(info["shape"]).clone()
    return out
