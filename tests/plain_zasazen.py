"""A plain, slow statement of the Zasazen design in PyTorch, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dict and the
tensors by their stored names, walks recurrences token by token, and keeps nothing
between calls.  Everything is computed in ``dtype`` (float64 by default) from the
weights as they are stored.  With ``rounded=True`` whatever a 16-bit engine hands
to a matrix product or keeps in its cache is rounded to bfloat16 first.

Notation: ``h`` is a sublayer's input ``[T, width]``; ``p(name)`` gives a tensor of
the current layer; positions count from 0.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces
def as_stored(x, rounded):
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(x, w, bias=None):
    """``out[t, c] = sum_j w[c, j] * x[t - taps + 1 + j, c]`` (+ bias), zeros before the start."""
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
    angle = position * base^(-2i/dims).  x: [T, heads, D]; positions: [T]."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    a = (positions.to(x.dtype)[:, None] * f[None, :])[:, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------ mixers
def selective_scan_mixer(h, p, m, rounded=False):
    """The 'mamba1' mixer: a diagonal state-space recurrence with a step size per channel."""
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    xz = hh @ p("in").T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, p("conv"), p("conv.b")))
    low = as_stored(x, rounded) @ p("x").T
    dt_low, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:R + 2 * N]
    dt = softplus(as_stored(dt_low, rounded) @ p("dt").T + p("dt.b"))         # [T, inner]
    A = -torch.exp(p("A_log"))                                                   # [inner, N]
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + p("D") * x[t]
    y = y * silu(z)
    return as_stored(y, rounded) @ p("o").T


def distance_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (n + 1) / H) for n in range(H)], dtype=torch.float64)


def biased_attention(h, p, m, eps, rounded=False):
    """The left half of the 'parallel' mixer: softmax attention with norms over the whole query and key
    projections, a query temperature growing with position and a linear distance penalty per head."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    q = hh @ p("q").T + p("q.b")
    k = hh @ p("k").T + p("k.b")
    v = hh @ p("v").T + p("v.b")
    q = rms_norm(q, p("q.norm"), eps)
    k = rms_norm(k, p("k.norm"), eps)
    pos = torch.arange(T, dtype=torch.float64)
    qt = m.get("q_temp")
    if qt is not None:
        temp = 1.0 + qt["coef"] * torch.log(torch.floor((pos + 1.0) / qt["every"]) + 1.0)
        q = q * temp.to(h.dtype)[:, None]
    q = as_stored(q, rounded).view(T, H, d)
    k = as_stored(k, rounded).view(T, G, d)
    v = as_stored(v, rounded).view(T, G, dv)
    slopes = distance_slopes(H).to(h.dtype)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)
    seen = dist >= 0
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"] - slopes[n] * dist
        s = s.masked_fill(~seen, float("-inf"))
        out[:, n] = torch.softmax(s, dim=-1) @ v[:, g]
    return as_stored(out.reshape(T, H * dv), rounded) @ p("o").T


def retention(h, p, m, eps, rounded=False):
    """The right half: linear attention with a fixed decay per head, no softmax and no denominator."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    hh = as_stored(h, rounded)
    q = (hh @ p("q").T).view(T, H, d)
    k = (hh @ p("k").T).view(T, H, d)
    v = (hh @ p("v").T).view(T, H, dv)
    g = hh @ p("g").T
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q = rotate_half_pairs(q, pos, rot["base"], rot["dims"])
        k = rotate_half_pairs(k, pos, rot["base"], rot["dims"])
    k = k * d ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(g)
    return as_stored(o, rounded) @ p("o").T


def parallel_mixer(h, p, m, eps, rounded=False):
    """Both halves read h; each output is RMS-normed over the width; half their sum."""
    left = biased_attention(h, lambda n: p("left." + n), m["left"], eps, rounded)
    right = retention(h, lambda n: p("right." + n), m["right"], eps, rounded)
    return 0.5 * (rms_norm(left, p("left.out"), eps) + rms_norm(right, p("right.out"), eps))


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, p, rounded=False):
    a = gelu_tanh(as_stored(h, rounded) @ p("up").T)
    return as_stored(a, rounded) @ p("down").T


def gated_expert(hh, p, name, rounded):
    a = silu(hh @ p(name + ".gate").T) * (hh @ p(name + ".up").T)
    return as_stored(a, rounded) @ p(name + ".down").T


def routed_ff(h, p, mlp, rounded=False):
    """Experts chosen by the largest router logits, weighted by the softmax over the chosen logits; a shared
    expert scaled by a sigmoid gate of one number per token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    hh = as_stored(h, rounded)
    z = hh @ p("router").T + p("router.b")
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += w[rows, j][:, None] * gated_expert(hh[rows], p, f"e{e}", rounded)
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(hh @ p("shared.sg").T)
        out = out + gate * gated_expert(hh, p, "shared", rounded)
    return out


def router_gap(h, p, mlp):
    """Per token: the gap between the last chosen and the first unchosen router logit."""
    top = mlp["router"]["top"]
    z = h @ p("router").T + p("router.b")
    s = torch.sort(z, dim=-1, descending=True).values
    return (s[:, top - 1] - s[:, top]) if z.shape[1] > top else torch.full((h.shape[0],), float("inf"), dtype=h.dtype)


# ------------------------------------------------------------------------- model
class PlainZasazen:
    def __init__(self, cfg, tensors, dtype=torch.float64, rounded=False):
        self.cfg, self.dtype, self.rounded = cfg, dtype, rounded
        self.t = tensors
        self._conv = {}
        self.gaps = []

    def w(self, name):
        if name not in self._conv:
            self._conv[name] = self.t[name].to(self.dtype)
        return self._conv[name]

    def order(self):
        """[(layer, pass number or None when the layer run does not open a pass)]"""
        n = len(self.cfg["layers"])
        loop = self.cfg.get("loop")
        if not loop:
            return [(i, None) for i in range(n)]
        out = [(i, None) for i in range(loop["start"])]
        for t in range(loop["times"]):
            for i in range(loop["start"], loop["stop"]):
                out.append((i, t if i == loop["start"] else None))
        return out + [(i, None) for i in range(loop["stop"], n)]

    def layer(self, i, x):
        cfg, eps, r = self.cfg, self.cfg["norm"]["eps"], self.rounded
        L = cfg["layers"][i]

        def pm(n):
            return self.w(f"l{i}.mix.{n}")

        def pf(n):
            return self.w(f"l{i}.mlp.{n}")

        h1 = rms_norm(x, self.w(f"l{i}.norm1"), eps)
        if L["type"] == "mamba1":
            y = selective_scan_mixer(h1, pm, L["mixer"], r)
        else:
            y = parallel_mixer(h1, pm, L["mixer"], eps, r)
        mlp = L.get("mlp")
        if mlp is not None:
            h2 = rms_norm(x, self.w(f"l{i}.norm2"), eps)
            y = y + (dense_ff(h2, pf, r) if mlp["kind"] == "dense" else routed_ff(h2, pf, mlp, r))
            if mlp["kind"] == "moe":
                self.gaps.append(router_gap(h2, pf, mlp))
        return x + y

    def forward(self, tokens, return_layers=False):
        """Logits ``[T, vocab]`` of a whole sequence (and the residual after every layer run)."""
        cfg, r = self.cfg, self.rounded
        x0 = self.w("embed")[torch.tensor(tokens)] * cfg["embedding"]["scale"]
        x = x0
        seen = []
        self.gaps = []          # per routed layer run: every position's gap between the last chosen and the next logit
        for i, enters in self.order():
            if enters is not None:
                x = as_stored(torch.cat([x, x0], dim=-1), r) @ self.w("loop.in").T + self.w("loop.step")[enters]
            x = self.layer(i, x)
            seen.append(x)
        n = rms_norm(x, self.w("final.norm"), cfg["norm"]["eps"])
        logits = as_stored(n, r) @ self.w("head").T
        return (logits, torch.stack(seen)) if return_layers else logits

    def smallest_gap(self, tokens):
        """Per position, the smallest router gap over all routed layer runs (inf without routed layers)."""
        self.forward(tokens)
        if not self.gaps:
            return torch.full((len(tokens),), float("inf"), dtype=self.dtype)
        return torch.stack(self.gaps).min(0).values
