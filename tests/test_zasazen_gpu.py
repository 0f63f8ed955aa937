"""Zasazen on the GPU.  Kernels alone against their plain PyTorch statements, with inputs made so that a fault shows
(one key that stands out far back and at a page's border, something written into a state hundreds of tokens ago,
positions on both sides of a temperature step); then the engine against the plain model: every mixer alone, four
configurations of unlike sizes under every cutting in both precisions, slots and pages that are used again, long
greedy decoding through the scheduler and the replayed graphs."""
import math
from types import SimpleNamespace

import pytest
import torch

import cuttings
import plain_zasazen as plain
from plain_ops import PlainOps
from zasazen_models import (CONFIGS, TOL, _dense, _left, _mamba, _moe, _parallel, _right, one_layer, references, row_error,
                            tokens, worst_ratio, write_model)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=True)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zasazen_gpu")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainZasazen(cfg, tensors))
    return out


def batch_of(lengths, slots, starts=None):
    """The fields of a step the kernels read, for requests that bring ``lengths`` tokens from ``starts`` on."""
    starts = starts or [0] * len(lengths)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    i32 = dict(dtype=torch.int32, device=DEV)
    return SimpleNamespace(
        num_requests=len(lengths), cu_q=torch.tensor(cu, **i32), state_slot=torch.tensor(slots, **i32),
        token_req=torch.tensor([r for r, n in enumerate(lengths) for _ in range(n)], **i32),
        positions=torch.tensor([s + i for s, n in zip(starts, lengths) for i in range(n)], **i32))


def to_cpu(b):
    return SimpleNamespace(**{k: (v.cpu() if torch.is_tensor(v) else v) for k, v in vars(b).items()})


def randn(*shape, seed=0, std=1.0):
    return (std * torch.randn(*shape, generator=torch.Generator().manual_seed(seed))).to(DEV)


# ============================================================== kernels alone
@pytest.mark.parametrize("inner,N", [(70, 5), (256, 16), (96, 40), (33, 1), (64, 130)])
def test_selective_scan_in_portions_with_slots_used_again(ops, inner, N):
    """Two requests fed in portions (1 to 273 tokens, within and past the kernel's tile) beside each other: every output
    equals the scan over the whole sequence; the state of a slot that is zeroed starts a new sequence; a write of
    300 tokens ago is still in the state when the decay is slow."""
    ref = PlainOps()
    L = [330, 61]
    g = torch.Generator().manual_seed(inner + N)
    seqs = [dict(x=randn(n, inner, seed=1 + i), dt=randn(n, inner, seed=3 + i) - 1.0, bc=randn(n, 2 * N, seed=5 + i),
                 z=randn(n, inner, seed=7 + i)) for i, n in enumerate(L)]
    A_log = (3.0 * torch.rand(inner, N, generator=g) - 2.0).to(DEV)
    A_log[0, 0] = -9.0                                         # channel 0, state 0 hardly forgets
    seqs[0]["x"][5, 0], seqs[0]["bc"][5, 0] = 40.0, 3.0        # ... what token 5 writes there
    dt_b, D = randn(inner, seed=9, std=0.5), randn(inner, seed=10)
    whole_state = torch.zeros(3, inner, N)
    whole = [ref.selective_scan(s["x"].cpu(), s["dt"].cpu(), s["bc"].cpu(), s["z"].cpu(), dt_b.cpu(), A_log.cpu(), D.cpu(),
                                whole_state, to_cpu(batch_of([n], [i])), torch.float32) for i, (s, n) in enumerate(zip(seqs, L))]
    state = torch.full((4, inner, N), 7.0, device=DEV)         # used slots ...
    state[[1, 2]] = 0.0                                        # ... are zeroed when a request takes them
    fed = [0, 0]
    cuts = [(40, 1), (1, 17), (16, 2), (273, 40), (0, 1)]
    for n0, n1 in cuts:
        lens, slots, which = [n for n in (n0, n1) if n], [s for s, n in ((2, n0), (1, n1)) if n], [i for i, n in ((0, n0), (1, n1)) if n]
        cat = {k: torch.cat([seqs[i][k][fed[i]:fed[i] + n] for i, n in zip(which, lens)]) for k in ("x", "dt", "bc", "z")}
        wide = torch.cat([randn(sum(lens), 3, seed=11), cat["x"], cat["z"]], dim=1)          # column slices
        got = ops.selective_scan(wide[:, 3:3 + inner], cat["dt"], cat["bc"], wide[:, 3 + inner:], dt_b, A_log, D, state,
                                 batch_of(lens, slots), torch.float32)
        want = torch.cat([whole[i][fed[i]:fed[i] + n] for i, n in zip(which, lens)])
        assert torch.allclose(got.cpu(), want, rtol=2e-4, atol=2e-4), (n0, n1)
        for i, n in zip(which, lens):
            fed[i] += n
    assert fed == [330, 61]
    assert torch.allclose(state[2].cpu(), whole_state[0], rtol=2e-4, atol=2e-4)
    assert abs(float(whole_state[0][0, 0])) > 1.0              # the old write is still there
    bf = ops.selective_scan(seqs[1]["x"], seqs[1]["dt"], seqs[1]["bc"], seqs[1]["z"], dt_b, A_log, D,
                            torch.zeros_like(state), batch_of([61], [0]), torch.bfloat16)
    assert torch.allclose(bf.float().cpu(), whole[1], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H,d,dv", [(3, 32, 16), (1, 46, 38), (5, 6, 10), (2, 64, 128)])
def test_scan_with_constant_decays_is_retention(ops, H, d, dv):
    """The state-space scan with fixed decays, step size 1 and no direct term, fed in portions with a slot used
    again, against the decayed sum over the past; a decay of 1 forgets nothing in 400 tokens."""
    ref = PlainOps()
    n = 400
    decay = torch.tensor([1.0, 0.9, 0.99, 0.5, 0.999][:H]).to(DEV)
    rows = randn(n, H * dv + 2 * H * d, seed=H + d, std=0.5)
    want_state = torch.zeros(2, H, d, dv)
    want = ref.ssm_scan(rows.cpu(), None, None, None, None, want_state, to_cpu(batch_of([n], [0])), H, dv, d, H,
                        fixed_decay=decay.cpu())
    v, k, q = (rows[:, a:b].cpu().double().reshape(n, H, -1) for a, b in ((0, H * dv), (H * dv, H * dv + H * d),
                                                                           (H * dv + H * d, H * dv + 2 * H * d)))
    i = n - 1
    direct = sum(decay.cpu().double()[:, None] ** (i - s) * (q[i] * k[s]).sum(-1, keepdim=True) * v[s] for s in range(n))
    assert torch.allclose(want[i].double().reshape(H, dv), direct, rtol=1e-3, atol=1e-3)
    state = torch.full((3, H, d, dv), 5.0, device=DEV)
    state[1] = 0.0
    fed, outs = 0, []
    for m in (1, 2, 17, 300, 80):
        wide = torch.cat([rows[fed:fed + m], randn(m, 5, seed=m)], dim=1)                     # a column slice
        outs.append(ops.ssm_scan(wide[:, :rows.shape[1]], None, None, None, None, state, batch_of([m], [1]), H, dv, d, H,
                                 fixed_decay=decay))
        fed += m
    assert torch.allclose(torch.cat(outs).cpu(), want, rtol=1e-3, atol=1e-3)
    assert torch.allclose(state[1].cpu(), want_state[0], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,D", [(6, 2, 24, 40, 48), (8, 1, 10, 6, 16), (4, 2, 64, 64, 64), (3, 3, 18, 26, 32),
                                           (8, 1, 128, 96, 128), (2, 1, 150, 70, 152)])
def test_norms_temperature_and_cache_write(ops, dtype, nh, nkv, d, dv, D):
    """Positions on both sides of every temperature step (period 5), a slot that is not stored (-1), heads padded
    with zeros up to the stored size."""
    ref = PlainOps()
    T, ps, pages = 23, 16, 6
    pos = torch.tensor([0, 1, 3, 4, 5, 8, 9, 10, 13, 14, 15, 19, 20, 24, 25, 99, 100, 101, 498, 499, 500, 4094, 4095],
                       dtype=torch.int32, device=DEV)
    wide = randn(T, 3 + (nh + nkv) * d + nkv * dv, seed=d)
    qkv = wide[:, 3:]
    qn, kn = randn(nh * d, seed=1) + 2.0, randn(nkv * d, seed=2) + 2.0
    slots = torch.randperm(ps * pages, generator=torch.Generator().manual_seed(3))[:T].to(DEV, torch.int32)
    slots[4] = -1
    for qn_w, kn_w, every in ((qn, kn, 5), (None, None, 0), (qn, None, 1)):
        caches = [torch.zeros(pages + 1, nkv, ps, D, dtype=dtype, device=DEV) for _ in range(2)]
        want_c = [c.cpu().clone() for c in caches]
        got = ops.qk_norm_write(qkv, pos, qn_w, kn_w, 1e-5, 0.7, every, slots, caches[0], caches[1], nh, nkv, d, dv, D, dtype)
        want = ref.qk_norm_write(qkv.cpu(), pos.cpu(), None if qn_w is None else qn_w.cpu(), None if kn_w is None else kn_w.cpu(),
                                 1e-5, 0.7, every, slots.cpu(), want_c[0], want_c[1], nh, nkv, d, dv, D, dtype)
        tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
        assert torch.allclose(got.float().cpu(), want.float(), **tol)
        for c, w in zip(caches, want_c):
            assert torch.allclose(c.float().cpu(), w.float(), **tol)
        if D > d:
            assert float(got.view(T, nh, D)[:, :, d:].abs().max()) == 0.0
    # the temperature itself, by hand: position 9 with period 5 -> 1 + 0.7 ln(3)
    base = ops.qk_norm_write(qkv, pos, qn, kn, 1e-5, 0.0, 0, None, caches[0], caches[1], nh, nkv, d, dv, D, torch.float32) \
        if dtype == torch.float32 else None
    if base is not None:
        hot = ops.qk_norm_write(qkv, pos, qn, kn, 1e-5, 0.7, 5, None, caches[0], caches[1], nh, nkv, d, dv, D, torch.float32)
        assert torch.allclose(hot[6], base[6] * (1.0 + 0.7 * math.log(3.0)), rtol=1e-6)
        assert torch.equal(hot[:3], base[:3])


@pytest.mark.parametrize("heads,dim,rot", [(3, 32, 16), (5, 6, 2), (1, 46, 46), (2, 64, 0), (4, 33, 32)])
def test_rotation_in_place(ops, heads, dim, rot):
    ref = PlainOps()
    T = 19
    pos = torch.randint(0, 5000, (T,), generator=torch.Generator().manual_seed(rot)).to(DEV, torch.int32)
    x = randn(T, 7 + 3 * heads * dim, seed=dim)
    freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV) if rot else None
    want = x.cpu().clone()
    ref.rotate_heads(want, pos.cpu(), None if freq is None else freq.cpu(), rot, heads, dim, 7 + heads * dim, dim ** -0.5,
                     7, 1.0)
    keep = x[:, 7 + 2 * heads * dim:].clone()
    ops.rotate_heads(x, pos, freq, rot, heads, dim, 7 + heads * dim, dim ** -0.5, 7, 1.0)
    assert torch.allclose(x.cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(x[:, 7 + 2 * heads * dim:], keep) and torch.equal(x[:, :7].cpu(), want[:, :7])


def test_small_pieces(ops):
    ref = PlainOps()
    T, H = 37, 90
    a, b, wa, wb = randn(T, H, seed=1), 3.0 * randn(T, H, seed=2), randn(H, seed=3) + 1.0, randn(H, seed=4) + 1.0
    for second in (b, None):
        resid, want = randn(T, H, seed=5), randn(T, H, seed=5).cpu()
        ops.branch_norm_add(resid, a, wa, second, None if second is None else wb, 1e-5, 0.5)
        ref.branch_norm_add(want, a.cpu(), wa.cpu(), None if second is None else second.cpu(), wb.cpu(), 1e-5, 0.5)
        assert torch.allclose(resid.cpu(), want, rtol=1e-5, atol=1e-5)
    for dt in (torch.float32, torch.bfloat16):
        assert torch.equal(ops.concat_rows(a, b, dt).cpu(), ref.concat_rows(a.cpu(), b.cpu(), dt))
    y, gate = randn(T, 6 * 15, seed=6), randn(T, 6 * 15, seed=7)
    got = ops.gated_rmsnorm(y, gate, None, 6, 1e-5, "silu_after", torch.float32)
    assert torch.allclose(got.cpu(), ref.gated_rmsnorm(y.cpu(), gate.cpu(), None, 6, 1e-5, "silu_after", torch.float32),
                          rtol=1e-5, atol=1e-5)
    z = 4.0 * randn(T, H, seed=8)
    assert torch.allclose(ops.activation(z, "gelu_tanh", torch.float32).cpu(), plain.gelu_tanh(z.cpu().double()).float(),
                          rtol=1e-5, atol=1e-6)
    assert torch.equal(ops.activation(z[:, 3:20], "copy", torch.bfloat16).cpu(), z[:, 3:20].cpu().to(torch.bfloat16))
    for dt in (torch.float32, torch.bfloat16):
        hh, w = randn(T, 64, seed=9).to(dt), (randn(48, 64, seed=10) / 8).to(dt)
        got = ops.linear_act(hh, w, "gelu_tanh")
        want = plain.gelu_tanh(hh.cpu().double() @ w.cpu().double().T)
        assert got.dtype == dt and torch.allclose(got.cpu().double(), want, rtol=2e-2, atol=2e-2 if dt == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,K,N", [(3, 64, 96), (16, 256, 1024), (40, 256, 512), (200, 128, 256), (700, 1024, 2048), (90, 90, 34),
                                   (2048, 512, 2048)])
def test_first_product_with_the_tanh_gelu_in_its_epilogue(ops, dtype, M, K, N):
    """`linear_act(..., "gelu_tanh")` on every product kernel the sizes reach (streaming, small-M, tcgen05 single and
    paired, warp-level, FMA) against the plain statement; and two norms of the same rows in one pass."""
    g = torch.Generator().manual_seed(M + K)
    h = torch.randn(M, K, generator=g).to(DEV, dtype)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K) * 2.0).to(DEV, dtype)
    got = ops.linear_act(h, w, "gelu_tanh")
    want = plain.gelu_tanh(h.cpu().double() @ w.cpu().double().T)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert got.dtype == dtype and torch.allclose(got.cpu().double(), want, atol=tol, rtol=tol)
    x, wa, wb = randn(M, K, seed=1) * 3.0, randn(K, seed=2) + 1.0, randn(K, seed=3) - 1.0
    a, b = ops.rmsnorm_pair(x, wa, wb, 1e-5, dtype)
    ra, rb = PlainOps().rmsnorm_pair(x.cpu(), wa.cpu(), wb.cpu(), 1e-5, dtype)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(a.float().cpu(), ra.float(), rtol=tol, atol=tol) and torch.allclose(b.float().cpu(), rb.float(), rtol=tol, atol=tol)
    torch.cuda.synchronize()
    ops.check_errors()


@pytest.mark.parametrize("T", [1, 9, 16, 17, 48, 49, 300, 700])
@pytest.mark.parametrize("E,k,gate", [(5, 2, True), (3, 3, False), (16, 3, True), (4, 1, False)])
def test_router_with_its_own_bias(ops, T, E, k, gate):
    """Every routing path (one launch up to 16 tokens, a block per token up to 48, three launches beyond): the bias
    joins the logits, so it moves the choice and the weights; the weights are the softmax over the chosen logits."""
    ref = PlainOps()
    H = 72
    resid = randn(T, H, seed=T + E)
    w = (randn(E + (1 if gate else 0), H, seed=2) * 0.4)
    bias = 2.0 * randn(E, seed=3)
    nw = randn(H, seed=4) + 1.0
    for dt in (torch.float32, torch.bfloat16):
        ids, wts, g, off, rows, dest = ops.route(resid, w.to(dt), E, k, True, gate, norm_weight=nw, eps=1e-5, logit_bias=bias)
        h = resid.cpu() / torch.sqrt((resid.cpu() ** 2).mean(-1, keepdim=True) + 1e-5) * nw.cpu()
        z = h @ w.to(dt).float().cpu().T
        logits = z[:, :E] + bias.cpu()
        val, idx = torch.topk(logits, k, dim=-1)
        gap = torch.sort(logits, dim=-1, descending=True).values
        sure = (gap[:, k - 1] - gap[:, k] > 1e-3) if k < E else torch.ones(T, dtype=torch.bool)
        assert torch.equal(torch.sort(ids.cpu()[sure].long(), dim=-1).values, torch.sort(idx[sure], dim=-1).values)
        want_w = torch.softmax(torch.gather(logits, 1, ids.cpu().long()), dim=-1)
        assert torch.allclose(wts.cpu()[sure], want_w[sure], rtol=1e-4, atol=1e-5)
        if gate:
            assert torch.allclose(g.cpu(), torch.sigmoid(z[:, E]), rtol=1e-4, atol=1e-5)
        assert int(off[-1]) == T * k
        # without the bias the choice differs somewhere (the bias is of the size of the logits)
        ids0 = ops.route(resid, w.to(dt), E, k, True, gate, norm_weight=nw, eps=1e-5)[0]
        assert k == E or T < 9 or not torch.equal(torch.sort(ids0, dim=-1).values, torch.sort(ids, dim=-1).values)
    torch.cuda.synchronize()
    ops.check_errors()


ATT = [  # nh, nkv, hd, page size, dtype: every attention kernel (FMA, warp-level prefill and decode, TMA-fed decode)
    (6, 2, 48, 16, torch.float32), (8, 1, 16, 16, torch.bfloat16), (4, 2, 64, 64, torch.bfloat16),
    (8, 1, 128, 64, torch.bfloat16), (3, 3, 32, 16, torch.bfloat16), (32, 2, 64, 64, torch.bfloat16),
    (2, 1, 152, 16, torch.bfloat16), (4, 4, 96, 32, torch.float32)]


@pytest.mark.parametrize("nh,nkv,hd,ps,dtype", ATT)
def test_attention_with_a_distance_penalty(ops, nh, nkv, hd, ps, dtype):
    """Prompts, portions and single tokens in one batch over pages in scrambled order.  One far key (position 3, and
    one right at a page's border) matches every query a hundredfold: the head with the smallest slope still finds it
    from 700 tokens away, the head with the largest slope has long lost it; both as the plain statement says."""
    ref = PlainOps()
    lens, news = [760, 130, 1, 64, 17], [1, 130, 1, 7, 1]
    R, T = len(lens), sum(news)
    g = torch.Generator().manual_seed(nh * hd)
    n_pages = sum(-(-n // ps) for n in lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // ps) for n in lens)
    table = torch.full((R, width), -1, dtype=torch.int32)
    k_cache = torch.zeros(n_pages + 1, nkv, ps, hd)
    v_cache = torch.zeros(n_pages + 1, nkv, ps, hd)
    direction = torch.randn(hd, generator=g)
    direction /= direction.norm()
    for r, n in enumerate(lens):
        for lp in range(-(-n // ps)):
            table[r, lp] = perm.pop()
        k = 0.3 * torch.randn(n, nkv, hd, generator=g)
        v = torch.randn(n, nkv, hd, generator=g)
        for far in (3, ps - 1, ps):
            if far < n:
                k[far] += 8.0 * direction
                v[far] += 10.0
        pos = torch.arange(n)
        k_cache[table[r, pos // ps].long(), :, pos % ps] = k
        v_cache[table[r, pos // ps].long(), :, pos % ps] = v
    q = 0.3 * torch.randn(T, nh, hd, generator=g) + 8.0 * direction
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)])
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32)
    kv = torch.tensor(lens, dtype=torch.int32)
    args = lambda f, dev: (f(q.reshape(T, nh * hd)).to(dev), f(k_cache).to(dev), f(v_cache).to(dev), table.to(dev),
                           cu.to(dev), kv.to(dev))
    cast = lambda t: t.to(dtype)
    single = sum(1 for n in news if n == 1)
    scale = 0.11
    for sl in (slopes, None):
        want = ref.attention(*args(cast, "cpu"), 0, scale, nh, nkv, hd, max(news), max(lens), single,
                             slopes=sl).float().reshape(T, nh, hd)
        got = ops.attention(*args(cast, DEV), 0, scale, nh, nkv, hd, max(news), max(lens), single,
                            slopes=None if sl is None else sl.to(DEV)).float().cpu().reshape(T, nh, hd)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        assert torch.allclose(got, want, rtol=tol, atol=tol * float(want.abs().max())), float((got - want).abs().max())
        if sl is not None and nh >= 4:
            # request 0's single token at position 759: the flattest head still draws on the far keys, the steepest not
            assert float(want[0, nh - 1].mean()) > 1.0 and abs(float(want[0, 0].mean())) < 0.5
    torch.cuda.synchronize()
    ops.check_errors()


# ====================================================== the engine against the plain model
def gpu_engine(folder, dtype, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype=dtype, device=DEV, page_size=16, num_pages=64, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


def worst_error(got, ref):
    return max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items())


LAYERS = {"scan": lambda mlp: _mamba(72, 10, 3, 4, mlp),
          "scan_one_tap": lambda mlp: _mamba(40, 3, 2, 1, mlp),
          "pair": lambda mlp: _parallel(_left(6, 2, 12, 20, 0.3, (0.4, 7)), _right(3, 10, 14, [0.9, 0.99, 0.6], (100.0, 6)), mlp),
          "pair_plain": lambda mlp: _parallel(_left(2, 2, 8, 8, 0.5), _right(2, 8, 8, [0.95, 0.8]), mlp)}


@pytest.mark.parametrize("kind", list(LAYERS))
@pytest.mark.parametrize("mlp,loop", [(None, None), (_moe(4, 2, 24, 20), None), (_dense(50), {"start": 0, "stop": 1, "times": 2}),
                                      (_moe(3, 3, 16), None)])
def test_each_mixer_alone(kind, mlp, loop, tmp_path):
    """A model of one layer: the mixer (and the feed-forward) alone, whole, token by token, and in portions of two;
    also the layer run twice with a cache and state for each pass."""
    cfg = one_layer(LAYERS[kind](mlp), loop=loop)
    tensors = write_model(cfg, str(tmp_path / "m"), seed=11)
    oracle = plain.PlainZasazen(cfg, tensors)
    reqs = {"a": tokens(1, 45, cfg["vocab"])}
    ref, lim, clear = references(oracle, reqs, "float32")
    eng = gpu_engine(str(tmp_path / "m"), "float32")
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 44), cuttings.portions(reqs, sizes=(2,))):
        worst, share = worst_ratio(cuttings.run_trace(eng, steps), ref, lim, clear)
        assert worst < 1.0 and share > 0.9


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_matches_the_plain_model(name, dtype, folders):
    """Prefill against decoding token by token, portions down to two tokens, unequal requests batched against each
    alone, requests long enough to cross pages' borders and many temperature steps in prompts and in decoding, the
    first tokens of a sequence (requests of one and two tokens)."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 2, 23, 150, 310])}
    ref, lim, clear = references(oracle, reqs, dtype)
    page = 64 if name == "C" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=1024 // page)
    mixed, _ = cuttings.mixed(reqs, max_live=4, seed=1, decode_tail=70 if name == "B" else 24)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 140)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        worst, share = worst_ratio(got, ref, lim, clear)
        print(f"{name} {dtype} {what}: worst error / limit {worst:.2f} over {share:.2f} of the positions")
        assert worst < 1.0 and share > (0.9 if dtype == "float32" else 0.25), (what, worst, share)
    assert all(p.used_pages == 0 for p in eng.cache.stats())


def test_cuttings_agree_to_the_last_bit_in_32_bit(folders):
    """In 32-bit every kernel adds in an order of its own that does not depend on the cut: logits are equal bit for
    bit whether a request came whole, token by token, or beside others."""
    folder, _ = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"r{i}": tokens(30 + i, n, V) for i, n in enumerate([5, 60, 33])}
    eng = gpu_engine(folder, "float32")
    base = cuttings.run_trace(eng, cuttings.whole(reqs))
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=4)
    for steps in (cuttings.tail_decode(reqs, 30), cuttings.portions(reqs, sizes=(2, 3)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert all(torch.equal(got[k], base[k]) for k in base)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype, folders):
    folder, oracle = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7, 64, 65])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    eng = gpu_engine(folder, dtype, num_pages=cuttings.peak_tokens(steps) // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    ref, lim, clear = references(oracle, reqs, dtype)
    worst, share = worst_ratio(got, ref, lim, clear)
    assert worst < 1.0 and share > 0.25
    assert all(s.used_pages == 0 for s in eng.cache.stats())


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "bfloat16"), ("C", "bfloat16")])
def test_long_greedy_generation_through_scheduler_and_graphs(name, dtype, folders):
    """Engine.generate: prompts in portions under a token budget, then 200 decode steps replayed from graphs, state
    carried in the slots all the way.  Every produced token is the plain model's choice wherever that is clear, and
    the logits of the last step agree."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    prompts = [tokens(60, 70, V), tokens(61, 3, V), tokens(62, 129, V)]
    page = 64 if name == "C" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=2048 // page, max_step_tokens=48, max_context=512)
    assert eng.use_graphs
    news = [200, 40, 90]
    ids = [eng.submit(p, max_new_tokens=n) for p, n in zip(prompts, news)]
    last = {}
    while eng.scheduler.has_work():
        produced = eng.run_step()
        if len(produced) == 1 and eng.last_logits.shape[0] == 1:
            last["row"] = eng.last_logits[0].float().cpu().clone()
    outs = [eng.result(i) for i in ids]
    assert eng.graphs_recorded > 0 and [len(o) for o in outs] == news
    seqs = {str(i): p + out[:-1] for i, (p, out) in enumerate(zip(prompts, outs))}
    ref, lim, clear = references(oracle, seqs, dtype)
    sure = 0
    for i, (p, out) in enumerate(zip(prompts, outs)):
        for j, tok in enumerate(out):
            at = len(p) - 1 + j
            row = ref[str(i)][at]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if bool(clear[str(i)][at]) and float(top2[0] - top2[1]) > 4 * float(lim[str(i)][at]) * spread:
                assert int(torch.argmax(row)) == tok, (name, dtype, i, j)
                sure += 1
    print(f"{name} {dtype}: {sure} of {sum(news)} tokens were clear choices")
    assert sure >= sum(news) // 16
    if bool(clear["0"][-1]):
        assert float(row_error(last["row"], ref["0"][-1]) / lim["0"][-1]) < 1.0


def test_command_line_with_random_weights(tmp_path):
    """`dlm-b200 generate --random CONFIG.json --save-random DIR`: the architecture is found through the registry,
    the weights are drawn and written, and the ids printed are the plain model's greedy choices on that folder."""
    import ast
    import json
    import os
    import subprocess
    import sys
    from dlm_b200.weights.safetensors_io import TensorStore
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path, folder = str(tmp_path / "config.json"), str(tmp_path / "model")
    with open(cfg_path, "w") as f:
        json.dump(CONFIGS["D"], f)
    prompts = [[5, 6, 7, 40, 3], [9]]
    cmd = [sys.executable, os.path.join(root, "bin", "dlm-b200"), "generate", "--random", cfg_path, "--seed", "3",
           "--save-random", folder, "--max-new-tokens", "6", "--dtype", "float32"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("generated ids:")]
    assert len(lines) == len(prompts)
    store = TensorStore(folder)
    oracle = plain.PlainZasazen(CONFIGS["D"], {n: store.tensor(n).clone() for n in store.names()})
    store.close()
    for p, ln in zip(prompts, lines):
        ids = ast.literal_eval(ln.split(":", 1)[1].strip())
        assert len(ids) == 6
        seq = list(p)
        for tok in ids:
            row = oracle.forward(seq)[-1]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if float(top2[0] - top2[1]) > 1e-3 * spread:
                assert int(torch.argmax(row)) == tok
            seq.append(tok)
