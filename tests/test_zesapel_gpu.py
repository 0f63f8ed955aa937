"""Zesapel on the GPU.  Kernels alone against their plain PyTorch statements, with inputs made so that a
fault shows (one key that stands out at a window's edge and at a page's border, a sink that takes all the
weight, something written into a state hundreds of tokens ago); then the engine against the plain model:
every mixer alone, three configurations of unlike sizes under every cutting in both precisions, slots
and pages that are used again, long greedy decoding through the scheduler and the replayed graphs."""
import math
from types import SimpleNamespace

import pytest
import torch

import cuttings
import plain_zesapel as plain
from plain_ops import PlainOps
from zesapel_models import (CONFIGS, TOL, _delta, _latent, _mamba, _moe, one_layer, references, row_error, tokens,
                            worst_ratio, write_model)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from dlm_b200.ops import native_ops
    return native_ops(fast=True)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zesapel_gpu")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainZesapel(cfg, tensors))
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
def test_streams_and_positions(ops):
    ref = PlainOps()
    T, S, H = 37, 3, 200
    x = randn(T, H, seed=1)
    table = randn(50, H, seed=2).to(torch.bfloat16)
    idx = torch.randint(0, 50, (T,), generator=torch.Generator().manual_seed(3)).to(DEV, torch.int32)
    want = x.clone()
    ref.add_rows(want, table, idx)
    ops.add_rows(x, table, idx)
    assert torch.equal(x, want)
    xs = ops.streams_expand(x, S)
    assert torch.equal(xs, ref.streams_expand(x, S))
    xs = xs + randn(T, S, H, seed=4)
    a, w = randn(S, seed=5), randn(H, seed=6)
    for norm_w in (None, w):
        got = ops.streams_reduce(xs, a, norm_w, 1e-5, torch.float32)
        assert torch.allclose(got, ref.streams_reduce(xs, a, norm_w, 1e-5, torch.float32), rtol=1e-5, atol=1e-5)
    assert torch.allclose(ops.streams_reduce(xs, None, None, 0.0, torch.float32), xs.sum(1), atol=1e-5)
    mix, outw, y = randn(S, S, seed=7), randn(S, seed=8), randn(T, H, seed=9)
    want = xs.clone()
    ref.streams_update(want, mix, outw, y)
    ops.streams_update(xs, mix, outw, y)
    assert torch.allclose(xs, want, rtol=1e-5, atol=1e-5)
    # the update and the next sublayer's read in one pass
    for norm_w in (None, w):
        a1, a2 = xs.clone(), xs.clone()
        got = ops.streams_update_reduce(a1, mix, outw, y, a, norm_w, 1e-5, torch.float32)
        want_h = ref.streams_update_reduce(a2, mix, outw, y, a, norm_w, 1e-5, torch.float32)
        assert torch.allclose(a1, a2, rtol=1e-5, atol=1e-5) and torch.allclose(got, want_h, rtol=1e-4, atol=1e-4)
    with pytest.raises(Exception):
        ops.add_rows(x, table, idx + 50)          # a position beyond the table: reported, not read
        torch.cuda.synchronize()
        ops.check_errors()
    ops.k.take_error_flag()


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_convolution_carries_its_inputs_across_steps(ops, taps):
    """Two requests fed in portions of 1, 2, 5, 1 and 3, 1, 1, 4 tokens: every output equals the convolution
    over the whole sequence; a slot that is zeroed starts a new sequence."""
    C, slots = 70, 5
    w, bias = randn(C, taps, seed=1), randn(C, seed=2)
    seqs = [randn(9, C, seed=3), randn(9, C, seed=4)]
    whole = [plain.causal_conv(s.cpu().double(), w.cpu().double(), bias.cpu().double()) for s in seqs]
    state = torch.zeros(slots + 1, max(taps - 1, 0), C, device=DEV)
    state[3] = 7.0                                    # a used slot ...
    state[3].zero_()                                  # ... is zeroed when a request takes it
    fed = [0, 0]
    for n0, n1 in [(1, 3), (2, 1), (5, 1), (1, 4)]:
        x = torch.cat([seqs[0][fed[0]:fed[0] + n0], seqs[1][fed[1]:fed[1] + n1]])
        wide = torch.cat([randn(n0 + n1, 3, seed=5), x, randn(n0 + n1, 2, seed=6)], dim=1)   # a column slice
        out = ops.causal_conv(wide[:, 3:3 + C], w, bias, state, batch_of([n0, n1], [3, 1]), False, False, torch.float32)
        want = torch.cat([whole[0][fed[0]:fed[0] + n0], whole[1][fed[1]:fed[1] + n1]])
        assert torch.allclose(out.cpu().double(), want, atol=1e-5)
        fed = [fed[0] + n0, fed[1] + n1]
    got = ops.causal_conv(seqs[0], w, None, torch.zeros_like(state), batch_of([9], [0]), True, True, torch.bfloat16)
    v = plain.causal_conv(seqs[0].cpu().double(), w.cpu().double()) + seqs[0].cpu().double()
    assert torch.allclose(got.cpu().double(), plain.silu(v), atol=2e-2, rtol=2e-2)


def test_gated_norm_activation_and_table(ops):
    ref = PlainOps()
    T, groups, gs = 19, 3, 40
    y, gate, w = randn(T, groups * gs, seed=1), randn(T, groups * gs + 8, seed=2), randn(groups * gs, seed=3)
    for mode in ("silu_before", "sigmoid_after"):
        got = ops.gated_rmsnorm(y, gate[:, 8:], w, groups, 1e-5, mode, torch.float32)
        assert torch.allclose(got, ref.gated_rmsnorm(y, gate[:, 8:], w, groups, 1e-5, mode, torch.float32), atol=1e-5, rtol=1e-5)
    a = ops.gated_rmsnorm(y, gate[:, 8:], w, 1, 1e-5, "silu_before", torch.float32)
    assert not torch.allclose(a, got)                 # one group is not three
    for op in ("tanh", "gelu", "silu"):
        assert torch.allclose(ops.activation(gate[:, 3:50], op, torch.float32), ref.activation(gate[:, 3:50], op, torch.float32),
                              atol=1e-6, rtol=1e-5)
    V, top, E = 31, 3, 7
    table = torch.argsort(torch.rand(V, E, generator=torch.Generator().manual_seed(4)), dim=1)[:, :top].to(DEV, torch.int32).contiguous()
    toks = torch.randint(0, V, (23,), generator=torch.Generator().manual_seed(5)).to(DEV, torch.int32)
    ids, wts, offsets, rows, dest = ops.table_route(toks, table, E)
    assert torch.equal(ids, table[toks.long()]) and torch.allclose(wts, torch.full_like(wts, 1 / 3))
    assert int(offsets[-1]) == 23 * top
    for e in range(E):
        got_rows = sorted(rows[int(offsets[e]):int(offsets[e + 1])].tolist())
        assert got_rows == sorted(t for t in range(23) if e in ids[t].tolist())


@pytest.mark.parametrize("heads,P,N,groups", [(4, 24, 16, 2), (2, 136, 64, 1), (3, 8, 40, 3)])
def test_state_space_scan(ops, heads, P, N, groups):
    ref = PlainOps()
    lens = [5, 1, 12]
    T = sum(lens)
    C = heads * P + 2 * groups * N
    xbc, dt = randn(T, C, seed=1), randn(T, heads + 3, seed=2)[:, 3:]
    dt_bias, A_log, D = randn(heads, seed=3, std=0.5), randn(heads, seed=4, std=0.5), randn(heads, seed=5)
    state = randn(6, heads, N, P, seed=6, std=0.3)
    b = batch_of(lens, [4, 0, 2])
    want_state = state.clone().cpu()
    want = ref.ssm_scan(xbc.cpu(), dt.cpu(), dt_bias.cpu(), A_log.cpu(), D.cpu(), want_state, to_cpu(b), heads, P, N, groups)
    got = ops.ssm_scan(xbc, dt, dt_bias, A_log, D, state, b, heads, P, N, groups)
    assert torch.allclose(got.cpu(), want, atol=2e-4, rtol=2e-4)
    assert torch.allclose(state.cpu(), want_state, atol=2e-4, rtol=2e-4)
    assert torch.equal(state[[1, 3, 5]].cpu(), randn(6, heads, N, P, seed=6, std=0.3)[[1, 3, 5]].cpu())   # others untouched


def test_state_space_scan_remembers_a_far_token(ops):
    """With hardly any decay, what token 0 wrote through B = e_3 is read 400 tokens later by C = e_3, and by no
    other C; the state is carried through steps of 399, 1 and 1 tokens."""
    heads, P, N = 2, 24, 16
    T = 401
    xbc = torch.zeros(T, heads * P + 2 * N, device=DEV)
    xbc[0, :heads * P] = torch.arange(1, heads * P + 1, device=DEV).float()
    xbc[0, heads * P + 3] = 1.0                                   # B_0 = e_3
    xbc[T - 1, heads * P + N + 3] = 1.0                           # C_last = e_3
    xbc[T - 2, heads * P + N + 4] = 1.0                           # C before = e_4: sees nothing
    dt = torch.zeros(T, heads, device=DEV)
    A_log = torch.full((heads,), -20.0, device=DEV)
    zeros = torch.zeros(heads, device=DEV)
    state = torch.zeros(3, heads, N, P, device=DEV)
    ys, at = [], 0
    for n in (399, 1, 1):
        ys.append(ops.ssm_scan(xbc[at:at + n], dt[at:at + n], zeros, A_log, zeros, state, batch_of([n], [1]), heads, P, N, 1))
        at += n
    y = torch.cat(ys)
    assert torch.allclose(y[T - 1], math.log(2.0) * xbc[0, :heads * P], rtol=1e-4)    # dt = softplus(0)
    assert float(y[T - 2].abs().max()) == 0.0


@pytest.mark.parametrize("heads,d", [(3, 24), (2, 128), (1, 48)])
def test_delta_scan(ops, heads, d):
    ref = PlainOps()
    lens = [7, 1, 10]
    T, HD = sum(lens), heads * d
    proj = randn(T, 4 * HD + 5, seed=1)
    lw, a_b = randn(T, HD, seed=2), randn(HD, seed=3)
    state = randn(5, heads, d, d, seed=4, std=0.2)
    b = batch_of(lens, [2, 4, 0])
    offs = (HD + 5, 0, 2 * HD + 5, 3 * HD + 5)        # r, k, v, a at offsets of their own
    want_state = state.clone().cpu()
    want = ref.delta_scan(proj.cpu(), offs, lw.cpu(), a_b.cpu(), want_state, to_cpu(b), heads, d, 1e-6, math.exp(-0.5))
    got = ops.delta_scan(proj, offs, lw, a_b, state, b, heads, d, 1e-6, math.exp(-0.5))
    assert torch.allclose(got.cpu(), want, atol=3e-4, rtol=3e-4)
    assert torch.allclose(state.cpu(), want_state, atol=3e-4, rtol=3e-4)


def test_delta_scan_keeps_and_removes_a_far_key(ops):
    """Decay 1 (raw decay very negative) and removal 0: the pair (k = 2 e_5, v) written at token 0 is read by
    r = e_5 at token 300.  With removal 1 a later token with the same key direction takes it out first."""
    heads, d, T = 1, 24, 301
    proj = torch.zeros(T, 4 * d, device=DEV)
    v0 = torch.arange(1, d + 1, device=DEV).float()
    proj[0, d + 5] = 2.0
    proj[0, 2 * d:3 * d] = v0
    proj[T - 1, 5] = 1.0                               # r = e_5
    proj[:, 3 * d:] = -40.0                            # a = sigmoid(-40) = 0
    lw = torch.full((T, d), -40.0, device=DEV)
    a_b = torch.zeros(d, device=DEV)
    state = torch.zeros(2, heads, d, d, device=DEV)
    outs, at = [], 0
    for n in (200, 2, 99):
        outs.append(ops.delta_scan(proj[at:at + n], (0, d, 2 * d, 3 * d), lw[at:at + n], a_b, state, batch_of([n], [0]),
                                   heads, d, 1e-6, math.exp(-0.5)))
        at += n
    assert torch.allclose(torch.cat(outs)[T - 1], 2.0 * v0, rtol=1e-4)
    proj[150, d + 5] = 1.0                             # the same direction with nothing to write (v = 0) ...
    proj[150, 3 * d:] = 40.0                           # ... and full removal
    state.zero_()
    o = ops.delta_scan(proj, (0, d, 2 * d, 3 * d), lw, a_b, state, batch_of([T], [0]), heads, d, 1e-6, math.exp(-0.5))
    assert float(o[T - 1].abs().max()) < 1e-2 * float(v0.max())


def _latent_case(ops, dtype, H, dn, dr, dv, rank, window, page, lens, starts, seed, rot_dims=None):
    """Fills a paged latent cache for requests of ``starts + lens`` tokens through latent_prep (in portions),
    then runs the attention of the last ``lens`` tokens; returns (engine result, plain result, pieces)."""
    ref = PlainOps()
    rot_dims = dr if rot_dims is None else rot_dims
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    total = [s + n for s, n in zip(starts, lens)]
    pages_each = [-(-t // page) for t in total]
    n_pages = sum(pages_each) + 2
    order = torch.randperm(n_pages - 1, generator=g).tolist()       # pages scattered over the pool
    table = torch.full((R, max(pages_each)), -1, dtype=torch.int32)
    k = 0
    for r in range(R):
        for lp in range(pages_each[r]):
            table[r, lp] = order[k]
            k += 1
    cache = torch.zeros(n_pages, 1, page, rank + dr, dtype=dtype, device=DEV)
    inv_freq = torch.tensor([10000.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(max(rot_dims // 2, 1))], device=DEV)
    qn, kvn = torch.ones(8, device=DEV), (1.0 + 0.1 * torch.randn(rank, generator=g)).to(DEV)
    rows = [torch.randn(t, 8 + rank + dr, generator=g).to(DEV) for t in total]
    for r in range(R):
        pos = torch.arange(total[r], dtype=torch.int32, device=DEV)
        slots = (table[r, (pos // page).long().cpu()].to(DEV) * page + pos % page).to(torch.int32)
        ops.latent_prep(rows[r], 0, 8, qn, 8, rank, kvn, dr, inv_freq, rot_dims, pos, slots, 1e-5, cache, dtype)
    b = batch_of(lens, list(range(R)), starts)
    T = sum(lens)
    q = torch.randn(T, H * (dn + dr), generator=g).to(DEV)
    gate = torch.randn(T, H, generator=g).to(DEV)
    w_uk = (torch.randn(H * dn, rank, generator=g) / math.sqrt(rank)).to(DEV, dtype)
    w_uv = (torch.randn(H * dv, rank, generator=g) / math.sqrt(rank)).to(DEV, dtype)
    sink = torch.randn(H, generator=g).to(DEV)
    return dict(q=q, gate=gate, w_uk=w_uk, w_uv=w_uv, sink=sink, cache=cache, table=table.to(DEV), b=b, inv_freq=inv_freq,
                rot_dims=rot_dims, args=(H, dn, dr, dv, rank, window), ref=ref, rows=rows)


def _run_latent(ops, c, scale=0.3, **over):
    """The whole way from projected queries to gated head outputs, on the kernels and on their plain statements."""
    from dlm_b200.parts.attention import latent_attend
    p = dict(c, **over)
    H, dn, dr, dv, rank, window = p["args"]
    w_ukT = p["w_uk"].reshape(H, dn, rank).transpose(1, 2).contiguous()
    w_uv = p["w_uv"].reshape(H, dv, rank).contiguous()

    def cpu(v):
        return v.cpu() if torch.is_tensor(v) else v
    got = latent_attend(ops, p["q"], p["gate"], w_ukT, w_uv, p["sink"], p["cache"], p["table"], p["b"], p["inv_freq"],
                        p["rot_dims"], window, scale)
    want = latent_attend(p["ref"], cpu(p["q"]), cpu(p["gate"]), w_ukT.cpu(), w_uv.cpu(), cpu(p["sink"]), p["cache"].cpu(),
                         p["table"].cpu(), to_cpu(p["b"]), p["inv_freq"].cpu(), p["rot_dims"], window, scale)
    return got.float().cpu(), want.float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dn,dr,dv,rank,window,rot_dims", [(3, 24, 16, 40, 48, 7, 8), (2, 40, 8, 24, 72, 16, 8),
                                                             (4, 64, 32, 64, 160, 33, 32), (1, 16, 24, 16, 300, 0, 24),
                                                             # latents the tensor-core kernel takes (in bfloat16)
                                                             (3, 24, 16, 40, 128, 7, 8), (20, 16, 8, 24, 256, 33, 8),
                                                             (16, 128, 64, 128, 512, 50, 64), (5, 32, 24, 16, 384, 0, 24)])
def test_latent_attention_against_its_statement(ops, dtype, H, dn, dr, dv, rank, window, rot_dims):
    """Prompt portions that start in the middle of a page beside single decoded tokens, pages of 16 scattered over
    the pool, windows shorter than, equal to and longer than a page."""
    c = _latent_case(ops, dtype, H, dn, dr, dv, rank, window, 16, lens=[1, 9, 1, 30], starts=[40, 13, 0, 3], seed=rank,
                     rot_dims=rot_dims)
    got, want = _run_latent(ops, c)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol)
    got2, want2 = _run_latent(ops, c, sink=None, gate=None)
    assert torch.allclose(got2, want2, atol=tol, rtol=tol) and not torch.allclose(got2, got, atol=tol)


@pytest.mark.parametrize("dtype,rank", [(torch.float32, 32), (torch.bfloat16, 128)])
@pytest.mark.parametrize("window,page", [(16, 16), (17, 16), (5, 16), (64, 64), (40, 64), (33, 16)])
def test_latent_attention_finds_the_key_at_the_windows_edge(ops, window, page, dtype, rank):
    """One cached token gets a rotated key part that the query's rotated part loves (no rotation: rot_dims 0).
    A query at distance window - 1 returns that token's value; at distance window it does not see it.  Decoded
    alone and inside a prompt portion, with the key at the last place of a page and at the first of the next."""
    H, dn, dr, dv = 2, 8, 8, 8
    tol = 1e-3 if dtype == torch.float32 else 4e-2
    for key_pos in (page - 1, page, 2 * page + 3, 31, 32):
        c = _latent_case(ops, dtype, H, dn, dr, dv, rank, window, page, lens=[1, 1, 6], starts=[key_pos + window - 1,
                         key_pos + window, key_pos + window - 3], seed=key_pos, rot_dims=0)
        # the three requests hold the same kind of cache; plant the key in each at key_pos
        cache, table = c["cache"], c["table"]
        for r in range(3):
            pg = int(table[r, key_pos // page])
            cache[pg, 0, key_pos % page, rank:] = torch.tensor([30.0, 0, 0, 0, 0, 0, 0, 0], device=DEV).to(dtype)
        q = torch.zeros_like(c["q"]).reshape(-1, H, dn + dr)
        q[:, :, dn] = 30.0                                   # every query loves that direction
        got, want = _run_latent(ops, c, q=q.reshape(c["q"].shape), gate=None, sink=None, scale=1.0)
        assert torch.allclose(got, want, atol=tol / 10, rtol=tol / 10)
        wv = c["w_uv"].float().reshape(H, dv, rank)

        def value_of(r):
            pg = int(table[r, key_pos // page])
            return torch.einsum("hdr,r->hd", wv, cache[pg, 0, key_pos % page, :rank].float()).reshape(-1).cpu()
        assert torch.allclose(got[0], value_of(0), atol=tol)                       # decoded, distance window - 1: seen
        assert not torch.allclose(got[1], value_of(1), atol=1e-1)                  # decoded, distance window: not seen
        # the portion holds positions key_pos + window - 3 .. + 2: the first three see the key, the others do not
        for i in range(6):
            assert torch.allclose(got[2 + i], value_of(2), atol=tol if i < 3 else 1e-1) == (i < 3)


def test_latent_attention_sink_takes_the_weight(ops):
    c = _latent_case(ops, torch.float32, 2, 8, 4, 8, 32, 9, 16, lens=[1, 4], starts=[20, 0], seed=3)
    got, want = _run_latent(ops, c, gate=None)
    big, want_big = _run_latent(ops, c, gate=None, sink=torch.full((2,), 60.0, device=DEV))
    assert torch.allclose(got, want, atol=1e-4) and torch.allclose(big, want_big, atol=1e-6)
    assert float(big.abs().max()) < 1e-6 * max(float(got.abs().max()), 1.0)
    first = _run_latent(ops, c, gate=None, sink=torch.zeros(2, device=DEV), q=torch.zeros_like(c["q"]))[0]
    # position 0 of the second request: one key with score 0 beside a sink of 0 -> half the value
    alone = _run_latent(ops, c, gate=None, sink=None, q=torch.zeros_like(c["q"]))[0]
    assert torch.allclose(first[1], 0.5 * alone[1], atol=1e-5)


# ====================================================== the engine against the plain model
def gpu_engine(folder, dtype, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype=dtype, device=DEV, page_size=16, num_pages=64, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


def worst_error(got, ref):
    return max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items())


LAYERS = {"state_space": _mamba(3, 24, 16, 3, 4, 2), "latent": _latent(3, 24, 16, 40, 48, 40, 7, 10000.0, dims=8, scale=0.17),
          "delta": _delta(3, 24)}


@pytest.mark.parametrize("kind", list(LAYERS))
@pytest.mark.parametrize("mlp,taps", [(None, 3), (_moe(4, 2, 24), 3), (_moe(4, 2, 24), 1)])
def test_each_mixer_alone(kind, mlp, taps, tmp_path):
    """A model of one layer: the mixer (and the experts) alone, whole, token by token, and in portions of two;
    also with an input convolution of a single tap (nothing carried from step to step)."""
    cfg = one_layer(LAYERS[kind], mlp=mlp, taps=taps)
    tensors = write_model(cfg, str(tmp_path / "m"), seed=11)
    oracle = plain.PlainZesapel(cfg, tensors)
    reqs = {"a": tokens(1, 45, cfg["vocab"])}
    ref = {"a": oracle.forward(reqs["a"])}
    eng = gpu_engine(str(tmp_path / "m"), "float32")
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 44), cuttings.portions(reqs, sizes=(2,))):
        assert worst_error(cuttings.run_trace(eng, steps), ref) < TOL["float32"]


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_matches_the_plain_model(name, dtype, folders):
    """Prefill against decoding token by token, portions down to two tokens, unequal requests batched against each
    alone, requests long enough for every window to pass over pages' borders in prompts and in decoding."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 2, 23, 150, 310])}
    ref, lim = references(oracle, reqs, dtype)
    page = 64 if name == "Z" else 16
    eng = gpu_engine(folder, dtype, page_size=page, num_pages=1024 // page)
    mixed, _ = cuttings.mixed(reqs, max_live=4, seed=1, decode_tail=70 if name == "Y" else 24)
    for what, steps in (("whole", cuttings.whole(reqs)), ("decode", cuttings.tail_decode(reqs, 140)),
                        ("portions", cuttings.portions(reqs)), ("mixed", mixed)):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        worst = worst_error(got, ref)
        print(f"{name} {dtype} {what}: worst relative error {worst:.2e}, worst error / limit {worst_ratio(got, ref, lim):.2f}")
        assert worst_ratio(got, ref, lim) < 1.0, (what, worst)
    assert all(p.used_pages == 0 for p in eng.cache.stats())


def test_cuttings_agree_to_the_last_bit_in_32_bit(folders):
    """In 32-bit every kernel adds in an order of its own that does not depend on the cut: logits are equal bit for
    bit whether a request came whole, token by token, or beside others."""
    folder, _ = folders["X"]
    V = CONFIGS["X"]["vocab"]
    reqs = {f"r{i}": tokens(30 + i, n, V) for i, n in enumerate([5, 60, 33])}
    eng = gpu_engine(folder, "float32")
    base = cuttings.run_trace(eng, cuttings.whole(reqs))
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=4)
    for steps in (cuttings.tail_decode(reqs, 30), cuttings.portions(reqs, sizes=(2, 3)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert all(torch.equal(got[k], base[k]) for k in base)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype, folders):
    folder, oracle = folders["X"]
    V = CONFIGS["X"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7, 64, 65])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    eng = gpu_engine(folder, dtype, num_pages=cuttings.peak_tokens(steps) // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    ref, lim = references(oracle, reqs, dtype)
    assert worst_ratio(got, ref, lim) < 1.0
    stats = eng.cache.stats()
    assert all(s.used_pages == 0 for s in stats)


@pytest.mark.parametrize("name,dtype", [("Y", "float32"), ("X", "bfloat16"), ("Z", "bfloat16")])
def test_long_greedy_generation_through_scheduler_and_graphs(name, dtype, folders):
    """Engine.generate: prompts in portions under a token budget, then 200 decode steps replayed from graphs, state
    carried in the slots all the way.  Every produced token is the plain model's choice wherever that is clear, and
    the logits of the last step agree."""
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    prompts = [tokens(60, 70, V), tokens(61, 3, V), tokens(62, 129, V)]
    page = 64 if name == "Z" else 16
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
    ref, lim = references(oracle, seqs, dtype)
    clear = 0
    for i, (p, out) in enumerate(zip(prompts, outs)):
        for j, tok in enumerate(out):
            at = len(p) - 1 + j
            row = ref[str(i)][at]
            top2 = torch.topk(row, 2).values
            spread = float((row - row.mean()).pow(2).mean().sqrt())
            if float(top2[0] - top2[1]) > 4 * float(lim[str(i)][at]) * spread:      # the plain model's choice is clear
                assert int(torch.argmax(row)) == tok, (name, dtype, i, j)
                clear += 1
    print(f"{name} {dtype}: {clear} of {sum(news)} tokens were clear choices")
    assert clear >= sum(news) // 8
    # the longest request decodes alone at the end: its last step's logits against the plain model
    assert float(row_error(last["row"], ref["0"][-1]) / lim["0"][-1]) < 1.0


def test_command_line_with_random_weights(tmp_path):
    """`dlm-b200 generate --random CONFIG.json --save-random DIR`: the architecture is found through the registry,
    the weights are drawn and written, and the ids printed are the plain model's greedy choices on that folder."""
    import ast
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path, folder = str(tmp_path / "config.json"), str(tmp_path / "model")
    with open(cfg_path, "w") as f:
        json.dump(CONFIGS["X"], f)
    prompts = [[5, 6, 7, 100, 3], [9]]
    cmd = [sys.executable, os.path.join(root, "bin", "dlm-b200"), "generate", "--random", cfg_path, "--seed", "3",
           "--save-random", folder, "--max-new-tokens", "6", "--dtype", "float32"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("generated ids:")]
    assert len(lines) == len(prompts)
    oracle = plain.PlainZesapel(folder)
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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,E,top,K,N", [(3, 4, 2, 64, 96), (200, 6, 2, 128, 256), (40, 16, 2, 256, 512), (17, 3, 1, 90, 34),
                                         (700, 8, 2, 1024, 1024), (9, 32, 2, 2048, 2048)])
def test_experts_first_product_with_gelu_in_its_epilogue(ops, dtype, T, E, top, K, N):
    """`grouped_act(..., "gelu")` on every product kernel the sizes reach (streaming, tcgen05 single and paired,
    warp-level, FMA) against the plain statement; silu goes through the separate activation kernel."""
    ref = PlainOps()
    g = torch.Generator().manual_seed(T + K)
    h = torch.randn(T, K, generator=g).to(DEV, dtype)
    w = (torch.randn(E, N, K, generator=g) / math.sqrt(K)).to(DEV, dtype)
    table = torch.argsort(torch.rand(50, E, generator=g), dim=1)[:, :top].to(DEV, torch.int32).contiguous()
    toks = torch.randint(0, 50, (T,), generator=g).to(DEV, torch.int32)
    _, _, offsets, rows, _ = ops.table_route(toks, table, E)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for act in ("gelu", "silu"):
        got = ops.grouped_act(h, w, offsets, rows, act)
        want = ref.grouped_act(h.cpu(), w.cpu(), offsets.cpu(), rows.cpu(), act)
        assert got.dtype == dtype and torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=tol), act
    torch.cuda.synchronize()
    ops.check_errors()
