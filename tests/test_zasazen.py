"""Zasazen without a GPU: the config reader and registry, the order of layer calls with repeated passes, tensor
names and shapes, the plain implementation's own hand-made cases, and the engine's host side (cache, state slots,
step function, scheduler, replay) with the plain PyTorch statement of the kernels standing in for them."""
import copy
import io
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

import cuttings
import plain_zasazen as plain
from plain_ops import PlainOps
from zasazen_models import (CONFIGS, TOL, _dense, _left, _mamba, _moe, _parallel, _right, make_weights, one_layer,
                            row_error, tokens, write_model)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zasazen")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainZasazen(cfg, tensors))
    return out


def cpu_engine(folder, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=40, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


# ------------------------------------------------------------------ config, registry, tensors
def test_registry_resolves_the_architecture_and_round_trips_the_config():
    from dlm_b200.config import ZasazenConfig
    from dlm_b200.registry import architectures, resolve
    assert "Zasazen" in architectures()
    for cfg in CONFIGS.values():
        name, typed, spec = resolve(copy.deepcopy(cfg))
        assert name == "Zasazen" and isinstance(typed, ZasazenConfig)
        assert len(spec.layers) == len(cfg["layers"]) and spec.embed_scale == cfg["embedding"]["scale"]
        assert spec.vocab_size == cfg["vocab"] and (spec.pass_entry is not None) == ("loop" in cfg)
        assert ZasazenConfig.from_dict(typed.to_dict()) == typed


def test_order_of_layer_calls_with_a_repeated_run():
    from dlm_b200.models.zasazen import layer_order
    calls = layer_order(5, {"start": 1, "stop": 3, "times": 3})
    assert [c.layer for c in calls] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [c.enters_pass for c in calls] == [None, 0, None, 1, None, 2, None, None, None]
    assert [c.layer for c in layer_order(3, None)] == [0, 1, 2]
    whole = layer_order(2, {"start": 0, "stop": 2, "times": 1})
    assert [(c.layer, c.enters_pass) for c in whole] == [(0, 0), (1, None)]
    one = layer_order(3, {"start": 2, "stop": 3, "times": 2})
    assert [(c.layer, c.enters_pass) for c in one] == [(0, None), (1, None), (2, 0), (2, 1)]


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("layers"), "layers"),
    (lambda c: c["layers"][0].update(type="conv_mixer"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "mlp"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_refusals(edit, what):
    from dlm_b200.config import ConfigError
    from dlm_b200.registry import resolve
    cfg = copy.deepcopy(CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        resolve(cfg)
    assert what.split(".")[0] in str(e.value)


def test_tensor_names_and_shapes_are_the_checkpoints():
    from dlm_b200.parts import DecoderModel, Runtime, WeightError
    from dlm_b200.registry import resolve
    for name, cfg in CONFIGS.items():
        _, _, spec = resolve(copy.deepcopy(cfg))
        model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
        tensors = make_weights(cfg)
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()})      # nothing missing, nothing extra
        for i, L in enumerate(cfg["layers"]):
            if L["mlp"] is None:
                assert not any(n.startswith(f"l{i}.mlp") or n == f"l{i}.norm2" for n in model.param_specs())
        assert ("loop.in" in model.param_specs()) == ("loop" in cfg)
    cfg = CONFIGS["A"]
    _, _, spec = resolve(copy.deepcopy(cfg))
    model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
    bad = make_weights(cfg)
    bad.pop("l0.mix.right.out")
    bad.pop("l1.mlp.router.b")
    bad["loop.step"] = torch.zeros(5, cfg["width"])
    bad["l2.mix.left.sink"] = torch.zeros(4)
    with pytest.raises(WeightError) as e:
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in bad.items()})
    for n in ("l0.mix.right.out", "l1.mlp.router.b", "loop.step", "l2.mix.left.sink"):
        assert n in str(e.value)


def test_random_weights_for_a_config_build_and_load(tmp_path):
    from dlm_b200.config import ZasazenConfig
    from dlm_b200.engine import Engine
    from dlm_b200.weights import write_random_model
    cfg = ZasazenConfig.from_dict(copy.deepcopy(CONFIGS["D"]))
    folder = write_random_model(cfg, 5, str(tmp_path / "m"))
    toks = tokens(1, 20, cfg.vocab)
    a = cpu_engine(folder)
    b = Engine.from_random(cfg, 5, dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=8, max_requests=2)
    sa, sb = a.cache.open(), b.cache.open()
    la, lb = a.step([(sa, toks, [19])]), b.step([(sb, toks, [19])])
    assert torch.allclose(la, lb, atol=1e-5)
    assert torch.isfinite(la).all() and float(la.std()) > 0


# --------------------------------------------------------- the plain implementation's own cases
def test_plain_retention_is_the_decayed_sum_over_the_past():
    """o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s, worked out directly (no rotation, one head)."""
    T, W, d, dv = 7, 5, 3, 2
    g = torch.Generator().manual_seed(0)
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    t = {n: torch.randn(r, W, generator=g, dtype=torch.float64) for n, r in (("q", d), ("k", d), ("v", dv), ("g", dv))}
    t["o"] = torch.eye(dv, dtype=torch.float64)
    m = {"heads": 1, "dim": d, "vdim": dv, "decay": [0.8]}
    got = plain.retention(h, t.__getitem__, m, 1e-6)
    q, k, v, gate = (h @ t[n].T for n in "qkvg")
    k = k * d ** -0.5
    for i in range(T):
        o = sum(0.8 ** (i - s) * float(q[i] @ k[s]) * v[s] for s in range(i + 1))
        o = o / torch.sqrt((o * o).mean() + 1e-6) * plain.silu(gate[i])
        assert torch.allclose(got[i], o, atol=1e-12)


def test_plain_attention_distance_penalty_temperature_and_far_keys():
    """One head, keys and values read off the input: without a penalty a far key that matches the query wins; the
    penalty slope * distance takes the weight back; the temperature multiplies the scores from its period on."""
    assert torch.allclose(plain.distance_slopes(4), torch.tensor([0.25, 0.0625, 0.015625, 0.00390625], dtype=torch.float64))
    T, W = 40, 4
    h = torch.zeros(T, W, dtype=torch.float64)
    h[:, 0] = 1.0
    h[3, 1] = 1.0                                    # token 3 carries a value that stands out
    eye = torch.eye(W, dtype=torch.float64)
    t = {"q": eye[:1], "k": eye[:1], "v": eye[1:2], "q.b": torch.zeros(1), "k.b": torch.zeros(1), "v.b": torch.zeros(1),
         "q.norm": torch.ones(1), "k.norm": torch.ones(1), "o": torch.ones(W, 1)}
    t = {k: v.double() for k, v in t.items()}
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0}
    out = plain.biased_attention(h, t.__getitem__, m, 0.0)
    # every score is 1 (unit q and k): weights are exp(-slope * distance) / sum with slope 2^-8
    s = 2.0 ** -8
    for i in (3, 10, 39):
        w = torch.exp(-s * (i - torch.arange(i + 1, dtype=torch.float64)))
        assert abs(float(out[i, 0]) - float(w[3] / w.sum())) < 1e-12
    # the temperature: 1 + coef * ln(floor((p + 1) / every) + 1)
    h2 = torch.randn(T, W, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    t2 = dict(t, **{"q.norm": torch.ones(1).double() * 3.0})
    a = plain.biased_attention(h2, t2.__getitem__, dict(m, q_temp={"coef": 0.5, "every": 8}), 1e-6)
    b = plain.biased_attention(h2, t2.__getitem__, m, 1e-6)
    assert torch.allclose(a[:7], b[:7], atol=1e-14) and not torch.allclose(a[7], b[7], atol=1e-6)
    c = plain.biased_attention(h2, t2.__getitem__, dict(m, scale=1.0 + 0.5 * math.log(2.0)), 1e-6)
    assert torch.allclose(a[7:15], c[7:15], atol=1e-12) and not torch.allclose(a[15], c[15], atol=1e-6)


def test_plain_routing_with_every_expert_chosen_is_the_softmax_of_all():
    W, E, ff, T = 6, 3, 4, 9
    g = torch.Generator().manual_seed(2)
    t = {"router": torch.randn(E, W, generator=g), "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        t.update({f"e{e}.gate": torch.randn(ff, W, generator=g), f"e{e}.up": torch.randn(ff, W, generator=g),
                  f"e{e}.down": torch.randn(W, ff, generator=g)})
    t = {k: v.double() for k, v in t.items()}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = plain.routed_ff(h, t.__getitem__, {"router": {"experts": E, "top": E}})
    w = torch.softmax(h @ t["router"].T + t["router.b"], dim=-1)
    want = sum(w[:, e:e + 1] * plain.gated_expert(h, t.__getitem__, f"e{e}", False) for e in range(E))
    assert torch.allclose(got, want, atol=1e-12)
    one = plain.routed_ff(h, t.__getitem__, {"router": {"experts": E, "top": 1}})
    best = torch.argmax(h @ t["router"].T + t["router.b"], dim=-1)
    for i in range(T):
        assert torch.allclose(one[i], plain.gated_expert(h[i:i + 1], t.__getitem__, f"e{int(best[i])}", False)[0], atol=1e-12)


def test_plain_selective_scan_forgets_at_the_rate_of_its_step_size():
    """With B = C = 1 (one state), x = 1 and a constant step size the state is the geometric sum."""
    T, inner = 6, 2
    h = torch.ones(T, 1, dtype=torch.float64)
    t = {"in": torch.tensor([[1.0], [1.0], [50.0], [50.0]]), "conv": torch.tensor([[1.0], [1.0]]), "conv.b": torch.zeros(2),
         "x": torch.tensor([[0.0, 0.0], [0.0, 0.0], [0.0, 0.0]]), "dt": torch.zeros(2, 1), "dt.b": torch.tensor([0.0, 1.0]),
         "A_log": torch.zeros(2, 1), "D": torch.zeros(2), "o": torch.eye(2)}
    t = {k: v.double() for k, v in t.items()}
    m = {"inner": inner, "state": 1, "dt_rank": 1, "conv": 1}
    # B = C = 0 from a zero projection: only D x would come through, and D is 0
    assert plain.selective_scan_mixer(h, t.__getitem__, m).abs().max() == 0
    t["x"] = torch.tensor([[0.0, 0.0], [1.0, 0.0], [1.0, 0.0]], dtype=torch.float64)     # B = C = silu(1) (x of channel 0)
    out = plain.selective_scan_mixer(h, t.__getitem__, m)
    x = float(plain.silu(torch.tensor(1.0, dtype=torch.float64)))
    # the gate is silu(50)
    z = 50.0 / (1.0 + math.exp(-50.0))
    out = out / z
    for c, dt in enumerate((math.log(2.0), math.log1p(math.e))):
        S = 0.0
        for i in range(T):
            S = math.exp(-dt) * S + dt * x * x
            assert abs(float(out[i, c]) - S * x) < 1e-12


# ----------------------------------------------------------------- engine host side on the CPU
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_every_cutting_matches_the_plain_model(name, folders):
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 2, 19, 44])}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=3, seed=1)
    worst = 0.0
    for steps in (cuttings.whole(reqs), cuttings.tail_decode(reqs, 20), cuttings.portions(reqs), mixed):
        got = cuttings.run_trace(eng, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (rid, p), row in got.items():
            worst = max(worst, float(row_error(row, ref[rid][p])))
    print(f"{name}: worst relative error {worst:.2e}")
    assert worst < TOL["float32"]
    assert all(p.used_pages == 0 for p in eng.cache.stats())


def test_residual_after_every_layer_run_matches(folders):
    """Every pass of a repeated run has a cache and state of its own: the residual after each call of the order
    against the plain model's, for a request fed in two portions."""
    folder, oracle = folders["A"]
    toks = tokens(3, 21, CONFIGS["A"]["vocab"])
    _, want = oracle.forward(toks, return_layers=True)
    eng = cpu_engine(folder)
    seen = []
    for block in eng.model.blocks:
        real = block.forward
        block.forward = (lambda real: lambda x, ctx, call: (real(x, ctx, call), seen.append((call, x.clone())))[0])(real)
    slot = eng.cache.open()
    eng.step([(slot, toks[:13], [])])
    eng.step([(slot, toks[13:], [])])
    calls = len(eng.model.order)
    assert calls == want.shape[0] == 6 and len(seen) == 2 * calls
    for call in range(calls):
        got = torch.cat([x for c, x in seen if c == call]).double()
        assert float((got - want[call]).abs().max()) < 1e-4 * float(want[call].abs().max())


def test_slots_and_pages_are_used_again_with_fresh_state(folders):
    folder, oracle = folders["A"]
    V = CONFIGS["A"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([40, 33, 65, 16, 50, 7])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    peak = cuttings.peak_tokens(steps)
    eng = cpu_engine(folder, num_pages=peak // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    worst = max(float(row_error(row, oracle.forward(reqs[rid][:p + 1])[-1])) for (rid, p), row in got.items()
                if p in (0, 1, 2, len(reqs[rid]) - 1))
    assert worst < TOL["float32"]
    assert all(s.used_pages == 0 for s in eng.cache.stats())


def test_greedy_generation_through_the_scheduler(folders):
    folder, oracle = folders["B"]
    V = CONFIGS["B"]["vocab"]
    prompts = [tokens(40, 5, V), tokens(41, 37, V), tokens(42, 1, V)]
    eng = cpu_engine(folder, max_step_tokens=16)
    outs = eng.generate(prompts, max_new_tokens=6)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            row = oracle.forward(seq)[-1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 1e-3:
                assert int(torch.argmax(row)) == tok
            seq.append(tok)
    alone = [cpu_engine(folder).generate(p, max_new_tokens=6) for p in prompts]
    assert alone == outs


def test_replay_program_on_the_stand_in(folders, tmp_path, monkeypatch):
    from dlm_b200.engine import replay, Engine
    folder, oracle = folders["D"]
    V = CONFIGS["D"]["vocab"]
    reqs = {"a": tokens(50, 30, V), "b": tokens(51, 9, V)}
    steps, _ = cuttings.mixed(reqs, max_live=2, seed=3)
    real = Engine.from_pretrained
    monkeypatch.setattr(Engine, "from_pretrained", classmethod(
        lambda cls, path, **kw: real(path, **dict(kw, device="cpu", ops=PlainOps()))))
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out_dir = str(tmp_path / "out")
    assert replay.main(["--model", folder, "--dtype", "float32", "--out", out_dir, "--max-tokens", "128",
                        "--page-size", "16", "--device", "cpu"]) == 0
    fed = {r: 0 for r in reqs}
    for st in steps:
        rows = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4").reshape(-1, V)
        k = 0
        for e in st["entries"]:
            ref = oracle.forward(reqs[e["id"]][:fed[e["id"]] + len(e["tokens"])])
            for w in e["want"]:
                assert float(row_error(torch.from_numpy(rows[k].copy()), ref[fed[e["id"]] + w])) < TOL["float32"]
                k += 1
            fed[e["id"]] += len(e["tokens"])


@pytest.mark.parametrize("kind", ["scan", "pair", "pair_dense_loop"])
def test_models_of_one_layer(kind, tmp_path):
    """A model without any paged cache (the scan only: tokens are still counted against the pool), a pair of mixers
    without a feed-forward, and a single layer repeated three times."""
    layer = {"scan": _mamba(24, 6, 2, 3, _moe(3, 2, 16)),
             "pair": _parallel(_left(2, 1, 8, 12, 0.3, (0.4, 3)), _right(2, 6, 10, [0.9, 0.5], (100.0, 4)), None),
             "pair_dense_loop": _parallel(_left(4, 2, 6, 4, 0.5), _right(1, 10, 6, [0.95]), _dense(40))}[kind]
    cfg = one_layer(layer, width=32, vocab=41, loop={"start": 0, "stop": 1, "times": 3} if kind.endswith("loop") else None)
    folder = str(tmp_path / "m")
    oracle = plain.PlainZasazen(cfg, write_model(cfg, folder, seed=5))
    reqs = {"a": tokens(1, 40, 41), "b": tokens(2, 7, 41)}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=2, seed=6)
    for steps in (cuttings.whole(reqs), cuttings.portions(reqs, sizes=(2, 5)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items()) < TOL["float32"]
