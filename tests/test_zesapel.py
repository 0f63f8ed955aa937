"""Zesapel without a GPU: the config reader and registry, tensor names and shapes, the plain
implementation's own hand-made cases, and the engine's host side (cache, state slots, step function,
scheduler, replay) with the plain PyTorch statement of the kernels standing in for them."""
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
import plain_zesapel as plain
from plain_ops import PlainOps
from zesapel_models import CONFIGS, TOL, make_weights, one_layer, row_error, tokens, write_model


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zesapel")
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(base / name)
        tensors = write_model(cfg, folder, seed=len(name) + ord(name))
        out[name] = (folder, plain.PlainZesapel(cfg, tensors))
    return out


def cpu_engine(folder, **kw):
    from dlm_b200.engine import Engine
    args = dict(dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=40, max_requests=4)
    args.update(kw)
    return Engine.from_pretrained(folder, **args)


# ------------------------------------------------------------------ config, registry, tensors
def test_registry_resolves_the_architecture_and_round_trips_the_config():
    from dlm_b200.config import ZesapelConfig
    from dlm_b200.registry import architectures, resolve
    assert "Zesapel" in architectures()
    for cfg in CONFIGS.values():
        name, typed, spec = resolve(copy.deepcopy(cfg))
        assert name == "Zesapel" and isinstance(typed, ZesapelConfig)
        assert len(spec.layers) == len(cfg["layers"]) and spec.residual_streams == cfg["streams"]
        assert spec.embed_scale == cfg["embedding"]["scale"] and spec.vocab_size == cfg["vocab"]
        again = ZesapelConfig.from_dict(typed.to_dict())
        assert again == typed and typed.max_position_embeddings == cfg["max_positions"]


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.pop("layers"), "layers"),
    (lambda c: c["layers"][0].update(type="conv_mixer"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(streams=40), "streams"),
])
def test_config_refusals(edit, what):
    from dlm_b200.config import ConfigError
    from dlm_b200.registry import resolve
    cfg = copy.deepcopy(CONFIGS["X"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        resolve(cfg)
    assert what.split(".")[0] in str(e.value)


def test_tensor_names_and_shapes_are_the_checkpoints(folders):
    from dlm_b200.parts import DecoderModel, Runtime, WeightError
    from dlm_b200.registry import resolve
    for name, cfg in CONFIGS.items():
        _, _, spec = resolve(copy.deepcopy(cfg))
        model = DecoderModel(spec, Runtime("cpu", torch.float32, None))
        tensors = make_weights(cfg)
        model.check({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()})      # nothing missing, nothing extra
        layer_without_ffn = [i for i, L in enumerate(cfg["layers"]) if L["mlp"] is None]
        for i in layer_without_ffn:
            assert not any(n.startswith(f"l{i}.mlp") or n.startswith(f"l{i}.hc2") for n in model.param_specs())
        bad = dict(tensors)
        bad.pop("l1.hc1.mix")
        bad["l0.norm1"] = torch.zeros(cfg["width"] + 1)
        bad["l1.mlp.table" if cfg["layers"][1]["mlp"] else "l2.mlp.table"] = torch.zeros(cfg["vocab"], 2)
        with pytest.raises(WeightError) as e:
            model.check({n: (t.dtype, tuple(t.shape)) for n, t in bad.items()})
        assert "l1.hc1.mix" in str(e.value) and "l0.norm1" in str(e.value) and "mlp.table" in str(e.value)


def test_random_weights_for_a_config_build_and_load(tmp_path):
    """The random-weights mode (what the command line's --random / --save-random use): tables hold distinct
    ids below the number of experts, the written folder loads again and gives the same logits."""
    from dlm_b200.config import ZesapelConfig
    from dlm_b200.engine import Engine
    from dlm_b200.weights import write_random_model
    from dlm_b200.weights.safetensors_io import TensorStore
    cfg = ZesapelConfig.from_dict(copy.deepcopy(CONFIGS["X"]))
    folder = write_random_model(cfg, 5, str(tmp_path / "m"))
    store = TensorStore(folder)
    table = store.tensor("l1.mlp.table")
    assert table.dtype == torch.int32 and int(table.max()) < 5 and int(table.min()) >= 0
    assert all(len(set(r)) == len(r) for r in table.tolist())
    assert store.tensor("l2.mix.w1").shape[1] == cfg.width
    store.close()
    toks = tokens(1, 20, cfg.vocab)
    a = cpu_engine(folder)
    b = Engine.from_random(cfg, 5, dtype="float32", device="cpu", ops=PlainOps(), page_size=16, num_pages=8, max_requests=2)
    sa, sb = a.cache.open(), b.cache.open()
    la, lb = a.step([(sa, toks, [19])]), b.step([(sb, toks, [19])])
    assert torch.allclose(la, lb, atol=1e-5)
    assert torch.isfinite(la).all() and float(la.std()) > 0


# --------------------------------------------------------- the plain implementation's own cases
def test_plain_convolution_and_rotation_by_hand():
    x = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 1.0, 2.0], [0.0, 0.0, 1.0]], dtype=torch.float64)      # the last tap is the current token's
    out = plain.causal_conv(x, w)
    assert out[:, 0].tolist() == [2.0, 5.0, 8.5] and out[:, 1].tolist() == [10.0, 20.0, 30.0]
    v = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 5.0]]], dtype=torch.float64)            # dims 4 rotate, the fifth passes
    r = plain.rotate_half_pairs(v, torch.tensor([1]), 100.0, 4)
    a0, a1 = 1.0, 100.0 ** -0.5
    want = [math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1), 5.0]
    assert torch.allclose(r[0, 0], torch.tensor(want, dtype=torch.float64))


def test_plain_window_edge_and_sink():
    """With one head, identity-like projections and a query that loves one key, the key just inside the window
    is found and the key just outside is not; a large sink takes the weight away from every key."""
    m = {"heads": 1, "dim": 2, "rot_dim": 2, "vdim": 2, "kv_rank": 2, "q_rank": 2, "mask": {"size": 4},
         "rot": {"base": 10.0, "dims": 0}, "scale": 1.0}
    T = 8
    h = torch.zeros(T, 4, dtype=torch.float64)
    h[:, 0] = 1.0                                   # every token: the same query direction and a constant latent part
    h[2, 1] = 30.0                                  # token 2 carries a key (and value) that stands out
    t = {"mix.dq": torch.tensor([[1.0, 0, 0, 0], [0, 0.0, 0, 0]]), "mix.dq.norm": torch.ones(2), "mix.uq": torch.tensor(
        [[0.0, 0], [0, 0], [20.0, 0], [0, 0]]), "mix.dkv": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [0, 1.0, 0, 0], [0, 0, 0, 0.0]]),
         "mix.dkv.norm": torch.ones(2), "mix.uk": torch.zeros(2, 2), "mix.uv": torch.eye(2), "mix.sink": torch.tensor([-50.0]),
         "mix.g": torch.tensor([[50.0, 0, 0, 0]]), "mix.o": torch.eye(4)[:, :2]}
    t = {k: v.double() for k, v in t.items()}
    out = plain.latent_attention(h, t.__getitem__, m, 0.0, torch.arange(T))
    # the value of token 2 is its normalised latent (about [0.047, 1.41]); others' is [1.41, 0]
    assert out[5, 1] > 1.3 and out[6, 1] < 1e-6      # position 5 still sees token 2 (5 - 2 < 4), position 6 does not
    t["mix.sink"] = torch.tensor([5000.0], dtype=torch.float64)
    assert plain.latent_attention(h, t.__getitem__, m, 0.0, torch.arange(T)).abs().max() < 1e-6


# ----------------------------------------------------------------- engine host side on the CPU
@pytest.mark.parametrize("name", ["X", "Y"])
def test_every_cutting_matches_the_plain_model(name, folders):
    folder, oracle = folders[name]
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": tokens(i, n, V) for i, n in enumerate([1, 17, 40, 75])}
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


def test_slots_and_pages_are_used_again_with_fresh_state(folders):
    """Six requests through three slots and a pool that holds only what is live: a request that takes a used
    slot starts from zero state, and window pages go back while a request runs."""
    folder, oracle = folders["X"]
    V = CONFIGS["X"]["vocab"]
    reqs = {f"q{i}": tokens(20 + i, n, V) for i, n in enumerate([70, 33, 129, 16, 90, 7])}
    steps, _ = cuttings.mixed(reqs, max_live=3, seed=2)
    peak = cuttings.peak_tokens(steps)
    eng = cpu_engine(folder, num_pages=peak // 16, max_requests=3)
    got = cuttings.run_trace(eng, steps)
    worst = max(float(row_error(row, oracle.forward(reqs[rid][:p + 1])[-1])) for (rid, p), row in got.items()
                if p in (0, 1, 2, len(reqs[rid]) - 1))
    assert worst < TOL["float32"]
    stats = eng.cache.stats()
    assert all(s.used_pages == 0 for s in stats) and min(s.high_water for s in stats) < max(s.high_water for s in stats)


def test_greedy_generation_through_the_scheduler(folders):
    """Engine.generate (scheduler, portions under a token budget, sampling, commit) against greedy decoding with
    the plain model; batched prompts give what each gives alone."""
    folder, oracle = folders["Y"]
    V = CONFIGS["Y"]["vocab"]
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
    folder, oracle = folders["X"]
    V = CONFIGS["X"]["vocab"]
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


@pytest.mark.parametrize("kinds", [("delta", "ssm"), ("latent", "latent"), ("ssm",)])
def test_models_of_one_kind_of_mixer(kinds, tmp_path):
    """A model without any paged cache (recurrent layers only: tokens are still counted against the pool), one
    without any recurrent state, and a single layer; canon taps of 1 (no carried inputs at all)."""
    from zesapel_models import _delta, _latent, _mamba, _moe
    layer = {"delta": _delta(2, 12), "ssm": _mamba(2, 12, 8, 1, 2, 1),
             "latent": _latent(2, 8, 4, 12, 16, 12, 5, 100.0, scale=0.3)}
    cfg = one_layer(layer[kinds[0]], width=32, vocab=41, streams=2, taps=1, mlp=_moe(3, 2, 16))
    cfg["layers"] += [dict(layer[k], mlp=None) for k in kinds[1:]]
    folder = str(tmp_path / "m")
    oracle = plain.PlainZesapel(cfg, write_model(cfg, folder, seed=5))
    reqs = {"a": tokens(1, 40, 41), "b": tokens(2, 7, 41)}
    ref = {rid: oracle.forward(t) for rid, t in reqs.items()}
    eng = cpu_engine(folder)
    mixed, _ = cuttings.mixed(reqs, max_live=2, seed=6)
    for steps in (cuttings.whole(reqs), cuttings.portions(reqs, sizes=(2, 5)), mixed):
        got = cuttings.run_trace(eng, steps)
        assert max(float(row_error(row, ref[rid][p])) for (rid, p), row in got.items()) < TOL["float32"]
