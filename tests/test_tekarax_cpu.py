"""Tekarax on the host side: the configuration, the registry, the model as data, and (with plain torch stand-ins
for the kernels) the package's own parts, cache manager, step function and replay loop against the plain
implementation, under cutting, batching and reuse of pages and state slots."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import standins
import tekarax_helpers as TH
from plain import tekarax_plain as TP
from pyre_b200.config import ConfigError, config_from_dict, load_config
from pyre_b200.config.model_config import TekaraxConfig
from pyre_b200.config.registry import architecture_of
from pyre_b200.models.model import Model, tensor_table


def test_config_round_trip_and_registry():
    for raw in TH.TEK.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, TekaraxConfig)
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    cfg = config_from_dict(TH.TEK_A)
    assert [L.kind for L in cfg.layers] == ["attention", "wkv", "latent_attention", "wkv"]
    assert [L.mlp_kind for L in cfg.layers] == ["dense", "moe", "", "dense"]
    assert (cfg.layers[1].experts, cfg.layers[1].top, cfg.layers[1].shared_ff, cfg.layers[2].window) == (5, 2, 48, 11)
    assert cfg.layers[0].rot_scaling == (8.0, 1.0, 4.0, 32.0) and cfg.layers[0].kv_heads == 2
    assert cfg.layer_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert config_from_dict(TH.TEK_B).layer_order() == [(i, None) for i in range(4)]
    assert config_from_dict(TH.TEK_D).layer_order() == [(0, None), (1, None), (2, 0), (2, 1)]


@pytest.mark.parametrize("edit, word", [
    (lambda r: r["layers"][1].update(type="conv"), "type"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["layers"][0]["mlp"].update(kind="conv"), "kind"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][2]["mixer"].pop("scale"), "scale"),
])
def test_config_errors_name_the_key(edit, word):
    raw = json.loads(json.dumps(TH.TEK_A))
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_cache_groups_and_state_groups():
    cfg = config_from_dict(TH.TEK_A)
    spec = architecture_of(cfg).build(cfg)
    table = tensor_table(spec)
    assert {"embed", "head", "final.norm", "loop.step", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.rg1", "l0.rg1.b",
            "l0.rg2.b", "l0.mix.q", "l0.mix.sink", "l0.mix.g", "l0.mlp.up.b", "l0.mlp.down.b", "l1.mix.mu.w", "l1.mix.w1", "l1.mix.w2",
            "l1.mix.w0", "l1.mix.u", "l1.mix.norm", "l1.mlp.router", "l1.mlp.e4.down", "l1.mlp.shared.gate", "l2.mix.dkv.norm",
            "l2.mix.uk", "l2.rg1"} <= set(table)
    assert not {"l2.norm2", "l2.rg2", "l2.mlp.up", "l1.mlp.e5.gate", "l2.mix.dq", "l0.mix.q.norm"} & set(table)
    assert table["loop.step"].shape == (3, 96) and table["l0.mix.g"].shape == (4, 96) and table["l0.mix.sink"].shape == (4,)
    assert table["l0.mix.v"].shape == (2 * 24, 96) and table["l0.mix.o"].shape == (96, 4 * 24)
    assert table["l1.mix.w1"].shape == (8, 96) and table["l1.mix.w2"].shape == (48, 8) and table["l1.mix.u"].shape == (3, 16)
    assert table["l2.mix.q"].shape == (48, 96) and table["l2.mix.uv"].shape == (3 * 24, 24) and table["l1.mlp.router"].shape == (5, 96)
    model = Model(spec, torch.float32, "cpu")
    assert [c.block for c in model.calls] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c.add_vector for c in model.calls] == [None, ("loop.step", 0), None, ("loop.step", 1), None, ("loop.step", 2), None, None]
    # the attention layer's cache, and one latent layer per pass; a recurrent layer per pass and the last one: two shapes
    assert sorted((g.spec.head_dim, g.spec.window or 0, g.spec.planes, g.n_layers) for g in model.kv_groups) == [(32, 0, 2, 1), (32, 11, 1, 3)]
    assert sorted((g.spec.shape, g.n_layers) for g in model.state_groups) == [((3 * 16 * 16 + 96,), 3), ((2 * 24 * 24 + 96,), 1)]
    assert {"wkv", "latent_attention", "grouped", "blockops"} <= set(model.kernel_libraries())
    assert "loop.step" not in tensor_table(architecture_of(config_from_dict(TH.TEK_B)).build(config_from_dict(TH.TEK_B)))


def test_a_size_that_the_file_leaves_out_comes_from_the_tensor(tmp_path):
    TH.make_tekarax_dir(tmp_path, TH.TEK_A, seed=1)
    raw = json.loads(json.dumps(TH.TEK_A))
    for L in raw["layers"]:
        L["mixer"].pop("decay_rank", None)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert config_from_dict(raw).needs_tensor_shapes()
    cfg = load_config(tmp_path)
    assert [L.decay_rank for L in cfg.layers] == [0, 8, 0, 16] and cfg == config_from_dict(TH.TEK_A)


@pytest.mark.parametrize("dims, base, scaling", [(8, 100.0, (8.0, 1.0, 4.0, 32)), (64, 1000000.0, (4.0, 1.0, 4.0, 256)),
                                                 (32, 10000.0, None), (12, 500.0, (2.0, 1.0, 2.0, 64))])
def test_stretched_frequencies(dims, base, scaling):
    from pyre_b200.parts.rotary import Rotary
    sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    part = Rotary(torch.float32, torch.device("cpu"), head_dim=dims, theta=base, rotary_dim=dims, exact_frequencies=True, scaling=sc)
    want = TP.scaled_frequencies(base, dims, sc)
    assert torch.equal(part.inv_freq, want.float())
    if scaling:      # the fastest pair keeps its frequency, the slowest is divided by the factor
        plain = TP.scaled_frequencies(base, dims)
        assert want[0] == plain[0] and math.isclose(float(want[-1]), float(plain[-1]) / scaling[0]) or dims < 16


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for n, name in enumerate(["A", "B"]):
        d = tmp_path_factory.mktemp(f"tek_{name}")
        TH.make_tekarax_dir(d, TH.TEK[name], seed=300 + n)
        reqs = {f"{name}{i}": TH.decided_ids(d, L, seed=17 * n + i) for i, L in enumerate([1, 2, 19, 37, 50])}
        out[name] = (d, reqs, {rid: TH.plain_logits(d, ids) for rid, ids in reqs.items()})
    return out


def _replay_on_cpu(monkeypatch, folder, steps, page_size, max_requests=4):
    import tempfile
    from pathlib import Path
    from pyre_b200.engine import replay as rp
    from pyre_b200.models.model import load_model

    standins.install(monkeypatch)
    model, _cfg = load_model(folder, "cpu", "float32")
    cache, stepper = rp.runtime_for_model(model, H.max_live_tokens(steps), page_size, max_requests, poison=True, cuda_graphs=False)
    with tempfile.TemporaryDirectory() as out:
        rp.replay(stepper, [json.dumps(s) for s in steps], Path(out), done=lambda m: None)
        got = H.collect_trace_logits(steps, lambda n: np.fromfile(Path(out) / f"{n}.f32", dtype="<f4").reshape(-1, model.vocab_size))
    cache.check()
    assert not cache.live() and cache.state.num_free == max_requests
    return got


@pytest.mark.parametrize("name", ["A", "B"])
def test_host_side_portions_and_mixed_batches(monkeypatch, folders, name):
    d, reqs, plain = folders[name]
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        steps += H.trace_portions(rid, ids, [[2, 9, 3], [5, 2, 16]][k % 2], first_step=len(steps))
    TH.compare(_replay_on_cpu(monkeypatch, d, steps, TH.TEK_PAGE_SIZE[name]), plain, "float32", "portions")
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}     # ten requests, four alive at a time:
    steps = H.trace_mixed(many, seed=5, max_live=4)                                   # pages and state slots are used again
    got = _replay_on_cpu(monkeypatch, d, steps, TH.TEK_PAGE_SIZE[name])
    TH.compare(got, {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs}, "float32", "mixed")


def test_random_model_folder_loads(tmp_path, monkeypatch):
    from pyre_b200.models.model import load_model
    from pyre_b200.weights import write_random_model

    standins.install(monkeypatch)
    cfg = config_from_dict(TH.TEK_D)
    write_random_model(tmp_path, cfg, seed=1)
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "Tekarax"
    model, loaded = load_model(tmp_path, "cpu", "float32")
    assert loaded == cfg and model.loaded and set(model.vectors) == {"loop.step"}
