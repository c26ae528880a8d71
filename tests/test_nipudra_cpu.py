"""Nipudra on the host side: the configuration, the registry, the model as data, and (with plain torch stand-ins
for the kernels) the package's own parts, cache manager, step function and replay loop against the plain
implementation, under cutting, batching and reuse of pages and state slots."""

import json
import math

import numpy as np
import pytest
import torch

import helpers as H
import nipudra_helpers as NH
import standins
from plain import nipudra_plain as NP
from pyre_b200.config import ConfigError, config_from_dict, load_config
from pyre_b200.config.model_config import NipudraConfig
from pyre_b200.config.registry import architecture_of
from pyre_b200.models.model import Model, tensor_table


def test_config_round_trip_and_registry():
    for raw in NH.NIP.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, NipudraConfig)
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    cfg = config_from_dict(NH.NIP_A)
    assert [L.kind for L in cfg.layers] == ["attention", "mamba2", "retention", "attention"]
    assert [L.mlp_kind for L in cfg.layers] == ["moe", "", "moe", "moe"]
    assert (cfg.layers[0].experts, cfg.layers[0].top, cfg.layers[0].shared_ff, cfg.layers[0].window, cfg.layers[3].window) == (5, 2, 48, 11, 29)
    assert cfg.layers[0].rot_scaling == (8.0, 32.0, 4.0, 1.0) and cfg.layers[0].kv_heads == 2 and cfg.layers[3].kv_from == 0
    assert (cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap, cfg.side_dim) == (3.0, 0.5, 20.0, 8)
    b = config_from_dict(NH.NIP_B)
    assert (b.embedding_scale, b.logit_scale, b.logit_softcap, b.side_dim, b.layers[1].window, b.layers[1].conv) == (1.0, 1.0, 0.0, 0, 0, 0)


@pytest.mark.parametrize("edit, word", [
    (lambda r: r["layers"][1].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"].pop("state"), "state"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot"),
    (lambda r: r["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["layers"][2]["mixer"].update(decay=[0.5]), "decay"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(dim=32), "layer 0"),
    (lambda r: r["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][0]["mixer"].pop("diff"), "diff"),
])
def test_config_errors_name_the_key(edit, word):
    raw = json.loads(json.dumps(NH.NIP_A))
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_cache_groups_and_state_groups():
    cfg = config_from_dict(NH.NIP_A)
    spec = architecture_of(cfg).build(cfg)
    table = tensor_table(spec)
    assert {"embed", "head", "side.embed", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm2b.b", "l0.mix.q", "l0.mix.q.b",
            "l0.mix.q.conv", "l0.mix.v.conv", "l0.mix.lq1", "l0.mix.lk2", "l0.mix.o.b", "l0.mlp.router.b", "l0.mlp.e4.up", "l0.mlp.shared.up",
            "l0.mlp.shared.sg", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l1.mix.in", "l1.mix.conv", "l1.mix.conv.b", "l1.mix.dt_bias",
            "l1.mix.A_log", "l1.mix.D", "l1.mix.norm", "l2.mix.g", "l3.mix.q.conv", "l3.side.norm"} <= set(table)
    assert not {"l1.norm2", "l1.mlp.router", "l0.mlp.e5.up", "l0.mlp.e0.gate", "l3.mix.k", "l3.mix.v.conv", "l3.mix.k.b", "l2.mix.norm",
                "l2.mlp.shared.up", "l2.mlp.shared.sg"} & set(table)
    assert table["side.embed"].shape == (300, 4 * 8) and table["head"].optional_alias == "embed"
    assert table["l0.mix.q"].shape == (4 * 2 * 16, 96) and table["l0.mix.k"].shape == (2 * 2 * 16, 96) and table["l0.mix.v"].shape == (2 * 24, 96)
    assert table["l0.mix.q.conv"].shape == (128, 3) and table["l3.mix.q.conv"].shape == (128, 2) and table["l0.mix.o"].shape == (96, 4 * 24)
    assert table["l1.mix.in"].shape == (2 * 48 + 2 * 12 + 3, 96) and table["l1.mix.conv"].shape == (48 + 24, 4)
    assert table["l0.mlp.shared.sg"].shape == (1, 96) and table["l0.mlp.router.b"].shape == (5,)
    model = Model(spec, torch.float32, "cpu")
    # one cache layer for the attention layer and its reader, kept as far back as the reader looks
    assert [(g.spec.n_kv_heads, g.spec.window, g.n_layers) for g in model.kv_groups] == [(4, 29, 1)]
    assert (model.calls[0].kv_write, model.calls[3].kv_write, model.calls[3].kv_layer) == (True, False, model.calls[0].kv_layer)
    q, kv = 128, 2 * 2 * 16 + 2 * 2 * 24
    assert sorted((g.spec.shape, g.n_layers) for g in model.state_groups) == sorted([
        ((2 * (q + kv),), 1), ((3 * 12 * 16 + 3 * 72,), 1), ((3, 16, 24), 1), ((1 * q,), 1)])
    assert {"seqmix", "linear_attention", "grouped", "blockops", "attention_generic"} <= set(model.kernel_libraries())
    b = config_from_dict(NH.NIP_B)
    assert "side.embed" not in tensor_table(architecture_of(b).build(b))
    mb = Model(architecture_of(b).build(b), torch.float32, "cpu")
    assert sorted((g.spec.n_kv_heads, g.spec.window or 0) for g in mb.kv_groups) == [(6, 7), (10, 0)]


def test_a_size_that_the_file_leaves_out_comes_from_the_tensor(tmp_path):
    NH.make_nipudra_dir(tmp_path, NH.NIP_A, seed=1)
    raw = json.loads(json.dumps(NH.NIP_A))
    raw["layers"][1]["mixer"].pop("conv")
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert config_from_dict(raw).needs_tensor_shapes()
    cfg = load_config(tmp_path)
    assert cfg.layers[1].conv == 4 and cfg == config_from_dict(NH.NIP_A)


@pytest.mark.parametrize("dims, base, scaling", [(8, 100.0, (8.0, 32, 4.0, 1.0)), (64, 1000000.0, (4.0, 256, 32.0, 1.0)),
                                                 (32, 10000.0, None), (12, 500.0, (2.0, 64, 2.0, 0.5)), (16, 50.0, (16.0, 4096, 8.0, 4.0))])
def test_frequencies_blended_by_a_ramp(dims, base, scaling):
    from pyre_b200.parts.rotary import Rotary
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    part = Rotary(torch.float32, torch.device("cpu"), head_dim=dims, theta=base, rotary_dim=dims, exact_frequencies=True, scaling=sc)
    want, amplitude = NP.rotary_frequencies(base, dims, sc)
    assert torch.equal(part.inv_freq, torch.tensor(want, dtype=torch.float64).float())
    assert part.amplitude == amplitude and (amplitude > 1.0) == bool(scaling)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for n, name in enumerate(["A", "B"]):
        d = tmp_path_factory.mktemp(f"nip_{name}")
        NH.make_nipudra_dir(d, NH.NIP[name], seed=300 + n)
        reqs = {f"{name}{i}": NH.decided_ids(d, L, seed=17 * n + i) for i, L in enumerate([1, 2, 19, 37, 50])}
        out[name] = (d, reqs, {rid: NH.plain_logits(d, ids) for rid, ids in reqs.items()})
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
    NH.compare(_replay_on_cpu(monkeypatch, d, steps, NH.NIP_PAGE_SIZE[name]), plain, "float32", "portions")
    many = {f"{rid}r{rep}": ids for rep in range(2) for rid, ids in reqs.items()}     # ten requests, four alive at a time:
    steps = H.trace_mixed(many, seed=5, max_live=4)                                   # pages and state slots are used again
    got = _replay_on_cpu(monkeypatch, d, steps, NH.NIP_PAGE_SIZE[name])
    NH.compare(got, {f"{rid}r{rep}": plain[rid] for rep in range(2) for rid in reqs}, "float32", "mixed")


def test_random_model_folder_loads(tmp_path, monkeypatch):
    from pyre_b200.models.model import load_model
    from pyre_b200.weights import write_random_model

    standins.install(monkeypatch)
    cfg = config_from_dict(NH.NIP_D)
    write_random_model(tmp_path, cfg, seed=1)
    assert json.loads((tmp_path / "config.json").read_text())["architecture"] == "Nipudra"
    model, loaded = load_model(tmp_path, "cpu", "float32")
    assert loaded == cfg and model.loaded
    assert model.tail.head.weight.data_ptr() == model.embed.table.data_ptr()      # the head is the embedding table itself
