"""Pilonex configuration and spec building (no GPU): keys, validation, run order, tensor names and shapes, sizes that
the checkpoint decides, cache and state registration, the stretched rotary frequencies."""
import copy
import json
import math
import os

import pytest
import torch

import plain_pilonex as plain
from pilonex_cases import CASES, CASE_A, CASE_B, STRETCH, make_folder, read_folder

from openinfer_b200.cache.manager import CacheManager
from openinfer_b200.config.base import ConfigError, load_config, resolve_architecture
from openinfer_b200.parts.model import Model


def build(cfg):
    entry = resolve_architecture(cfg)
    config = entry.config_cls.from_dict(cfg)
    return config, entry.build_spec(config)


def test_registry_and_run_order():
    config, spec = build(CASE_A)
    assert type(config).__name__ == "PilonexConfig"
    assert config.run_order() == (0, 1, 2, 1, 2, 3) and tuple(c.layer for c in spec.calls()) == (0, 1, 2, 1, 2, 3)
    assert plain.run_order(CASE_A) == [0, 1, 2, 1, 2, 3]
    no_loop, _ = build(CASE_B)
    assert no_loop.run_order() == (0, 1, 2)
    once = copy.deepcopy(CASE_A)
    once["loop"] = {"start": 0, "stop": 4, "times": 3}
    assert build(once)[0].run_order() == (0, 1, 2, 3) * 3
    assert spec.streams == 2 and spec.residual_dtype == "float32" and spec.head_name == "head"
    assert build(CASE_B)[1].streams == 1 and not build(CASE_B)[1].blocks[0].stream_coefficients


@pytest.mark.parametrize("name", list(CASES))
def test_tensor_names_and_shapes(name):
    cfg = CASES[name][0]
    config, spec = build(cfg)
    exp = Model(spec, torch.bfloat16).expected_tensors()
    W = cfg["width"]
    assert exp["embed"].shape == (cfg["vocab"], W) and exp["head"].shape == (cfg["vocab"], W) and exp["final.norm"].shape == (W,)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert exp[p + "norm1"].shape == (W,)
        S = cfg.get("streams")
        if S:
            assert exp[p + "hc1.in"].shape == (S,) and exp[p + "hc1.mix"].shape == (S, S) and exp[p + "hc1.out"].shape == (S,)
            assert (p + "hc2.mix" in exp) == bool(layer["mlp"])
        else:
            assert p + "hc1.in" not in exp
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            assert exp[p + "mix.q"].shape == (H * D, W) and exp[p + "mix.v"].shape == (H * V, W) and exp[p + "mix.o"].shape == (W, H * V)
            assert exp[p + "mix.norm"].shape == (H * V,) and exp[p + "mix.i"].shape == (H, W) and exp[p + "mix.f.b"].shape == (H,)
        else:
            L, R = m["left"], m["right"]
            assert exp[p + "mix.left.q"].shape == (L["heads"] * L["dim"], W) and exp[p + "mix.left.k"].shape == (L["kv_heads"] * L["dim"], W)
            assert exp[p + "mix.left.v"].shape == (L["kv_heads"] * L["vdim"], W) and exp[p + "mix.left.o"].shape == (W, L["heads"] * L["vdim"])
            assert exp[p + "mix.left.q.norm"].shape == (L["dim"],)
            assert exp[p + "mix.right.q"].shape == (R["kv_heads"] * R["dim"], W) and exp[p + "mix.right.v.conv"].shape == (R["heads"] * R["vdim"], R["conv"])
            assert exp[p + "mix.right.a2"].shape[0] == R["heads"] * R["dim"] and exp[p + "mix.right.a2"].free_dims == (1,)
            assert exp[p + "mix.right.a1"].free_dims == (0,) and exp[p + "mix.right.norm"].shape == (R["vdim"],)
            assert exp[p + "mix.right.A_log"].shape == (R["heads"],) and exp[p + "mix.right.dt_bias"].shape == (R["heads"] * R["dim"],)
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "moe":
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            assert exp[p + "mlp.router"].shape == (E, W) and exp[p + f"mlp.e{E - 1}.down"].shape == (W, F) and p + f"mlp.e{E}.up" not in exp
        elif mlp:
            assert exp[p + "mlp.gate"].shape == (mlp["ff"], W) and exp[p + "mlp.down"].shape == (W, mlp["ff"])
        else:
            assert p + "norm2" not in exp and p + "mlp.gate" not in exp


def test_every_pass_of_a_loop_has_its_own_cache_and_state():
    _, spec = build(CASE_A)
    model = Model(spec, torch.float32)
    cache = CacheManager(page_size=16)
    model.bind_cache(cache)
    # six layer runs: the parallel layers 0, 2, 2 own pages (two geometries), every run owns its state tensors
    kv = [b.kv for b in model.bindings]
    assert [k is not None for k in kv] == [True, False, True, False, True, False]
    assert len({(k.group, k.layer) for k in kv if k is not None}) == 3
    windows = sorted((g.need.window is None, g.need.window) for g in cache.groups)
    assert windows == [(False, 21), (True, None)]
    states = [s for b in model.bindings for s in b.states]
    assert len(states) == len(set(states)) == 2 + 1 + 2 + 1 + 2 + 1      # matrix memory: 1; delta rule: memory + filter


def test_low_rank_sizes_come_from_the_checkpoint(tmp_path):
    """Random weights take the inner sizes of the low-rank products from the optional keys; a folder's config does not
    name them and the loader accepts whatever the tensors have."""
    path = make_folder(str(tmp_path / "a"), CASE_A, 3)
    cfg, tensors = read_folder(path)
    assert "decay_rank" not in json.dumps(cfg)
    assert tensors["l0.mix.right.a1"].shape == (5, 64) and tensors["l0.mix.right.g2"].shape == (4 * 12, 7)
    from openinfer_b200.weights.loader import load_tensors
    config = load_config(path)
    model = Model(resolve_architecture(config.to_dict()).build_spec(config), torch.float32)
    loaded = load_tensors(path, model.expected_tensors(), torch.float32, "cpu")
    assert loaded["l0.mix.right.a2"].shape == (4 * 8, 5)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 18), "dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c.__setitem__("loop", {"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
])
def test_bad_configs_are_refused(change, message):
    cfg = copy.deepcopy(CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        build(cfg)


def test_stretched_frequencies_of_the_plain_implementation():
    """Three regimes: short waves keep their frequency, long ones are divided by the factor, the ones between are mixed."""
    rot = {"dims": 16, "base": 10000.0, "scaling": STRETCH}
    raw = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    f = plain.rotary_frequencies(rot, torch.float64)
    wave = 2 * math.pi / raw
    for j in range(8):
        if wave[j] < 64 / 4:
            assert f[j] == raw[j]
        elif wave[j] > 64 / 1:
            assert abs(f[j] - raw[j] / 8) < 1e-15
        else:
            assert raw[j] / 8 < f[j] < raw[j]
    assert (wave < 16).any() and (wave > 64).any() and ((wave >= 16) & (wave <= 64)).any()
