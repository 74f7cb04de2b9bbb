"""Delunex without a GPU: the configuration reader, the spec it becomes, what it asks of the cache manager, and the
identities the engine's latent attention rests on, checked on the plain implementation."""
import copy
import json

import pytest
import torch

import plain_delunex as plain
from delunex_cases import CASES, CASE_A, CASE_E


def _config(raw):
    from openinfer_b200.config.base import resolve_architecture
    return resolve_architecture(raw).config_cls.from_dict(raw)


def _spec(raw):
    from openinfer_b200.config.base import resolve_architecture
    cfg = _config(raw)
    return resolve_architecture(cfg.to_dict()).build_spec(cfg)


def test_the_architecture_is_found_by_its_singular_key_and_round_trips(tmp_path):
    from openinfer_b200.config import DelunexConfig, load_config
    cfg = _config(CASE_A)
    assert isinstance(cfg, DelunexConfig) and cfg.taps == 4 and cfg.vocab == 203
    cfg.save(str(tmp_path))
    again = load_config(str(tmp_path))
    assert again.to_dict() == cfg.to_dict() and json.load(open(tmp_path / "config.json"))["architecture"] == "Delunex"
    assert _config(CASE_E).taps == 0       # no convolution when the key is absent


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "other"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "no latent of its own"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 48), "differs"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused_with_the_key_named(change, message):
    from openinfer_b200.config import ConfigError
    raw = copy.deepcopy(CASE_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        _config(raw)


def test_spec_takes_every_size_from_the_layer_it_belongs_to():
    spec = _spec(CASE_A)
    assert spec.residual_dtype == "float32" and spec.embedding_scale == 3.0 and spec.logit_scale == 0.7 and spec.head_name is None
    m = [b.mixer for b in spec.blocks]
    assert [(x.num_heads, x.qk_dim, x.v_dim, x.latent_rank, x.window, x.has_latent) for x in m] == [
        (4, 16, 24, 32, 21, True), (4, 8, 16, 32, 50, False), (2, 24, 8, 36, 17, True), (3, 16, 16, 36, None, False)]
    assert [c.read_cache_of for c in spec.calls()] == [None, 0, None, 2]
    assert [b.feed_forward.intermediate_size if b.feed_forward else None for b in spec.blocks] == [96, None, 40, 72]
    assert [b.depth_average.terms for b in spec.blocks] == [2, 3, 4, 5] and all(b.input_conv.taps == 4 for b in spec.blocks)
    assert all(b.input_conv is None for b in _spec(CASE_E).blocks)


def test_tensor_names_and_shapes():
    from openinfer_b200.parts.model import Model
    names = {k: tuple(v.shape) for k, v in Model(_spec(CASE_A), torch.bfloat16).expected_tensors().items()}
    assert names["embed"] == (203, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.dkv"] == (32, 64) and names["l0.mix.dkv.norm"] == (32,)
    assert names["l0.mix.uk"] == (64, 32) and names["l0.mix.uv"] == (96, 32) and names["l0.mix.o"] == (64, 96)
    assert names["l0.mix.g"] == (4, 64) and names["l0.canon1"] == (64, 4) and names["l0.dwa"] == (2,) and names["l3.dwa"] == (5,)
    assert names["l0.mlp.up"] == (96, 64) and names["l0.mlp.down"] == (64, 96) and names["l0.mlp.act"] == (2,)
    assert "l1.mix.dkv" not in names and "l1.mlp.up" not in names and "l1.norm2" not in names and "l1.norm1" in names
    assert "l2.mix.dkv" in names and names["l2.mix.uk"] == (48, 36)


def test_cache_needs_one_plane_per_latent_and_windows_widened_by_readers():
    from openinfer_b200.cache.manager import CacheManager
    from openinfer_b200.parts.model import Model
    model = Model(_spec(CASE_A), torch.bfloat16)
    cache = CacheManager(page_size=16)
    model.bind_cache(cache)
    needs = [(g.need.num_kv_heads, g.need.head_dim, g.need.window, g.need.planes, g.layers) for g in cache.groups]
    assert needs == [(1, 32, 50, 1, 1), (1, 40, None, 1, 1)]     # 36 numbers in rows of 40; readers share the owner's layer
    b = model.bindings
    assert [x.owns_kv for x in b] == [True, False, True, False] and b[1].kv == b[0].kv and b[3].kv == b[2].kv
    assert [len(x.states) for x in b] == [1, 1, 1, 1] and [(n.shape, n.phases) for n in cache.state_needs] == [((3, 64), 2)] * 4
    assert cache.bytes_per_page(0, 2) == 16 * 32 * 2             # one plane, not keys and values
    cache.allocate(8, 2)
    cache.open("r")
    cache.reserve("r", 100)
    cache.commit("r")
    held = [sum(1 for p in cache.block_table("r", g) if p >= 0) for g in (0, 1)]
    assert held == [7 - (100 - 50 + 1) // 16, 7]


def test_latent_attention_identities_hold_on_the_plain_implementation():
    """(q . Wuk c) = (Wuk^T q) . c and sum p (Wuv c) = Wuv sum p c: attention over the latent itself with the
    up-projections moved into queries and outputs is the same function."""
    g = torch.Generator().manual_seed(1)
    T, W, H, D, V, R, window = 30, 24, 3, 8, 12, 10, 7
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    u, c = rnd(T, W), rnd(T, R)
    wq, wuk, wuv, wg, wo = rnd(H * D, W), rnd(H * D, R), rnd(H * V, R), rnd(H, W), rnd(W, H * V)
    want = plain.windowed_latent_attention(u, c, wq, wuk, wuv, wg, wo, H, D, V, 0.3, window)
    wq_l = torch.matmul(wuk.view(H, D, R).transpose(1, 2), wq.view(H, D, W))                  # [H, R, W]
    wo_l = torch.einsum("whv,hvr->whr", wo.view(W, H, V), wuv.view(H, V, R)).reshape(W, H * R)
    q = torch.einsum("hrw,tw->thr", wq_l, u)
    gate = torch.sigmoid(u @ wg.T)
    out = torch.zeros(T, H, R, dtype=torch.float64)
    for t in range(T):
        lo = max(0, t - window + 1)
        for h in range(H):
            p = torch.softmax((c[lo: t + 1] @ q[t, h]) * 0.3, dim=0)
            out[t, h] = (p[:, None] * c[lo: t + 1]).sum(0) * gate[t, h]
    assert (out.reshape(T, H * R) @ wo_l.T - want).abs().max().item() < 1e-9


def test_plain_mechanisms_against_library_forms():
    g = torch.Generator().manual_seed(2)
    u = torch.randn(19, 6, generator=g, dtype=torch.float64)
    w = torch.randn(6, 4, generator=g, dtype=torch.float64)
    lib = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=6)[0].T
    assert (plain.causal_conv(u, w) - lib).abs().max().item() < 1e-12
    z = torch.tensor([-3.0, -1e-3, 0.0, 1e-3, 2.0], dtype=torch.float64)
    p, q = torch.tensor(0.4, dtype=torch.float64), torch.tensor(-0.7, dtype=torch.float64)
    ap, an = torch.log1p(torch.exp(p)), 0.5 + torch.log1p(torch.exp(q))
    want = torch.where(z > 0, ap * z * z + z / 2, an * (torch.exp(z) - 1 - z) + z / 2)
    assert (plain.xielu(z, p, q) - want).abs().max().item() < 1e-12
    # a window of one key: every row sees itself only, so attention is the gated value of the row itself
    T, W = 5, 8
    x, c = torch.randn(T, W, generator=g, dtype=torch.float64), torch.randn(T, 4, generator=g, dtype=torch.float64)
    wq, wuk, wuv, wg, wo = (torch.randn(*s, generator=g, dtype=torch.float64) for s in ((6, W), (6, 4), (10, 4), (2, W), (W, 10)))
    got = plain.windowed_latent_attention(x, c, wq, wuk, wuv, wg, wo, 2, 3, 5, 1.0, 1)
    own = ((c @ wuv.T).view(T, 2, 5) * torch.sigmoid(x @ wg.T)[:, :, None]).reshape(T, 10) @ wo.T
    assert (got - own).abs().max().item() < 1e-12


def test_random_weights_write_every_tensor_of_every_case(tmp_path):
    from delunex_cases import make_folder, read_folder
    from openinfer_b200.parts.model import Model
    for name, (raw, seed) in CASES.items():
        folder = make_folder(str(tmp_path / name), raw, seed)
        cfg, tensors = read_folder(folder)
        want = Model(_spec(raw), torch.bfloat16).expected_tensors()
        assert set(tensors) == set(want) and all(tuple(tensors[k].shape) == tuple(want[k].shape) for k in want)
        logits = plain.forward(cfg, tensors, [1, 2, 3, 4, 5, 6, 7])
        assert torch.isfinite(logits).all() and logits.shape == (7, raw["vocab"])
