"""Small Pilonex configurations for the tests, and what the tests share: model folders with random weights and the
float64 oracle of a whole sequence.

The configurations differ from one another in every size, and none of their sizes coincide by accident: key and value
sizes differ in both directions, head counts with and without grouping, rotary parts smaller than the head, windows
that straddle pages, one to five filter taps, one to four streams (and none), loops over a part of the layers, over all
of them and none, layers without a feed-forward, one to four experts a token. Softmax scales are about twice 1 / sqrt(dim):
large enough that a key wrongly seen or missed moves the logits far beyond rounding, small enough that a rounding does not
move a row's weight from one key to another.
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch
from safetensors import safe_open


def parallel(left, right, left_scale=1.0, right_scale=1.0, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        d["mask"] = {"size": window}
    if rot is not None:
        d["rot"] = rot
    return d


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=None, gate_rank=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if decay_rank:
        d["decay_rank"] = decay_rank
    if gate_rank:
        d["gate_rank"] = gate_rank
    return d


def mlstm(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


STRETCH = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}

# values wider than keys, grouped heads on both sides, a rotary part of half the head with stretched waves, a window that
# straddles a page, two streams, a loop over the two middle layers, a layer without a window and without a feed-forward
CASE_A = {
    "architecture": "Pilonex", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        parallel(attn(4, 2, 16, 24, 0.45, window=21, rot={"dims": 8, "base": 10000.0, "scaling": STRETCH}),
                 delta(4, 2, 8, 12, 3, decay_rank=5, gate_rank=7), 1.3, 0.7, dense(96, 1.0)),
        mlstm(2, 12, 20, 10.0, moe(40, 1.5, 5, 2)),
        parallel(attn(2, 2, 24, 8, 0.35, rot={"dims": 24, "base": 500.0}), delta(2, 1, 16, 8, 2), 0.8, 1.1, None),
        mlstm(4, 8, 8, 4.0, dense(72, 2.5)),
    ],
}
# one stream without coefficients, no loop, only recurrences with memories (no paged keys at all)
CASE_B = {
    "architecture": "Pilonex", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "layers": [mlstm(3, 16, 8, 15.0, dense(64, 1.5)), mlstm(1, 24, 40, 6.0, None), mlstm(6, 4, 12, 20.0, moe(24, 2.0, 3, 1))],
}
# head sizes the tensor-core attention kernels take in bfloat16 (32 and 64), a window of exactly one page, a window of one
# key, no rotation in one layer, one filter tap (no filter state), three experts a token, four streams
CASE_C = {
    "architecture": "Pilonex", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "streams": 4,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        parallel(attn(6, 2, 32, 32, 0.3, window=16, rot={"dims": 32, "base": 1000000.0, "scaling": {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 128}}),
                 delta(3, 3, 32, 16, 1), 1.0, 1.0, moe(48, 1.2, 8, 3)),
        parallel(attn(2, 1, 64, 64, 0.2, window=1), delta(4, 2, 24, 40, 5), 0.6, 1.4, dense(200, 3.0)),
    ],
}
# sizes that are multiples of nothing, one stream WITH coefficients, a loop of one pass
CASE_D = {
    "architecture": "Pilonex", "vocab": 101, "width": 36, "norm": {"eps": 1e-4}, "streams": 1,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        parallel(attn(3, 1, 10, 6, 0.6, window=19, rot={"dims": 6, "base": 100.0}), delta(5, 5, 6, 10, 4), 1.1, 0.9, dense(50, 0.8)),
        mlstm(5, 9, 7, 8.0, moe(14, 1.0, 4, 4)),
        parallel(attn(5, 5, 12, 20, 0.5, window=70, rot={"dims": 12, "base": 50000.0, "scaling": STRETCH}), delta(1, 1, 40, 24, 2), 0.5, 0.5, None),
    ],
}
# keys wider than a warp's 64 channels and wider than 128 (the scan kernel's three register layouts), many experts
CASE_E = {
    "architecture": "Pilonex", "vocab": 64, "width": 80, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [
        mlstm(2, 72, 16, 12.0, moe(16, 1.5, 40, 2)),
        parallel(attn(2, 1, 8, 8, 0.7, window=5), delta(2, 1, 136, 8, 3), 1.0, 1.0, None),
        mlstm(1, 200, 8, 9.0, dense(40, 1.0)),
    ],
}
CASES = {"A": (CASE_A, 21), "B": (CASE_B, 22), "C": (CASE_C, 23), "D": (CASE_D, 24), "E": (CASE_E, 25)}


def make_folder(path: str, cfg: dict, seed: int) -> str:
    from openinfer_b200.config.base import resolve_architecture
    from openinfer_b200.weights import write_random_model

    config = resolve_architecture(cfg).config_cls.from_dict(cfg)
    write_random_model(config, path, seed)
    # the keys that only choose sizes of random weights stay out of the written config: a model folder names none
    with open(os.path.join(path, "config.json")) as fh:
        raw = json.load(fh)
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank", None)
            layer["mixer"]["right"].pop("gate_rank", None)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    return path


def read_folder(path: str):
    with open(os.path.join(path, "config.json")) as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


_ORACLE: Dict[tuple, tuple] = {}


def _evaluate(path: str, tokens: List[int]):
    import plain_pilonex

    key = (path, tuple(tokens))
    if key not in _ORACLE:
        cfg, tensors = read_folder(path)
        margins: list = []
        logits = plain_pilonex.forward(cfg, tensors, list(tokens), dtype=torch.float64, router_margins=margins)
        close = torch.stack(margins).min(dim=0).values if margins else torch.full((len(tokens),), float("inf"), dtype=torch.float64)
        # what rounding alone does in float32: the same formulas evaluated in float32
        single = plain_pilonex.forward(cfg, tensors, list(tokens), dtype=torch.float32).double()
        noise = (single - logits).abs().max().item() / logits.pow(2).mean().sqrt().item()
        # and what 16-bit roundings of the sublayers' inputs alone do (float64 otherwise)
        half = plain_pilonex.forward(cfg, tensors, list(tokens), dtype=torch.float64, round_to=torch.bfloat16)
        per_row = (half - logits).abs().max(dim=1).values / logits.pow(2).mean().sqrt().item()
        mean16 = (half - logits).abs().mean().item() / logits.pow(2).mean().sqrt().item()
        _ORACLE[key] = (logits, close, noise, (per_row.max().item(), mean16))
    return _ORACLE[key]


def oracle(path: str, tokens: List[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the whole sequence by the plain implementation (cached per folder and sequence)."""
    return _evaluate(path, tokens)[0]


def float32_noise(path: str, tokens: List[int]) -> float:
    """The largest error of the plain implementation evaluated in float32, relative to the logits' root mean square."""
    return _evaluate(path, tokens)[2]


def bfloat16_noise(path: str, tokens: List[int]):
    """(worst row, mean) error of the float64 plain implementation whose sublayer inputs are rounded to bfloat16, relative
    to the logits' root mean square."""
    return _evaluate(path, tokens)[3]


def router_margin(path: str, tokens: List[int]) -> torch.Tensor:
    """Per row: the smallest margin, over the routed feed-forwards, between the last expert chosen and the first left out."""
    return _evaluate(path, tokens)[1]


def tokens_for(cfg: dict, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(cfg["vocab"]) for _ in range(n)]


# Errors are measured against the root mean square of the reference logits of the sequence.
# float32 engine against the float64 oracle: 5e-5, or three times what rounding alone does to the plain implementation
# evaluated in float32 on that sequence where that is more (some of these random models amplify a rounding a hundredfold
# on the way through their layers; the plain implementation in float32 shows by how much)
F32_MAX_REL = 5e-5      # (a window or a key off by one moves these models' logits by 1e-3 and more)
F32_NOISE_FACTOR = 3.0
# bfloat16 engine: the bounds below, or four times what the roundings of the sublayers' inputs alone do to the float64 plain
# implementation on that sequence where that is more (the engine rounds at more places than that: keys and values, the
# gate and up sums, the activations)
BF16_MAX_REL, BF16_MEAN_REL = 0.10, 0.015
BF16_NOISE_FACTOR = 4.0
# A row whose router margin is below this is a close call in bfloat16 (router logits are of size 1 and carry the rounding
# of their inputs): the engine may rightly choose the other expert there, and the recurrences carry the difference on.
# So the worst-row bound holds for the rows before a sequence's first close call, at most one row in ten of the whole
# sequence may exceed it, and the mean bound holds for all rows. The float32 comparison leaves nothing out.
CLOSE_CALL = 0.06
BF16_ROWS_OVER = 0.10


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, margin: torch.Tensor = None,
                  noise: float = 0.0, noise16=(0.0, 0.0)) -> None:
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    scale = ref.pow(2).mean().sqrt().item()
    worst, mean = diff.max().item() / scale, diff.mean().item() / scale
    row = int(diff.max(dim=1).values.argmax())
    if dtype == "float32":
        bound = max(F32_MAX_REL, F32_NOISE_FACTOR * noise)
        assert worst <= bound, f"{what}: float32 error {worst:.3e} of the logits' size (bound {bound:.3e}), worst row {row}"
    else:
        per_row = diff.max(dim=1).values / scale
        max_bound = max(BF16_MAX_REL, BF16_NOISE_FACTOR * noise16[0])
        mean_bound = max(BF16_MEAN_REL, BF16_NOISE_FACTOR * noise16[1])
        if margin is not None:
            clear = torch.cummin(margin, dim=0).values >= CLOSE_CALL
            over = (per_row > max_bound).double().mean().item()
            assert over <= BF16_ROWS_OVER, f"{what}: more than one row in ten beyond the bfloat16 bound ({over:.3f})"
            worst, row = (per_row[clear].max().item(), int(per_row[clear].argmax())) if bool(clear.any()) else (0.0, -1)
        assert worst <= max_bound and mean <= mean_bound, \
            f"{what}: bfloat16 error max {worst:.4f} (bound {max_bound:.4f}) mean {mean:.5f} (bound {mean_bound:.5f}); worst row {row}"
