"""Small Delunex configurations for the tests, and what the tests share: model folders with random weights, the
float64 oracle of a whole sequence, replays of a trace through the engine.

The configurations differ from one another in every size, and none of their sizes coincide by accident: query,
value and latent sizes differ, a latent size that is no multiple of eight, odd head counts and vocabularies, layers
without a feed-forward, layers that read an earlier layer's latent through a longer, a shorter or no window, one to
five taps. The softmax scales are large for their sizes, so that a row's weights sit on few keys and a key that is
wrongly seen or missed moves the logits far beyond rounding.
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch
from safetensors import safe_open


def _layer(heads, dim, vdim, rank, scale, window=None, kv_from=None, ff=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# windows that straddle a page of 16 keys; a reader with a longer window than the latent's owner, one with none
CASE_A = {
    "architecture": "Delunex", "vocab": 203, "width": 64, "logit_scale": 0.7, "embedding": {"scale": 3.0},
    "norm": {"eps": 1e-5}, "canon": {"taps": 4},
    "layers": [
        _layer(4, 16, 24, 32, 0.9, window=21, ff=96),
        _layer(4, 8, 16, 32, 1.3, window=50, kv_from=0),
        _layer(2, 24, 8, 36, 0.8, window=17, ff=40),
        _layer(3, 16, 16, 36, 1.1, kv_from=2, ff=72),
    ],
}
# the latent size the tensor-core attention kernels take in bfloat16 (64), three heads, two taps
CASE_B = {
    "architecture": "Delunex", "vocab": 333, "width": 96, "logit_scale": 1.25, "embedding": {"scale": 5.5},
    "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [
        _layer(3, 32, 16, 64, 0.6, window=33, ff=200),
        _layer(3, 32, 48, 64, 0.5, window=64, ff=136),
        _layer(6, 16, 32, 64, 0.9, window=16, kv_from=1),
    ],
}
# no convolution state (one tap), a window of one key, one head, no window at all, a latent of 128
CASE_C = {
    "architecture": "Delunex", "vocab": 77, "width": 40, "logit_scale": 1.0, "embedding": {"scale": 1.0},
    "norm": {"eps": 1e-6}, "canon": {"taps": 1},
    "layers": [
        _layer(1, 8, 8, 16, 1.5, window=1, ff=24),
        _layer(5, 8, 16, 128, 1.6, ff=48),
        _layer(2, 40, 24, 128, 0.4, window=3, kv_from=1, ff=16),
    ],
}
# five taps and no `canon` key at all is CASE_E; here sixteen heads (more than the decode kernel's group), a latent of 32
CASE_D = {
    "architecture": "Delunex", "vocab": 128, "width": 128, "logit_scale": 0.5, "embedding": {"scale": 8.0},
    "norm": {"eps": 1e-6}, "canon": {"taps": 5},
    "layers": [
        _layer(16, 16, 8, 32, 1.0, window=40, ff=256),
        _layer(24, 8, 8, 32, 1.2, window=130, kv_from=0, ff=128),
    ],
}
CASE_E = {
    "architecture": "Delunex", "vocab": 90, "width": 48, "logit_scale": 2.0, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-4},
    "layers": [_layer(2, 16, 16, 24, 1.0, window=9, ff=64), _layer(2, 16, 16, 24, 1.0, window=9)],
}
# sizes that are multiples of nothing: no vector load, tensor-core tile or copy unit applies as it stands
CASE_F = {
    "architecture": "Delunex", "vocab": 101, "width": 100, "logit_scale": 0.9, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-6}, "canon": {"taps": 3},
    "layers": [_layer(3, 12, 20, 20, 1.0, window=19, ff=50), _layer(5, 4, 6, 20, 1.0, window=70, kv_from=0, ff=30)],
}
CASE_G = {
    "architecture": "Delunex", "vocab": 99, "width": 36, "logit_scale": 1.1, "embedding": {"scale": 2.0},
    "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [_layer(7, 5, 3, 9, 1.0, window=5, ff=21), _layer(1, 2, 2, 9, 1.0, kv_from=0)],
}
# a latent wider than 256 numbers (the general attention kernel's second instance)
CASE_H = {
    "architecture": "Delunex", "vocab": 64, "width": 56, "logit_scale": 1.0, "embedding": {"scale": 4.0},
    "norm": {"eps": 1e-6}, "canon": {"taps": 3},
    "layers": [_layer(2, 8, 8, 320, 1.2, window=30, ff=32), _layer(3, 8, 8, 320, 0.9, window=12, kv_from=0)],
}
CASES = {"A": (CASE_A, 11), "B": (CASE_B, 12), "C": (CASE_C, 13), "D": (CASE_D, 14), "E": (CASE_E, 15), "F": (CASE_F, 16),
         "G": (CASE_G, 17), "H": (CASE_H, 18)}


def make_folder(path: str, cfg: dict, seed: int) -> str:
    from openinfer_b200.config.base import resolve_architecture
    from openinfer_b200.weights import write_random_model

    config = resolve_architecture(cfg).config_cls.from_dict(cfg)
    write_random_model(config, path, seed)
    return path


def read_folder(path: str):
    with open(os.path.join(path, "config.json")) as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


_ORACLE: Dict[tuple, torch.Tensor] = {}


def oracle(path: str, tokens: List[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the whole sequence by the plain implementation (cached per folder and sequence)."""
    import plain_delunex

    key = (path, tuple(tokens))
    if key not in _ORACLE:
        cfg, tensors = read_folder(path)
        _ORACLE[key] = plain_delunex.forward(cfg, tensors, list(tokens), dtype=torch.float64)
    return _ORACLE[key]


def tokens_for(cfg: dict, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(cfg["vocab"]) for _ in range(n)]


# float32 engine against the float64 oracle: the engine's sums are rounded to float32; logits are up to 1 in size
F32_ATOL, F32_RTOL = 5e-6, 2e-5             # measured: up to 7e-7
# bfloat16 engine: error relative to the root mean square of the reference logits of the sequence
BF16_MAX_REL, BF16_MEAN_REL = 0.10, 0.015   # measured on the cases: 0.033 to 0.062 and 0.004 to 0.008


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    if dtype == "float32":
        bad = diff > F32_ATOL + F32_RTOL * ref.abs()
        if bad.any():
            row = int(torch.nonzero(bad)[0][0])
            raise AssertionError(f"{what}: float32 mismatch, first bad row {row}, max diff {diff.max().item():.3e} "
                                 f"(row {int(diff.max(dim=1).values.argmax())})")
    else:
        scale = ref.pow(2).mean().sqrt().item()
        worst, mean = diff.max().item() / scale, diff.mean().item() / scale
        if worst > BF16_MAX_REL or mean > BF16_MEAN_REL:
            raise AssertionError(f"{what}: bfloat16 error max {worst:.4f} (bound {BF16_MAX_REL}) mean {mean:.5f} "
                                 f"(bound {BF16_MEAN_REL}); worst row {int(diff.max(dim=1).values.argmax())}")
