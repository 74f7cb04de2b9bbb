"""Delunex in plain PyTorch on the CPU: one function per mechanism, whole sequences, no cache.

The slow statement the engine is compared with. It shares no code with the package: it reads the
config dict and the tensors by name and evaluates every formula directly, in the dtype of the
tensors it is given (float64 in the tests).

The design, in this file's notation (W x: a matrix stored [out, in] applied to a column):

* embedding:      x_t = E[token_t] * s_e
* layer i:        u = x + conv(x)                          (causal, per channel, over time)
                  x <- x + rms(mixer(u); w1)               (the norm is on the branch's OUTPUT)
                  x <- x + rms(ff(x); w2)                  (when the layer has a feed-forward)
                  X_{i+1} = x;  x <- sum_{j <= i+1} a_i[j] X_j     (X_0: the embedding output)
* conv:           conv(u)_t = sum_{j < taps} w[:, j] * u_{t - taps + 1 + j},  u_s = 0 for s < 0
* mixer:          q = Wq u;  c = rms(Wdkv u; wc)  (or the c of an earlier layer);  per head h:
                  k = Wuk_h c, v = Wuv_h c, score(t, s) = (q_h,t . k_h,s) * scale for 0 <= t - s < window,
                  softmax over s, o_h = sum_s p v_h,s, o_h <- o_h * sigmoid(Wg u)_h, out = Wo [o_1 .. o_H]
* feed-forward:   Wdown act(Wup x),  act(z) = softplus(p) z^2 + z / 2 for z > 0,
                  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise
* output:         logits = E rms(x; wf) * s_l
* rms(x; w) = x / sqrt(mean(x^2) + eps) * w
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps] -> conv(u) [T, C]."""
    T, taps = u.shape[0], w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def latent(u: torch.Tensor, w_dkv: torch.Tensor, w_norm: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(u @ w_dkv.T, w_norm, eps)


def windowed_latent_attention(u: torch.Tensor, c: torch.Tensor, wq, wuk, wuv, wg, wo, heads: int, dim: int, vdim: int,
                              scale: float, window: Optional[int]) -> torch.Tensor:
    T = u.shape[0]
    q = (u @ wq.T).view(T, heads, dim)
    k = (c @ wuk.T).view(T, heads, dim)
    v = (c @ wuv.T).view(T, heads, vdim)
    gate = torch.sigmoid(u @ wg.T)                       # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=u.dtype)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for h in range(heads):
            s = (k[lo: t + 1, h] @ q[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = (p[:, None] * v[lo: t + 1, h]).sum(dim=0) * gate[t, h]
    return out.reshape(T, heads * vdim) @ wo.T


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(x))


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(x: torch.Tensor, w_up, w_down, act) -> torch.Tensor:
    return xielu(x @ w_up.T, act[0], act[1]) @ w_down.T


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence. ``layers_out``: a list that receives the stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    taps = int(cfg.get("canon", {}).get("taps", 0) or 0)
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    history = [x]
    latents: Dict[int, torch.Tensor] = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        u = x + causal_conv(x, W[pre + "canon1"]) if taps else x
        src = m.get("kv_from")
        if src is None:
            latents[i] = latent(u, W[pre + "mix.dkv"], W[pre + "mix.dkv.norm"], eps)
            c = latents[i]
        else:
            c = latents[int(src)]
        window = m.get("mask", {}).get("size") if m.get("mask") else None
        a = windowed_latent_attention(u, c, W[pre + "mix.q"], W[pre + "mix.uk"], W[pre + "mix.uv"], W[pre + "mix.g"],
                                      W[pre + "mix.o"], int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]), window)
        x = x + rms(a, W[pre + "norm1"], eps)
        if layer.get("mlp"):
            x = x + rms(dense_ff(x, W[pre + "mlp.up"], W[pre + "mlp.down"], W[pre + "mlp.act"]), W[pre + "norm2"], eps)
        history.append(x)
        a_i = W[pre + "dwa"]
        x = sum(a_i[j] * history[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    y = rms(x, W["final.norm"], eps)
    return (y @ W["embed"].T) * float(cfg["logit_scale"])
