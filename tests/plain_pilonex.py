"""Pilonex in plain PyTorch on the CPU: one function per mechanism, whole sequences, no cache, no state.

The slow statement the engine is compared with. It shares no code with the package: it reads the config
dict and the tensors by name and evaluates every formula directly in the dtype it is asked for (float64
in the tests).

Notation of this file (W x: a matrix stored [out, in] applied to a column; t: time; h: head):

* streams:   X = (x_1 .. x_S), all E[token] at the start. Sublayer q of a layer (1 mixer, 2 feed-forward), with the
             three tensors a_q [S], M_q [S, S], b_q [S]:  u = sum_s a_q[s] x_s;  y = f(rms1(u));
             x'_r = sum_s M_q[s, r] x_s + b_q[r] y  (all r from the OLD streams).  Without streams: x <- x + f(rms1(x)).
             The layer's result, and what the final norm reads, is sum_s x_s.
* rms1(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w);  rms(x; w) the same with w itself;  unit(x) without a weight.
* run order: layers [start, stop) repeated `times` times in a row, every pass with a memory of its own.
* mixer "mlstm": per head a matrix C [dim, vdim], a vector n [dim] and a scalar m, all 0 at the start:
             i = cap tanh((Wi x + bi) / cap),  f = logsigmoid(cap tanh((Wf x + bf) / cap)),
             m' = max(f + m, i),  C' = e^(f + m - m') C + e^(i - m') k v^T,  n' likewise with k,
             o = C'^T q / (max(|n' . q|, e^(-m')) + 1e-6)  with q = Wq x / sqrt(dim);
             out = Wo ( [unit(o_1) .. unit(o_H)] * w * sigmoid(Wg x) ).
* mixer "parallel": c_l * window_attention(x) + c_r * delta_rule(x).
  window_attention: grouped queries; q and k per head through rms(.; w_q), rms(.; w_k), then the first R numbers of
             each head turned by angle p * f_j in pairs (j, j + R/2); f_j = base^(-2j/R), stretched for long waves;
             score = q . k * scale over keys s with 0 <= t - s < window; softmax; values of size vdim; Wo.
  delta_rule: q, k (kv heads x dim), v (heads x vdim) each through a causal filter over time and silu; q, k to unit
             length (1e-6 inside the root), q / sqrt(dim); beta = sigmoid(Wb x); per head and key channel a decay
             g = exp(-exp(A_h) softplus(Wa2 Wa1 x + dt));  C <- g C (rows);  d = beta (v - C^T k);  C <- C + k d^T;
             o = C^T q;  out = Wo ( unit(o_h) * w * sigmoid(Wg2 Wg1 x)_h ).
* feed-forward: y = g sigmoid(1.702 g) (u + 1) with g = min(Wgate x, L), u = clamp(Wup x, -L, L); Wdown y.
  Experts: the `top` largest router logits choose; their softmax weighs the chosen experts' outputs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def rms_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * (1.0 + w)


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


# ----------------------------------------------------------------------------- feed-forward
def clamped_glu(x: torch.Tensor, w_gate, w_up, w_down, limit: float) -> torch.Tensor:
    g = torch.clamp(x @ w_gate.T, max=limit)
    u = torch.clamp(x @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def routed_experts(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, experts: int, top: int, limit: float,
                   margins: Optional[list] = None) -> torch.Tensor:
    """``margins``: receives, per row, how far the last chosen logit lies above the first one left out."""
    z = x @ W[pre + "router"].T                         # [T, experts]
    out = torch.zeros_like(x)
    if margins is not None:
        ranked = torch.sort(z, dim=1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < experts else torch.full((x.shape[0],), float("inf"), dtype=x.dtype))
    for t in range(x.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(z[t, e]), e))[:top]
        zs = torch.stack([z[t, e] for e in order])
        p = torch.softmax(zs, dim=0)
        for w, e in zip(p, order):
            ep = f"{pre}e{e}."
            out[t] += w * clamped_glu(x[t: t + 1], W[ep + "gate"], W[ep + "up"], W[ep + "down"], limit)[0]
    return out


def feed_forward(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, mlp: dict, margins: Optional[list] = None) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return clamped_glu(x, W[pre + "gate"], W[pre + "up"], W[pre + "down"], float(mlp["limit"]))
    if mlp["kind"] == "moe":
        return routed_experts(x, W, pre, int(mlp["router"]["experts"]), int(mlp["router"]["top"]), float(mlp["expert"]["limit"]), margins)
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------------------- matrix memory
def matrix_memory(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, D, V, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (x @ W[pre + "q"].T).view(T, H, D) / math.sqrt(D)
    k = (x @ W[pre + "k"].T).view(T, H, D)
    v = (x @ W[pre + "v"].T).view(T, H, V)
    gi = cap * torch.tanh((x @ W[pre + "i"].T + W[pre + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x @ W[pre + "f"].T + W[pre + "f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=x.dtype)
    for h in range(H):
        C = torch.zeros(D, V, dtype=x.dtype)
        n = torch.zeros(D, dtype=x.dtype)
        mx = torch.zeros((), dtype=x.dtype)
        for t in range(T):
            m_new = torch.maximum(gf[t, h] + mx, gi[t, h])
            keep, put = torch.exp(gf[t, h] + mx - m_new), torch.exp(gi[t, h] - m_new)
            C = keep * C + put * torch.outer(k[t, h], v[t, h])
            n = keep * n + put * k[t, h]
            mx = m_new
            den = torch.maximum((n @ q[t, h]).abs(), torch.exp(-mx)) + 1e-6
            out[t, h] = (C.T @ q[t, h]) / den
    o = unit_rms(out, eps).reshape(T, H * V) * W[pre + "norm"] * torch.sigmoid(x @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


# ----------------------------------------------------------------------------- window attention
def rotary_frequencies(rot: dict, dtype) -> torch.Tensor:
    R = int(rot["dims"])
    j = torch.arange(R // 2, dtype=dtype)
    f = float(rot["base"]) ** (-2.0 * j / R)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wave = 2.0 * math.pi / f
        s = (orig / wave - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, mid))
    return f


def rotate(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, dim]: the first 2 * len(freqs) numbers of each head turn, pairs (j, j + half)."""
    T, half = x.shape[0], freqs.numel()
    ang = torch.arange(T, dtype=x.dtype)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half: 2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)


def window_attention(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms((x @ W[pre + "q"].T).view(T, H, D), W[pre + "q.norm"], eps)
    k = rms((x @ W[pre + "k"].T).view(T, G, D), W[pre + "k.norm"], eps)
    v = (x @ W[pre + "v"].T).view(T, G, V)
    if m.get("rot"):
        f = rotary_frequencies(m["rot"], x.dtype)
        q, k = rotate(q, f), rotate(k, f)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    out = torch.zeros(T, H, V, dtype=x.dtype)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for h in range(H):
            g = h // (H // G)
            p = torch.softmax((k[lo: t + 1, g] @ q[t, h]) * float(m["scale"]), dim=0)
            out[t, h] = p @ v[lo: t + 1, g]
    return out.reshape(T, H * V) @ W[pre + "o"].T


# ----------------------------------------------------------------------------- delta rule
def causal_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps] (the last column meets the current token) -> [T, C]; zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    out = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * u[: T - back]
    return out


def unit_length(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def delta_rule(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    T = x.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    silu = torch.nn.functional.silu
    q = silu(causal_filter(x @ W[pre + "q"].T, W[pre + "q.conv"])).view(T, G, D)
    k = silu(causal_filter(x @ W[pre + "k"].T, W[pre + "k.conv"])).view(T, G, D)
    v = silu(causal_filter(x @ W[pre + "v"].T, W[pre + "v.conv"])).view(T, H, V)
    q, k = unit_length(q) / math.sqrt(D), unit_length(k)
    beta = torch.sigmoid(x @ W[pre + "b"].T)                                        # [T, H]
    dt = torch.nn.functional.softplus((x @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(W[pre + "A_log"])[None, :, None] * dt)             # [T, H, D]
    out = torch.zeros(T, H, V, dtype=x.dtype)
    for h in range(H):
        g = h // (H // G)
        C = torch.zeros(D, V, dtype=x.dtype)
        for t in range(T):
            C = decay[t, h][:, None] * C
            d = beta[t, h] * (v[t, h] - C.T @ k[t, g])
            C = C + torch.outer(k[t, g], d)
            out[t, h] = C.T @ q[t, g]
    gate = torch.sigmoid((x @ W[pre + "g1"].T) @ W[pre + "g2"].T).view(T, H, V)
    o = (unit_rms(out, eps) * W[pre + "norm"] * gate).reshape(T, H * V)
    return o @ W[pre + "o"].T


def mixer(x: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, layer: dict, eps: float) -> torch.Tensor:
    m = layer["mixer"]
    if layer["type"] == "mlstm":
        return matrix_memory(x, W, pre, m, eps)
    if layer["type"] == "parallel":
        return (float(m["left_scale"]) * window_attention(x, W, pre + "left.", m["left"], eps)
                + float(m["right_scale"]) * delta_rule(x, W, pre + "right.", m["right"], eps))
    raise ValueError(layer["type"])


# ----------------------------------------------------------------------------- the model
def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None, router_margins: Optional[list] = None, round_to=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. ``layers_out``: receives the stream after every layer run;
    ``router_margins``: per routed feed-forward that ran, every row's margin between chosen and left-out experts;
    ``round_to``: every sublayer's normed input is rounded to this type (what an engine that hands 16-bit rows to its
    products does at the least), to see how far such roundings alone move the logits of a model."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    S = cfg.get("streams")

    def rounded(v):
        return v if round_to is None else v.to(round_to).to(dtype)

    x0 = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    X = [x0.clone() for _ in range(int(S))] if S else [x0]
    for i in run_order(cfg):
        layer, pre = cfg["layers"][i], f"l{i}."
        subs = [(1, lambda u: mixer(u, W, pre + "mix.", layer, eps))]
        if layer.get("mlp"):
            subs.append((2, lambda u: feed_forward(u, W, pre + "mlp.", layer["mlp"], router_margins)))
        for qn, f in subs:
            if S:
                a, M, b = W[f"{pre}hc{qn}.in"], W[f"{pre}hc{qn}.mix"], W[f"{pre}hc{qn}.out"]
                u = sum(a[s] * X[s] for s in range(len(X)))
                y = f(rounded(rms_one_plus(u, W[f"{pre}norm{qn}"], eps)))
                X = [sum(M[s, r] * X[s] for s in range(len(X))) + b[r] * y for r in range(len(X))]
            else:
                X = [X[0] + f(rounded(rms_one_plus(X[0], W[f"{pre}norm{qn}"], eps)))]
        if layers_out is not None:
            layers_out.append(sum(X))
    return rounded(rms_one_plus(sum(X), W["final.norm"], eps)) @ W["head"].T
