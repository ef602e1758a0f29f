"""A plain, slow implementation of the Medodra decoder: one function per mechanism, 64-bit, whole sequences, no cache.

It shares no code with the library: tensors come as a ``{name: tensor}`` mapping, sizes and constants from the nested
configuration (a dict shaped like config.json). Every function works on ONE sequence given from its first token on;
recurrences are written token by token, attention as an explicit double loop over (query, key) reduced with tensor
operations per query.

Notation: ``h`` is a mixer's or feed-forward's input ``[T, width]``; linear weights are ``[out, in]``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def load_model(model_dir: str):
    """(the JSON object of config.json, {name: tensor}) of a model folder"""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))


def _w(t: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    return t[name].to(F64)


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose gain is stored around zero"""
    return rms(x, eps) * (1.0 + w)


def sinusoid(positions: torch.Tensor, width: int) -> torch.Tensor:
    """[T, width]: column 2i holds sin(p f_i), column 2i + 1 holds cos(p f_i), f_i = 10000^(-2i / width)"""
    out = torch.zeros((positions.numel(), width), dtype=F64)
    for c in range(width):
        i = c // 2
        ang = positions.to(F64) * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def embedding(t, tokens: List[int], scale: float, width: int, first_pos: int = 0) -> torch.Tensor:
    pos = torch.arange(first_pos, first_pos + len(tokens))
    return _w(t, "embed")[torch.tensor(tokens, dtype=torch.long)] * scale + sinusoid(pos, width)


def _conv(t, name: str, u: torch.Tensor) -> torch.Tensor:
    """the projection's short convolution, where the model has one"""
    return short_conv(u, _w(t, name)) if name in t else u


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """causal convolution over time per channel: u [T, C], w [C, taps]; the last tap meets the current token and
    zeros stand before the sequence's start"""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for tt in range(T):
        for j in range(taps):
            src = tt - (taps - 1) + j
            if src >= 0:
                y[tt] += w[:, j] * u[src]
    return y


# ----------------------------------------------------------------------------------------------- gated delta rule
def delta_recurrence(q, k, v, beta, decay, states: Optional[list] = None):
    """q, k [T, G, d], v [T, H, dv], beta and decay [T, H]: per head S <- decay S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q, token by token from S = 0 (or from ``states[h]``, which is left as the last S)"""
    T, H, dv = v.shape
    G, d = k.shape[1], k.shape[2]
    out = torch.zeros((T, H, dv), dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros((d, dv), dtype=F64) if states is None else states[hh]
        for tt in range(T):
            S = decay[tt, hh] * S
            u = beta[tt, hh] * (v[tt, hh] - S.T @ k[tt, g])
            S = S + torch.outer(k[tt, g], u)
            out[tt, hh] = S.T @ q[tt, g]
        if states is not None:
            states[hh] = S
    return out


def gated_delta_mixer(t, p: str, m: Mapping, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = silu(_conv(t, p + "q.conv", h @ _w(t, p + "q").T)).view(T, G, d)
    k = silu(_conv(t, p + "k.conv", h @ _w(t, p + "k").T)).view(T, G, d)
    v = silu(_conv(t, p + "v.conv", h @ _w(t, p + "v").T)).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ _w(t, p + "b").T)                                              # [T, H]
    decay = torch.exp(-torch.exp(_w(t, p + "A_log")) * softplus(h @ _w(t, p + "a").T + _w(t, p + "dt_bias")))
    out = delta_recurrence(q, k, v, beta, decay)
    out = rms(out, eps) * _w(t, p + "norm")
    out = out.reshape(T, H * dv) * silu(h @ _w(t, p + "g").T)
    return out @ _w(t, p + "o").T


# ----------------------------------------------------------------------------------------------- left: biased sigmoid attention
def distance_bucket(n: int, n_rows: int, far: float) -> int:
    half = n_rows // 2
    if n < half:
        return n
    return min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (n_rows - half))))


def sigmoid_attention(q, k, v, scale: float, rel, far: float, pb, first_query: int = 0):
    """q [Tq, H, d] (the last Tq positions of the sequence when ``first_query`` > 0), k [T, G, d], v [T, G, dv],
    rel [rows, H], pb [H]: out[i, h] = sum over j <= i of sigmoid(q_i . k_j * scale + rel[bucket(i - j), h] + pb[h]) v_j"""
    Tq, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    n_rows = rel.shape[0]
    out = torch.zeros((Tq, H, dv), dtype=F64)
    row_of = torch.tensor([distance_bucket(n, n_rows, far) for n in range(first_query + Tq)], dtype=torch.long)
    for r in range(Tq):
        i = first_query + r
        bias = rel[row_of[i - torch.arange(i + 1)]]                                               # [i + 1, H]
        for hh in range(H):
            g = hh // (H // G)
            s = (k[: i + 1, g] @ q[r, hh]) * scale + bias[:, hh]
            out[r, hh] = sigmoid(s + pb[hh]) @ v[: i + 1, g]
    return out


def sigmoid_attention_mixer(t, p: str, m: Mapping, h: torch.Tensor, eps: float, first_pos: int = 0) -> torch.Tensor:
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = _conv(t, p + "q.conv", h @ _w(t, p + "q").T + _w(t, p + "q.b")).view(T, H, d)
    k = _conv(t, p + "k.conv", h @ _w(t, p + "k").T + _w(t, p + "k.b")).view(T, G, d)
    v = _conv(t, p + "v.conv", h @ _w(t, p + "v").T + _w(t, p + "v.b")).view(T, G, dv)
    coef, every = float(m["q_temp"]["coef"]), int(m["q_temp"]["every"])
    for tt in range(T):
        pp = first_pos + tt
        q[tt] = q[tt] * (1.0 + coef * math.log((pp + 1) // every + 1))
    v = rms(v, eps)
    rel, pb = _w(t, p + "rel"), _w(t, p + "pb")
    far, scale = float(m["bias_max"]), float(m["scale"])
    out = sigmoid_attention(q, k, v, scale, rel, far, pb)
    return out.reshape(T, H * dv) @ _w(t, p + "o").T + _w(t, p + "o.b")


# ----------------------------------------------------------------------------------------------- right: minGRU
def min_gru_scan(z, u, S: Optional[torch.Tensor] = None):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t with c = u + 1/2 where u >= 0 and sigmoid(u) where u < 0; [T, W] of the S_t"""
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    S = torch.zeros(z.shape[1], dtype=F64) if S is None else S
    states = []
    for tt in range(z.shape[0]):
        S = (1.0 - z[tt]) * S + z[tt] * cand[tt]
        states.append(S)
    return torch.stack(states)


def min_gru_mixer(t, p: str, m: Mapping, h: torch.Tensor) -> torch.Tensor:
    z = sigmoid(h @ _w(t, p + "z").T + _w(t, p + "z.b"))
    u = h @ _w(t, p + "x").T + _w(t, p + "x.b")
    return (min_gru_scan(z, u) * silu(h @ _w(t, p + "g").T)) @ _w(t, p + "o").T


def parallel_mixer(t, p: str, m: Mapping, h: torch.Tensor, eps: float) -> torch.Tensor:
    left = sigmoid_attention_mixer(t, p + "left.", m["left"], h, eps)
    right = min_gru_mixer(t, p + "right.", m["right"], h)
    return 0.5 * (rms(left, eps) * _w(t, p + "left.out") + rms(right, eps) * _w(t, p + "right.out"))


# ----------------------------------------------------------------------------------------------- feed-forward
def gated_expert(t, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ _w(t, p + "gate").T) * (h @ _w(t, p + "up").T)) @ _w(t, p + "down").T


def moe_feed_forward(t, p: str, m: Mapping, h: torch.Tensor) -> torch.Tensor:
    E, top = int(m["router"]["experts"]), int(m["router"]["top"])
    s = sigmoid(h @ _w(t, p + "router").T)                                           # [T, E]
    out = torch.zeros_like(h)
    for tt in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[tt, e]), e))[:top]
        for e in order:
            out[tt] += gated_expert(t, p + "e%d." % e, (s[tt, e] * h[tt])[None])[0]
    if m.get("shared") is not None:
        out = out + gated_expert(t, p + "shared.", h) * sigmoid(h @ _w(t, p + "shared.sg").T)
    return out


# ----------------------------------------------------------------------------------------------- the model
def run_order(cfg: Mapping) -> List[tuple]:
    """(layer, starts a pass) in the order the layers run"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg: Mapping, t: Mapping[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None):
    """logits [T, vocab] (64-bit) of one sequence given from its first token on"""
    width, eps = int(cfg["width"]), float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    x0 = embedding(t, tokens, float((cfg.get("embedding") or {}).get("scale", 1.0)), width)
    x = x0
    for i, starts in run_order(cfg):
        layer = cfg["layers"][i]
        p = "l%d." % i
        if starts:
            x = torch.cat([x, x0], dim=1) @ _w(t, "loop.in").T
        h1 = norm_one_plus(x, _w(t, p + "norm1"), eps)
        if layer["type"] == "delta":
            y = gated_delta_mixer(t, p + "mix.", layer["mixer"], h1, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(t, p + "mix.", layer["mixer"], h1, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + moe_feed_forward(t, p + "mlp.", layer["mlp"], norm_one_plus(x, _w(t, p + "norm2"), eps))
        x = x + mult * y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return norm_one_plus(x, _w(t, "final.norm"), eps) @ _w(t, "head").T
