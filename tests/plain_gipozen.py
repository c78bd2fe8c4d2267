"""Gipozen, plainly: float64 torch on whole sequences, one function per mechanism, no cache, no batching.

The engine's kernels are compared with this; it shares no code with them.  `weights` maps tensor names to float64
tensors; `cfg` is the config.json dict.
"""
from __future__ import annotations

import math

import torch

F = torch.float64
GELU_FREE_ALPHA = 1.702      # the constant inside the gated expert's sigmoid


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def causal_conv(u: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps_w [C, K]: y[t] = sum_k taps_w[:, k] * u[t - (K - 1) + k], with u = 0 before the sequence."""
    T, C = u.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for k in range(K):
            src = t - (K - 1) + k
            if src >= 0:
                y[t] += taps_w[:, k] * u[src]
    return y


def in_sight(T: int, window, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & ((i - j < window) | (j < keep_first))
    return see


def diff_lambda(w: dict, p: str, diff: float) -> float:
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def softmax_map(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, see: torch.Tensor) -> torch.Tensor:
    """One attention map: q, k [T, d], v [T, dv]."""
    out = torch.zeros(q.shape[0], v.shape[1], dtype=F)
    for i in range(q.shape[0]):
        js = torch.nonzero(see[i]).flatten()
        s = (k[js] @ q[i]) * scale
        p = torch.exp(s - s.max())
        out[i] = (p / p.sum()) @ v[js]
    return out


def keys_and_values(w: dict, p: str, m: dict, h: torch.Tensor):
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = causal_conv(h @ w[p + "k"].T, w[p + "k.conv"]).view(-1, G, 2, d)
    v = causal_conv(h @ w[p + "v"].T, w[p + "v.conv"]).view(-1, G, dv)
    return k, v


def diff_attention(w: dict, p: str, m: dict, h: torch.Tensor, kv, eps: float) -> torch.Tensor:
    """h [T, width] -> the mixer's output; kv = (k [T, G, 2, d], v [T, G, dv]), this layer's own or another's."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = causal_conv(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, H, 2, d)
    k, v = kv
    mask = m.get("mask") or {}
    see = in_sight(T, mask.get("size"), mask.get("keep_first") or 0)
    lam = diff_lambda(w, p, m["diff"])
    gate = torch.sigmoid(h @ w[p + "g"].T).view(T, H, dv)
    heads = []
    for a in range(H):
        g = a // (H // G)
        first = softmax_map(q[:, a, 0], k[:, g, 0], v[:, g], m["scale"], see)
        second = softmax_map(q[:, a, 1], k[:, g, 1], v[:, g], m["scale"], see)
        heads.append(rms(first - lam * second, eps) * (1.0 - m["diff"]) * gate[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    return coef[0] * rms(z, eps) + coef[1] * rms(z * z, eps) + coef[2] * rms(z * z * z, eps) + coef[3]


def dense(w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    return polynorm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def gated_expert(w: dict, p: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GELU_FREE_ALPHA * g) * (u + 1.0)) @ w[p + "down"].T


def route(w: dict, p: str, h: torch.Tensor, top: int):
    """(chosen [T, top], scores [T, outputs]): softmax scores; chosen by score + correction, largest first."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    order = torch.argsort(s + w[p + "correction"], dim=-1, descending=True, stable=True)
    return order[:, :top], s


def experts(w: dict, p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    r = mlp["router"]
    n_real = r["experts"]
    chosen, s = route(w, p, h, r["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            y = gated_expert(w, p + f"e{e}.", h[t:t + 1], mlp["expert"]["limit"])[0] if e < n_real else h[t]
            out[t] += s[t, e] * y
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(w, p + "shared.", h, mlp["shared"]["limit"])
    return out


def layers_of(cfg: dict, w: dict, tokens):
    """The stream after every layer (after its depth average), and the last one's: list of [T, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    results, kept, after = [x], {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms(x, eps) * w[p + "norm1"]
        if m.get("kv_from") is None:
            kept[i] = keys_and_values(w, p + "mix.", m, h)
        x = x + diff_attention(w, p + "mix.", m, h, kept[i if m.get("kv_from") is None else m["kv_from"]], eps)
        if layer.get("mlp"):
            h = rms(x, eps) * w[p + "norm2"]
            x = x + (dense(w, p + "mlp.", h, eps) if layer["mlp"]["kind"] == "dense" else experts(w, p + "mlp.", layer["mlp"], h))
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        after.append(x)
    return after


def forward(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """float64 logits [T, vocab]."""
    x = layers_of(cfg, w, tokens)[-1]
    return (rms(x, cfg["norm"]["eps"]) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)
