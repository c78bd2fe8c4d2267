"""Vilodra, plainly: float64 torch on whole sequences, one function per mechanism, no cache, no batching.

The engine's kernels are compared with this; it shares no code with them.  `w` maps tensor names to float64
tensors; `cfg` is the config.json dict.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


# ------------------------------------------------------------------ small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of the layers and of the model's end: the tensor holds the factor's offset from one."""
    return rms(x, eps) * (1.0 + weight)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# ------------------------------------------------------------------ rotation
def plain_frequencies(base: float, dims: int) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=F)
    return base ** (-2.0 * i / dims)


def stretched_by_wavelength(freq: torch.Tensor, s: dict) -> torch.Tensor:
    """Short waves stay, long waves slow down by `factor`, those between are blended by where their wavelength lies."""
    factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = freq.clone()
    for i, f in enumerate(freq.tolist()):
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out[i] = f
        elif wave > original / low:
            out[i] = f / factor
        else:
            t = (original / wave - low) / (high - low)
            out[i] = (1.0 - t) * f / factor + t * f
    return out


def stretched_by_ramp(freq: torch.Tensor, base: float, dims: int, s: dict):
    """A ramp over the pair index between the pairs that make `fast` and `slow` turns over the original length; returns
    the frequencies and the factor both tables are multiplied by."""
    factor, original = float(s["factor"]), float(s["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(s["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(s["slow"]))), dims - 1)
    out = freq.clone()
    for i, f in enumerate(freq.tolist()):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f / factor * ramp + f * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def turn_pairs(x: torch.Tensor, freq: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """x [T, ..., n]: coordinates (2i, 2i + 1) for i < len(freq) turn by position * freq[i]; the rest pass."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=F)
    shape = [T] + [1] * (x.dim() - 2)
    for i, f in enumerate(freq.tolist()):
        c = (torch.cos(pos * f) * magnitude).view(shape)
        s = (torch.sin(pos * f) * magnitude).view(shape)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ------------------------------------------------------------------ lightning mixer
def lightning_recurrence(q, k, v, decay):
    """q, k [T, H, d], v [T, H, dv], decay [H]: S <- decay S + k v^T, o = S^T q, token by token from S = 0."""
    T, H, d = q.shape
    dv = v.shape[2]
    o = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = decay[a] * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    return o


def lightning(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o = lightning_recurrence(q, k, v, torch.tensor(m["decay"], dtype=F)).reshape(T, H * dv)
    o = rms(o, eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------ differential attention
def softmax_rows(scores: torch.Tensor, see: torch.Tensor, sink=None) -> torch.Tensor:
    """Row-wise softmax over the keys in sight; `sink`: one more term exp(sink) in the denominator only."""
    out = torch.zeros_like(scores)
    for i in range(scores.shape[0]):
        js = torch.nonzero(see[i]).flatten()
        s = scores[i, js]
        top = s.max() if sink is None else max(float(s.max()), float(sink))
        e = torch.exp(s - top)
        den = e.sum() + (0.0 if sink is None else math.exp(float(sink) - float(top)))
        out[i, js] = e / den
    return out


def causal(T: int, window=None) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & (i - j < window)
    return see


def diff_attention(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    rot = m["rot"]
    freq = plain_frequencies(float(rot["base"]), int(rot["dims"]))
    if rot.get("scaling"):
        freq = stretched_by_wavelength(freq, rot["scaling"])
    q = turn_pairs((h @ w[p + "q"].T).view(T, H, 2, d), freq)
    k = turn_pairs((h @ w[p + "k"].T).view(T, G, 2, d), freq)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    lam = (math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum()))
           + float(m["diff"]))
    see = causal(T)
    heads = []
    for a in range(H):
        g = a // (H // G)
        maps = [softmax_rows((q[:, a, n] @ k[:, g, n].T) * m["scale"], see) @ v[:, g] for n in range(2)]
        heads.append(rms(maps[0] - lam * maps[1], eps) * (1.0 - float(m["diff"])))
    return torch.cat(heads, dim=1) @ w[p + "o"].T


# ------------------------------------------------------------------ latent attention
def latent_rows(w: dict, p: str, m: dict, h: torch.Tensor, eps: float):
    """What a layer with a down projection keeps per token: the normed latent and the turned key part."""
    rank, r = m["kv_rank"], m["rot_dim"]
    rot = m["rot"]
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    freq = plain_frequencies(float(rot["base"]), int(rot["dims"]))
    magnitude = 1.0
    if rot.get("scaling"):
        freq, magnitude = stretched_by_ramp(freq, float(rot["base"]), int(rot["dims"]), rot["scaling"])
    return c, turn_pairs(down[:, rank:rank + r], freq, magnitude)


def latent_attention(w: dict, p: str, m: dict, h: torch.Tensor, kept) -> torch.Tensor:
    """`kept` = (latent [T, rank], turned key part [T, rot_dim]) of this layer or of the layer it reads."""
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    rot = m["rot"]
    c, k_rot = kept
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    freq = plain_frequencies(float(rot["base"]), int(rot["dims"]))
    magnitude = 1.0
    if rot.get("scaling"):
        freq, magnitude = stretched_by_ramp(freq, float(rot["base"]), int(rot["dims"]), rot["scaling"])
    q_rot = turn_pairs(q[:, :, d:], freq, magnitude)
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    see = causal(T, (m.get("mask") or {}).get("size"))
    heads = []
    for a in range(H):
        scores = (q[:, a, :d] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        heads.append(softmax_rows(scores, see, sink=float(w[p + "sink"][a])) @ v[:, a])
    return torch.cat(heads, dim=1) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(w: dict, p: str, router: dict, h: torch.Tensor):
    """Per token: the chosen experts (best first) and their weights."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    top = int(router["top"])
    best = torch.topk(s, top, dim=-1)
    weight = best.values / (best.values.sum(dim=-1, keepdim=True) + 1e-20) * float(router["scale"])
    return best.indices, weight


def expert(w: dict, p: str, e: int, h: torch.Tensor) -> torch.Tensor:
    return gelu_erf(h @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T


def routed_ff(w: dict, p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    chosen, weight = route(w, p, mlp["router"], h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * expert(w, p, e, h[t:t + 1])[0]
    return out


# ------------------------------------------------------------------ the model
def forward(cfg: dict, w: dict, tokens, after_layer=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; `after_layer(i, x)` is called with the stream after every layer."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if kind == "lightning":
            y = lightning(w, p + "mix.", m, h, eps)
        elif kind == "attention":
            y = diff_attention(w, p + "mix.", m, h, eps)
        elif kind == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_rows(w, p + "mix.", m, h, eps)
            y = latent_attention(w, p + "mix.", m, h, kept[i if m.get("kv_from") is None else int(m["kv_from"])])
        else:
            raise ValueError(kind)
        x = x + mult * y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            y = dense_ff(w, p + "mlp.", h) if mlp["kind"] == "dense" else routed_ff(w, p + "mlp.", mlp, h)
            x = x + mult * y
        if after_layer is not None:
            after_layer(i, x)
    return layer_norm(x, w["final.norm"], eps) @ w["embed"].T
