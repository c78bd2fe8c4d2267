"""Small Gipozen configurations and seeded weights for the tests.

The shapes differ in what a configuration can set: head counts with and without grouping, map and value widths whose
attention rows need padding and ones that are tensor-core widths (64, 128), windows of a few keys with and without kept
first keys, no mask at all, one to five taps, layers that read an earlier layer's keys and values, layers without a
feed-forward, dense and routed feed-forwards, routers with and without identity and shared experts, top 1 and top all.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def mixer(heads, kv_heads, dim, vdim, scale, conv=3, diff=0.5, window=None, keep_first=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window} if keep_first is None else {"size": window, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, identity=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mix, mlp):
    return {"type": "attention", "mixer": mix, "mlp": mlp}


def model(vocab, width, layers, eps=1e-5, logit_scale=0.5):
    return {"architecture": "Gipozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


# padded rows (2 x 24 and 40 -> 48); shared keys and values; identity and shared experts; a layer without a feed-forward
GA = model(151, 80, [
    layer(mixer(4, 2, 24, 40, 0.21, conv=3, diff=0.55, window=21, keep_first=5), dense(136)),
    layer(mixer(4, 2, 24, 40, 0.19, conv=2, diff=0.3, window=13, keep_first=18, kv_from=0), moe(40, 1.5, 5, 2, identity=2, shared=(24, 0.8))),
    layer(mixer(3, 3, 16, 24, 0.3, conv=4, diff=0.7, window=9), None),
    layer(mixer(6, 3, 16, 24, 0.25, conv=1, diff=0.2, window=40, keep_first=1, kv_from=2), moe(56, 0.7, 3, 1)),
])

# tensor-core row widths: 2 x 32 | 64 -> 64, 2 x 64 | 96 -> 128; windows beyond one query tile and one key range; wide groups
GB = model(263, 128, [
    layer(mixer(8, 2, 32, 64, 0.18, conv=4, diff=0.6, window=150, keep_first=20), dense(200)),
    layer(mixer(2, 1, 64, 96, 0.12, conv=2, diff=0.4, window=70, keep_first=3), moe(64, 1.2, 4, 2, identity=1, shared=(32, 2.0))),
    layer(mixer(4, 2, 32, 64, 0.2, conv=3, diff=0.5, window=300, keep_first=130, kv_from=0), dense(96)),
], eps=1e-6, logit_scale=0.25)

# sizes that fit no 16-byte group; no mask at all; five taps; every router output taken (no choice)
GC = model(97, 52, [
    layer(mixer(3, 1, 10, 12, 0.3, conv=5, diff=0.45), moe(20, 1.0, 3, 5, identity=2)),
    layer(mixer(2, 2, 6, 25, 0.35, conv=2, diff=0.1, window=6, keep_first=2), dense(50)),
    layer(mixer(3, 1, 10, 12, 0.28, conv=3, diff=0.8, window=17, keep_first=0, kv_from=0), None),
], eps=3e-6, logit_scale=1.0)

CASES = {"ga": (GA, 61), "gb": (GB, 62), "gc": (GC, 63)}


def no_choice(cfg: dict) -> dict:
    """The same model with every router output taken: no close call between two experts can change the path."""
    out = json.loads(json.dumps(cfg))
    for spec in out["layers"]:
        if spec.get("mlp") and spec["mlp"]["kind"] == "moe":
            r = spec["mlp"]["router"]
            r["top"] = r["experts"] + (r.get("identity") or 0)
    return out


def tensor_shapes(cfg: dict) -> dict:
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "head": (v, w), "final.norm": ()}
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv", 1)
        shapes.update({p + "norm1": (), p + "dwa": (i + 2,), p + "mix.q": (H * 2 * d, w), p + "mix.q.conv": (H * 2 * d, taps),
                       p + "mix.g": (H * dv, w), p + "mix.o": (w, H * dv)})
        for name in ("lq1", "lk1", "lq2", "lk2"):
            shapes[p + "mix." + name] = (d,)
        if m.get("kv_from") is None:
            shapes.update({p + "mix.k": (G * 2 * d, w), p + "mix.k.conv": (G * 2 * d, taps), p + "mix.v": (G * dv, w),
                           p + "mix.v.conv": (G * dv, taps)})
        mlp = spec.get("mlp")
        if not mlp:
            continue
        shapes[p + "norm2"] = ()
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], w), p + "mlp.down": (w, mlp["ff"]), p + "mlp.act": (4,)})
            continue
        r, ff = mlp["router"], mlp["expert"]["ff"]
        outputs = r["experts"] + (r.get("identity") or 0)
        shapes.update({p + "mlp.router": (outputs, w), p + "mlp.correction": (outputs,)})
        for e in range(r["experts"]):
            shapes.update({p + f"mlp.e{e}.gate": (ff, w), p + f"mlp.e{e}.up": (ff, w), p + f"mlp.e{e}.down": (w, ff)})
        if mlp.get("shared"):
            fs = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (fs, w), p + "mlp.shared.up": (fs, w), p + "mlp.shared.down": (w, fs),
                           p + "mlp.shared.sg": (1, w)})
    return shapes


def make_weights(cfg: dict, seed: int, gain: float = 1.0) -> dict:
    """Seeded weights, every value representable in bfloat16 (so a bfloat16 engine and a float oracle start alike).
    `gain` scales the query and key projections (a larger one makes the softmax peaked).  Norm weights, averaging
    weights, taps, router corrections and the lambda vectors are spread widely, so that leaving one out moves the logits."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            value = 1.0 + 0.3 * rng.standard_normal(shape)
        elif leaf == "dwa":
            value = 0.25 * rng.standard_normal(shape) + (np.arange(shape[0]) == shape[0] - 1) * 0.8 + 0.1
        elif leaf == "conv":
            value = 0.5 * rng.standard_normal(shape) + (np.arange(shape[1]) == shape[1] - 1) * 0.6
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            value = 0.25 * rng.standard_normal(shape)
        elif leaf == "act":
            value = np.array([0.6, 0.3, 0.2, 0.05]) + 0.1 * rng.standard_normal(shape)
        elif leaf == "correction":
            value = 0.1 * rng.standard_normal(shape)
        elif leaf == "router":
            value = 3.0 / np.sqrt(shape[1]) * rng.standard_normal(shape)
        elif name == "embed":
            value = rng.standard_normal(shape)
        elif ".mix." in name and leaf in ("q", "k"):
            value = gain / np.sqrt(shape[1]) * rng.standard_normal(shape)
        elif leaf in ("gate", "up") and ".mlp.e" in name or ".shared." in name and leaf in ("gate", "up"):
            value = 1.5 / np.sqrt(shape[1]) * rng.standard_normal(shape)      # wide enough that the clamps bite
        else:
            value = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.tensor(np.asarray(value), dtype=torch.float32).to(torch.bfloat16).to(torch.float64)
    return out


def write_model_dir(directory, cfg: dict, weights: dict) -> Path:
    from safetensors.torch import save_file
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    (directory / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, str(directory / "model.safetensors"))
    return directory


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def one_layer(mix, mlp=None, width=64, vocab=101):
    return model(vocab, width, [layer(mix, mlp)])
