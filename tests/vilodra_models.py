"""Small Vilodra configurations and seeded weights for the tests.

The shapes differ in what a configuration can set: every order of the three mixers; lightning heads with key rows that
fill no warp, exactly one, and two; a decay of exactly 1; differential attention with and without grouping, part and
whole rotation, with and without stretched frequencies; latent attention with windows of a few keys, beyond one query
tile, and none, readers whose window is wider and narrower than their owner's; cache rows that need padding and rows of
tensor-core widths; layers without a feed-forward; routers that take one, two and all experts; a residual multiplier of 1.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def lightning(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def attention(heads, kv_heads, dim, vdim, scale, diff, rot_dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return "attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff, "rot": rot}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, window=None, base=50000.0, scaling=None, kv_from=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "latent_attention", m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def layer(mix, mlp):
    return {"type": mix[0], "mixer": mix[1], "mlp": mlp}


def model(vocab, width, layers, eps=1e-5, mult=0.6):
    return {"architecture": "Vilodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


YARN_A, YARN_B = (4.0, 64, 8.0, 1.0), (6.0, 96, 24.0, 2.0)

# padded cache rows (40 + 8 -> 48; 2 x 24 | 40 -> 48), a reader with a wider window than its owner, a decay of 1
VA = model(157, 72, [
    layer(lightning(3, 20, 12, (0.7, 0.93, 1.0)), dense(100)),
    layer(latent(3, 24, 8, 20, 40, 0.21, window=19, scaling=YARN_A), moe(40, 5, 2, 1.7)),
    layer(attention(4, 2, 24, 40, 0.2, 0.55, 12, scaling=(4.0, 1.0, 4.0, 48)), None),
    layer(latent(2, 16, 8, 28, 40, 0.25, window=33, scaling=YARN_A, kv_from=1), dense(56)),
    layer(lightning(2, 40, 24, (0.85, 0.99)), moe(24, 3, 1, 0.8)),
], mult=0.6)

# tensor-core row widths (64 and 128), windows beyond a query tile and a key range, wide query groups, whole rotation
VB = model(263, 128, [
    layer(attention(4, 1, 32, 64, 0.18, 0.3, 32), dense(192)),
    layer(lightning(2, 64, 64, (0.9, 0.995)), moe(64, 4, 2, 2.5)),
    layer(latent(8, 32, 16, 32, 48, 0.15, window=150), dense(96)),
    layer(latent(4, 48, 16, 24, 48, 0.17, window=70, kv_from=2), moe(64, 4, 2, 1.0)),
    layer(attention(2, 2, 64, 128, 0.12, 0.7, 16, base=500.0, scaling=(8.0, 1.0, 2.0, 40)), None),
    layer(latent(2, 64, 64, 64, 64, 0.1, window=300, base=1000.0, scaling=YARN_B), dense(64)),
], eps=1e-6, mult=0.8)

# sizes that fit no 16-byte group; one head everywhere; no window at all; every expert taken; a multiplier of 1
VC = model(97, 52, [
    layer(latent(1, 10, 6, 7, 13, 0.4), moe(20, 3, 3, 1.0)),
    layer(lightning(1, 10, 7, (0.8,)), dense(50)),
    layer(attention(1, 1, 10, 25, 0.3, 0.45, 4), None),
    layer(latent(3, 6, 6, 9, 13, 0.35, window=5, kv_from=0), dense(30)),
    layer(lightning(5, 34, 3, (0.5, 0.6, 0.97, 0.999, 0.75)), None),
], eps=3e-6, mult=1.0)

CASES = {"va": (VA, 71), "vb": (VB, 72), "vc": (VC, 73)}


def no_choice(cfg: dict) -> dict:
    """The same model with every expert taken: no close call between two experts can change the path."""
    out = json.loads(json.dumps(cfg))
    for spec in out["layers"]:
        if spec.get("mlp") and spec["mlp"]["kind"] == "moe":
            spec["mlp"]["router"]["top"] = spec["mlp"]["router"]["experts"]
    return out


def tensor_shapes(cfg: dict) -> dict:
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,)}
    for i, spec in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", spec["mixer"], spec["type"]
        shapes[p + "norm1"] = (w,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if kind == "lightning":
            shapes.update({p + "mix.q": (H * d, w), p + "mix.k": (H * d, w), p + "mix.v": (H * dv, w), p + "mix.g": (H * dv, w),
                           p + "mix.norm": (H * dv,), p + "mix.o": (w, H * dv)})
        elif kind == "attention":
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * 2 * d, w), p + "mix.k": (G * 2 * d, w), p + "mix.v": (G * dv, w), p + "mix.o": (w, H * dv)})
            for name in ("lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + name] = (d,)
        else:
            r, rank = m["rot_dim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (d + r), w), p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.sink": (H,),
                           p + "mix.o": (w, H * dv)})
            if m.get("kv_from") is None:
                shapes.update({p + "mix.dkv": (rank + r, w), p + "mix.dkv.norm": (rank,)})
        mlp = spec.get("mlp")
        if not mlp:
            continue
        shapes[p + "norm2"] = (w,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], w), p + "mlp.up": (mlp["ff"], w), p + "mlp.down": (w, mlp["ff"])})
            continue
        ff = mlp["expert"]["ff"]
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], w)
        for e in range(mlp["router"]["experts"]):
            shapes.update({p + f"mlp.e{e}.up": (ff, w), p + f"mlp.e{e}.down": (w, ff)})
    return shapes


def make_weights(cfg: dict, seed: int, gain: float = 1.0) -> dict:
    """Seeded weights, every value representable in bfloat16 (so a bfloat16 engine and a float oracle start alike).
    `gain` scales the query projections of the softmax mixers (a larger one makes the softmax peaked).  Norm weights
    (offsets from one), sinks, the lambda vectors and routers are spread widely, so that leaving one out, or using a
    weight without its offset, moves the logits."""
    rng = np.random.default_rng(seed)
    out = {}
    lightning_layers = {f"l{i}." for i, spec in enumerate(cfg["layers"]) if spec["type"] == "lightning"}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            value = 0.3 * rng.standard_normal(shape)
        elif leaf == "norm":                                   # plain weights: of the latent and of the lightning output
            value = 1.0 + 0.3 * rng.standard_normal(shape)
        elif leaf == "sink":
            value = 1.5 * rng.standard_normal(shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            value = 0.25 * rng.standard_normal(shape)
        elif leaf == "router":
            value = 3.0 / np.sqrt(shape[1]) * rng.standard_normal(shape)
        elif name == "embed":
            value = rng.standard_normal(shape)
        elif ".mix." in name and leaf == "q" and name[:name.index("mix.")] not in lightning_layers:
            value = gain / np.sqrt(shape[1]) * rng.standard_normal(shape)
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


def one_layer(mix, mlp=None, width=64, vocab=101, mult=0.7):
    return model(vocab, width, [layer(mix, mlp)], mult=mult)
