"""Typed configuration of Gipozen, a decoder of differential-attention layers whose residual stream is a
depth-weighted average of all earlier layers' results.

config.json of this design, key by key:

    architecture        "Gipozen"
    vocab, width        sizes of the token table and of the residual stream
    norm.eps            eps of every RMS norm: the layers' (one weight for all channels), the per-head norm of the
                        attention's output, the feed-forward's PolyNorm
    logit_scale         the logits are multiplied by it
    layers[i]           type: "attention";
                        mixer: heads, kv_heads, dim (per map), vdim, conv (taps of the causal convolution on q, k and v),
                        scale, diff, mask.size (a window of keys) and mask.keep_first (the first keys that stay in sight),
                        kv_from (optional: an earlier layer whose keys and values this one reads; it has none of its own);
                        mlp: null, or kind "dense" with ff (up, PolyNorm, down), or kind "moe" with expert.ff,
                        expert.limit, router.experts / identity / top, and shared (ff, limit; optional)
    max_positions       optional: longest sequence the block tables are made for

Tensor names: embed, head, l<i>.norm1 / norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.dwa, final.norm.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17
EXPERT_NAMES = {"router": "router", "gate": "e{}.gate", "up": "e{}.up", "down": "e{}.down", "choice_bias": "correction",
                "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down", "shared_scale": "shared.sg"}


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or key not in mapping:
        raise ConfigError(f"config.json lacks {where}{key}")
    return mapping[key]


@dataclass(frozen=True)
class GipozenConfig:
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "GipozenConfig":
        config = cls(dict(raw))
        config.to_spec()          # every refusal is raised here, before any weight is read
        return config

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ---------------------------------------------------------------- the parts of a layer
    @staticmethod
    def _mixer(layers, i: int, width: int, eps: float) -> PartSpec:
        layer, where = layers[i], f"layers[{i}]."
        kind = _need(layer, "type", where)
        if kind != "attention":
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design; known: attention")
        m = _need(layer, "mixer", where)
        at = where + "mixer."
        heads, kv_heads = int(_need(m, "heads", at)), int(_need(m, "kv_heads", at))
        dim, vdim = int(_need(m, "dim", at)), int(_need(m, "vdim", at))
        taps = int(m.get("conv", 1))
        if min(heads, kv_heads, dim, vdim, taps) <= 0 or heads % kv_heads:
            raise ConfigError(f"{at}: sizes must be positive and heads a multiple of kv_heads")
        if max(2 * dim, vdim) > 256:
            raise ConfigError(f"{at}: two maps of dim {dim} (or values of {vdim}) do not fit the attention kernels' rows of 256")
        mask = m.get("mask") or {}
        window = int(mask["size"]) if mask.get("size") is not None else None
        keep_first = int(mask.get("keep_first") or 0)
        if (window is not None and window < 1) or keep_first < 0:
            raise ConfigError(f"{at}mask: size must be at least 1 and keep_first not negative")
        source = m.get("kv_from")
        if source is not None:
            source = int(source)
            if not 0 <= source < i:
                raise ConfigError(f"{at}kv_from names layer {source}, which must come earlier")
            other = _need(layers[source], "mixer", f"layers[{source}].")
            if other.get("kv_from") is not None:
                raise ConfigError(f"{at}kv_from names layer {source}, which has no keys and values of its own")
            if (int(other.get("kv_heads", 0)), int(other.get("dim", 0)), int(other.get("vdim", 0))) != (kv_heads, dim, vdim):
                raise ConfigError(f"{at}kv_from: layer {source} has other key/value heads or widths")
        return PartSpec("diff_attention", {
            "hidden_size": width, "num_heads": heads, "num_kv_heads": kv_heads, "key_dim": dim, "value_dim": vdim,
            "scale": float(_need(m, "scale", at)), "diff": float(_need(m, "diff", at)), "eps": eps, "conv": taps,
            "window": window, "keep_first": keep_first, "shared_kv": source is not None})

    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int, eps: float):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        at = where + "mlp."
        kind = _need(mlp, "kind", at)
        if kind == "dense":
            ff = int(_need(mlp, "ff", at))
            if ff <= 0:
                raise ConfigError(f"{at}ff must be positive")
            return PartSpec("polynorm_mlp", {"hidden_size": width, "intermediate_size": ff, "eps": eps})
        if kind != "moe":
            raise ConfigError(f"{at}kind {kind!r} is not a feed-forward of this design; known: dense, moe")
        expert, router = _need(mlp, "expert", at), _need(mlp, "router", at)
        experts, top = int(_need(router, "experts", at + "router.")), int(_need(router, "top", at + "router."))
        identity = int(router.get("identity") or 0)
        ff, limit = int(_need(expert, "ff", at + "expert.")), float(_need(expert, "limit", at + "expert."))
        if experts < 1 or identity < 0 or not 0 < top <= experts + identity or ff <= 0 or not limit > 0:
            raise ConfigError(f"{at}: at least one expert, 0 < top <= experts + identity, ff and limit positive")
        shared = mlp.get("shared")
        if shared:
            shared = {"size": int(_need(shared, "ff", at + "shared.")), "limit": float(_need(shared, "limit", at + "shared."))}
            if shared["size"] <= 0 or not shared["limit"] > 0:
                raise ConfigError(f"{at}shared: ff and limit must be positive")
        return PartSpec("routed_experts", {
            "hidden_size": width, "expert_size": ff, "experts": experts, "top": top, "identity": identity, "scores": "softmax",
            "choice_bias": True, "activation": "gated_clamp", "limit": limit, "shared": shared or None, "names": EXPERT_NAMES})

    # ---------------------------------------------------------------- the model
    def to_spec(self) -> ModelSpec:
        raw = self.raw
        if raw.get("architecture") != "Gipozen":
            raise ConfigError(f"architecture {raw.get('architecture')!r} is not Gipozen")
        vocab, width = int(_need(raw, "vocab", "")), int(_need(raw, "width", ""))
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if vocab <= 0 or width <= 0 or not eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        layer_list = _need(raw, "layers", "")
        if not layer_list:
            raise ConfigError("a model needs at least one layer")
        norm = PartSpec("rms_norm_scalar", {"size": width, "eps": eps, "weight_name": ""})
        names = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2", "depth": "dwa"}
        layers, run = [], []
        for i, layer in enumerate(layer_list):
            where = f"layers[{i}]."
            ffn = self._feed_forward(layer, where, width, eps)
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=self._mixer(layer_list, i, width, eps), mixer_norm=norm, feed_forward=ffn,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="pre_norm_depth", names=names,
                                    extras={"depth": PartSpec("depth_weights", {"count": i + 2})}))
            source = layer["mixer"].get("kv_from")
            run.append(RunEntry(layer=i, cache_of=None if source is None else int(source)))
        spec = ModelSpec(
            hidden_size=width, vocab_size=vocab, max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": width, "weight_name": ""}),
            embedding_prefix="embed", layers=tuple(layers), run=tuple(run),
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": width, "tied_to": None, "weight_name": "",
                                          "scale": float(raw.get("logit_scale", 1.0))}),
            head_prefix="head",
            stream=PartSpec("depth_average", {"entries": len(layers)}))
        spec.validate()
        return spec


register_architecture("Gipozen", GipozenConfig)
