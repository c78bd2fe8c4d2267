"""Typed configuration of Vilodra, a decoder that mixes three kinds of layers: lightning attention (a linear recurrence
with a matrix state per head), differential attention with rotary positions, and latent attention behind a sliding
window with a learned softmax sink per head; dense gated and routed feed-forwards; every residual branch multiplied by
one constant; the token table doubles as the output head.

config.json of this design, key by key:

    architecture        "Vilodra"
    vocab, width        sizes of the token table and of the residual stream
    norm.eps            eps of every RMS norm (the layers' and the final norm, whose weights are offsets from one: the factor is
                        1 + w; the lightning mixer's output norm; the latent's norm; the per-head norm of the
                        differential attention)
    residual_mult       x <- x + residual_mult * f(norm(x)) for the mixer and for the feed-forward
    layers[i]           type, mixer, mlp:
      type "lightning"          mixer: heads, dim, vdim, decay (one number per head)
      type "attention"          mixer: heads, kv_heads, dim (per map), vdim, scale, diff, rot (base, dims, optional scaling:
                                factor, low, high, original)
      type "latent_attention"   mixer: heads, dim (unrotated), rot_dim, vdim, kv_rank, scale, rot (base, dims = rot_dim,
                                optional scaling: factor, original, fast, slow), mask.size (optional window), kv_from
                                (optional: an earlier layer whose cached latent and key part this one reads; it has no
                                down projection of its own)
      mlp                       null, or kind "dense" with ff, or kind "moe" with expert.ff and router.experts / top / scale
    max_positions       optional: longest sequence the block tables are made for

Tensor names: embed, l<i>.norm1 / norm2, l<i>.mix.*, l<i>.mlp.*, final.norm.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17
MIXER_TYPES = ("lightning", "attention", "latent_attention")
HEAD_STEP, HEAD_MAX = 16, 256        # the attention kernels take rows that are multiples of 16 up to 256
LIGHTNING_MAX_KEY_DIM = 256          # the recurrence kernels hold up to this many rows per state column


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or key not in mapping:
        raise ConfigError(f"config.json lacks {where}{key}")
    return mapping[key]


def _rotation(rot: Mapping[str, Any], at: str, kind: str) -> PartSpec:
    """The rotary encoding of a mixer: neighbouring coordinates paired, `dims` of them turned, frequencies stretched by
    the mixer's own rule where `scaling` is given ("wavelength" for the differential attention, "yarn" for the latent)."""
    dims, base = int(_need(rot, "dims", at)), float(_need(rot, "base", at))
    if dims <= 0 or dims % 2 or not base > 0:
        raise ConfigError(f"{at}: dims must be positive and even, base positive")
    params = {"theta": base, "dim": dims}
    scaling = rot.get("scaling")
    if scaling:
        keys = ("factor", "low", "high", "original") if kind == "wavelength" else ("factor", "original", "fast", "slow")
        params["scaling"] = {"kind": kind, **{key: float(_need(scaling, key, at + "scaling.")) for key in keys}}
        if kind == "wavelength" and params["scaling"]["high"] == params["scaling"]["low"]:
            raise ConfigError(f"{at}scaling: high and low must differ")
    return PartSpec("rotary_interleaved", params)


@dataclass(frozen=True)
class VilodraConfig:
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VilodraConfig":
        config = cls(dict(raw))
        config.to_spec()          # every refusal is raised here, before any weight is read
        return config

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ---------------------------------------------------------------- mixers
    @staticmethod
    def _lightning(m, at: str, width: int, eps: float) -> PartSpec:
        heads, dim, vdim = int(_need(m, "heads", at)), int(_need(m, "dim", at)), int(_need(m, "vdim", at))
        decay = [float(d) for d in _need(m, "decay", at)]
        if min(heads, dim, vdim) <= 0 or len(decay) != heads or not all(0.0 < d <= 1.0 for d in decay):
            raise ConfigError(f"{at}: sizes must be positive, with one decay in (0, 1] per head")
        if dim > LIGHTNING_MAX_KEY_DIM:
            raise ConfigError(f"{at}dim {dim} is not supported: the recurrence takes key heads up to {LIGHTNING_MAX_KEY_DIM}")
        return PartSpec("lightning", {"hidden_size": width, "num_heads": heads, "key_dim": dim, "value_dim": vdim, "decay": tuple(decay),
                                      "eps": eps})

    @staticmethod
    def _attention(m, at: str, width: int, eps: float) -> PartSpec:
        heads, kv_heads = int(_need(m, "heads", at)), int(_need(m, "kv_heads", at))
        dim, vdim = int(_need(m, "dim", at)), int(_need(m, "vdim", at))
        if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
            raise ConfigError(f"{at}: sizes must be positive and heads a multiple of kv_heads")
        if max(2 * dim, vdim) > HEAD_MAX:
            raise ConfigError(f"{at}: two maps of dim {dim} (or values of {vdim}) do not fit the attention kernels' rows of {HEAD_MAX}")
        position = _rotation(_need(m, "rot", at), at + "rot.", "wavelength")
        if position["dim"] > dim:
            raise ConfigError(f"{at}rot.dims must not exceed dim")
        return PartSpec("diff_attention", {
            "hidden_size": width, "num_heads": heads, "num_kv_heads": kv_heads, "key_dim": dim, "value_dim": vdim,
            "scale": float(_need(m, "scale", at)), "diff": float(_need(m, "diff", at)), "eps": eps, "conv": 0, "gate": False,
            "position": position, "window": None, "keep_first": 0, "shared_kv": False, "in_place": True})

    @staticmethod
    def _latent(layers, i: int, at: str, width: int, eps: float) -> PartSpec:
        m = layers[i]["mixer"]
        heads, dim, rot_dim = int(_need(m, "heads", at)), int(_need(m, "dim", at)), int(_need(m, "rot_dim", at))
        vdim, kv_rank = int(_need(m, "vdim", at)), int(_need(m, "kv_rank", at))
        if min(heads, dim, rot_dim, vdim, kv_rank) <= 0:
            raise ConfigError(f"{at}: sizes must be positive")
        position = _rotation(_need(m, "rot", at), at + "rot.", "yarn")
        if position["dim"] != rot_dim:
            raise ConfigError(f"{at}rot.dims must equal rot_dim")
        if -(-(kv_rank + rot_dim) // HEAD_STEP) * HEAD_STEP > HEAD_MAX:
            raise ConfigError(f"{at}kv_rank + rot_dim = {kv_rank + rot_dim} is not supported: the attention kernels take cache rows up to {HEAD_MAX} wide")
        mask = m.get("mask") or {}
        window = int(mask["size"]) if mask.get("size") is not None else None
        if window is not None and window < 1:
            raise ConfigError(f"{at}mask.size must be at least 1")
        source = m.get("kv_from")
        if source is not None:
            source = int(source)
            if not 0 <= source < i:
                raise ConfigError(f"{at}kv_from names layer {source}, which must come earlier")
            other = layers[source]
            if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                raise ConfigError(f"{at}kv_from names layer {source}, which has no down projection of its own")
            same = ("kv_rank", "rot_dim", "rot")
            if any(other["mixer"].get(key) != m.get(key) for key in same):
                raise ConfigError(f"{at}kv_from: layer {source} has another kv_rank, rot_dim or rotation")
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": heads, "plain_dim": dim, "rot_dim": rot_dim, "value_dim": vdim, "kv_rank": kv_rank,
            "q_rank": 0, "gate": False, "position": position, "scale": float(_need(m, "scale", at)), "eps": eps, "window": window,
            "sink": True, "shared_kv": source is not None,
            "names": {"q": "q", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o", "sink": "sink"}})

    def _mixer(self, layers, i: int, width: int, eps: float) -> PartSpec:
        where = f"layers[{i}]."
        kind = _need(layers[i], "type", where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design; known: {', '.join(MIXER_TYPES)}")
        m, at = _need(layers[i], "mixer", where), where + "mixer."
        if kind == "lightning":
            return self._lightning(m, at, width, eps)
        if kind == "attention":
            return self._attention(m, at, width, eps)
        return self._latent(layers, i, at, width, eps)

    # ---------------------------------------------------------------- feed-forwards
    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int) -> Optional[PartSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        at = where + "mlp."
        kind = _need(mlp, "kind", at)
        if kind == "dense":
            ff = int(_need(mlp, "ff", at))
            if ff <= 0:
                raise ConfigError(f"{at}ff must be positive")
            return PartSpec("swiglu", {"hidden_size": width, "intermediate_size": ff, "names": {"gate": "gate", "up": "up", "down": "down"}})
        if kind != "moe":
            raise ConfigError(f"{at}kind {kind!r} is not a feed-forward of this design; known: dense, moe")
        router = _need(mlp, "router", at)
        experts, top = int(_need(router, "experts", at + "router.")), int(_need(router, "top", at + "router."))
        ff = int(_need(_need(mlp, "expert", at), "ff", at + "expert."))
        if min(experts, top, ff) <= 0 or top > experts:
            raise ConfigError(f"{at}: experts, top and ff must be positive and top at most experts")
        return PartSpec("routed_experts", {
            "hidden_size": width, "expert_size": ff, "experts": experts, "top": top, "scores": "softmax", "renormalize": True,
            "route_scale": float(_need(router, "scale", at + "router.")), "activation": "gelu",
            "names": {"router": "router", "up": "e{}.up", "down": "e{}.down"}})

    # ---------------------------------------------------------------- the model
    def to_spec(self) -> ModelSpec:
        raw = self.raw
        if raw.get("architecture") != "Vilodra":
            raise ConfigError(f"architecture {raw.get('architecture')!r} is not Vilodra")
        vocab, width = int(_need(raw, "vocab", "")), int(_need(raw, "width", ""))
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        mult = float(_need(raw, "residual_mult", ""))
        if vocab <= 0 or width <= 0 or not eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        layer_list = _need(raw, "layers", "")
        if not layer_list:
            raise ConfigError("a model needs at least one layer")
        norm = PartSpec("rms_norm_offset", {"size": width, "eps": eps, "weight_name": ""})
        branch = PartSpec("channel_scale", {"size": width, "value": mult})        # one constant for every channel: no tensor
        names = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2"}
        layers, run = [], []
        for i, layer in enumerate(layer_list):
            where = f"layers[{i}]."
            ffn = self._feed_forward(layer, where, width)
            extras = {"mixer_scale": branch} | ({"feed_forward_scale": branch} if ffn is not None else {})
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=self._mixer(layer_list, i, width, eps), mixer_norm=norm, feed_forward=ffn,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="pre_norm_scaled", names=names,
                                    extras=extras))
            source = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            run.append(RunEntry(layer=i, cache_of=None if source is None else int(source)))
        spec = ModelSpec(
            hidden_size=width, vocab_size=vocab, max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": width, "weight_name": ""}),
            embedding_prefix="embed", layers=tuple(layers), run=tuple(run),
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": width, "tied_to": "embed", "weight_name": ""}),
            head_prefix="head")
        spec.validate()
        return spec


register_architecture("Vilodra", VilodraConfig)
