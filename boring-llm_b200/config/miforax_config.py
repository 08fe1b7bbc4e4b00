"""Typed configuration of the Miforax decoder, read from its own config.json keys.

    {"architecture": "Miforax", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

    mixer:  {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "mask": {"size"}, "kv_from": j (optional),
             "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"} (optional)}}
    mlp:    {"kind": "dense", "ff"}
            {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"} (optional)}

Every size and every constant that can differ between models of the design is a field.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from .model_config import ConfigError, _get, _positive, architecture_name


@dataclass(frozen=True)
class YarnScaling:
    """Stretched rotation angles: pairs that make more than `fast` turns over `original` positions keep their angle,
    pairs that make fewer than `slow` turns have it divided by `factor`, a linear ramp over the pair index between."""
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention over a cached latent of `kv_rank` values and one rotated key part of `rot_dim` values per token. A head
    has `dim` unrotated and `rot_dim` rotated query/key values and `vdim` value channels; queries pass through a latent
    of `q_rank`. `window` 0 sees every earlier token. `kv_from` names the layer whose cached rows this one reads."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int
    rot_base: float
    rot_dims: int
    scaling: Optional[YarnScaling] = None
    kv_from: Optional[int] = None

    def to_dict(self):
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = self.scaling.to_dict()
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
             "kv_rank": self.kv_rank, "scale": self.scale, "rot": rot}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DenseFFConfig:
    """down(gelu_tanh(gate h) * (up h)) with hidden size `ff`."""
    ff: int

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class TableExpertsConfig:
    """`experts` clamped-GLU experts of hidden size `ff`, `top` a token, picked by a table over token ids, each with
    weight 1 / top; an optional expert of hidden size `shared_ff` that every token uses."""
    ff: int
    limit: float
    experts: int
    top: int
    shared_ff: int = 0
    shared_limit: float = 0.0

    def to_dict(self):
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class MiforaxLayerConfig:
    type: str
    mixer: LatentAttentionConfig
    mlp: Union[DenseFFConfig, TableExpertsConfig, None] = None

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None}


def _limit(m: dict, where: str) -> float:
    v = _get(m, "limit", float)
    if not v > 0:
        raise ConfigError(f"config.json: {where}.limit must be positive, got {v}")
    return float(v)


def _mixer(m: dict, where: str, index: int) -> LatentAttentionConfig:
    n = {k: _positive(f"{where}.{k}", _get(m, k, int)) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")}
    window = _get(m.get("mask") or {}, "size", int, 0)
    if window < 0:
        raise ConfigError(f"config.json: {where}.mask.size must not be negative, got {window}")
    rot = _get(m, "rot", dict)
    base = _get(rot, "base", float)
    if not base > 1:
        raise ConfigError(f"config.json: {where}.rot.base must be above 1, got {base}")
    dims = _get(rot, "dims", int, n["rot_dim"])
    if dims < 0 or dims % 2 != 0 or dims > n["rot_dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims ({dims}) must be even and at most rot_dim ({n['rot_dim']})")
    scaling = None
    if rot.get("scaling") is not None:
        s = _get(rot, "scaling", dict)
        scaling = YarnScaling(*(float(_get(s, k, float)) for k in ("factor", "original", "fast", "slow")))
        if not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0):
            raise ConfigError(f"config.json: {where}.rot.scaling: factor, original, fast and slow must be positive")
    src = m.get("kv_from")
    if src is not None:
        src = _get(m, "kv_from", int)
        if not 0 <= src < index:
            raise ConfigError(f"config.json: {where}.kv_from ({src}) must name an earlier layer")
    return LatentAttentionConfig(n["heads"], n["dim"], n["rot_dim"], n["vdim"], n["q_rank"], n["kv_rank"],
                                 float(_get(m, "scale", float)), window, float(base), dims, scaling, src)


def _mlp(mlp, where: str, vocab: int):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    kind = _get(mlp, "kind", str)
    if kind == "dense":
        return DenseFFConfig(_positive(f"{where}.ff", _get(mlp, "ff", int)))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense, moe)")
    expert = _get(mlp, "expert", dict)
    router = _get(mlp, "router", dict)
    experts = _positive(f"{where}.router.experts", _get(router, "experts", int))
    top = _positive(f"{where}.router.top", _get(router, "top", int))
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: {top} experts a token out of {experts}")
    shared_ff, shared_limit = 0, 0.0
    if mlp.get("shared") is not None:
        sh = _get(mlp, "shared", dict)
        shared_ff, shared_limit = _positive(f"{where}.shared.ff", _get(sh, "ff", int)), _limit(sh, where + ".shared")
    return TableExpertsConfig(_positive(f"{where}.expert.ff", _get(expert, "ff", int)), _limit(expert, where + ".expert"),
                              experts, top, shared_ff, shared_limit)


@dataclass(frozen=True)
class MiforaxConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[MiforaxLayerConfig, ...]
    max_position_embeddings: int = 1 << 20      # the design has no position limit of its own; engines clamp to their cache
    eos_token_ids: Tuple[int, ...] = ()
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURES = ("Miforax",)

    @classmethod
    def from_dict(cls, d: dict) -> "MiforaxConfig":
        arch = architecture_name(d)
        vocab = _positive("vocab", _get(d, "vocab", int))
        width = _positive("width", _get(d, "width", int))
        eps = _get(_get(d, "norm", dict), "eps", float)
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        scale = float(_get(d.get("embedding") or {}, "scale", float, 1.0))
        entries = _get(d, "layers", list)
        if not entries:
            raise ConfigError("config.json: 'layers' lists no layer")
        layers = []
        for i, e in enumerate(entries):
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = _get(e, "type", str)
            if kind != "latent_attention":
                raise ConfigError(f"config.json: layers[{i}]: unknown layer type {kind!r} (latent_attention)")
            mixer = _mixer(_get(e, "mixer", dict), f"layers[{i}].mixer", i)
            if mixer.kv_from is not None:
                owner = layers[mixer.kv_from].mixer
                if owner.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {mixer.kv_from}, which keeps no rows of its own")
                same = ("kv_rank", "rot_dim", "rot_base", "rot_dims", "scaling")
                if any(getattr(owner, k) != getattr(mixer, k) for k in same):
                    raise ConfigError(f"config.json: layers[{i}].mixer reads layer {mixer.kv_from}'s rows, but their kv_rank, rot_dim or rotation differ")
            layers.append(MiforaxLayerConfig(kind, mixer, _mlp(e.get("mlp"), f"layers[{i}].mlp", vocab)))
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "embedding", "layers",
                 "max_position_embeddings", "eos_token_id"}
        unknown = sorted(k for k in d if k not in known and not k.startswith("_"))
        if unknown:
            warnings.warn(f"config.json: keys not used by {arch}: {', '.join(unknown)}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(architecture=arch, vocab_size=vocab, width=width, norm_eps=float(eps), embedding_scale=scale,
                   layers=tuple(layers),
                   max_position_embeddings=_positive("max_position_embeddings", _get(d, "max_position_embeddings", int, 1 << 20)),
                   eos_token_ids=eos_ids, raw=dict(d))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "layers": [l.to_dict() for l in self.layers]}
        if self.max_position_embeddings != 1 << 20:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
