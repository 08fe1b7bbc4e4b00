"""Typed configuration of the Dapuzen decoder, read from its own config.json keys.

    {"architecture": "Dapuzen", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "attention" | "retention" | "parallel", "mixer": {...}, "mlp": {...} | null, "weights_of": j (optional)}, ...]}

    attention mixer:  {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"}}
    retention mixer:  {"heads", "dim", "vdim", "decay": [one per head], "rot": {"base", "dims"}}
    parallel mixer:   {"left":  {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size"}},
                       "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "left_scale", "right_scale"}
    mlp:              {"kind": "dense", "ff"}
                      {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity", "groups": {"count", "keep"}},
                       "shared": {"ff"} (optional)}

Every size and every constant that can differ between models of the design is a field. A layer with `weights_of: j` runs
with layer j's tensors and keeps a cache of its own; the rest of its entry equals layer j's.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from .model_config import ConfigError, _get, _positive, architecture_name


def _window(m: dict, where: str) -> int:
    w = _get(m.get("mask") or {}, "size", int, 0)
    if w < 0:
        raise ConfigError(f"config.json: {where}.mask.size must not be negative, got {w}")
    return w


def _rot(m: dict, where: str, dim: int):
    """(base, rotated values) of a mixer; without a 'rot' entry nothing is rotated."""
    if m.get("rot") is None:
        return 10000.0, 0
    rot = _get(m, "rot", dict)
    base = float(_get(rot, "base", float))
    dims = _get(rot, "dims", int, dim)
    if not base > 0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base}")
    if dims < 0 or dims % 2 != 0 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims ({dims}) must be even and at most dim ({dim})")
    return base, dims


def _heads(m: dict, where: str, keys) -> dict:
    return {k: _positive(f"{where}.{k}", _get(m, k, int)) for k in keys}


@dataclass(frozen=True)
class GatedAttentionConfig:
    """'attention': grouped queries, rotation of the first `rot_dims` values of a head in halves, a window (0: every earlier
    token), a sigmoid gate per head on the head's output, no biases."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_base: float
    rot_dims: int

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class RetentionConfig:
    """'retention': a matrix state per head with a fixed decay (`decay`, one per head), rotation on q and k."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float
    rot_dims: int

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class CappedAttentionConfig:
    """The left half of 'parallel': windowed attention with biases, no rotation, scores capped by `softcap` (0: no cap)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    softcap: float

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.softcap:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    """The right half of 'parallel': `heads` heads of `vdim` channels over a state of `state` values, B and C in `groups`
    groups, a causal convolution of `conv` taps, the output norm in `norm_groups` parts."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self):
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class ParallelPairConfig:
    """'parallel': left_scale * left + right_scale * right."""
    left: CappedAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class DenseFFConfig:
    """down(xIELU(up h)) with hidden size `ff`."""
    ff: int

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class ExpertsConfig:
    """`experts` SwiGLU experts of hidden size `ff` and `identity` identity experts behind one router with softmax scores;
    `top` a token out of the `keep` best of `groups` groups (a group's score: its largest choice score); an optional
    expert of hidden size `shared_ff` that every token uses, behind a sigmoid gate of one number per token."""
    ff: int
    experts: int
    top: int
    identity: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0

    def to_dict(self):
        d = {"kind": "moe", "expert": {"ff": self.ff},
             "router": {"experts": self.experts, "top": self.top, "identity": self.identity,
                        "groups": {"count": self.groups, "keep": self.keep}}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class DapuzenLayerConfig:
    type: str
    mixer: Union[GatedAttentionConfig, RetentionConfig, ParallelPairConfig]
    mlp: Union[DenseFFConfig, ExpertsConfig, None] = None
    weights_of: Optional[int] = None

    def to_dict(self):
        d = {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _mixer(kind: str, m: dict, where: str):
    if kind == "attention":
        n = _heads(m, where, ("heads", "kv_heads", "dim", "vdim"))
        if n["heads"] % n["kv_heads"] != 0:
            raise ConfigError(f"config.json: {where}: {n['heads']} heads cannot share {n['kv_heads']} key/value heads")
        base, dims = _rot(m, where, n["dim"])
        return GatedAttentionConfig(n["heads"], n["kv_heads"], n["dim"], n["vdim"], float(_get(m, "scale", float)),
                                    _window(m, where), base, dims)
    if kind == "retention":
        n = _heads(m, where, ("heads", "dim", "vdim"))
        decay = _get(m, "decay", list)
        if len(decay) != n["heads"] or any(isinstance(c, bool) or not isinstance(c, (int, float)) or not 0 <= c <= 1 for c in decay):
            raise ConfigError(f"config.json: {where}.decay must list one number in [0, 1] for each of the {n['heads']} heads")
        base, dims = _rot(m, where, n["dim"])
        return RetentionConfig(n["heads"], n["dim"], n["vdim"], tuple(float(c) for c in decay), base, dims)
    if kind == "parallel":
        l, r = _get(m, "left", dict), _get(m, "right", dict)
        ln = _heads(l, where + ".left", ("heads", "kv_heads", "dim", "vdim"))
        if ln["heads"] % ln["kv_heads"] != 0:
            raise ConfigError(f"config.json: {where}.left: {ln['heads']} heads cannot share {ln['kv_heads']} key/value heads")
        cap = float(_get(l, "softcap", float, 0.0))
        if cap < 0:
            raise ConfigError(f"config.json: {where}.left.softcap must not be negative, got {cap}")
        left = CappedAttentionConfig(ln["heads"], ln["kv_heads"], ln["dim"], ln["vdim"], float(_get(l, "scale", float)),
                                     _window(l, where + ".left"), cap)
        rn = _heads(r, where + ".right", ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
        if rn["heads"] % rn["groups"] != 0:
            raise ConfigError(f"config.json: {where}.right: {rn['heads']} heads cannot share {rn['groups']} groups")
        if (rn["heads"] * rn["vdim"]) % rn["norm_groups"] != 0:
            raise ConfigError(f"config.json: {where}.right: {rn['heads'] * rn['vdim']} channels do not split into {rn['norm_groups']} parts")
        right = StateSpaceConfig(rn["heads"], rn["vdim"], rn["state"], rn["groups"], rn["conv"], rn["norm_groups"])
        return ParallelPairConfig(left, right, float(_get(m, "left_scale", float, 1.0)), float(_get(m, "right_scale", float, 1.0)))
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (attention, retention, parallel)")


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where} must be an object or null")
    kind = _get(mlp, "kind", str)
    if kind == "dense":
        return DenseFFConfig(_positive(f"{where}.ff", _get(mlp, "ff", int)))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense, moe)")
    router = _get(mlp, "router", dict)
    experts = _positive(f"{where}.router.experts", _get(router, "experts", int))
    top = _positive(f"{where}.router.top", _get(router, "top", int))
    identity = _get(router, "identity", int, 0)
    if identity < 0:
        raise ConfigError(f"config.json: {where}.router.identity must not be negative, got {identity}")
    g = router.get("groups") or {}
    groups, keep = _positive(f"{where}.router.groups.count", _get(g, "count", int, 1)), _positive(f"{where}.router.groups.keep", _get(g, "keep", int, 1))
    total = experts + identity
    if total % groups != 0 or keep > groups:
        raise ConfigError(f"config.json: {where}.router: {total} router outputs in {groups} groups, {keep} kept")
    if top > keep * (total // groups):
        raise ConfigError(f"config.json: {where}.router: {top} experts a token out of {keep} groups of {total // groups}")
    shared = 0
    if mlp.get("shared") is not None:
        shared = _positive(f"{where}.shared.ff", _get(_get(mlp, "shared", dict), "ff", int))
    return ExpertsConfig(_positive(f"{where}.expert.ff", _get(_get(mlp, "expert", dict), "ff", int)), experts, top, identity,
                         groups, keep, shared)


@dataclass(frozen=True)
class DapuzenConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[DapuzenLayerConfig, ...]
    max_position_embeddings: int = 1 << 20      # the design has no position limit of its own; engines clamp to their cache
    eos_token_ids: Tuple[int, ...] = ()
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURES = ("Dapuzen",)

    @classmethod
    def from_dict(cls, d: dict) -> "DapuzenConfig":
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
            layer = DapuzenLayerConfig(kind, _mixer(kind, _get(e, "mixer", dict), f"layers[{i}].mixer"),
                                       _mlp(e.get("mlp"), f"layers[{i}].mlp"), None)
            src = e.get("weights_of")
            if src is not None:
                src = _get(e, "weights_of", int)
                if not 0 <= src < i:
                    raise ConfigError(f"config.json: layers[{i}].weights_of ({src}) must name an earlier layer")
                owner = layers[src]
                if owner.weights_of is not None:
                    raise ConfigError(f"config.json: layers[{i}].weights_of names layer {src}, which has no tensors of its own")
                if (owner.type, owner.mixer, owner.mlp) != (layer.type, layer.mixer, layer.mlp):
                    raise ConfigError(f"config.json: layers[{i}] runs with layer {src}'s tensors, but its entry differs from that layer's")
                layer = DapuzenLayerConfig(layer.type, layer.mixer, layer.mlp, src)
            layers.append(layer)
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
