"""The Miforax decoder as a list of parts, and its checkpoint tensor names.

A layer is a `PreNormBlock` around a `LatentAttention` mixer (window, sink, output gate, stretched rotation) and an optional
feed-forward: `GluMLP` with the tanh form of GELU, or `TableExperts` (experts picked by a table over token ids) plus a
`GluMLP` that every token uses. A layer with `kv_from: j` has no down-projection to the key/value latent: its entry of the run
order reads the cache layer that layer j writes. The embedding rows are scaled; an RMS norm and an untied head end the model.
Layer i's tensors are `l<i>.*`: `norm1`, `norm2`, `mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, g, o}`,
`mlp.{gate, up, down}` or `mlp.{table, e<j>.gate / .up / .down, shared.gate / .up / .down}`.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.miforax_config import MiforaxConfig, DenseFFConfig, TableExpertsConfig
from ..parts import (DecoderModel, Embedding, GluMLP, LatentAttention, LayerCall, OutputHead, PreNormBlock, RMSNorm,
                     RotaryTable, SumFeedForward, TableExperts)


def _norm(cfg, name):
    return RMSNorm(cfg.width, cfg.norm_eps, {"weight": name})


def _rotary(m) -> RotaryTable:
    if m.scaling is None:
        return RotaryTable(m.rot_dim, m.rot_base, n_rot=m.rot_dims, pairs="halves")
    s = m.scaling
    return RotaryTable.yarn(m.rot_dim, m.rot_base, m.rot_dims, s.factor, s.original, s.fast, s.slow, pairs="halves")


def cache_windows(cfg: MiforaxConfig):
    """What the cache layer of every layer with rows of its own keeps: the widest window among the layer and the layers
    that read its rows, 0 (everything) if one of them sees every earlier token."""
    windows = {}
    for i, layer in enumerate(cfg.layers):
        owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
        windows.setdefault(owner, []).append(layer.mixer.window)
    return {owner: (0 if min(w) == 0 else max(w)) for owner, w in windows.items()}


def _mixer(cfg: MiforaxConfig, m, p: str, cache_window: int) -> LatentAttention:
    names = {"wdq": p + "dq", "dq_norm": p + "dq.norm", "wuq": p + "uq", "wdkv": p + "dkv", "dkv_norm": p + "dkv.norm",
             "wuk": p + "uk", "wuv": p + "uv", "sink": p + "sink", "wg": p + "g", "wo": p + "o"}
    return LatentAttention(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, _rotary(m), names,
                           window=m.window, scale=m.scale, norm_eps=cfg.norm_eps, sink=True, out_gate=True,
                           own_kv=m.kv_from is None, cache_window=cache_window)


def _feed_forward(cfg: MiforaxConfig, f, p: str):
    d = cfg.width
    if isinstance(f, DenseFFConfig):
        return GluMLP(d, f.ff, {"w_gate": p + "gate", "w_up": p + "up", "w_down": p + "down"}, activation="gelu_tanh")
    if isinstance(f, TableExpertsConfig):
        names = {"table": p + "table"}
        for j in range(f.experts):
            names.update({f"gate{j}": f"{p}e{j}.gate", f"up{j}": f"{p}e{j}.up", f"down{j}": f"{p}e{j}.down"})
        experts = TableExperts(d, f.ff, f.experts, f.top, cfg.vocab_size, names, activation="clamped", limit=f.limit)
        if not f.shared_ff:
            return experts
        shared = GluMLP(d, f.shared_ff, {"w_gate": p + "shared.gate", "w_up": p + "shared.up", "w_down": p + "shared.down"},
                        activation="clamped", limit=f.shared_limit)
        return SumFeedForward([experts, shared])
    raise TypeError(f"no feed-forward for {type(f).__name__}")


def build_miforax(cfg: MiforaxConfig) -> DecoderModel:
    d = cfg.width
    keeps = cache_windows(cfg)
    blocks, order, cache_of, spare = [], [], {}, []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        owner = i if m.kv_from is None else m.kv_from
        if m.kv_from is None:
            cache_of[i] = len(cache_of)
        ff = {}
        if layer.mlp is None:
            spare.append(p + "norm2")         # a file may keep the norm of a feed-forward that the layer does not have
        else:
            ff = dict(ffn_norm=_norm(cfg, p + "norm2"), ffn=_feed_forward(cfg, layer.mlp, p + "mlp."))
        blocks.append(PreNormBlock(_norm(cfg, p + "norm1"), _mixer(cfg, m, p + "mix.", keeps[owner]), **ff))
        order.append(LayerCall(i, cache_of[owner], write_cache=m.kv_from is None))
    return DecoderModel(Embedding(cfg.vocab_size, d, {"table": "embed"}, scale=cfg.embedding_scale), blocks,
                        _norm(cfg, "final.norm"), OutputHead(cfg.vocab_size, d, {"weight": "head"}), schedule=order,
                        ignorable_tensors=spare)


register_architecture(MiforaxConfig.ARCHITECTURES, MiforaxConfig, build_miforax)
