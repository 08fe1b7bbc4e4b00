"""The Dapuzen decoder as a list of parts, and its checkpoint tensor names.

A layer is a `ParallelBlock` (ONE RMS norm whose weight is a single number; the mixer and the feed-forward both read its
rows and both add into the stream) around one of three mixers, `GatedSinkAttention` with an output gate per head
('attention'), `Retention` ('retention'), or `ParallelMixers` of a `GatedSinkAttention` with biases and capped scores and a
`StateSpaceDuality` mixer, joined with two constants ('parallel'), and an optional feed-forward: `DenseMLP` with xIELU, or
`RoutedExperts` with softmax scores and identity experts plus a shared `GluMLP` behind a gate of one number per token.
A layer with `weights_of: j` is an entry of the run order that names layer j's block and a cache of its own. The embedding
rows are scaled; the same kind of norm and an untied head end the model. Layer i's tensors are `l<i>.*`: `norm1`,
`mix.{q, k, v, g, o}` (attention, retention), `mix.left.{q, k, v, o}` (+ `.b`), `mix.right.{in, conv, conv.b, dt_bias,
A_log, D, norm, o}`, `mlp.{up, down, act}` or `mlp.{router, correction, e<j>.gate / .up / .down, shared.gate / .up / .down / .sg}`.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.dapuzen_config import (DapuzenConfig, DenseFFConfig, ExpertsConfig, GatedAttentionConfig, ParallelPairConfig,
                                     RetentionConfig)
from ..parts import (DecoderModel, DenseMLP, Embedding, GatedSinkAttention, GluMLP, LayerCall, OutputHead, ParallelBlock,
                     ParallelMixers, Retention, RMSNorm, RotaryTable, RoutedExperts, RowGatedFeedForward, StateSpaceDuality,
                     SumFeedForward)


def _norm(cfg, name):
    return RMSNorm(cfg.width, cfg.norm_eps, {"weight": name}, scalar_weight=True)


def _rotary(m):
    return RotaryTable(m.dim, m.rot_base, n_rot=m.rot_dims, pairs="halves") if m.rot_dims else None


def _mixer(cfg: DapuzenConfig, m, p: str):
    d, eps = cfg.width, cfg.norm_eps
    if isinstance(m, GatedAttentionConfig):
        return GatedSinkAttention(d, m.heads, m.kv_heads, m.dim, m.vdim, _rotary(m),
                                  {"wq": p + "q", "wk": p + "k", "wv": p + "v", "wg": p + "g", "wo": p + "o"},
                                  window=m.window, scale=m.scale, out_gate=True)
    if isinstance(m, RetentionConfig):
        return Retention(d, m.heads, m.dim, m.vdim, m.decay, _rotary(m), eps,
                         {"wq": p + "q", "wk": p + "k", "wv": p + "v", "wg": p + "g", "wo": p + "o"})
    if isinstance(m, ParallelPairConfig):
        l, r = m.left, m.right
        lp, rp = p + "left.", p + "right."
        left = GatedSinkAttention(d, l.heads, l.kv_heads, l.dim, l.vdim, None,
                                  {"wq": lp + "q", "wk": lp + "k", "wv": lp + "v", "wo": lp + "o", "bq": lp + "q.b", "bk": lp + "k.b",
                                   "bv": lp + "v.b", "bo": lp + "o.b"},
                                  window=l.window, scale=l.scale, qkv_bias=True, out_bias=True, softcap=l.softcap)
        right = StateSpaceDuality(d, r.heads, r.vdim, r.state, r.groups, r.conv, r.norm_groups, eps,
                                  {"w_in": rp + "in", "conv": rp + "conv", "conv_bias": rp + "conv.b", "dt_bias": rp + "dt_bias",
                                   "a_log": rp + "A_log", "skip": rp + "D", "norm": rp + "norm", "wo": rp + "o"})
        return ParallelMixers(d, left, right, combine="weighted", scales=(m.left_scale, m.right_scale))
    raise TypeError(f"no mixer for {type(m).__name__}")


def _feed_forward(cfg: DapuzenConfig, f, p: str):
    d = cfg.width
    if f is None:
        return None
    if isinstance(f, DenseFFConfig):
        return DenseMLP(d, f.ff, {"w_up": p + "up", "w_down": p + "down", "act": p + "act"}, activation="xielu")
    if isinstance(f, ExpertsConfig):
        names = {"router": p + "router", "correction": p + "correction"}
        for j in range(f.experts):
            names.update({f"gate{j}": f"{p}e{j}.gate", f"up{j}": f"{p}e{j}.up", f"down{j}": f"{p}e{j}.down"})
        experts = RoutedExperts(d, f.ff, f.experts, f.top, names, n_groups=f.groups, keep_groups=f.keep, score="softmax",
                                group_score="max", n_identity=f.identity)
        if not f.shared_ff:
            return experts
        shared = GluMLP(d, f.shared_ff, {"w_gate": p + "shared.gate", "w_up": p + "shared.up", "w_down": p + "shared.down"})
        return SumFeedForward([experts, RowGatedFeedForward(d, shared, {"gate": p + "shared.sg"}, logit_from=experts)])
    raise TypeError(f"no feed-forward for {type(f).__name__}")


def build_dapuzen(cfg: DapuzenConfig) -> DecoderModel:
    d = cfg.width
    blocks, order, block_of, n_cache = [], [], {}, 0
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            p = f"l{i}."
            block_of[i] = len(blocks)
            blocks.append(ParallelBlock(_norm(cfg, p + "norm1"), _mixer(cfg, layer.mixer, p + "mix."),
                                        _feed_forward(cfg, layer.mlp, p + "mlp.")))
        b = block_of[i if layer.weights_of is None else layer.weights_of]
        spec = blocks[b].cache_spec()                  # every entry of the run order has cache layers of its own
        if isinstance(spec, tuple):
            order.append(LayerCall(b, tuple(range(n_cache, n_cache + len(spec)))))
            n_cache += len(spec)
        else:
            order.append(LayerCall(b, n_cache))
            n_cache += 1
    return DecoderModel(Embedding(cfg.vocab_size, d, {"table": "embed"}, scale=cfg.embedding_scale), blocks,
                        _norm(cfg, "final.norm"), OutputHead(cfg.vocab_size, d, {"weight": "head"}), schedule=order)


register_architecture(DapuzenConfig.ARCHITECTURES, DapuzenConfig, build_dapuzen)
