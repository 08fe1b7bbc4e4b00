"""How a norm, a mixer and a feed-forward are arranged in one layer."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS
from .base import Part, takes_pending_norm, to_device_matrix, to_device_vector
from .linear import linear, EPI_BIAS, EPI_NONE
from .norm import LayerNorm


class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x)): sequential residuals around pre-norms, the
    arrangement of the reference's plain layer (src/model.br:1297-1358 with residual_type 0)."""

    def __init__(self, mixer_norm, mixer, ffn_norm=None, ffn=None):
        """A block without a feed-forward (`ffn` None) has only the first of the two."""
        super().__init__()
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("PreNormBlock: a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.mixer, "graph_safe", False) and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def forward(self, ctx, x, cache_layer: Optional[int], write_cache: bool = True) -> None:
        # a mixer or feed-forward may take the norm in front of it into its first kernel (steps with few rows)
        # (and the product that adds into the stream may begin the norm that reads it next: ctx.next_norm says which,
        # and a part that can finish such a norm says so with `takes_pending_norm`, or, by the step's number of rows,
        # with `takes_pending_norm_at`)
        if self.ffn is None:
            ctx.next_norm = ctx.norm_after_block
        else:
            ctx.next_norm = self.ffn_norm if takes_pending_norm(self.ffn, x.shape[0]) else None
        if not self.mixer.forward_fused_norm(ctx, x, self.mixer_norm, cache_layer, write_cache):
            h = self._normed(ctx, self.mixer_norm, x, self.mixer)
            self.mixer.forward(ctx, h, x, cache_layer, write_cache)
        if self.ffn is None:
            ctx.next_norm = None
            return
        ctx.next_norm = ctx.norm_after_block
        if not self.ffn.forward_fused_norm(ctx, x, self.ffn_norm):
            h = self._normed(ctx, self.ffn_norm, x, self.ffn)
            self.ffn.forward(ctx, h, x)
        ctx.next_norm = None

    @staticmethod
    def _normed(ctx, norm, x, reader):
        if takes_pending_norm(reader, x.shape[0]) and hasattr(norm, "dim"):
            try:
                return norm.forward(ctx, x, pending_ok=True)
            except TypeError:                    # a norm part without the option
                pass
        return norm.forward(ctx, x)


class ParallelBlock(Part):
    """ONE norm in front of both sublayers, which read the same rows and whose results join the stream together:

        h = norm(x);   x += mixer(h) + ffn(h)          (a block without a feed-forward has only the first)

    Both sublayers add into the 32-bit stream in place (the rows h were made before either wrote)."""

    def __init__(self, norm, mixer, ffn=None):
        super().__init__()
        self.mixer_norm, self.mixer, self.ffn = norm, mixer, ffn

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.mixer, "graph_safe", False) and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def forward(self, ctx, x, cache_layer, write_cache: bool = True) -> None:
        h = self.mixer_norm.forward(ctx, x)
        # only the sublayer that adds LAST leaves the finished row: it alone may begin the norm that reads the stream next
        ctx.next_norm = None if self.ffn is not None else ctx.norm_after_block
        self.mixer.forward(ctx, h, x, cache_layer, write_cache)
        if self.ffn is not None:
            ctx.next_norm = ctx.norm_after_block
            self.ffn.forward(ctx, h, x)
        ctx.next_norm = None


class ResidualGate(Part):
    """The logits of a gate on a sublayer's result: h . W^T (+ b), one per channel of the stream, 32-bit. The sigmoid and
    the product with the sublayer's result belong to the kernel that adds the result to the stream."""

    def __init__(self, dim: int, names, bias: bool = True):
        super().__init__(names)
        self.dim, self.has_bias = dim, bool(bias)
        self.weight = self.bias = None

    def local_specs(self):
        s = {"weight": TensorSpec((self.dim, self.dim), MATRIX)}
        if self.has_bias:
            s["bias"] = TensorSpec((self.dim,), BIAS)
        return s

    def logits(self, ctx, h):
        out = ctx.empty((h.shape[0], self.dim), torch.float32)
        linear(ctx, h, self.weight, out, self.bias, EPI_BIAS if self.has_bias else EPI_NONE)
        return out

    def join_into(self, part) -> bool:
        """Hands this gate's matrix to a sublayer whose first product reads the same rows (`part.join_rows`): the gate's
        logits then come out of that product as further columns (`part.joined_out`), and the bias is added by the kernel
        that applies the gate. True when the part took it."""
        if self.weight is None or not hasattr(part, "join_rows"):
            return False
        part.join_rows(self.weight)
        self.weight = None
        return True


class GatedSandwichBlock(Part):
    """Norms on both sides of each sublayer and a gate on its result:

        x += post1(mixer(h) * sigmoid(gate1(h))),  h = pre1(x)
        x += post2(ffn(h)   * sigmoid(gate2(h))),  h = pre2(x)      (a block without a feed-forward has only the first)

    The gates read what the sublayer reads and act before the norm behind it. `post*` are `LayerNorm` parts (the gate,
    that norm and the residual sum are one kernel); a gate may be None. The sublayers write their results instead of
    adding them (`Mixer.mix`, `FeedForward.apply`)."""

    def __init__(self, mixer_norm, mixer, mixer_post_norm, mixer_gate, ffn_norm=None, ffn=None, ffn_post_norm=None, ffn_gate=None):
        super().__init__()
        self.mixer_norm, self.mixer, self.mixer_post_norm, self.mixer_gate = mixer_norm, mixer, mixer_post_norm, mixer_gate
        self.ffn_norm, self.ffn, self.ffn_post_norm, self.ffn_gate = ffn_norm, ffn, ffn_post_norm, ffn_gate
        if ffn is not None and (ffn_norm is None or ffn_post_norm is None):
            raise ValueError("GatedSandwichBlock: a feed-forward needs the norms on both of its sides")
        self._joined = None                      # (mixer's gate joined, feed-forward's gate joined), once the weights are there

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.mixer_gate, self.ffn_norm, self.ffn,
                                 self.ffn_post_norm, self.ffn_gate) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.mixer, "graph_safe", False) and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    def forward(self, ctx, x, cache_layer: Optional[int], write_cache: bool = True) -> None:
        ctx.next_norm = None                     # no product of this block may begin a norm for its successor
        if self._joined is None:                 # the first step: a gate reads what its sublayer reads, so one product serves both
            self._joined = (self.mixer_gate is not None and self.mixer_gate.join_into(self.mixer),
                            self.ffn is not None and self.ffn_gate is not None and self.ffn_gate.join_into(self.ffn))
        # the rows this block's first norm would make may be there already: the kernel that ended the block before made them
        h = ctx.memo.pop(("normed rows", id(self.mixer_norm)), None)
        if h is None:
            h = self.mixer_norm.forward(ctx, x)
        after, ctx.after_block = ctx.after_block, None     # what the model wants done with the stream behind this block
        sub = ctx.empty(tuple(x.shape), torch.float32)
        self.mixer.mix(ctx, h, sub, cache_layer, write_cache)
        if self.ffn is None:
            self._add(ctx, x, sub, h, self.mixer_gate, self.mixer_post_norm, self.mixer if self._joined[0] else None, after=after)
            return
        h = self._add(ctx, x, sub, h, self.mixer_gate, self.mixer_post_norm, self.mixer if self._joined[0] else None,
                      then=self.ffn_norm)
        self.ffn.apply(ctx, h, sub)
        self._add(ctx, x, sub, h, self.ffn_gate, self.ffn_post_norm, self.ffn if self._joined[1] else None, after=after)

    @staticmethod
    def _add(ctx, x, sub, h, gate, post, joined_into, then=None, after=None):
        """x += post(sub * sigmoid(gate)), then what reads x next, in one launch where the rows allow it: `then` (a norm
        of this block; its rows are returned) or `after` (the model's: the average over the streams, and the next block's
        first norm, whose rows are left in the step's memo)."""
        if gate is None:
            g = gb = None
        elif joined_into is not None:
            g, gb = joined_into.joined_out, gate.bias
        else:
            g, gb = gate.logits(ctx, h), None
        chain = isinstance(post, LayerNorm) and ops.norm_chain_supported(x, g)
        if not chain:
            ops.gated_norm_residual(x, sub, g, post.weight, getattr(post, "bias", None), post.eps, gb)
            if after is not None:
                after.run_unfused(ctx)
            return then.forward(ctx, x) if then is not None else None
        pst = (post.weight, post.bias, post.eps)
        if then is not None:
            y = ctx.empty(tuple(x.shape))
            ops.norm_chain(x, sub, g, gb, pst, then=(then.weight, then.bias, then.eps), y=y)
            return y
        if after is None:
            ops.norm_chain(x, sub, g, gb, pst)
            return None
        if after.mix.n > ops.NORM_CHAIN_MAX_STREAMS:             # more layers than the fused average takes
            ops.norm_chain(x, sub, g, gb, pst)
            return None
        nxt = after.next_norm if isinstance(after.next_norm, LayerNorm) else None
        y = ctx.empty(tuple(x.shape)) if nxt is not None else None
        ops.norm_chain(x, sub, g, gb, pst, streams=after.streams, coeffs=after.mix.weight, n=after.mix.n, mix_out=after.out,
                       then=(nxt.weight, nxt.bias, nxt.eps) if nxt is not None else None, y=y)
        if nxt is not None:
            ctx.memo[("normed rows", id(nxt))] = y
        after.done = True
        return None


class PostNormBlock(Part):
    """The norm stands BEHIND each sublayer and the sublayers read the residual stream itself:

        x += norm1(mixer(x));   x += norm2(ffn(x))          (a block without a feed-forward has only the first)

    `mixer_post_norm` / `ffn_post_norm` are `LayerNorm` parts without bias. The stream is 32-bit; what the sublayers'
    products read are its rows in the activation dtype, which the kernel that adds to the stream also writes (one launch
    for norm, residual sum and hand-over), the stream itself in the 32-bit path. A mixer that works on the 32-bit rows
    (a token shift) finds them in the step's memo under ("rows32", id(h)). A mixer made of two (`ParallelMixers`) hands
    its two results to the same kernel, which norms each, takes their mean, norms again and adds."""

    def __init__(self, mixer, mixer_post_norm, ffn=None, ffn_post_norm=None):
        super().__init__()
        self.mixer, self.mixer_post_norm, self.ffn, self.ffn_post_norm = mixer, mixer_post_norm, ffn, ffn_post_norm
        if ffn is not None and ffn_post_norm is None:
            raise ValueError("PostNormBlock: a feed-forward needs the norm behind it")
        for n in (mixer_post_norm, ffn_post_norm):
            if n is not None and (not isinstance(n, LayerNorm) or n.has_bias):
                raise ValueError("PostNormBlock: the norms behind the sublayers are layer norms without bias")
        self.mixer_norm = None                   # nothing in front of the mixer: no product before this block may begin a norm for it

    def children(self):
        return tuple(p for p in (self.mixer, self.mixer_post_norm, self.ffn, self.ffn_post_norm) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.mixer, "graph_safe", False) and (self.ffn is None or getattr(self.ffn, "graph_safe", False)))

    @staticmethod
    def _rows(ctx, x):
        """The stream's rows as the products read them."""
        h = ctx.memo.pop(("stream rows", id(x)), None)
        if h is None:
            if ctx.dtype == torch.float32:
                h = x
            else:
                h = ctx.empty(tuple(x.shape))
                ops.cast_rows(x, h)
        ctx.memo[("rows32", id(h))] = x
        return h

    def _add(self, ctx, x, a, norm, b=None, pair=None):
        y = ctx.empty(tuple(x.shape)) if ctx.dtype != torch.float32 else None
        if b is None:
            ops.post_norm_residual(x, a, norm.weight, norm.eps, y)
        else:
            ops.post_norm_residual(x, a, norm.weight, norm.eps, y, b=b, wa=pair.left_out, wb=pair.right_out, rms_eps=pair.eps)
        if y is not None:
            ctx.memo[("stream rows", id(x))] = y

    def forward(self, ctx, x, cache_layer, write_cache: bool = True) -> None:
        ctx.next_norm = None
        h = self._rows(ctx, x)
        a = ctx.empty(tuple(x.shape), torch.float32)
        if hasattr(self.mixer, "mix_pair"):
            b = ctx.empty(tuple(x.shape), torch.float32)
            self.mixer.mix_pair(ctx, h, a, b, cache_layer, write_cache)
            self._add(ctx, x, a, self.mixer_post_norm, b, self.mixer)
        else:
            self.mixer.mix(ctx, h, a, cache_layer, write_cache)
            self._add(ctx, x, a, self.mixer_post_norm)
        ctx.memo.pop(("rows32", id(h)), None)
        if self.ffn is None:
            return
        h = self._rows(ctx, x)
        self.ffn.apply(ctx, h, a)
        ctx.memo.pop(("rows32", id(h)), None)
        self._add(ctx, x, a, self.ffn_post_norm)
