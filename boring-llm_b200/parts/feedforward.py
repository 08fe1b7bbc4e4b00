"""Feed-forward parts: rows in, rows out, no cache."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS, INT_TABLE
from .base import Part, to_device_matrix
from .linear import linear, EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU


FF_FUSED_MAX_ROWS = 16    # more rows: a separate norm and the tcgen05 product are faster (measured: 6% of a step at 24 and 32 rows)


class FeedForward(Part):
    """Interface: `forward(ctx, h, residual)` reads the normed rows `h` [T, dim] and adds its
    result into the 32-bit `residual` [T, dim] in place. `graph_safe` as for mixers."""
    graph_safe = False

    def forward(self, ctx, h, residual) -> None:
        raise NotImplementedError

    def forward_fused_norm(self, ctx, x, norm) -> bool:
        """Optional: run `norm` and this feed-forward on the residual stream `x` in fused kernels and return
        True, or return False to be called with the normed rows as usual."""
        return False

    def apply(self, ctx, h, out) -> None:
        """Writes the result into the 32-bit `out` [T, dim] instead of adding it to a stream (for arrangements
        that treat a sublayer's result before the residual sum: gates, norms behind the sublayer)."""
        out.zero_()
        self.forward(ctx, h, out)


class DenseMLP(FeedForward):
    """down(act(up(h))), no biases, no gate branch; `activation`: "gelu" (exact, erf), "gelu_tanh", "silu" or "xielu",
    evaluated in 32-bit on the up product's 32-bit sums. xIELU has two learned numbers p, q (a tensor `act` [2]):
    z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    graph_safe = True
    ACTIVATIONS = {"silu": ops.ACT_SILU, "gelu": ops.ACT_GELU_ERF, "gelu_tanh": ops.ACT_GELU_TANH, "xielu": None}

    def __init__(self, dim: int, hidden: int, names: Dict[str, str], activation: str = "gelu"):
        super().__init__(names)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"DenseMLP: activation must be one of {sorted(self.ACTIVATIONS)}, got {activation!r}")
        self.dim, self.hidden, self.activation = dim, hidden, activation
        self.w_up = self.w_down = self.act_args = None

    def local_specs(self):
        s = {"w_up": TensorSpec((self.hidden, self.dim), MATRIX), "w_down": TensorSpec((self.dim, self.hidden), MATRIX)}
        if self.activation == "xielu":
            s["act"] = TensorSpec((2,), BIAS)
        return s

    def place(self, local, dtype, device):
        self.w_up = to_device_matrix(local["w_up"], dtype, device)
        self.w_down = to_device_matrix(local["w_down"], dtype, device)
        if self.activation == "xielu":
            p, q = (float(v) for v in local["act"].to(torch.float32))
            self.act_args = ops.xielu_args(p, q, device)

    def join_rows(self, weight) -> None:
        """Further rows for the up product's matrix, from a part that reads the same rows (a gate on this feed-forward's
        result); after each run their 32-bit sums are `self.joined_out` [T, rows]."""
        pad = -self.w_up.shape[0] % 8            # the further columns start on a 16-byte boundary of the 32-bit sums
        self.n_own = self.w_up.shape[0] + pad
        self.w_up = torch.cat([self.w_up, self.w_up.new_zeros((pad, self.w_up.shape[1])),
                               weight.to(device=self.w_up.device, dtype=self.w_up.dtype)], dim=0).contiguous()

    def _run(self, ctx, h, out, epilogue):
        act = ctx.empty((h.shape[0], self.hidden))
        if self.activation == "xielu":
            sums = ctx.empty((h.shape[0], self.w_up.shape[0]), torch.float32)
            linear(ctx, h, self.w_up, sums, None, EPI_NONE)
            ops.xielu(sums, act, self.act_args)
            rest = sums[:, self.hidden:] if self.w_up.shape[0] > self.hidden else None
        else:
            rest = ops.linear_act(h, self.w_up, act, self.ACTIVATIONS[self.activation], fast=ctx.fast)
        self.joined_out = rest[:, self.n_own - self.hidden:] if rest is not None else None
        linear(ctx, act, self.w_down, out, None, epilogue)

    def forward(self, ctx, h, residual):
        self._run(ctx, h, residual, EPI_RESIDUAL)

    def apply(self, ctx, h, out):
        self._run(ctx, h, out, EPI_NONE)


class SwiGLU(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases (src/math.br:232-233, 246-261). Gate and up run as
    one joined product over [Wg; Wu] (src/model.br:788-792) whose epilogue combines them
    (src/math_gpu.br:2673-2692); the down product adds into the residual stream."""
    graph_safe = True
    takes_pending_norm = True            # its first product can finish an RMS norm that the product before has begun

    def __init__(self, dim: int, hidden: int, names: Dict[str, str]):
        super().__init__(names)
        self.dim, self.hidden = dim, hidden
        self.w_gate_up = self.w_down = None

    def local_specs(self):
        return {"w_gate": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_up": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_down": TensorSpec((self.dim, self.hidden), MATRIX)}

    def place(self, local, dtype, device):
        self.w_gate_up = to_device_matrix(torch.cat([local["w_gate"], local["w_up"]], dim=0), dtype, device)
        self.w_down = to_device_matrix(local["w_down"], dtype, device)

    def takes_pending_norm_at(self, rows: int) -> bool:
        """gate/up finishes a norm that the product before has begun where it runs on pairs of SMs (many rows) or on the
        register-streaming kernel (a decode step's 2 to 16 rows, a matrix of up to 592 blocks of 16 columns that does
        not stream better through TMA); elsewhere the product before need not begin one."""
        if rows >= ops.PAIR_MIN_ROWS:
            return True
        return (ops.SKINNY_LINK_MIN_ROWS <= rows <= ops.SKINNY_LINK_MAX_ROWS and self.w_gate_up is not None
                and -(-self.hidden // 16) <= ops.SKINNY_LINK_MAX_BLOCKS and not ops.gemm_streams_better(self.w_gate_up))

    def forward_fused_norm(self, ctx, x, norm) -> bool:
        from .norm import RMSNorm
        if not (ctx.fast and ctx.dtype == torch.bfloat16 and x.shape[0] <= FF_FUSED_MAX_ROWS and isinstance(norm, RMSNorm)
                and ops.norm_gemm_supported(x, self.w_gate_up) and not ops.gemm_streams_better(self.w_gate_up)):
            return False
        held = ctx.memo.get(("pending norm", id(x)))
        if held is not None and held.norm is norm:
            return False                # the product before has begun this norm: `forward` finishes it in gate/up's epilogue
        act = ctx.empty((x.shape[0], self.hidden))
        ops.norm_gemm(x, norm.weight, norm.eps, self.w_gate_up, act, None, EPI_SWIGLU)
        linear(ctx, act, self.w_down, x, None, EPI_RESIDUAL)
        return True

    def forward(self, ctx, h, residual):
        act = ctx.empty((h.shape[0], self.hidden))
        linear(ctx, h, self.w_gate_up, act, None, EPI_SWIGLU)
        linear(ctx, act, self.w_down, residual, None, EPI_RESIDUAL)


class GluMLP(FeedForward):
    """down(glu(gate(h), up(h))), no biases, with the gated activation as an argument:

    * "silu":       silu(g) * u (what `SwiGLU` computes with fused epilogues);
    * "gelu_tanh":  0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u;
    * "clamped":    g' = min(g, limit), u' = clamp(u, -limit, limit); g' sigmoid(1.702 g') (u' + 1).

    Gate and up are one joined product over [Wg; Wu] whose epilogue evaluates the activation on the 32-bit sums (the
    epilogue of `SwiGLU`, told which activation by two numbers on the device); the down product adds into the residual
    stream."""
    graph_safe = True
    KINDS = {"silu": ops.GLU_SILU, "gelu_tanh": ops.GLU_GELU_TANH, "clamped": ops.GLU_CLAMPED}

    def __init__(self, dim: int, hidden: int, names: Dict[str, str], activation: str = "silu", limit: float = 0.0):
        super().__init__(names)
        if activation not in self.KINDS:
            raise ValueError(f"GluMLP: activation must be one of {sorted(self.KINDS)}, got {activation!r}")
        if activation == "clamped" and not limit > 0:
            raise ValueError(f"GluMLP: the clamped activation needs a positive limit, got {limit}")
        self.dim, self.hidden, self.activation, self.limit = dim, hidden, activation, float(limit)
        self.w_gate_up = self.w_down = self.act_args = None

    def local_specs(self):
        return {"w_gate": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_up": TensorSpec((self.hidden, self.dim), MATRIX),
                "w_down": TensorSpec((self.dim, self.hidden), MATRIX)}

    def place(self, local, dtype, device):
        self.w_gate_up = to_device_matrix(torch.cat([local["w_gate"], local["w_up"]], dim=0), dtype, device)
        self.w_down = to_device_matrix(local["w_down"], dtype, device)
        self.act_args = ops.glu_args(self.KINDS[self.activation], self.limit, device)

    def takes_pending_norm_at(self, rows: int) -> bool:
        """gate/up finishes a norm that the product before has begun on the register-streaming kernel (a decode step's 2
        to 16 rows), and, with SiLU, on pairs of SMs (many rows), as `SwiGLU` does."""
        if rows >= ops.PAIR_MIN_ROWS:
            return self.act_args is None and self.w_gate_up is not None and self.w_gate_up.dtype == torch.bfloat16
        return (ops.SKINNY_LINK_MIN_ROWS <= rows <= ops.SKINNY_LINK_MAX_ROWS and self.w_gate_up is not None
                and self.w_gate_up.dtype == torch.bfloat16 and -(-self.hidden // 16) <= ops.SKINNY_LINK_MAX_BLOCKS
                and not ops.gemm_streams_better(self.w_gate_up))

    def _run(self, ctx, h, out, epilogue):
        act = ctx.empty((h.shape[0], self.hidden))
        linear(ctx, h, self.w_gate_up, act, self.act_args, EPI_SWIGLU)
        linear(ctx, act, self.w_down, out, None, epilogue)

    def forward(self, ctx, h, residual):
        self._run(ctx, h, residual, EPI_RESIDUAL)

    def apply(self, ctx, h, out):
        self._run(ctx, h, out, EPI_NONE)


class SumFeedForward(FeedForward):
    """Several feed-forwards that read the same rows; their results are added (routed experts and an expert that every
    token uses)."""

    def __init__(self, parts):
        super().__init__()
        self.parts = list(parts)

    def children(self):
        return tuple(self.parts)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts)

    def forward(self, ctx, h, residual):
        # only the LAST part's addition may begin the norm that reads the stream next: the others' sums are not the row yet
        after = ctx.next_norm
        for i, p in enumerate(self.parts):
            ctx.next_norm = after if i == len(self.parts) - 1 else None
            p.forward(ctx, h, residual)
        ctx.next_norm = after

    def apply(self, ctx, h, out):
        self.parts[0].apply(ctx, h, out)
        for p in self.parts[1:]:
            p.forward(ctx, h, out)


class RowGatedFeedForward(FeedForward):
    """A feed-forward whose result is multiplied by sigmoid(w . h), ONE number per token (`gate` [1, dim]), before it joins
    the stream: x += sigmoid(h gate^T) * inner(h). The gate's logit is 32-bit. `logit_from`: a part that runs BEFORE this one
    on the same rows and begins with a product of them (`join_rows`, `joined_out`: routed experts' router): the gate's row
    becomes one more row of that product's matrix, and the logit costs no launch of its own."""

    def __init__(self, dim: int, inner: FeedForward, names: Dict[str, str], logit_from=None):
        super().__init__(names)
        self.dim, self.inner, self.logit_from = dim, inner, logit_from
        self.gate = None
        self._joined = False

    def children(self):
        return (self.inner,)

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.inner, "graph_safe", False))

    def local_specs(self):
        return {"gate": TensorSpec((1, self.dim), MATRIX)}

    def place(self, local, dtype, device):
        self.gate = to_device_matrix(local["gate"], dtype, device)
        src = self.logit_from
        if src is not None and getattr(src, "router", None) is not None and hasattr(src, "join_rows"):
            src.join_rows(self.gate)                     # (the other part's tensors are placed already: it comes first)
            self._joined = True

    def forward(self, ctx, h, residual):
        after, ctx.next_norm = ctx.next_norm, None       # the inner result is not the stream: its product begins no norm
        y = ctx.empty(tuple(residual.shape), torch.float32)
        self.inner.apply(ctx, h, y)
        ctx.next_norm = after
        logit = self.logit_from.joined_out if self._joined else None
        if logit is None or logit.shape[0] != h.shape[0]:
            logit = ctx.empty((h.shape[0], 1), torch.float32)
            linear(ctx, h, self.gate, logit, None, EPI_NONE)
        ops.add_row_gated(residual, y, logit)


class RoutedExperts(FeedForward):
    """A mixture of experts: `n_experts` small SwiGLU feed-forwards without biases, of which each token uses `top`.

    Router logits z = h Wr^T in 32-bit, scores s = sigmoid(z). The CHOICE runs on s + correction (a learned vector), the
    weights are the chosen experts' s as they are (not renormalised). The experts form `n_groups` equal runs of
    neighbours; a group's score is the sum of its two largest choice scores, and only experts of the `keep_groups` best
    groups can be chosen. The result is the weighted sum of the chosen experts' outputs, added in the order of the choice.
    The experts' matrices are stacked ([E, 2 * hidden, dim] gate rows then up rows, [E, dim, hidden]); every (token,
    chosen expert) pair is a row of two products whose rows each use the matrix of their own expert. `activation` /
    `limit`: the experts' gated activation, as in `GluMLP`, evaluated in the first product's epilogue.

    Further choices: `score` "sigmoid" or "softmax" (the softmax of z over ALL router outputs); `group_score` "top2" (the sum
    of a group's two largest choice scores) or "max" (its largest); `n_identity`: the router has `n_experts + n_identity`
    outputs, and the last `n_identity` are identity experts without tensors whose output is the input row h itself (times
    the weight); groups are formed over experts and identity experts together."""
    graph_safe = True
    SCORES = {"sigmoid": ops.SCORE_SIGMOID, "softmax": ops.SCORE_SOFTMAX}

    def __init__(self, dim: int, hidden: int, n_experts: int, top: int, names: Dict[str, str], n_groups: int = 1,
                 keep_groups: int = 1, correction: bool = True, activation: str = "silu", limit: float = 0.0,
                 score: str = "sigmoid", group_score: str = "top2", n_identity: int = 0):
        super().__init__(names)
        if score not in self.SCORES or group_score not in ("top2", "max") or n_identity < 0:
            raise ValueError(f"RoutedExperts: score {score!r}, group_score {group_score!r}, {n_identity} identity experts")
        self.score, self.group_top, self.n_identity = self.SCORES[score], 2 if group_score == "top2" else 1, int(n_identity)
        self.n_out = n_experts + self.n_identity          # the router's outputs
        if activation not in GluMLP.KINDS:
            raise ValueError(f"experts: activation must be one of {sorted(GluMLP.KINDS)}, got {activation!r}")
        if activation == "clamped" and not limit > 0:
            raise ValueError(f"experts: the clamped activation needs a positive limit, got {limit}")
        self.activation, self.limit = activation, float(limit)
        if self.n_out % n_groups != 0 or not 1 <= keep_groups <= n_groups:
            raise ValueError(f"RoutedExperts: {self.n_out} experts in {n_groups} groups, {keep_groups} kept")
        if not 1 <= top <= keep_groups * (self.n_out // n_groups):
            raise ValueError(f"RoutedExperts: {top} experts a token out of {keep_groups} groups of {self.n_out // n_groups}")
        self.dim, self.hidden, self.E, self.top = dim, hidden, n_experts, top
        self.n_groups, self.keep_groups, self.has_correction = n_groups, keep_groups, bool(correction)
        self.router = self.correction = self.w_gate_up = self.w_down = self.act_args = self.joined_out = None
        self.record = None               # a list: every step appends a copy of the experts it chose [T, top] (tests; kernels launched singly)

    def choice_specs(self):
        """The tensors that choose a token's experts."""
        s = {"router": TensorSpec((self.n_out, self.dim), MATRIX)}
        if self.has_correction:
            s["correction"] = TensorSpec((self.n_out,), BIAS)
        return s

    def local_specs(self):
        s = self.choice_specs()
        for e in range(self.E):
            s[f"gate{e}"] = TensorSpec((self.hidden, self.dim), MATRIX)
            s[f"up{e}"] = TensorSpec((self.hidden, self.dim), MATRIX)
            s[f"down{e}"] = TensorSpec((self.dim, self.hidden), MATRIX)
        return s

    def place_choice(self, local, dtype, device):
        self.router = to_device_matrix(local["router"], dtype, device)
        if self.has_correction:
            self.correction = local["correction"].to(device=device, dtype=torch.float32).contiguous()

    def place(self, local, dtype, device):
        self.place_choice(local, dtype, device)
        self.w_gate_up = to_device_matrix(torch.stack([torch.cat([local[f"gate{e}"], local[f"up{e}"]], dim=0) for e in range(self.E)]),
                                          dtype, device)
        self.w_down = to_device_matrix(torch.stack([local[f"down{e}"] for e in range(self.E)]), dtype, device)
        self.act_args = ops.glu_args(GluMLP.KINDS[self.activation], self.limit, device)

    def join_rows(self, weight) -> None:
        """Further rows for the router's matrix, from a part that reads the same rows (a gate of one number per token on
        another feed-forward); after each run their 32-bit sums are `self.joined_out` [T, rows]."""
        pad = -self.router.shape[0] % 8          # the further columns start on a 32-byte boundary of the 32-bit sums
        self.n_own = self.router.shape[0] + pad
        self.router = torch.cat([self.router, self.router.new_zeros((pad, self.router.shape[1])),
                                 weight.to(device=self.router.device, dtype=self.router.dtype)], dim=0).contiguous()

    def route(self, ctx, h):
        """(experts [T, top] int32, weights [T, top] 32-bit) of the rows h."""
        T = h.shape[0]
        z = ctx.empty((T, self.router.shape[0]), torch.float32)
        linear(ctx, h, self.router, z, None, EPI_NONE)            # 32-bit sums of exact products (the rows may be bfloat16 roundings)
        n_own = getattr(self, "n_own", None)
        self.joined_out = z[:, n_own:] if n_own is not None else None
        if n_own is not None:
            z = z[:, :self.n_out]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=ctx.device)
        wts = ctx.empty((T, self.top), torch.float32)
        ops.moe_route(z, self.correction, self.top, self.n_groups, self.keep_groups, ids, wts, self.score, self.group_top)
        if self.record is not None:
            self.record.append(ids.clone())
        return ids, wts

    def _run(self, ctx, h, out, add):
        T = h.shape[0]
        ids, wts = self.route(ctx, h)
        if ctx.fast and ops.grouped_gemm_supported(h, self.w_gate_up) and self.hidden % 8 == 0:
            # tensor cores: the pairs lie expert by expert in tiles of 128 rows, each tile multiplied by its expert's matrices
            pos, row_src, tile_expert = ops.moe_plan(ids, self.E)
            rows = ctx.empty((row_src.numel(), self.dim))
            ops.gather_rows(h, row_src, self.top, rows)
            act = ctx.empty((row_src.numel(), self.hidden))
            ops.gemm_grouped(rows, self.w_gate_up, tile_expert, act, EPI_SWIGLU, self.act_args)
            y = ctx.empty((row_src.numel(), self.dim), torch.float32)
            ops.gemm_grouped(act, self.w_down, tile_expert, y, EPI_NONE)
            ops.moe_combine_rows(y, pos, wts, out, add=add, x=h if self.n_identity else None)
            return
        act = ctx.empty((T * self.top, self.hidden))
        ops.expert_gemm_plain(h, self.top, self.w_gate_up, ids, act, EPI_SWIGLU, self.act_args)
        y = ctx.empty((T * self.top, self.dim), torch.float32)
        ops.expert_gemm_plain(act, 1, self.w_down, ids, y, EPI_NONE)
        if self.n_identity:
            ops.moe_combine(y, wts, out, add=add, ids=ids, n_real=self.E, x=h)
        else:
            ops.moe_combine(y, wts, out, add=add)

    def forward(self, ctx, h, residual):
        self._run(ctx, h, residual, True)

    def apply(self, ctx, h, out):
        self._run(ctx, h, out, False)


class TableExperts(RoutedExperts):
    """Experts without a router: a table [vocabulary, top] of expert numbers gives every TOKEN ID its experts (the numbers
    of a row differ), each with weight 1 / top. Everything behind the choice is `RoutedExperts`."""

    def __init__(self, dim: int, hidden: int, n_experts: int, top: int, vocab: int, names: Dict[str, str],
                 activation: str = "silu", limit: float = 0.0):
        if not 1 <= top <= n_experts:
            raise ValueError(f"TableExperts: {top} experts a token out of {n_experts}")
        super().__init__(dim, hidden, n_experts, top, names, correction=False, activation=activation, limit=limit)
        self.vocab = vocab
        self.table = None

    def choice_specs(self):
        return {"table": TensorSpec((self.vocab, self.top), INT_TABLE, high=self.E)}

    def place_choice(self, local, dtype, device):
        t = local["table"].to(torch.int64)
        if int(t.min()) < 0 or int(t.max()) >= self.E:
            raise ValueError(f"TableExperts: the table names experts outside 0..{self.E - 1}")
        if self.top > 1:
            srt = torch.sort(t, dim=1).values
            if bool((srt[:, 1:] == srt[:, :-1]).any()):
                raise ValueError("TableExperts: a row of the table names an expert twice")
        self.table = t.to(device=device, dtype=torch.int32).contiguous()

    def route(self, ctx, h):
        T = h.shape[0]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=ctx.device)
        wts = ctx.empty((T, self.top), torch.float32)
        ops.table_route(self.table, ctx.token_ids, ids, wts)
        if self.record is not None:
            self.record.append(ids.clone())
        return ids, wts
