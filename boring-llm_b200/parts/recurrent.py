"""Mixers that carry a matrix state per head from token to token instead of caching keys and values.

Each request owns a state slot (`cache.StateSpec`); a step's kernels walk the tokens of every request in order from
the state the step before left, prompts' portions and single decoded tokens alike, and are pure device work (the
batch's structure comes from `ctx.cu_q` and `ctx.slots`), so steps with these mixers can be captured and replayed.
State, decays, gates and every sum of the recurrences are 32-bit in both engine dtypes.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import StateSpec
from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS, NORM
from .attention import Mixer
from .base import StepPlan, to_device_matrix, to_device_vector
from .linear import linear, EPI_BIAS, EPI_NONE, EPI_RESIDUAL


def _rank(t_a: torch.Tensor, t_b: torch.Tensor, what: str) -> int:
    """The inner size of a product in two factors, read from the tensors: t_a [r, dim], t_b [out, r]."""
    if t_a.shape[0] != t_b.shape[1]:
        raise ValueError(f"{what}: the first factor has {t_a.shape[0]} rows, the second {t_b.shape[1]} columns")
    return int(t_a.shape[0])


class _StateMixer(Mixer):
    graph_safe = True

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        self._run(ctx, h, residual, cache_layer, write_cache, EPI_RESIDUAL)

    def mix(self, ctx, h, out, cache_layer, write_cache=True):
        self._run(ctx, h, out, cache_layer, write_cache, EPI_NONE)

    RULE = None                      # ops.RULE_GLA or ops.RULE_DELTA

    def _parts(self, q_lens) -> int:
        n_long = sum(1 for n in q_lens if n >= ops.SCAN_PART_MIN_TOKENS)
        return ops.recurrent_scan_parts(self.RULE, self.H, self.dk, self.dv, n_long) if n_long else 1

    def plan_step(self, q_lens, ctx_lens, filler=None):
        """Into how many parts this step's long portions are cut (they run side by side): a launch shape, so part of what
        names a captured step."""
        parts = self._parts(q_lens)
        return self._plan_key(), StepPlan(host={"parts": parts}, shape=(parts,))

    def _plan_key(self) -> str:
        return f"recurrence parts {self.RULE} {self.H}x{self.dk}x{self.dv}"       # layers of equal sizes share the plan

    def _step_parts(self, ctx) -> int:
        if not ctx.fast:
            return 1
        plan = ctx.plans.get(self._plan_key())
        if plan is not None:
            return plan.host["parts"]
        return self._parts(ctx.q_lens) if ctx.q_lens else 1       # a step put together without asking the parts

    @staticmethod
    def _check(write_cache):
        if not write_cache:
            raise ValueError("a mixer with recurrent state cannot read the state another entry of the run order wrote")


class GatedLinearAttention(_StateMixer):
    """Per head, with a decay per key channel:

        S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t)^(1 / tau),
        z = (h A1^T) A2^T + b,   q = (h Wq^T) / sqrt(key_dim)

    then each head's o is RMS-normed over its value channels (one plain weight shared by the heads), the heads are
    joined, multiplied by silu(h Wg^T) and projected by Wo. `decay_rank` is the inner size of the decay's two factors
    (None: taken from the tensors when they are loaded)."""
    RULE = ops.RULE_GLA

    def __init__(self, dim: int, n_heads: int, key_dim: int, value_dim: int, tau: float, norm_eps: float,
                 names: Dict[str, str], decay_rank: Optional[int] = None):
        super().__init__(names)
        self.dim, self.H, self.dk, self.dv = dim, n_heads, key_dim, value_dim
        self.tau, self.eps, self.rank = float(tau), float(norm_eps), decay_rank
        self.off_k = self.H * self.dk
        self.off_v = 2 * self.H * self.dk
        self.off_g = self.off_v + self.H * self.dv
        self.off_a = self.off_g + self.H * self.dv
        self.w_in = self.wo = self.a2 = self.a2_bias = self.norm = self.coef = None

    def local_specs(self):
        r = -1 if self.rank is None else self.rank
        return {"wq": TensorSpec((self.H * self.dk, self.dim), MATRIX), "wk": TensorSpec((self.H * self.dk, self.dim), MATRIX),
                "wv": TensorSpec((self.H * self.dv, self.dim), MATRIX), "wg": TensorSpec((self.H * self.dv, self.dim), MATRIX),
                "wo": TensorSpec((self.dim, self.H * self.dv), MATRIX), "norm": TensorSpec((self.dv,), NORM),
                "a1": TensorSpec((r, self.dim), MATRIX), "a2": TensorSpec((self.H * self.dk, r), MATRIX),
                "a2_bias": TensorSpec((self.H * self.dk,), BIAS)}

    def place(self, local, dtype, device):
        self.rank = _rank(local["a1"], local["a2"], "the decay's factors")
        self.w_in = to_device_matrix(torch.cat([local[n] for n in ("wq", "wk", "wv", "wg", "a1")], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        self.a2 = to_device_matrix(local["a2"], dtype, device)
        self.a2_bias = to_device_vector(local["a2_bias"], dtype, device)
        self.norm = to_device_vector(local["norm"], dtype, device)
        self.coef = torch.full((self.H,), 1.0 / self.tau, dtype=torch.float32, device=device)

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv,), "float32")

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        T, H, dk, dv = h.shape[0], self.H, self.dk, self.dv
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        decay = ctx.empty((T, H * dk), torch.float32)              # sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau)
        ops.gemm_plain_decay(proj[:, self.off_a:self.off_a + self.rank], self.a2, self.a2_bias, self.coef, dk, -1.0, decay)
        o = ctx.empty((T, H * dv), torch.float32)
        ops.recurrent_scan(ops.RULE_GLA, proj[:, :self.off_k], proj[:, self.off_k:self.off_v], proj[:, self.off_v:self.off_g],
                           decay, None, dk ** -0.5, ctx.state(cache_layer), ctx.slots, ctx.cu_q, o, H, H, dk, dv,
                           parts=self._step_parts(ctx))
        y = ctx.empty((T, H * dv))
        ops.head_norm_gate(o, self.norm, proj[:, self.off_g:self.off_a], ops.GATE_SILU, self.eps, y, H, dv)
        linear(ctx, y, self.wo, out, None, epilogue)



class ChannelDeltaRule(_StateMixer):
    """The gated delta rule with a decay per head AND key channel. q, k (`n_qk_heads` heads of `key_dim`; head h of the
    `n_heads` value heads reads q/k head h // (n_heads / n_qk_heads)) and v pass a short causal convolution over time
    per channel and a SiLU; q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times
    1 / sqrt(key_dim). Per head

        S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q       (the read-out sees the token's write)
        g = exp(-exp(A_log[head]) * softplus((h A1^T) A2^T + dt_bias)),   beta = sigmoid(h Wb^T)

    then o is divided by its root mean square over the value channels, times a plain weight shared by the heads, times
    sigmoid((h G1^T) G2^T), and projected by Wo. The state slot holds S and the convolution's last taps - 1 inputs."""
    UNIT_EPS = 1e-6
    RULE = ops.RULE_DELTA

    def __init__(self, dim: int, n_heads: int, n_qk_heads: int, key_dim: int, value_dim: int, conv_taps: int,
                 norm_eps: float, names: Dict[str, str], decay_rank: Optional[int] = None, gate_rank: Optional[int] = None):
        super().__init__(names)
        if n_heads % n_qk_heads != 0:
            raise ValueError(f"{n_heads} value heads cannot share {n_qk_heads} query/key heads")
        self.dim, self.H, self.G, self.dk, self.dv = dim, n_heads, n_qk_heads, key_dim, value_dim
        self.taps, self.eps = int(conv_taps), float(norm_eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.C = 2 * self.G * self.dk + self.H * self.dv          # channels that pass the convolution: q | k | v
        self.off_b = self.C
        self.off_a = self.off_b + self.H
        self.w_in = self.wo = self.a2 = self.dt_bias = self.g2 = self.norm = self.coef = self.conv = None

    def local_specs(self):
        ra = -1 if self.decay_rank is None else self.decay_rank
        rg = -1 if self.gate_rank is None else self.gate_rank
        G, H, dk, dv, d = self.G, self.H, self.dk, self.dv, self.dim
        return {"wq": TensorSpec((G * dk, d), MATRIX), "q_conv": TensorSpec((G * dk, self.taps), MATRIX),
                "wk": TensorSpec((G * dk, d), MATRIX), "k_conv": TensorSpec((G * dk, self.taps), MATRIX),
                "wv": TensorSpec((H * dv, d), MATRIX), "v_conv": TensorSpec((H * dv, self.taps), MATRIX),
                "wb": TensorSpec((H, d), MATRIX), "a_log": TensorSpec((H,), BIAS), "norm": TensorSpec((dv,), NORM),
                "a1": TensorSpec((ra, d), MATRIX), "a2": TensorSpec((H * dk, ra), MATRIX), "dt_bias": TensorSpec((H * dk,), BIAS),
                "g1": TensorSpec((rg, d), MATRIX), "g2": TensorSpec((H * dv, rg), MATRIX), "wo": TensorSpec((d, H * dv), MATRIX)}

    def place(self, local, dtype, device):
        self.decay_rank = _rank(local["a1"], local["a2"], "the decay's factors")
        self.gate_rank = _rank(local["g1"], local["g2"], "the output gate's factors")
        self.off_g = self.off_a + self.decay_rank
        self.w_in = to_device_matrix(torch.cat([local[n] for n in ("wq", "wk", "wv", "wb", "a1", "g1")], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        self.a2 = to_device_matrix(local["a2"], dtype, device)
        self.g2 = to_device_matrix(local["g2"], dtype, device)
        self.dt_bias = to_device_vector(local["dt_bias"], dtype, device)
        self.norm = to_device_vector(local["norm"], dtype, device)
        self.conv = torch.cat([local[n].to(torch.float32) for n in ("q_conv", "k_conv", "v_conv")], dim=0).to(device).contiguous()
        self.coef = torch.exp(local["a_log"].to(torch.float32)).to(device).contiguous()

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv + (self.taps - 1) * self.C,), "float32")

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        T, H, G, dk, dv, C = h.shape[0], self.H, self.G, self.dk, self.dv, self.C
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        state = ctx.state(cache_layer)
        tail = state[:, H * dk * dv:]
        qkv = ctx.empty((T, C), torch.float32)
        ops.conv_silu_unit(proj, self.conv, tail, ctx.slots, ctx.tok_req, ctx.cu_q, qkv, 2 * G, G, dk, dk ** -0.5, self.UNIT_EPS)
        ops.conv_tail_update(proj, self.taps, tail, ctx.slots, ctx.cu_q, C)
        decay = ctx.empty((T, H * dk), torch.float32)              # exp(-exp(A_log) * softplus(z + dt_bias))
        ops.gemm_plain_decay(proj[:, self.off_a:self.off_g], self.a2, self.dt_bias, self.coef, dk, 1.0, decay)
        glog = ctx.empty((T, H * dv), torch.float32)
        ops.gemm_plain(proj[:, self.off_g:self.off_g + self.gate_rank], self.g2, glog, None, EPI_NONE)
        o = ctx.empty((T, H * dv), torch.float32)
        ops.recurrent_scan(ops.RULE_DELTA, qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], decay,
                           proj[:, self.off_b:self.off_a], 1.0, state, ctx.slots, ctx.cu_q, o, H, G, dk, dv,
                           parts=self._step_parts(ctx))
        y = ctx.empty((T, H * dv))
        ops.head_norm_gate(o, self.norm, glog, ops.GATE_SIGMOID, self.eps, y, H, dv)
        linear(ctx, y, self.wo, out, None, epilogue)


class MatrixMemory(_StateMixer):
    """A matrix memory per head with exponential gates held against a running maximum (the mLSTM of xLSTM). With
    q = h Wq^T / sqrt(key_dim), k = h Wk^T, v = h Wv^T and, per head, a log input gate i = cap tanh((h Wi^T + bi) / cap) and a
    log forget gate f = log sigmoid(cap tanh((h Wf^T + bf) / cap)):

        m' = max(f + m, i);   S' = e^(f + m - m') S + e^(i - m') k v^T;   n' = e^(f + m - m') n + e^(i - m') k
        o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)

    S, n and m start at zero. Each head's o is divided by its root mean square, the heads are joined, multiplied by a
    weight per head and channel and by sigmoid(h Wg^T), and projected by Wo. One joined product makes q | k | v | g | i | f;
    a kernel walks the gates (scalars per head) and leaves decays and weighted keys, which the scan of
    `GatedLinearAttention` consumes with one more value column, a column of ones: the state's last value column is then the
    normaliser n and the read-out's last column n . q. The slot holds S | n as [H, dk, dv + 1], and m [H]."""
    RULE = ops.RULE_GLA

    def __init__(self, dim: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float, names: Dict[str, str]):
        super().__init__(names)
        self.dim, self.H, self.dk, self.dv = dim, n_heads, key_dim, value_dim
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        H, dk, dv = self.H, self.dk, self.dv
        self.off_k, self.off_v, self.off_g = H * dk, 2 * H * dk, 2 * H * dk + H * dv
        self.off_i = self.off_g + H * dv
        self.off_f = self.off_i + H
        self.off_m = H * dk * (dv + 1)                # the normaliser is the state's last value column
        self.w_in = self.wo = self.norm = self.bias_i = self.bias_f = None

    def local_specs(self):
        H, dk, dv, d = self.H, self.dk, self.dv, self.dim
        return {"wq": TensorSpec((H * dk, d), MATRIX), "wk": TensorSpec((H * dk, d), MATRIX), "wv": TensorSpec((H * dv, d), MATRIX),
                "wg": TensorSpec((H * dv, d), MATRIX), "wi": TensorSpec((H, d), MATRIX), "wf": TensorSpec((H, d), MATRIX),
                "bias_i": TensorSpec((H,), BIAS), "bias_f": TensorSpec((H,), BIAS), "norm": TensorSpec((H * dv,), NORM),
                "wo": TensorSpec((d, H * dv), MATRIX)}

    def place(self, local, dtype, device):
        self.w_in = to_device_matrix(torch.cat([local[n] for n in ("wq", "wk", "wv", "wg", "wi", "wf")], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        self.norm = to_device_vector(local["norm"], dtype, device)
        self.bias_i = to_device_vector(local["bias_i"], dtype, device)
        self.bias_f = to_device_vector(local["bias_f"], dtype, device)

    def cache_spec(self):
        return StateSpec((self.H * self.dk * (self.dv + 1) + self.H,), "float32")

    def _parts(self, q_lens) -> int:
        n_long = sum(1 for n in q_lens if n >= ops.SCAN_PART_MIN_TOKENS)
        return ops.recurrent_scan_parts(self.RULE, self.H, self.dk, self.dv + 1, n_long) if n_long else 1

    def _plan_key(self) -> str:
        return f"recurrence parts {self.RULE} {self.H}x{self.dk}x{self.dv + 1}"

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        T, H, dk, dv = h.shape[0], self.H, self.dk, self.dv
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        state = ctx.state(cache_layer)
        decay, keys, values, floor = ops.memory_gates(proj, self.off_k, self.off_v, self.off_i, self.off_f, self.bias_i, self.bias_f,
                                                      self.cap, state, self.off_m, ctx.slots, ctx.cu_q, H, dk, dv)
        o = ctx.empty((T, H * (dv + 1)), torch.float32)      # a head's last column: n . q
        ops.recurrent_scan(ops.RULE_GLA, proj[:, :self.off_k], keys, values, decay, None, dk ** -0.5, state, ctx.slots, ctx.cu_q, o,
                           H, H, dk, dv + 1, parts=self._step_parts(ctx))
        y = ctx.empty((T, H * dv))
        ops.head_norm_gate_ext(o, self.norm, proj[:, self.off_g:self.off_i], ops.GATE_SIGMOID, self.eps, y, H, dv, floor=floor)
        linear(ctx, y, self.wo, out, None, epilogue)


class ShiftedDecayRecurrence(_StateMixer):
    """A linear recurrence whose inputs are mixed with the token before (the time mixing of RWKV). With h' the row of the
    request's token before (zeros before the first), each of r, k, v, the gate and the decay reads its own
    h + (h' - h) * mu_s. Per head (keys and values of `head_dim`), with a bonus u per head and key channel for the
    current token only:

        o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T;   w = exp(-exp(tanh(mix_w W1^T) W2^T + w0))

    Each head's o is divided by its root mean square, the heads are joined, multiplied by a weight per head and channel
    and by silu(mix_g Wg^T), and projected by Wo. The mixes are made from the 32-bit rows (the block leaves them in the
    step's memo), the slot holds S [H, dk, dk] and h' [dim]."""
    RULE = ops.RULE_BONUS
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, dim: int, n_heads: int, head_dim: int, norm_eps: float, names: Dict[str, str], decay_rank: Optional[int] = None):
        super().__init__(names)
        self.dim, self.H, self.dk, self.dv = dim, n_heads, head_dim, head_dim
        self.eps, self.rank = float(norm_eps), decay_rank
        self.off_prev = self.H * self.dk * self.dk
        self.mu = self.wr = self.wk = self.wv = self.wg = self.w1 = self.w2 = self.w0 = self.u = self.norm = self.wo = None

    def local_specs(self):
        H, dk, d = self.H, self.dk, self.dim
        r = -1 if self.rank is None else self.rank
        s = {f"mu_{m}": TensorSpec((d,), NORM) for m in self.MIXES}
        s.update({"wr": TensorSpec((H * dk, d), MATRIX), "wk": TensorSpec((H * dk, d), MATRIX), "wv": TensorSpec((H * dk, d), MATRIX),
                  "wg": TensorSpec((H * dk, d), MATRIX), "w1": TensorSpec((r, d), MATRIX), "w2": TensorSpec((H * dk, r), MATRIX),
                  "w0": TensorSpec((H * dk,), BIAS), "u": TensorSpec((H, dk), MATRIX), "norm": TensorSpec((H * dk,), NORM),
                  "wo": TensorSpec((d, H * dk), MATRIX)})
        return s

    def place(self, local, dtype, device):
        self.rank = _rank(local["w1"], local["w2"], "the decay's factors")
        self.mu = torch.stack([local[f"mu_{m}"].to(torch.float32) for m in self.MIXES], dim=0).to(device).contiguous()
        for n in ("wr", "wk", "wv", "wg", "w1", "w2", "wo"):
            setattr(self, n, to_device_matrix(local[n], dtype, device))
        self.w0 = to_device_vector(local["w0"], dtype, device)
        self.norm = to_device_vector(local["norm"], dtype, device)
        self.u = local["u"].to(device=device, dtype=torch.float32).contiguous()

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dk + self.dim,), "float32")

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        x32 = h if h.dtype == torch.float32 else ctx.memo.get(("rows32", id(h)))
        if x32 is None:
            raise TypeError("ShiftedDecayRecurrence mixes its inputs in 32-bit: the block must leave the 32-bit rows that `h` was made "
                            "from in the step's memo under ('rows32', id(h))")
        T, H, dk = h.shape[0], self.H, self.dk
        state = ctx.state(cache_layer)
        prev = state[:, self.off_prev:]
        mixes = ctx.empty((len(self.MIXES), T, self.dim))
        ops.shift_mix(x32, self.mu, prev, ctx.slots, ctx.tok_req, ctx.cu_q, mixes)
        ops.conv_tail_update(x32, 2, prev, ctx.slots, ctx.cu_q, self.dim)
        r, k, v, g = (ctx.empty((T, H * dk), torch.float32) for _ in range(4))
        for i, (w, dst) in enumerate(((self.wr, r), (self.wk, k), (self.wv, v), (self.wg, g))):
            linear(ctx, mixes[i], w, dst, None, EPI_NONE)
        low = ctx.empty((T, self.rank), torch.float32)
        linear(ctx, mixes[4], self.w1, low, None, EPI_NONE)
        decay = ctx.empty((T, H * dk), torch.float32)
        ops.gemm_plain_decay_exp(low, self.w2, self.w0, decay, x_tanh=True)
        bonus = ctx.empty((T, H), torch.float32)
        ops.bonus_dot(r, k, self.u, bonus, H, dk)
        o = ctx.empty((T, H * dk), torch.float32)
        ops.recurrent_scan(ops.RULE_BONUS, r, k, v, decay, bonus, 1.0, state, ctx.slots, ctx.cu_q, o, H, H, dk, dk,
                           parts=self._step_parts(ctx))
        y = ctx.empty((T, H * dk))
        ops.head_norm_gate_ext(o, self.norm, g, ops.GATE_SILU, self.eps, y, H, dk)
        linear(ctx, y, self.wo, out, None, epilogue)


class Retention(_StateMixer):
    """Linear attention with a FIXED decay per head and no softmax or denominator. With q = h Wq^T and k = h Wk^T (heads of
    `key_dim`), both rotated by the token's position (any `RotaryTable` with pairs in halves; partial rotation), k then times
    key_dim^(-1/2), and v = h Wv^T (heads of `value_dim`):

        S_t = c_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t                (c_h: `decays`, one constant per head)

    Each head's o is divided by its root mean square (no weight), the heads are joined, multiplied by silu(h Wg^T) and
    projected by Wo. One joined product makes q | k | v | g with 32-bit sums; rotation, the key's factor and the decays are one
    kernel in 32-bit; the scan is `GatedLinearAttention`'s. The slot holds S [H, key_dim, value_dim]."""
    RULE = ops.RULE_GLA

    def __init__(self, dim: int, n_heads: int, key_dim: int, value_dim: int, decays, rotary, norm_eps: float, names: Dict[str, str]):
        super().__init__(names)
        decays = [float(c) for c in decays]
        if len(decays) != n_heads:
            raise ValueError(f"Retention: {len(decays)} decays for {n_heads} heads")
        if any(not 0.0 <= c <= 1.0 for c in decays):
            raise ValueError(f"Retention: decays must lie in [0, 1], got {decays}")
        if rotary is not None and rotary.pairs != "halves":
            raise ValueError("Retention: the rotation pairs value i with i + n / 2")
        self.dim, self.H, self.dk, self.dv = dim, n_heads, key_dim, value_dim
        self.decays, self.rotary, self.eps = decays, rotary, float(norm_eps)
        self.off_k, self.off_v = self.H * self.dk, 2 * self.H * self.dk
        self.off_g = self.off_v + self.H * self.dv
        self.w_in = self.wo = self.head_decay = self.no_freq = None

    def local_specs(self):
        H, dk, dv, d = self.H, self.dk, self.dv, self.dim
        return {"wq": TensorSpec((H * dk, d), MATRIX), "wk": TensorSpec((H * dk, d), MATRIX), "wv": TensorSpec((H * dv, d), MATRIX),
                "wg": TensorSpec((H * dv, d), MATRIX), "wo": TensorSpec((d, H * dv), MATRIX)}

    def place(self, local, dtype, device):
        self.w_in = to_device_matrix(torch.cat([local[n] for n in ("wq", "wk", "wv", "wg")], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        self.head_decay = torch.tensor(self.decays, dtype=torch.float32, device=device)
        self.no_freq = torch.zeros(1, dtype=torch.float32, device=device)
        if self.rotary is not None:
            self.rotary.to(device)

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv,), "float32")

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        T, H, dk, dv = h.shape[0], self.H, self.dk, self.dv
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        rot = self.rotary
        q, k, decay = ops.rope_decay_prep(proj, self.off_k, ctx.positions, rot.inv_freq if rot is not None else self.no_freq,
                                          rot.rot_half if rot is not None else 0, self.head_decay, dk ** -0.5, H, dk)
        o = ctx.empty((T, H * dv), torch.float32)
        ops.recurrent_scan(ops.RULE_GLA, q, k, proj[:, self.off_v:self.off_g], decay, None, 1.0, ctx.state(cache_layer), ctx.slots,
                           ctx.cu_q, o, H, H, dk, dv, parts=self._step_parts(ctx))
        y = ctx.empty((T, H * dv))
        ops.head_norm_gate(o, None, proj[:, self.off_g:self.off_g + H * dv], ops.GATE_SILU, self.eps, y, H, dv)
        linear(ctx, y, self.wo, out, None, epilogue)


class StateSpaceDuality(_StateMixer):
    """A selective state-space mixer whose decay is one number per head and token (Mamba-2). With inner = heads * value_dim,
    N = `state`, G = `groups`, the joined product W_in h is laid out [z: inner | x: inner | B: G N | C: G N | dt: heads]. x, B
    and C pass a short causal convolution per channel (taps [channels, n], the last column the current token's, a bias per
    channel, zeros before the start) and a SiLU; dt <- softplus(dt + dt_bias). Per head h (it reads B and C of group
    h // (heads / G)):

        S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T   (S: N x value_dim),     y_t = S_t^T C_t + D_h x_t

    then y (heads joined) is multiplied by silu(z) and after that RMS-normed in `norm_groups` equal parts of the row (each by
    its own root mean square), times a weight, and projected by Wo. B is the scan's key, C its query, dt x its value: the
    scan is `GatedLinearAttention`'s. The slot holds S [H, N, value_dim] and the convolution's last n - 1 inputs; dt, decays,
    state, gate and norm are 32-bit."""
    RULE = ops.RULE_GLA

    def __init__(self, dim: int, n_heads: int, value_dim: int, state: int, groups: int, conv_taps: int, norm_groups: int,
                 norm_eps: float, names: Dict[str, str]):
        super().__init__(names)
        if n_heads % groups != 0:
            raise ValueError(f"StateSpaceDuality: {n_heads} heads cannot share {groups} groups of B and C")
        inner = n_heads * value_dim
        if norm_groups < 1 or inner % norm_groups != 0:
            raise ValueError(f"StateSpaceDuality: {inner} inner channels do not split into {norm_groups} equal parts")
        self.dim, self.H, self.dk, self.dv, self.G = dim, n_heads, state, value_dim, groups
        self.taps, self.norm_groups, self.eps = int(conv_taps), int(norm_groups), float(norm_eps)
        self.inner = inner
        self.C = inner + 2 * groups * state              # channels that pass the convolution: x | B | C
        self.off_dt = inner + self.C
        self.n_in = self.off_dt + n_heads
        self.w_in = self.wo = self.conv = self.conv_bias = self.dt_bias = self.rate = self.skip = self.norm = None

    def local_specs(self):
        H, d = self.H, self.dim
        return {"w_in": TensorSpec((self.n_in, d), MATRIX), "conv": TensorSpec((self.C, self.taps), MATRIX),
                "conv_bias": TensorSpec((self.C,), BIAS), "dt_bias": TensorSpec((H,), BIAS), "a_log": TensorSpec((H,), BIAS),
                "skip": TensorSpec((H,), BIAS), "norm": TensorSpec((self.inner,), NORM), "wo": TensorSpec((d, self.inner), MATRIX)}

    def place(self, local, dtype, device):
        self.w_in = to_device_matrix(local["w_in"], dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.conv, self.conv_bias = f32(local["conv"]), f32(local["conv_bias"])
        self.dt_bias, self.skip = f32(local["dt_bias"]), f32(local["skip"])
        self.rate = torch.exp(local["a_log"].to(torch.float32)).to(device).contiguous()
        self.norm = to_device_vector(local["norm"], dtype, device)

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv + (self.taps - 1) * self.C,), "float32")

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        self._check(write_cache)
        T, H, G, N, dv, inner, C = h.shape[0], self.H, self.G, self.dk, self.dv, self.inner, self.C
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        state = ctx.state(cache_layer)
        tail = state[:, H * N * dv:]
        xbc_in = proj[:, inner:inner + C]
        xbc = ctx.empty((T, C), torch.float32)
        ops.conv_silu_unit(xbc_in, self.conv, tail, ctx.slots, ctx.tok_req, ctx.cu_q, xbc, 0, 0, 1, 1.0, 0.0, bias=self.conv_bias)
        ops.conv_tail_update(xbc_in, self.taps, tail, ctx.slots, ctx.cu_q, C)
        x = xbc[:, :inner]
        decay, v = ops.ssd_prep(proj[:, self.off_dt:self.off_dt + H], self.dt_bias, self.rate, x, H, N, dv)
        o = ctx.empty((T, inner), torch.float32)
        ops.recurrent_scan(ops.RULE_GLA, xbc[:, inner + G * N:], xbc[:, inner:inner + G * N], v, decay, None, 1.0, state, ctx.slots,
                           ctx.cu_q, o, H, G, N, dv, parts=self._step_parts(ctx))
        y = ctx.empty((T, inner))
        ops.gated_group_norm(o, x, self.skip, dv, proj[:, :inner], self.norm, self.norm_groups, self.eps, y)
        linear(ctx, y, self.wo, out, None, epilogue)
