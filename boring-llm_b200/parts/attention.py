"""Mixers: the parts of a block that let tokens see one another."""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from ..cache import PagedKVSpec
from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS, NORM
from .base import PendingNormRows, Part, StepPlan, to_device_matrix, to_device_vector
from .linear import linear, EPI_BIAS, EPI_NONE, EPI_RESIDUAL
from .norm import RMSNorm
from .rotary import RotaryTable

FUSED_MAX_ROWS = 64       # steps with at most this many rows take the fused norm + product kernels

QKV_EPILOGUE_MIN_ROWS = ops.PAIR_MIN_ROWS  # from here the joined product runs on pairs of SMs, whose epilogue can rotate and write the cache
PREFILL_TC_MIN_TOKENS = 256          # steps with fewer prompt tokens keep the 64-row tiles of the mma.sync kernel (measured: 512-token portions gain 8%)
DECODE_MAX_SPLITS = ops.DECODE_CLUSTER_SPLITS   # the slices of a request are one cluster of blocks that merge in shared memory
PLAN_KEY = "paged attention"         # one plan per step for all attention layers: its lists do not depend on head sizes


def tc_attention_tiles(q_lens, ctx_lens):
    """The launch list of the tcgen05 prefill attention: (request, first token) of every tile of 128 new tokens of
    the requests with more than one, the tile with the fewest keys first (the kernel starts from the end of the
    list, so that the long tiles run first and the short ones fill the tail). Key blocks are counted without the
    window (an upper bound)."""
    tiles = []                                           # [key blocks, request, first token]
    for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        if n <= 1:
            continue
        for t0 in range(0, n, 128):
            tiles.append([-(-(c - n + min(t0 + 128, n)) // 128), r, t0])
    tiles.sort()
    return [[r, t0] for _, r, t0 in tiles]


def attention_plan(q_lens, ctx_lens, filler=None) -> StepPlan:
    """What the attention kernels walk in one step: the 64-token tiles (and, for steps with many prompt tokens, the
    128-token tiles in launch order) of the requests with several new tokens, and the list of requests with a
    single one, with the longest context among those. For a step that will be replayed (`filler` given) the lists
    are padded to multiples of 8 with entries of the request without tokens, and the longest context is rounded up
    to a power of two: launches then depend on these sizes only."""
    tiles64 = [[r, t0] for r, n in enumerate(q_lens) if n > 1 for t0 in range(0, n, 64)]
    singles = [r for r, n in enumerate(q_lens) if n == 1]
    use_tc = sum(n for n in q_lens if n > 1) >= PREFILL_TC_MIN_TOKENS
    tiles128 = tc_attention_tiles(q_lens, ctx_lens) if use_tc else []
    longest = max((ctx_lens[r] for r in singles), default=0)
    if filler is not None:
        pad = lambda n: -(-n // 8) * 8 - n
        tiles64 = tiles64 + [[filler, 0]] * pad(len(tiles64))
        tiles128 = [[filler, 0]] * pad(len(tiles128)) + tiles128          # the front of this list is launched last
        singles = singles + [filler] * pad(len(singles))
        bucket = 256
        while bucket < longest:
            bucket *= 2
        longest = bucket if singles else 0
    return StepPlan(
        arrays={"tiles64": np.asarray(tiles64, dtype=np.int32).reshape(-1, 2),
                "tiles128": np.asarray(tiles128, dtype=np.int32).reshape(-1, 2),
                "singles": np.asarray(singles, dtype=np.int32)},
        host={"longest_single": longest},
        shape=(len(tiles64), len(tiles128), len(singles), longest))


def paged_attention(ctx, q, k_cache, v_cache, table, out, H: int, KV: int, dh: int, window: int, scale: float,
                    sinks=None, gate=None, softcap: float = 0.0) -> None:
    """Causal attention of the step's tokens over the paged cache. Tensor-core kernels for bfloat16 where they are built
    (pages of 16, common head sizes, values of the keys' head size): one launch for the requests with several new tokens
    (the tcgen05 kernel for head sizes 64 and 128 when the step has many of them), one for those with a single token.
    Otherwise, and always in float32, the plain kernel. Which requests those are comes from the step's plan
    (`attention_plan`). `sinks` [H] and `gate` (32-bit logits [T, >= H]) are what may follow the softmax: a score per
    head that joins the denominator, a sigmoid per (token, head) on the output. `softcap` c > 0: scaled scores pass
    c tanh(s / c) before the softmax (every attention kernel has it)."""
    dv = v_cache.shape[3]
    if not (ctx.fast and dv == dh and ops.attention_mma_supported(q.dtype, dh, k_cache.shape[2])):
        ops.attention_plain(q, k_cache, v_cache, ctx.tok_req, ctx.cu_q, ctx.ctx_len, table, out, H, window, scale, sinks, gate,
                            softcap=softcap)
        return
    plan = ctx.plans.get(PLAN_KEY)
    if plan is None:                                 # a step put together without asking the parts: plan it now
        plan = attention_plan(ctx.q_lens, ctx.ctx_lens)
        plan.arrays = {k: torch.from_numpy(v).to(ctx.device) for k, v in plan.arrays.items()}
        ctx.plans[PLAN_KEY] = plan
    tiles64, tiles128, singles = plan.arrays["tiles64"], plan.arrays["tiles128"], plan.arrays["singles"]
    if tiles64.shape[0]:
        if tiles128.shape[0] and ops.attention_prefill_tc_supported(q.dtype, dh, k_cache.shape[2]):
            ops.attention_prefill_tc(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, tiles128, out, H, window, scale, sinks, gate,
                                     softcap=softcap)
        else:
            ops.attention_prefill(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, tiles64, out, H, window, scale, sinks, gate,
                                  softcap=softcap)
    n = singles.shape[0]
    if n:
        # as many slices of the keys as fill the device once (the kernel knows how many of its blocks fit)
        longest = plan.host["longest_single"]
        if window > 0:
            longest = min(longest, window + 64)
        G = H // KV
        if ops.attention_decode_tma_supported(q.dtype, dh, k_cache.shape[2]):
            # head sizes 64 and 128: the TMA-fed kernel, which knows how many slices pay for this many requests
            n_splits = ops.attention_decode_tma_splits(n, KV, G, dh, longest)
            ops.attention_decode_tma(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, singles, n_splits, out, H, window, scale,
                                     sinks, gate, softcap=softcap)
            return
        groups = KV * (-(-G // 16))
        resident = ops.attention_decode_resident_blocks(dh)
        n_splits = max(1, min(-(-longest // 64), resident // (n * groups), DECODE_MAX_SPLITS))
        ops.attention_decode(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, singles, n_splits, out, H, window, scale,
                             sinks=sinks, gate=gate, softcap=softcap)


class Mixer(Part):
    """Interface of a mixer.

    `cache_spec()` says what one cache layer of this mixer needs (`PagedKVSpec`, `StateSpec` or
    None). `forward(ctx, h, residual, cache_layer, write_cache)` reads the normed rows `h` [T, dim],
    adds its result into the 32-bit `residual` [T, dim] in place, and may read and write the cache
    layer it is given through `ctx.kv(cache_layer)` / `ctx.state(cache_layer)`. With `write_cache`
    false it reads a layer that another call has written in this step.
    """

    # True when forward() only launches work on the current stream from device-side inputs (no host loops
    # over the batch, no host reads): such a mixer may be captured in a CUDA graph and replayed.
    graph_safe = False

    def cache_spec(self):
        return None

    def forward(self, ctx, h, residual, cache_layer: Optional[int], write_cache: bool = True) -> None:
        raise NotImplementedError

    def forward_fused_norm(self, ctx, x, norm, cache_layer: Optional[int], write_cache: bool = True) -> bool:
        """Optional: run `norm` and this mixer on the residual stream `x` in fused kernels and return True,
        or return False to be called with the normed rows as usual."""
        return False

    def join_rows(self, weight) -> None:
        """For mixers that begin with ONE joined product of their input rows (its matrix in `self.w_in`, its 32-bit sums
        in `proj`): further rows for that matrix, from a part that reads the same rows (a gate on the mixer's result).
        After each run their sums are `self.joined_out` (a view [T, rows])."""
        pad = -self.w_in.shape[0] % 8            # the further columns start on a 16-byte boundary of the 32-bit sums
        self.n_own = self.w_in.shape[0] + pad
        self.w_in = torch.cat([self.w_in, self.w_in.new_zeros((pad, self.w_in.shape[1])),
                               weight.to(device=self.w_in.device, dtype=self.w_in.dtype)], dim=0).contiguous()

    def _joined(self, proj):
        n_own = getattr(self, "n_own", None)
        self.joined_out = proj[:, n_own:] if n_own is not None else None

    def mix(self, ctx, h, out, cache_layer: Optional[int], write_cache: bool = True) -> None:
        """Writes the result into the 32-bit `out` [T, dim] instead of adding it to a stream (for arrangements that
        treat a sublayer's result before the residual sum). Mixers whose last product can write as well as add
        override this; the default clears `out` and adds."""
        out.zero_()
        self.forward(ctx, h, out, cache_layer, write_cache)


class GQAAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    q, k, v = h.Wq^T + bq, h.Wk^T + bk, h.Wv^T + bv as ONE joined product (src/model.br:765-768,
    864-869, 1113-1115); q and k rotated by position; k cached after rotation, v as projected
    (:1814-1820); softmax(q.k^T * scale) over the keys a token may see (src/math.br:304-359);
    out.Wo^T added to the residual stream (src/model.br:1328-1334).
    """
    graph_safe = True
    takes_pending_norm = True            # its first product can finish an RMS norm that the product before has begun

    def takes_pending_norm_at(self, rows: int) -> bool:
        """... in steps with enough rows for the product on pairs of SMs (with few rows the norm is part of the q/k/v
        kernel, which reads the stream itself: measured, a norm begun by the layer before's down projection made a
        batch-8 decode step 4 % slower)."""
        return rows >= QKV_EPILOGUE_MIN_ROWS

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, rotary: Optional[RotaryTable],
                 names: Dict[str, str], qkv_bias: bool = True, out_bias: bool = False, window: int = 0,
                 scale: Optional[float] = None):
        super().__init__(names)
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} query heads cannot share {n_kv_heads} key/value heads")
        self.out_bias = bool(out_bias)
        self.dim, self.H, self.KV, self.dh = dim, n_heads, n_kv_heads, head_dim
        self.rotary = rotary if rotary is not None else RotaryTable(head_dim, 10000.0, n_rot=0)
        self.qkv_bias, self.window = qkv_bias, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.w_qkv = self.b_qkv = self.wo = self.bo = None

    def local_specs(self):
        s = {"wq": TensorSpec((self.H * self.dh, self.dim), MATRIX),
             "wk": TensorSpec((self.KV * self.dh, self.dim), MATRIX),
             "wv": TensorSpec((self.KV * self.dh, self.dim), MATRIX),
             "wo": TensorSpec((self.dim, self.H * self.dh), MATRIX)}
        if self.qkv_bias:
            s.update({"bq": TensorSpec((self.H * self.dh,), BIAS), "bk": TensorSpec((self.KV * self.dh,), BIAS),
                      "bv": TensorSpec((self.KV * self.dh,), BIAS)})
        if self.out_bias:                       # read per file in the reference (src/model.br:500, 1328)
            s["bo"] = TensorSpec((self.dim,), BIAS)
        return s

    def place(self, local, dtype, device):
        self.w_qkv = to_device_matrix(torch.cat([local["wq"], local["wk"], local["wv"]], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        if self.qkv_bias:
            b = [local["bq"], local["bk"], local["bv"]]
            if any(t.dtype == torch.float32 for t in b):
                b = [t.to(torch.float32) for t in b]
            self.b_qkv = to_device_vector(torch.cat(b, dim=0), dtype, device)
        if self.out_bias:
            self.bo = to_device_vector(local["bo"], dtype, device)
        self.rotary.to(device)

    def cache_spec(self):
        return PagedKVSpec(self.KV, self.dh, self.window)

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        T = h.shape[0]
        width = (self.H + 2 * self.KV) * self.dh
        k_cache, v_cache, table = ctx.kv(cache_layer)
        q = ctx.empty((T, self.H * self.dh))
        pending = h if isinstance(h, PendingNormRows) else None
        rows = pending.rows if pending is not None else h
        if (ctx.fast and T >= QKV_EPILOGUE_MIN_ROWS and self.rotary.pair_layout == 0 and self.rotary.rot_half * 2 == self.dh
                and ops.qkv_rope_tc_supported(rows, self.w_qkv, self.H, self.KV, self.dh, k_cache.shape[2])):
            # many rows: bias, rotation and the writes of q, k and v are the epilogue of the joined product (and the
            # scale of a norm that the product before has begun)
            cs, sn = self.rotary.step_table(ctx)
            ops.qkv_rope_tc(rows, self.w_qkv, self.b_qkv if self.qkv_bias else None, ctx.positions, ctx.tok_req, table, cs, sn,
                            q, k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV, self.dh,
                            row_sums=pending.sums if pending is not None else None, eps=pending.eps if pending is not None else 0.0)
        else:
            if pending is not None:
                h = pending.normed(ctx)
            qkv = ctx.empty((T, width), torch.float32)
            linear(ctx, h, self.w_qkv, qkv, self.b_qkv, EPI_BIAS if self.qkv_bias else EPI_NONE)
            ops.rope_kv_write(qkv, ctx.positions, ctx.tok_req, table, self.rotary.inv_freq, self.rotary.rot_half,
                              self.rotary.mscale, q, k_cache if write_cache else None,
                              v_cache if write_cache else None, self.H, self.KV, self.dh, self.rotary.pair_layout)
        attn = ctx.empty((T, self.H * self.dh))
        self.attend(ctx, q, k_cache, v_cache, table, attn)
        self.project_out(ctx, attn, residual)

    def project_out(self, ctx, attn, residual):
        """residual += attn . Wo^T (+ bo)."""
        if self.out_bias:
            ops.add_row_vector(residual, self.bo)
        linear(ctx, attn, self.wo, residual, None, EPI_RESIDUAL)

    def forward_fused_norm(self, ctx, x, norm, cache_layer, write_cache=True) -> bool:
        """Few rows in bfloat16: norm, joined product, bias, rotation and cache write are ONE kernel."""
        T = x.shape[0]
        if not (ctx.fast and ctx.dtype == torch.bfloat16 and T <= FUSED_MAX_ROWS and isinstance(norm, RMSNorm)
                and self.rotary.rot_half * 2 == self.dh and self.dh % 16 == 0
                and ops.norm_gemm_supported(x, self.w_qkv)):
            return False
        k_cache, v_cache, table = ctx.kv(cache_layer)
        q = ctx.empty((T, self.H * self.dh))
        ops.norm_qkv_rope(x, norm.weight, norm.eps, self.w_qkv, self.b_qkv if self.qkv_bias else None,
                          ctx.positions, ctx.tok_req, table, self.rotary.inv_freq, self.rotary.mscale, q,
                          k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV, self.dh,
                          self.rotary.pair_layout)
        attn = ctx.empty((T, self.H * self.dh))
        self.attend(ctx, q, k_cache, v_cache, table, attn)
        self.project_out(ctx, attn, x)
        return True

    def plan_step(self, q_lens, ctx_lens, filler=None):
        return PLAN_KEY, attention_plan(q_lens, ctx_lens, filler)

    def attend(self, ctx, q, k_cache, v_cache, table, out):
        paged_attention(ctx, q, k_cache, v_cache, table, out, self.H, self.KV, self.dh, self.window, self.scale)

class GatedSinkAttention(Mixer):
    """Causal grouped-query attention over the paged cache with the options of newer designs, each a constructor
    argument:

    * `v_head_dim`: values of another head size than queries and keys;
    * `qk_norm="whole"`: an RMS norm over a token's whole q projection, and one over its whole k projection (all heads
      at once, plain weights), before the rotation (None: no norm);
    * `rotary`: any `RotaryTable` (pairs "halves" or "interleaved", partial rotation);
    * `window`: position i sees j with 0 <= i - j < window (0: every j <= i);
    * `sink=True`: a learned score per head whose exponential joins the softmax's denominator once, unscaled, with no
      key and no value;
    * `out_gate=True`: head h's output is multiplied by sigmoid(h . Wg^T)[h], one number per token and head, read from
      the same rows as the projections;
    * `qkv_bias=True` / `out_bias=True`: a bias on q, k and v, added in the joined product, and one on the output projection;
    * `softcap` c > 0: score <- c tanh(score / c) on the scaled score, before the softmax.

    q, k, v and the gate's logits are ONE joined product with 32-bit sums; norm, rotation and the cache write are one
    kernel; scores, softmax and the sink are 32-bit.
    """
    graph_safe = True

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: Optional[int],
                 rotary: Optional[RotaryTable], names: Dict[str, str], window: int = 0, scale: Optional[float] = None,
                 qk_norm: Optional[str] = None, qk_norm_eps: float = 1e-6, sink: bool = False, out_gate: bool = False,
                 qkv_bias: bool = False, out_bias: bool = False, softcap: float = 0.0):
        super().__init__(names)
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} query heads cannot share {n_kv_heads} key/value heads")
        if softcap < 0:
            raise ValueError(f"a cap on the scores must not be negative, got {softcap}")
        self.qkv_bias, self.out_bias, self.softcap = bool(qkv_bias), bool(out_bias), float(softcap)
        self.b_in = self.bo = None
        if qk_norm not in (None, "whole"):
            raise ValueError(f"qk_norm must be None or 'whole', got {qk_norm!r}")
        self.dim, self.H, self.KV, self.dk = dim, n_heads, n_kv_heads, head_dim
        self.dv = head_dim if v_head_dim is None else int(v_head_dim)
        self.rotary = rotary if rotary is not None else RotaryTable(head_dim, 10000.0, n_rot=0)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qk_norm, self.qk_norm_eps, self.has_sink, self.out_gate = qk_norm, float(qk_norm_eps), bool(sink), bool(out_gate)
        self.off_k = self.H * self.dk
        self.off_v = self.off_k + self.KV * self.dk
        self.off_g = self.off_v + self.KV * self.dv
        self.n_in = self.off_g + (self.H if self.out_gate else 0)
        self.w_in = self.wo = self.q_norm = self.k_norm = self.sinks = None

    def local_specs(self):
        s = {"wq": TensorSpec((self.H * self.dk, self.dim), MATRIX), "wk": TensorSpec((self.KV * self.dk, self.dim), MATRIX),
             "wv": TensorSpec((self.KV * self.dv, self.dim), MATRIX), "wo": TensorSpec((self.dim, self.H * self.dv), MATRIX)}
        if self.qk_norm:
            s["q_norm"] = TensorSpec((self.H * self.dk,), NORM)
            s["k_norm"] = TensorSpec((self.KV * self.dk,), NORM)
        if self.has_sink:
            s["sink"] = TensorSpec((self.H,), BIAS)
        if self.out_gate:
            s["wg"] = TensorSpec((self.H, self.dim), MATRIX)
        if self.qkv_bias:
            s.update({"bq": TensorSpec((self.H * self.dk,), BIAS), "bk": TensorSpec((self.KV * self.dk,), BIAS),
                      "bv": TensorSpec((self.KV * self.dv,), BIAS)})
        if self.out_bias:
            s["bo"] = TensorSpec((self.dim,), BIAS)
        return s

    def place(self, local, dtype, device):
        joined = [local["wq"], local["wk"], local["wv"]] + ([local["wg"]] if self.out_gate else [])
        self.w_in = to_device_matrix(torch.cat(joined, dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        if self.qkv_bias:                        # the gate's logits (further columns of the joined product) have none
            b = [local[n].to(torch.float32) for n in ("bq", "bk", "bv")] + ([torch.zeros(self.H)] if self.out_gate else [])
            self.b_in = torch.cat(b, dim=0).to(device).contiguous()
        if self.out_bias:
            self.bo = to_device_vector(local["bo"], dtype, device)
        if self.qk_norm:
            self.q_norm = to_device_vector(local["q_norm"], dtype, device)
            self.k_norm = to_device_vector(local["k_norm"], dtype, device)
        if self.has_sink:
            self.sinks = to_device_vector(local["sink"], dtype, device)
        self.rotary.to(device)

    def cache_spec(self):
        return PagedKVSpec(self.KV, self.dk, self.window, 0 if self.dv == self.dk else self.dv)

    def plan_step(self, q_lens, ctx_lens, filler=None):
        return PLAN_KEY, attention_plan(q_lens, ctx_lens, filler)

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        T = h.shape[0]
        k_cache, v_cache, table = ctx.kv(cache_layer)
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, self._bias_in(), EPI_BIAS if self.qkv_bias else EPI_NONE)
        self._joined(proj)
        q = ctx.empty((T, self.H * self.dk))
        ops.qk_norm_rope_write(proj, self.off_k, self.off_v, self.q_norm, self.k_norm, self.qk_norm_eps, ctx.positions,
                               ctx.tok_req, table, self.rotary.inv_freq, self.rotary.rot_half, self.rotary.pair_layout, q,
                               k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV,
                               self.dk, self.dv)
        attn = ctx.empty((T, self.H * self.dv))
        gate = proj[:, self.off_g:self.off_g + self.H] if self.out_gate else None
        self.attend(ctx, q, k_cache, v_cache, table, attn, gate)
        if self.out_bias:
            if epilogue == EPI_RESIDUAL:
                ops.add_row_vector(out, self.bo)
                linear(ctx, attn, self.wo, out, None, EPI_RESIDUAL)
            else:
                linear(ctx, attn, self.wo, out, self.bo, EPI_BIAS)
            return
        linear(ctx, attn, self.wo, out, None, epilogue)

    def _bias_in(self):
        """The joined product's bias, as long as its matrix (a part that joined further rows has none for them)."""
        if not self.qkv_bias:
            return None
        if self.b_in.shape[0] != self.w_in.shape[0]:
            self.b_in = torch.cat([self.b_in, self.b_in.new_zeros(self.w_in.shape[0] - self.b_in.shape[0])]).contiguous()
        return self.b_in

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        self._run(ctx, h, residual, cache_layer, write_cache, EPI_RESIDUAL)

    def mix(self, ctx, h, out, cache_layer, write_cache=True):
        self._run(ctx, h, out, cache_layer, write_cache, EPI_NONE)

    def attend(self, ctx, q, k_cache, v_cache, table, out, gate):
        paged_attention(ctx, q, k_cache, v_cache, table, out, self.H, self.KV, self.dk, self.window, self.scale, self.sinks, gate,
                        softcap=self.softcap)


class ChunkedTalkingAttention(Mixer):
    """Grouped-query attention over the query's own chunk of positions, with the heads' softmax weights mixed afterwards:

    * q and k get an RMS norm per head (`qk_norm_eps`; weights of the head size, shared by the heads) before the rotation;
    * `rotary`: any `RotaryTable` (partial rotation, pairs in halves or interleaved);
    * score = q . k * scale * temp[head], `temp` a learned number per head (of either sign: it is multiplied into q as q is
      written, in 32-bit);
    * `chunk` n > 0: position i sees j <= i with floor(i / n) = floor(j / n), chunks counted from position 0 of the
      sequence (0: every j <= i); `window` as in `GQAAttention`, on top of it;
    * softmax per head over the visible keys; then W'_h = sum_g talk[h, g] W_g (`talk` [H, H]), and head h applies W'_h to
      the values of its own key/value head; values may have another head size than keys.

    The mix is linear, so the kernels apply every head's softmax to the values of every key/value head in one pass over
    the keys and mix the results (`ops.attention_talk_plain`, `ops.talk_mix`); the cache manager gives back the pages that
    lie before the chunk of the next position."""
    graph_safe = True

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: Optional[int],
                 rotary: Optional[RotaryTable], names: Dict[str, str], chunk: int = 0, window: int = 0,
                 scale: Optional[float] = None, qk_norm_eps: float = 1e-6):
        super().__init__(names)
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} query heads cannot share {n_kv_heads} key/value heads")
        self.dim, self.H, self.KV, self.dk = dim, n_heads, n_kv_heads, head_dim
        self.dv = head_dim if v_head_dim is None else int(v_head_dim)
        self.rotary = rotary if rotary is not None else RotaryTable(head_dim, 10000.0, n_rot=0)
        self.chunk, self.window = int(chunk), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qk_norm_eps = float(qk_norm_eps)
        self.off_k = self.H * self.dk
        self.off_v = self.off_k + self.KV * self.dk
        self.w_in = self.wo = self.q_norm = self.k_norm = self.talk = self.temp = None

    def local_specs(self):
        return {"wq": TensorSpec((self.H * self.dk, self.dim), MATRIX), "wk": TensorSpec((self.KV * self.dk, self.dim), MATRIX),
                "wv": TensorSpec((self.KV * self.dv, self.dim), MATRIX), "wo": TensorSpec((self.dim, self.H * self.dv), MATRIX),
                "q_norm": TensorSpec((self.dk,), NORM), "k_norm": TensorSpec((self.dk,), NORM),
                "talk": TensorSpec((self.H, self.H), MATRIX), "temp": TensorSpec((self.H,), BIAS)}

    def place(self, local, dtype, device):
        self.w_in = to_device_matrix(torch.cat([local["wq"], local["wk"], local["wv"]], dim=0), dtype, device)
        self.wo = to_device_matrix(local["wo"], dtype, device)
        self.q_norm = to_device_vector(local["q_norm"], dtype, device)
        self.k_norm = to_device_vector(local["k_norm"], dtype, device)
        self.talk = local["talk"].to(device=device, dtype=torch.float32).contiguous()
        self.temp = local["temp"].to(device=device, dtype=torch.float32).contiguous()
        self.rotary.to(device)

    def cache_spec(self):
        return PagedKVSpec(self.KV, self.dk, self.window, 0 if self.dv == self.dk else self.dv, self.chunk)

    def plan_step(self, q_lens, ctx_lens, filler=None):
        return PLAN_KEY, attention_plan(q_lens, ctx_lens, filler)

    def attend(self, ctx, q, k_cache, v_cache, table, attn):
        """Every head's softmax over its chunk applied to the values of every key/value head, then the mix of the heads."""
        T = q.shape[0]
        # (the heads' factors on the scores are in q already; the tensor-core kernels want a positive scale)
        fast = (ctx.fast and self.dv == self.dk and self.scale > 0
                and ops.attention_mma_supported(q.dtype, self.dk, k_cache.shape[2]))
        if not fast:
            spread = ctx.empty((T, self.H, self.KV, self.dv), torch.float32)
            ops.attention_talk_plain(q, k_cache, v_cache, ctx.tok_req, ctx.cu_q, ctx.ctx_len, table, spread, self.H, self.chunk,
                                     self.window, self.scale, None)
            ops.talk_mix(spread, self.talk, attn)
            return
        plan = ctx.plans.get(PLAN_KEY)
        if plan is None:                                 # a step put together without asking the parts: plan it now
            plan = attention_plan(ctx.q_lens, ctx.ctx_lens)
            plan.arrays = {k: torch.from_numpy(v).to(ctx.device) for k, v in plan.arrays.items()}
            ctx.plans[PLAN_KEY] = plan
        tiles64, singles = plan.arrays["tiles64"], plan.arrays["singles"]
        spread = ctx.empty((T, self.H, self.KV, self.dv))
        if tiles64.shape[0]:
            ops.attention_prefill_talk(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, tiles64, spread, self.H, self.chunk,
                                       self.window, self.scale, None)
        n = singles.shape[0]
        if n:
            longest = plan.host["longest_single"]
            for bound in (self.chunk, self.window + 64 if self.window > 0 else 0):
                if bound > 0:
                    longest = min(longest, bound)
            groups = self.KV * (-(-(self.H // self.KV) // 16))
            resident = ops.attention_decode_resident_blocks(self.dk)
            n_splits = max(1, min(-(-longest // 64), resident // (n * groups), DECODE_MAX_SPLITS))
            ops.attention_decode_talk(q, k_cache, v_cache, ctx.cu_q, ctx.ctx_len, table, singles, n_splits, spread, self.H,
                                      self.chunk, self.window, self.scale, None)
        ops.talk_mix(spread, self.talk, attn)

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        T = h.shape[0]
        k_cache, v_cache, table = ctx.kv(cache_layer)
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        self._joined(proj)
        q = ctx.empty((T, self.H * self.dk))
        ops.qk_head_norm_rope_write(proj, self.off_k, self.off_v, self.q_norm, self.k_norm, self.qk_norm_eps, ctx.positions,
                                    ctx.tok_req, table, self.rotary.inv_freq, self.rotary.rot_half, self.rotary.pair_layout, q,
                                    k_cache if write_cache else None, v_cache if write_cache else None, self.H, self.KV,
                                    self.dk, self.dv, q_head_scale=self.temp)
        attn = ctx.empty((T, self.H * self.dv))
        self.attend(ctx, q, k_cache, v_cache, table, attn)
        linear(ctx, attn, self.wo, out, None, epilogue)

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        self._run(ctx, h, residual, cache_layer, write_cache, EPI_RESIDUAL)

    def mix(self, ctx, h, out, cache_layer, write_cache=True):
        self._run(ctx, h, out, cache_layer, write_cache, EPI_NONE)


class ParallelMixers(Mixer):
    """Two mixers side by side that read the same rows. Each mixer keeps its own cache, so this part's `cache_spec()` is the
    pair of theirs and it is handed a pair of cache layers. How the two results join is `combine`:

    * "rms_mean" (the default): the mean of the two, each RMS-normed over the model width first with a plain weight of its
      own: (rms_norm(left(h)) * left_out + rms_norm(right(h)) * right_out) / 2. A block that adds the result to the stream
      through a norm can take the two results as they are (`mix_pair`) and do the means in the kernel that adds.
    * "weighted": left_scale * left(h) + right_scale * right(h) with two constants (`scales`), no tensors of its own; it can
      add into a stream (`forward`)."""

    def __init__(self, dim: int, left: Mixer, right: Mixer, norm_eps: float = 0.0, names: Optional[Dict[str, str]] = None,
                 combine: str = "rms_mean", scales=(1.0, 1.0)):
        super().__init__(names)
        if combine not in ("rms_mean", "weighted"):
            raise ValueError(f"ParallelMixers: combine must be 'rms_mean' or 'weighted', got {combine!r}")
        self.dim, self.left, self.right, self.eps = dim, left, right, float(norm_eps)
        self.combine, self.scales = combine, (float(scales[0]), float(scales[1]))
        self.left_out = self.right_out = None

    def children(self):
        return (self.left, self.right)

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def local_specs(self):
        if self.combine == "weighted":
            return {}
        return {"left_out": TensorSpec((self.dim,), NORM), "right_out": TensorSpec((self.dim,), NORM)}

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def mix_pair(self, ctx, h, a, b, cache_layers, write_cache=True) -> None:
        """a = left(h), b = right(h), both 32-bit [T, dim]."""
        rows32 = ctx.memo.get(("rows32", id(h)))
        self.left.mix(ctx, h, a, cache_layers[0], write_cache)
        if rows32 is not None:
            ctx.memo[("rows32", id(h))] = rows32
        self.right.mix(ctx, h, b, cache_layers[1], write_cache)

    def mix(self, ctx, h, out, cache_layers, write_cache=True) -> None:
        a = ctx.empty(tuple(out.shape), torch.float32)
        b = ctx.empty(tuple(out.shape), torch.float32)
        self.mix_pair(ctx, h, a, b, cache_layers, write_cache)
        if self.combine == "weighted":
            out.zero_()
            ops.add_scaled_pair(out, a, self.scales[0], b, self.scales[1])
            return
        ops.pair_rms_mean(a, self.left_out, b, self.right_out, self.eps, out)

    def forward(self, ctx, h, residual, cache_layers, write_cache=True) -> None:
        if self.combine != "weighted":
            raise NotImplementedError("ParallelMixers with the normed mean writes its result (`mix`); blocks that add a mixer's result unchanged do not use it")
        a = ctx.empty(tuple(residual.shape), torch.float32)
        b = ctx.empty(tuple(residual.shape), torch.float32)
        after, ctx.next_norm = ctx.next_norm, None       # the two results are not the stream: neither product may begin a norm
        self.mix_pair(ctx, h, a, b, cache_layers, write_cache)
        ctx.next_norm = after
        ops.add_scaled_pair(residual, a, self.scales[0], b, self.scales[1])
