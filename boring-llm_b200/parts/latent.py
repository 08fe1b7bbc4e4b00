"""Attention over one cached latent per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import PagedKVSpec
from ..kernels import ops
from ..weights import TensorSpec, MATRIX, BIAS, NORM
from .attention import Mixer, PLAN_KEY, attention_plan
from .base import to_device_matrix, to_device_vector
from .linear import linear, EPI_NONE, EPI_RESIDUAL
from .rotary import RotaryTable


class LatentAttention(Mixer):
    """Multi-head attention whose keys and values are made from a small vector per token:

    * queries pass through a latent: cq = RMSnorm(h Wdq^T) * dq_norm, q = cq Wuq^T, per head `nope_dim` values that are
      not rotated followed by `rot_dim` rotated ones;
    * h Wdkv^T has kv_rank + rot_dim values: the first kv_rank, RMS-normed with `dkv_norm`, are the latent c; the rest,
      rotated by the position, are a key part that all heads share. Head h's key is [Uk_h c | shared part], its value
      Uv_h c (`wuk` [H * nope_dim, kv_rank], `wuv` [H * v_dim, kv_rank], head by head);
    * score = (q_nope . k_nope + q_rot . k_rot) * scale; `window` n > 0: position i sees j with 0 <= i - j < n;
      `sink=True`: exp(sink_h) joins head h's softmax denominator once, unscaled, with no value;
    * `out_gate=True`: the concatenated heads are multiplied by sigmoid(h Wg^T), one number per channel;
    * `own_kv=False`: the mixer has no Wdkv and reads the latent and rotated part that another layer cached (its run-order
      entry names that cache layer with `write_cache=False`); `cache_window` is then what the owner and all its readers
      agree the cache keeps (the widest of their windows, 0 if any sees everything).

    Only [c | rotated part] is cached (one row of kv_rank + rot_dim values per token, `values_in_keys`). The products with
    Uk and Uv are moved to the query's side, q' = Uk_h^T q_nope and out_h = Uv_h (sum_j p_j c_j), so every head of every
    token reads the same cached rows. All of the mixer's first products (Wdq, Wdkv, Wg) are ONE joined product with
    32-bit sums; both norms, the rotation and the cache write are one kernel; the gate is applied where the product with
    Uv is read. Norms, angles, scores and the softmax are 32-bit.

    In bfloat16 (and where the sizes allow: pages of 16, kv_rank, rot_dim and nope_dim multiples of 8, kv_rank <= 512) the
    part between the two joined products runs head-major: queries, attention results and the products with Uk and Uv
    lie as [H, Tp, .] with Tp the step's rows rounded up to 128, so that each of the two per-head products is ONE grouped
    tensor-core product whose tiles take the matrix of their head, and the attention kernel (`ops.latent_attention_mma`)
    reads and writes that layout. Otherwise, and always in float32, the plain kernels run on token rows.
    """
    graph_safe = True

    def __init__(self, dim: int, n_heads: int, nope_dim: int, rot_dim: int, v_dim: int, q_rank: int, kv_rank: int,
                 rotary: Optional[RotaryTable], names: Dict[str, str], window: int = 0, scale: Optional[float] = None,
                 norm_eps: float = 1e-6, sink: bool = False, out_gate: bool = False, own_kv: bool = True,
                 cache_window: Optional[int] = None):
        super().__init__(names)
        self.dim, self.H, self.dn, self.dr, self.dv = dim, n_heads, nope_dim, rot_dim, v_dim
        self.q_rank, self.rank = q_rank, kv_rank
        self.rotary = rotary if rotary is not None else RotaryTable(max(rot_dim, 2), 10000.0, n_rot=0)
        if self.rotary.pairs != "halves" or 2 * self.rotary.rot_half > rot_dim:
            raise ValueError(f"LatentAttention: the rotation ({self.rotary.n_rot} values in {self.rotary.pairs}) does not fit a rotated part of {rot_dim}")
        self.window = int(window)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window != 0 and (self.window == 0 or self.window > self.cache_window):
            raise ValueError(f"LatentAttention: a window of {self.window} over a cache that keeps {self.cache_window}")
        self.scale = float(scale) if scale is not None else float(nope_dim + rot_dim) ** -0.5
        self.eps, self.has_sink, self.out_gate, self.own_kv = float(norm_eps), bool(sink), bool(out_gate), bool(own_kv)
        pad = lambda n: -(-n // 8) * 8              # every part of the joined product starts on a 32-byte boundary of the sums
        self.off_kv = pad(q_rank)
        self.off_g = self.off_kv + (pad(kv_rank + rot_dim) if self.own_kv else 0)
        self.n_in = self.off_g + (n_heads * v_dim if self.out_gate else 0)
        self.w_in = self.wuq = self.wuk = self.wuv = self.wo = self.dq_norm = self.dkv_norm = self.sinks = None

    def local_specs(self):
        s = {"wdq": TensorSpec((self.q_rank, self.dim), MATRIX), "dq_norm": TensorSpec((self.q_rank,), NORM),
             "wuq": TensorSpec((self.H * (self.dn + self.dr), self.q_rank), MATRIX),
             "wuk": TensorSpec((self.H * self.dn, self.rank), MATRIX), "wuv": TensorSpec((self.H * self.dv, self.rank), MATRIX),
             "wo": TensorSpec((self.dim, self.H * self.dv), MATRIX)}
        if self.own_kv:
            s["wdkv"] = TensorSpec((self.rank + self.dr, self.dim), MATRIX)
            s["dkv_norm"] = TensorSpec((self.rank,), NORM)
        if self.has_sink:
            s["sink"] = TensorSpec((self.H,), BIAS)
        if self.out_gate:
            s["wg"] = TensorSpec((self.H * self.dv, self.dim), MATRIX)
        return s

    def place(self, local, dtype, device):
        w_in = torch.zeros((self.n_in, self.dim), dtype=local["wdq"].dtype)
        w_in[:self.q_rank] = local["wdq"]
        if self.own_kv:
            w_in[self.off_kv:self.off_kv + self.rank + self.dr] = local["wdkv"]
            self.dkv_norm = to_device_vector(local["dkv_norm"], dtype, device)
        if self.out_gate:
            w_in[self.off_g:] = local["wg"]
        self.w_in = to_device_matrix(w_in, dtype, device)
        self.dq_norm = to_device_vector(local["dq_norm"], dtype, device)
        self.wuq = to_device_matrix(local["wuq"], dtype, device)
        self.wuk = to_device_matrix(local["wuk"], dtype, device)              # [H * nope_dim, kv_rank] as stored
        # Uk_h^T stacked [H, kv_rank, nope_dim]: the matrices of the grouped product that moves the queries into the latent's space
        self.wuk_t = to_device_matrix(local["wuk"].view(self.H, self.dn, self.rank).transpose(1, 2).contiguous(), dtype, device)
        self.wuv = to_device_matrix(local["wuv"], dtype, device)              # [H * v_dim, kv_rank] as stored
        self.wo = to_device_matrix(local["wo"], dtype, device)
        if self.has_sink:
            self.sinks = to_device_vector(local["sink"], dtype, device)
        self.rotary.to(device)

    def cache_spec(self):
        return PagedKVSpec(1, self.rank + self.dr, self.cache_window, self.rank, values_in_keys=True)

    def takes_pending_norm_at(self, rows: int) -> bool:
        """The joined first product finishes an RMS norm that the product before has begun where it runs on the
        register-streaming kernel (a decode step's 2 to 16 rows); elsewhere the product before need not begin one."""
        return (ops.SKINNY_LINK_MIN_ROWS <= rows <= ops.SKINNY_LINK_MAX_ROWS and self.w_in is not None
                and self.w_in.dtype == torch.bfloat16 and -(-self.n_in // 16) <= ops.SKINNY_LINK_MAX_BLOCKS
                and not ops.gemm_streams_better(self.w_in))

    def plan_step(self, q_lens, ctx_lens, filler=None):
        return PLAN_KEY, attention_plan(q_lens, ctx_lens, filler)

    # -- the steps of a pass, each one kernel or product ----------------------------------------------------------------
    def absorbed_queries(self, ctx, cq):
        """[T, H, kv_rank + rot_dim]: per head Uk_h^T q_nope, then the rotated part of q."""
        T = cq.shape[0]
        q = ctx.empty((T, self.H * (self.dn + self.dr)), torch.float32)
        linear(ctx, cq, self.wuq, q, None, EPI_NONE)
        q3 = q.view(T, self.H, self.dn + self.dr)
        qa = ctx.empty((T, self.H, self.rank + self.dr))
        uk_t = self.wuk.view(self.H, self.dn, self.rank).transpose(1, 2)      # [H, kv_rank, nope_dim]: Uk_h^T as it lies
        ops.head_gemm_plain(q3[:, :, :self.dn], uk_t, qa[:, :, :self.rank])
        ops.rope_heads(q3[:, :, self.dn:], ctx.positions, self.rotary.inv_freq, self.rotary.rot_half, self.rotary.mscale,
                       qa[:, :, self.rank:])
        return qa

    def attend(self, ctx, qa, cache, table, out):
        ops.latent_attention_plain(qa, cache, ctx.tok_req, ctx.cu_q, ctx.ctx_len, table, out, self.window, self.scale, self.sinks)

    def head_major(self, ctx, cache) -> bool:
        """Whether this step runs on the tensor-core kernels in the head-major layout."""
        return bool(ctx.fast and self.dn % 8 == 0 and ops.latent_attention_mma_supported(cache.dtype, self.rank, self.dr, cache.shape[2]))

    def _attend_head_major(self, ctx, cq, cache, table, gate, heads):
        """heads [T, H * v_dim] from the normed query latent cq, over the cached rows, everything in between head-major."""
        T, H = cq.shape[0], self.H
        Tp = -(-T // ops.GROUPED_TILE) * ops.GROUPED_TILE
        key = ("head tiles", H, Tp)
        if key not in ctx.memo:                       # the same list for every layer of the step with as many heads
            ctx.memo[key] = ops.head_tiles(H, Tp // ops.GROUPED_TILE, ctx.device)
        tile_head = ctx.memo[key]
        q = ctx.empty((T, H * (self.dn + self.dr)), torch.float32)
        linear(ctx, cq, self.wuq, q, None, EPI_NONE)
        q3 = q.view(T, H, self.dn + self.dr)
        qn = ctx.empty((H, Tp, self.dn))
        q_rot = None
        if self.dr:                                   # one launch: the rotated part rotated, the other part cast, both head-major
            q_rot = ctx.empty((H, Tp, self.dr))
            ops.rope_heads(q3[:, :, self.dn:], ctx.positions, self.rotary.inv_freq, self.rotary.rot_half, self.rotary.mscale,
                           q_rot.transpose(0, 1)[:T], lead=q3[:, :, :self.dn], lead_out=qn.transpose(0, 1)[:T])
        else:
            ops.rope_heads(q3[:, :, :self.dn], ctx.positions, self.rotary.inv_freq, 0, 1.0, qn.transpose(0, 1)[:T])     # a cast
        q_lat = ctx.empty((H, Tp, self.rank))
        ops.gemm_grouped(qn.view(H * Tp, self.dn), self.wuk_t, tile_head, q_lat.view(H * Tp, self.rank), EPI_NONE)
        lat = ctx.empty((H, Tp, self.rank))
        plan = ctx.plans.get(PLAN_KEY)
        if plan is None:                              # a step put together without asking the parts: plan it now
            plan = attention_plan(ctx.q_lens, ctx.ctx_lens)
            plan.arrays = {k: torch.from_numpy(v).to(ctx.device) for k, v in plan.arrays.items()}
            ctx.plans[PLAN_KEY] = plan
        longest = plan.host["longest_single"]
        if self.window > 0:
            longest = min(longest, self.window + 64)
        for work, single in ((plan.arrays["tiles64"], False), (plan.arrays["singles"], True)):
            if work.shape[0]:
                splits = ops.latent_attention_splits(work.shape[0], H, longest) if single else 1
                ops.latent_attention_mma(q_lat, q_rot, cache, ctx.cu_q, ctx.ctx_len, table, work, single, lat, self.window, self.scale,
                                         self.sinks, splits)
        hv = ctx.empty((H, Tp, self.dv), torch.float32)
        ops.gemm_grouped(lat.view(H * Tp, self.rank), self.wuv.view(H, self.dv, self.rank), tile_head, hv.view(H * Tp, self.dv), EPI_NONE)
        ops.heads_gate_rows(hv, gate, heads)

    def _run(self, ctx, h, out, cache_layer, write_cache, epilogue):
        T = h.shape[0]
        if write_cache != self.own_kv:
            raise ValueError("LatentAttention: a mixer with a Wdkv of its own writes its cache layer, one without reads another's")
        cache, _, table = ctx.kv(cache_layer)
        proj = ctx.empty((T, self.n_in), torch.float32)
        linear(ctx, h, self.w_in, proj, None, EPI_NONE)
        cq = ctx.empty((T, self.q_rank))
        ops.latent_prep(proj, 0, self.q_rank, self.off_kv, self.rank, self.dr, self.rotary.rot_half, self.dq_norm, self.dkv_norm,
                        self.eps, ctx.positions, ctx.tok_req, table, self.rotary.inv_freq, self.rotary.mscale, cq,
                        cache if write_cache else None)
        if self.head_major(ctx, cache):
            heads = ctx.empty((T, self.H * self.dv))
            self._attend_head_major(ctx, cq, cache, table, proj[:, self.off_g:] if self.out_gate else None, heads)
            linear(ctx, heads, self.wo, out, None, epilogue)
            return
        qa = self.absorbed_queries(ctx, cq)
        lat = ctx.empty((T, self.H, self.rank))
        self.attend(ctx, qa, cache, table, lat)
        heads = ctx.empty((T, self.H * self.dv))
        ops.head_gemm_plain(lat, self.wuv.view(self.H, self.dv, self.rank), heads.view(T, self.H, self.dv),
                            proj[:, self.off_g:] if self.out_gate else None)
        linear(ctx, heads, self.wo, out, None, epilogue)

    def forward(self, ctx, h, residual, cache_layer, write_cache=True):
        self._run(ctx, h, residual, cache_layer, write_cache, EPI_RESIDUAL)

    def mix(self, ctx, h, out, cache_layer, write_cache=True):
        self._run(ctx, h, out, cache_layer, write_cache, EPI_NONE)
