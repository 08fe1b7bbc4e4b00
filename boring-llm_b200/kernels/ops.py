"""Typed Python front of the kernel library: every function takes torch CUDA tensors, checks what
the C side cannot see (devices, dtypes, shapes, contiguity) and launches on torch's current stream.
Nothing here computes on the CPU or through a library model: without the built library and an
sm_100a device these functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library

F32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
PAIRS_HALVES, PAIRS_INTERLEAVED = 0, 1

_checked_device = False


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported tensor dtype {t.dtype}: kernels take float32 or bfloat16")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """torch's current stream as a pointer. The two C entry points cost a fraction of a microsecond; a step of
    the engine asks hundreds of times, and `torch.cuda.current_stream()` builds a Python object each time."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_ready = None             # the library, once the device has been checked


def _lib():
    global _checked_device, _ready
    if _ready is not None:
        return _ready
    lib = library.load()
    if not _checked_device:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on an sm_100a GPU only (there is no CPU path)")
        if lib.bl_device_check() != 0:
            raise KernelError(lib.bl_last_error().decode())
        _checked_device = True
    _ready = lib
    return lib


launch_count = 0          # kernels launched through this module since import (the benchmark reads it)


_trace = None             # a StepTrace while one is recording


def _call(fn, *args):
    global launch_count
    launch_count += 1
    if fn(*args) != 0:
        raise KernelError(library.load().bl_last_error().decode())
    if _trace is not None and fn.__name__ != "bl_stamp":
        _trace.after(fn.__name__)


class StepTrace:
    """Time line of the kernels launched while it records: a time stamp kernel goes between every two of them
    (also inside a CUDA graph that is being captured), and `durations()` turns the stamps of the last run or
    replay into (kernel, microseconds) pairs. Stamps serialise the kernels, so overlap between neighbours
    (programmatic dependent launch) is not in these figures: they are each kernel's own time in place."""

    def __init__(self, device, capacity: int = 4096):
        self.buf = torch.zeros(capacity, dtype=torch.int64, device=device)
        self.names = []

    def __enter__(self):
        global _trace
        _trace = self
        self.names = []
        _call(_lib().bl_stamp, ctypes.c_void_p(self.buf.data_ptr()), 0, _stream())
        return self

    def __exit__(self, *exc):
        global _trace
        _trace = None

    def after(self, name: str) -> None:
        self.names.append(name)
        if len(self.names) < self.buf.numel():
            library.load().bl_stamp(ctypes.c_void_p(self.buf.data_ptr()), len(self.names), _stream())

    def durations(self):
        torch.cuda.synchronize()
        t = self.buf[:len(self.names) + 1].cpu().tolist()
        return [(n, (t[i + 1] - t[i]) / 1000.0) for i, n in enumerate(self.names)]


def _need(t: torch.Tensor, name: str, dtype=None, shape=None):
    if not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name}: must have shape {tuple(shape)}, got {tuple(t.shape)}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] widened to 32-bit (times `scale`). The caller has checked that ids lie inside the table."""
    T = ids.shape[0]
    V, d = table.shape
    _need(table, "table"); _need(ids, "ids", torch.int32, (T,)); _need(out, "out", torch.float32, (T, d))
    if scale == 1.0:
        _call(_lib().bl_embed, _p(table), _dt(table), _p(ids), _p(out), T, d, V, _stream())
    else:
        _call(_lib().bl_embed_scaled, _p(table), _dt(table), _p(ids), _p(out), T, d, V, ctypes.c_float(scale), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_idx: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[row_idx[r]] if row_idx is given else x[r]) * weight."""
    d = x.shape[1]
    rows = out.shape[0]
    _need(x, "x", torch.float32); _need(weight, "weight", None, (d,)); _need(out, "out", None, (rows, d))
    if row_idx is not None:
        _need(row_idx, "row_idx", torch.int32, (rows,))
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call(_lib().bl_rmsnorm, _p(x), _p(row_idx), _p(weight), _dt(weight), _p(out), _dt(out),
          rows, d, ctypes.c_float(eps), _stream())


def add_row_vector(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[r] += v for every row of the 32-bit residual stream."""
    rows, d = x.shape
    _need(x, "x", torch.float32); _need(v, "v", None, (d,))
    _call(_lib().bl_add_row_vector, _p(x), _p(v), _dt(v), rows, d, _stream())


def glu_args(kind: int, limit: float, device) -> Optional[torch.Tensor]:
    """What a product with the gated epilogue (EPI_SWIGLU) takes in the place of a bias to compute another gated activation
    than SiLU: the two 32-bit numbers {kind, limit} on the device (GLU_GELU_TANH, GLU_CLAMPED with its limit). None for SiLU."""
    if kind == GLU_SILU:
        return None
    if kind not in (GLU_GELU_TANH, GLU_CLAMPED):
        raise KernelError(f"glu_args: unknown gated activation {kind}")
    return torch.tensor([float(kind), float(limit)], dtype=torch.float32, device=device)


def _need_bias(bias: torch.Tensor, N: int, epilogue: int) -> None:
    """A bias of N values; with the gated epilogue, which adds none, the two numbers of `glu_args`."""
    if epilogue == EPI_SWIGLU:
        _need(bias, "activation", torch.float32, (2,))
    else:
        _need(bias, "bias", None, (N,))


def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
               epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) on CUDA cores with 32-bit accumulation. x may be a range of columns of a wider
    row-major matrix (its rows `x.stride(0)` values apart)."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    if not x.is_cuda or x.stride(1) != 1 or x.stride(0) < K:
        raise KernelError("x: must be a CUDA matrix whose rows are contiguous")
    _need(w, "w", None, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need_bias(bias, N, epilogue)
    _call(_lib().bl_gemm_plain_ld, _p(x), _dt(x), x.stride(0), _p(w), _dt(w), _p(bias), _dt(bias) if bias is not None else 0,
          _p(out), _dt(out), M, N, K, epilogue, _stream())


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                  block_table: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, mscale: float,
                  q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  H: int, KV: int, dh: int, pair_layout: int = 0) -> None:
    """Rotates q and k of joined [q | k | v] rows and writes k, v into the request's pages. `pair_layout`: which
    dimensions turn together, PAIRS_HALVES (j, j + rot_half) or PAIRS_INTERLEAVED (2j, 2j + 1)."""
    T = qkv.shape[0]
    _need(qkv, "qkv", torch.float32, (T, (H + 2 * KV) * dh))
    _need(positions, "positions", torch.int32, (T,)); _need(tok_req, "tok_req", torch.int32, (T,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32, (dh // 2,))
    _need(q_out, "q_out", None, (T, H * dh))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_rope_kv_write, _p(qkv), _p(positions), _p(tok_req), _p(block_table),
          block_table.shape[1], _p(inv_freq), rot_half, ctypes.c_float(mscale), _p(q_out), _p(k_cache),
          _p(v_cache), _dt(q_out), T, H, KV, dh, page_size, pair_layout, _stream())


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, mscale: float):
    """(cos, sin) of every token's rotation, float32 [T, rot_half] each, scaled by `mscale`: worked out once per step
    for the kernels that take the rotation from a table."""
    T = positions.shape[0]
    _need(positions, "positions", torch.int32, (T,)); _need(inv_freq, "inv_freq", torch.float32)
    both = torch.empty((2, T, rot_half), dtype=torch.float32, device=positions.device)
    _call(_lib().bl_rope_table, _p(positions), _p(inv_freq), rot_half, ctypes.c_float(mscale), _p(both[0]), _p(both[1]), T, _stream())
    return both[0], both[1]


def qkv_rope_tc_supported(x: torch.Tensor, w: torch.Tensor, H: int, KV: int, dh: int, page_size: int) -> bool:
    """Whether `qkv_rope_tc` takes this layer's joined product: bfloat16 operands, 16-byte aligned, head size 64 or
    128 with every pair of a head rotated, pages of 16."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library.load().bl_gemm_tc_pair_qkv_rope_supported(H, KV, dh, page_size, x.shape[1])))


def qkv_rope_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                tok_req: torch.Tensor, block_table: torch.Tensor, cs: torch.Tensor, sn: torch.Tensor, q_out: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], H: int, KV: int, dh: int,
                row_sums: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """The joined q/k/v product of many rows on pairs of SMs (tcgen05) with bias, rotation (pairs j, j + dh / 2, from
    the step's table `rope_table`) and the writes of q and of k and v into the requests' pages in its epilogue.
    `row_sums` (with `eps`): x holds rows whose RMS norm is pending (`gemm_residual_norm`); the product's rows are
    scaled by 1 / sqrt(row_sums[m].sum() / K + eps) before the bias."""
    M, K = x.shape
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, ((H + 2 * KV) * dh, K))
    _need(positions, "positions", torch.int32, (M,)); _need(tok_req, "tok_req", torch.int32, (M,))
    _need(block_table, "block_table", torch.int32)
    _need(cs, "cs", torch.float32, (M, dh // 2)); _need(sn, "sn", torch.float32, (M, dh // 2))
    _need(q_out, "q_out", torch.bfloat16, (M, H * dh))
    if bias is not None:
        _need(bias, "bias", None, ((H + 2 * KV) * dh,))
    page_size = 16
    if k_cache is not None:
        _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_gemm_tc_pair_qkv_rope, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, M, K, _p(tok_req),
          _p(positions), _p(block_table), block_table.shape[1], _p(cs), _p(sn), _p(q_out), _p(k_cache), _p(v_cache),
          H, KV, dh, page_size, _p(row_sums), 0 if row_sums is None else row_sums.shape[1], ctypes.c_float(1.0 / K),
          ctypes.c_float(eps), _stream())


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_req: torch.Tensor,
                    cu_q: torch.Tensor, ctx_len: torch.Tensor, block_table: torch.Tensor,
                    out: torch.Tensor, H: int, window: int, scale: float, sinks: Optional[torch.Tensor] = None,
                    gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Paged causal grouped-query attention, one warp per (token, head). `softcap` c > 0: the scaled scores pass
    c * tanh(s / c) before the softmax. The values' head size may differ from the
    keys' (v_cache `[pages, kv heads, page, dv]`, out `[T, H * dv]`). `sinks` [H]: exp(sinks[h]) joins head h's softmax
    denominator (once, unscaled, no value). `gate` (32-bit, [T, >= H], rows contiguous, possibly a column range of a
    wider matrix): head h of token t is multiplied by sigmoid(gate[t, h])."""
    T = q.shape[0]
    n_pages, KV, page_size, dh = k_cache.shape
    dv = v_cache.shape[3]
    _need(q, "q", k_cache.dtype, (T, H * dh)); _need(k_cache, "k_cache")
    _need(v_cache, "v_cache", k_cache.dtype, (n_pages, KV, page_size, dv))
    _need(tok_req, "tok_req", torch.int32, (T,)); _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32)
    _need(block_table, "block_table", torch.int32); _need(out, "out", q.dtype, (T, H * dv))
    if sinks is not None:
        _need(sinks, "sinks", None, (H,))
    ld_gate = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < H:
            raise KernelError("gate: must be 32-bit CUDA rows [T, >= H] with contiguous rows")
        ld_gate = gate.stride(0)
    _call(_lib().bl_attention_plain_cap, _p(q), _p(k_cache), _p(v_cache), _dt(q), _p(tok_req), _p(cu_q),
          _p(ctx_len), _p(block_table), block_table.shape[1], _p(out), T, H, KV, dh, dv, page_size, window,
          ctypes.c_float(scale), _p(sinks), _dt(sinks) if sinks is not None else 0, _p(gate), ld_gate, ctypes.c_float(softcap),
          _stream())


def argmax(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    rows, V = logits.shape
    _need(logits, "logits", torch.float32); _need(out_ids, "out_ids", torch.int32, (rows,))
    _call(_lib().bl_argmax, _p(logits), _p(out_ids), rows, V, _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out_ids: torch.Tensor) -> None:
    """One token per row: greedy where temperature <= 0, else temperature sampling after the top-k,
    top-p and min-p cuts, with the row's uniform random number."""
    rows, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(temperature, "temperature", torch.float32, (rows,)); _need(top_k, "top_k", torch.int32, (rows,))
    _need(top_p, "top_p", torch.float32, (rows,)); _need(min_p, "min_p", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,)); _need(out_ids, "out_ids", torch.int32, (rows,))
    _call(_lib().bl_sample, _p(logits), rows, V, _p(temperature), _p(top_k), _p(top_p), _p(min_p),
          _p(uniform), _p(out_ids), _stream())


def repeat_penalty(logits: torch.Tensor, tokens: torch.Tensor, offsets: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: logits[r, t] /= penalty[r] if positive else *= penalty[r], for the listed tokens of row r."""
    rows, V = logits.shape
    _need(logits, "logits", torch.float32); _need(tokens, "tokens", torch.int32)
    _need(offsets, "offsets", torch.int32, (rows + 1,)); _need(penalty, "penalty", torch.float32, (rows,))
    _call(_lib().bl_repeat_penalty, _p(logits), rows, V, _p(tokens), _p(offsets), _p(penalty), _stream())


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) for few rows: W streams once from HBM into tensor-core registers."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need_bias(bias, N, epilogue)
    _call(_lib().bl_gemm_skinny, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def _tail(T: int, H: int, sinks: Optional[torch.Tensor], gate: Optional[torch.Tensor]):
    """The arguments (sinks, their dtype, gate, its row stride) of the attention kernels' `_tail` entry points."""
    if sinks is not None:
        _need(sinks, "sinks", None, (H,))
    ld = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < H:
            raise KernelError("gate: must be 32-bit CUDA rows [T, >= H] with contiguous rows")
        ld = gate.stride(0)
    return _p(sinks), _dt(sinks) if sinks is not None else 0, _p(gate), ld


def attention_mma_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_mma_supported(dh, page_size))


def attention_prefill(q, k_cache, v_cache, cu_q, ctx_len, block_table, tiles, out, H: int, window: int,
                      scale: float, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      softcap: float = 0.0) -> None:
    """Tensor-core attention for requests with several new tokens. tiles: int32 [n, 2] = (request, first token
    of a 64-token tile among the request's new tokens). `softcap` c > 0: scaled scores pass c tanh(s / c)."""
    T = q.shape[0]
    _, KV, page_size, dh = k_cache.shape
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(tiles, "tiles", torch.int32)
    if softcap > 0:
        _call(_lib().bl_attention_prefill_cap, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), H, KV, dh, page_size, window,
          ctypes.c_float(scale), *_tail(T, H, sinks, gate), ctypes.c_float(softcap), _stream())
    elif sinks is None and gate is None:
        _call(_lib().bl_attention_prefill, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), H, KV, dh, page_size, window,
          ctypes.c_float(scale), _stream())
    else:
        _call(_lib().bl_attention_prefill_tail, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), H, KV, dh, page_size, window,
          ctypes.c_float(scale), *_tail(T, H, sinks, gate), _stream())


def attention_prefill_tc_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_prefill_tc_supported(dh, page_size))


def attention_prefill_tc(q, k_cache, v_cache, cu_q, ctx_len, block_table, tiles, out, H: int, window: int,
                         scale: float, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                         softcap: float = 0.0) -> None:
    """The tcgen05 form of `attention_prefill` (head size 64, pages of 16). tiles: int32 [n, 2] = (request,
    first token of a tile of 128 among the request's new tokens); the last entries are launched first. `softcap` c > 0:
    scaled scores pass c tanh(s / c) (a second build of the kernel; without a cap the kernel is the one it was)."""
    T = q.shape[0]
    n_pages, KV, page_size, dh = k_cache.shape
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(tiles, "tiles", torch.int32, (tiles.shape[0], 2))
    if softcap > 0:
        _call(_lib().bl_attention_prefill_tc_cap, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), T, n_pages, H, KV, dh, page_size, window,
          ctypes.c_float(scale), *_tail(T, H, sinks, gate), ctypes.c_float(softcap), _stream())
    elif sinks is None and gate is None:
        _call(_lib().bl_attention_prefill_tc, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), T, n_pages, H, KV, dh, page_size, window,
          ctypes.c_float(scale), _stream())
    else:
        _call(_lib().bl_attention_prefill_tc_tail, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(tiles), tiles.shape[0], _p(out), T, n_pages, H, KV, dh, page_size, window,
          ctypes.c_float(scale), *_tail(T, H, sinks, gate), _stream())


DECODE_CLUSTER_SPLITS = 16     # up to this many slices merge through distributed shared memory (one cluster a request and head group)


def attention_decode(q, k_cache, v_cache, cu_q, ctx_len, block_table, reqs, n_splits: int, out, H: int, window: int,
                     scale: float, scratch: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Tensor-core attention for requests with one new token; `reqs` int32 [n] lists them. The keys of each are
    cut into `n_splits` slices. Up to `DECODE_CLUSTER_SPLITS` slices without `scratch`: the slices of a request are
    the blocks of a cluster and merge in shared memory. More slices, or a `scratch` tensor (float32,
    `attention_decode_scratch(...)` elements): the partial results go through scratch and the last block merges."""
    T = q.shape[0]
    _, KV, page_size, dh = k_cache.shape
    n = reqs.shape[0]
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(reqs, "reqs", torch.int32, (n,))
    need = attention_decode_scratch(n, H, dh, n_splits)
    if scratch is None and n_splits <= DECODE_CLUSTER_SPLITS:
        need = 0                               # the slices of a request form a cluster and merge in shared memory: no scratch
    if need:
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"scratch: {scratch.numel()} floats, {need} needed")
    counters = None
    if need:
        n_counters = n * KV * (-(-(H // KV) // 16))
        counters = _decode_counters.get(q.device)
        if counters is None or counters.numel() < n_counters:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("attention_decode: its counters must exist before a capture (run the step once first)")
            # zero once; every launch leaves them at zero again
            counters = _decode_counters[q.device] = torch.zeros(max(n_counters, 4096), dtype=torch.int32, device=q.device)
    if softcap > 0:
        _call(_lib().bl_attention_decode_cap, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(scratch if need else None), _p(counters), _p(out), H, KV, dh,
          page_size, window, ctypes.c_float(scale), *_tail(T, H, sinks, gate), ctypes.c_float(softcap), _stream())
    elif sinks is None and gate is None:
        _call(_lib().bl_attention_decode, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(scratch if need else None), _p(counters), _p(out), H, KV, dh,
          page_size, window, ctypes.c_float(scale), _stream())
    else:
        _call(_lib().bl_attention_decode_tail, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(scratch if need else None), _p(counters), _p(out), H, KV, dh,
          page_size, window, ctypes.c_float(scale), *_tail(T, H, sinks, gate), _stream())


def attention_decode_tma_supported(dtype: torch.dtype, dh: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(library.load().bl_attention_decode_tma_supported(dh, page_size))


def attention_decode_tma(q, k_cache, v_cache, cu_q, ctx_len, block_table, reqs, n_splits: int, out, H: int, window: int,
                         scale: float, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                         softcap: float = 0.0) -> None:
    """`attention_decode` for head sizes 64 and 128 with keys and values streamed by TMA into per-warp rings and the
    query heads of a key/value head as the columns of the MMAs; 1 to `DECODE_CLUSTER_SPLITS` slices, which are the
    blocks of one cluster and send their partial rows to the blocks that finish them."""
    T = q.shape[0]
    n_pages, KV, page_size, dh = k_cache.shape
    n = reqs.shape[0]
    _need(q, "q", torch.bfloat16, (T, H * dh)); _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape); _need(out, "out", torch.bfloat16, (T, H * dh))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(reqs, "reqs", torch.int32, (n,))
    # Large clusters of a launch with more blocks than SMs start only when the kernel before has finished: placed while
    # its blocks still hold SMs they pile up two to an SM beside empty SMs (measured at batch 8: 54 -> 44 us a layer at
    # 32,000 tokens, 81 -> 62 at 64,000; small launches gain 2.5 us a layer from the early start)
    G = H // KV
    blocks = n * KV * (-(-G // (8 if G <= 8 else 16))) * n_splits
    early = not (n_splits >= DECODE_TMA_LATE_CLUSTER and blocks > _sms())
    if softcap > 0:                          # a cap on the scaled scores: a second build of the kernel
        _call(_lib().bl_attention_decode_tma_cap, _p(q), _p(k_cache), _p(v_cache), n_pages, _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(out), H, KV, dh, page_size, window, ctypes.c_float(scale),
          1 if early else 0, *_tail(T, H, sinks, gate), ctypes.c_float(softcap), _stream())
    elif sinks is None and gate is None:
        _call(_lib().bl_attention_decode_tma, _p(q), _p(k_cache), _p(v_cache), n_pages, _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(out), H, KV, dh, page_size, window, ctypes.c_float(scale),
          1 if early else 0, _stream())
    else:
        _call(_lib().bl_attention_decode_tma_tail, _p(q), _p(k_cache), _p(v_cache), n_pages, _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(reqs), n, n_splits, _p(out), H, KV, dh, page_size, window, ctypes.c_float(scale),
          1 if early else 0, *_tail(T, H, sinks, gate), _stream())


def attention_decode_tma_resident_blocks(dh: int, heads_per_kv: int) -> int:
    """Blocks of `attention_decode_tma` that the device holds at once (the kernel's own occupancy, asked once)."""
    key = (torch.cuda.current_device(), dh, heads_per_kv > 8)
    if key not in _decode_tma_resident:
        _decode_tma_resident[key] = max(1, int(_lib().bl_attention_decode_tma_resident_blocks(dh, heads_per_kv)))
    return _decode_tma_resident[key]


_decode_tma_resident = {}
_decode_tma_clusters = {}
_sm_count = {}
DECODE_TMA_LATE_CLUSTER = 8           # clusters from this size on, in launches of more blocks than SMs, are launched late


def _sms() -> int:
    dev = torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]

DECODE_TMA_UNIT = 32                  # keys a warp of `attention_decode_tma` takes at a time
DECODE_TMA_MIN_UNITS = 4              # a slice is worth a block from four units on (one for each warp)
DECODE_TMA_FEW_UNITS = 12             # up to this many units a warp, one block an SM is best: it may start under its predecessor (measured inside a layer's chain of kernels: 8 requests of 8,000 tokens 27.1 us a layer against 29.5, of 16,000 33.0 against 34.7; 32 requests of 3,900 want four slices)


def attention_decode_tma_splits(n: int, KV: int, heads_per_kv: int, dh: int, longest: int) -> int:
    """Slices for `attention_decode_tma` with n requests whose longest context (or window) has `longest` keys.
    Measured on a B200: a launch should run in one round (more clusters than the device holds at once cost a second
    round), slices below 128 keys cost more than they save, and while a warp has only a few units to walk, one block
    per SM beats two (the step is a chain of latencies); with long walks two blocks per SM keep more bytes in
    flight. Among the slice counts that qualify, the smallest that gives a warp the fewest units."""
    dev = torch.cuda.current_device()
    sms = _sms()
    groups = KV * (-(-heads_per_kv // (8 if heads_per_kv <= 8 else 16)))
    clusters = n * groups
    units = -(-max(1, longest) // DECODE_TMA_UNIT)
    most = max(1, min(DECODE_CLUSTER_SPLITS, units // DECODE_TMA_MIN_UNITS))

    def per_warp(s):
        return -(-(-(-units // s)) // 4)

    def fits(s):
        key = (dev, dh, heads_per_kv > 8)
        if key not in _decode_tma_clusters:                # asked once, for every cluster size (never inside a later capture)
            _decode_tma_clusters[key] = [0] + [int(_lib().bl_attention_decode_tma_max_clusters(dh, heads_per_kv, c))
                                               for c in range(1, DECODE_CLUSTER_SPLITS + 1)]
        return clusters <= _decode_tma_clusters[key][s]

    one_per_sm = max(1, min(most, sms // clusters))
    if per_warp(one_per_sm) <= DECODE_TMA_FEW_UNITS:
        top = one_per_sm
    else:
        top = next((s for s in range(most, 0, -1) if fits(s)), 1)
    return min(range(1, top + 1), key=lambda s: (per_warp(s), s))
_decode_counters = {}
_decode_resident = {}


def attention_decode_resident_blocks(dh: int) -> int:
    """Blocks of `attention_decode` that the device holds at once for this head size (asked of the kernel's own
    occupancy on the current device, once per head size)."""
    key = (torch.cuda.current_device(), dh)
    if key not in _decode_resident:
        _decode_resident[key] = max(1, int(_lib().bl_attention_decode_resident_blocks(dh)))
    return _decode_resident[key]


def attention_decode_scratch(n: int, H: int, dh: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else n * H * n_splits * (dh + 2)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_NONE) -> None:
    """out = epilogue(x @ w.T) for many rows: tcgen05 tensor cores, TMA-fed tiles, accumulator in tensor memory.
    Same operand rules as `gemm_skinny` (`gemm_skinny_supported`)."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need_bias(bias, N, epilogue)
    _call(_lib().bl_gemm_tc, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def gemm_tc_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 epilogue: int = EPI_NONE) -> None:
    """`gemm_tc` on pairs of SMs (tcgen05 cta_group::2): 256 x 256 tiles, for a few hundred rows and more."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need_bias(bias, N, epilogue)
    _call(_lib().bl_gemm_tc_pair, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


def gemm_tc_splitk(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   epilogue: int = EPI_NONE) -> None:
    """`gemm_tc` for shapes with few output tiles: clusters of up to eight blocks share a tile and cut K among them,
    their partial tiles added in block order through distributed shared memory."""
    M, K = x.shape
    N = out.shape[1]
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (rows_w, K)); _need(out, "out", None, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_tc_splitk, _p(x), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _stream())


_splitk_split = {}


def gemm_tc_splitk_split(M: int, N: int, K: int, epilogue: int) -> int:
    """Blocks that would share a tile of this product in `gemm_tc_splitk` (1: it has nothing over `gemm_tc`)."""
    key = (-(-M // 128), N, K, epilogue == EPI_SWIGLU)
    if key not in _splitk_split:
        _splitk_split[key] = int(_lib().bl_gemm_tc_splitk_split(M, N, K, epilogue))
    return _splitk_split[key]


def gemm_tc_cols_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `gemm_tc_cols` takes these operands: bfloat16, up to 64 rows, 16-byte aligned, x fits shared memory."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(library.load().bl_gemm_tc_cols_supported(x.shape[0], w.shape[0], x.shape[1])))


def gemm_tc_cols(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ w.T for few rows and very many columns (an output head): the tcgen05 kernel that streams W once
    through a deep TMA ring with W as the M side of the product."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16, (M, K)); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", None, (M, N))
    _call(_lib().bl_gemm_tc_cols, _p(x), _p(w), _p(out), _dt(out), M, N, K, _stream())


# Which matrix-product kernel takes a bfloat16 product of M rows by N columns. The thresholds were measured on a
# B200 (148 SMs) and live here, beside the kernels they choose between, not in the parts that call them.
SKINNY_MAX_ROWS = 64                  # up to here W streams through registers (faster than 128-row tcgen05 tiles at 64 rows)
TC_MIN_COLUMNS_FEW_ROWS = 4096        # 17..64 rows: wide products have enough 128-column tiles for TMA to stream W at full rate
TC_MIN_COLUMNS_VERY_FEW_ROWS = 32768  # an output head: up to 64 rows take the kernel made for it; without it 128-row tiles win from 9 rows
PAIR_MIN_ROWS = 256                   # from here on pairs of SMs share 256 x 256 tiles (tcgen05 cta_group::2)
SPLITK_MIN_ROWS, SPLITK_MAX_ROWS = 32, 640   # products with few tiles in this range of rows are cut along K over clusters ...
SPLITK_VERY_LONG_K = 16384            # ... or, below 32 rows, very long (K 18,944 by N 3,584 at 8 rows: 43 us against 72 us through registers)
STREAM_MIN_BYTES = 128 << 20          # matrices from this size on stream faster through TMA and tcgen05 than through registers, at any number of rows
SPLITK_LONG_K = 2048                  # ... when K is long (measured: K 4,864 by N 896 gains 2x at 128 rows, 1.25x at 512; K 896 gains only up to 128 rows)


def gemm_streams_better(w: torch.Tensor) -> bool:
    """Whether a matrix is so large that few rows of x are better served by the TMA-fed tcgen05 kernels than by the
    kernels that stream W through registers (measured on 272 MB at 8 rows: 4.3 TB/s against 2.6 TB/s)."""
    return w.numel() * w.element_size() >= STREAM_MIN_BYTES


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
         epilogue: int = EPI_NONE, fast: bool = True) -> None:
    """out = epilogue(x @ w.T) by the kernel that suits the operands: float32 operands, operands the tensor-core
    kernels cannot take, and `fast=False` run the plain CUDA-core kernel; bfloat16 operands a tensor-core kernel
    chosen by the number of rows (and, for few rows, of columns)."""
    kind = gemm_kernel(x, w, out.shape[1], bias, epilogue, fast)
    if kind == "plain":
        gemm_plain(x, w, out, bias, epilogue)
    elif kind == "cols":
        gemm_tc_cols(x, w, out)
    elif kind == "splitk":
        gemm_tc_splitk(x, w, out, bias, epilogue)
    elif kind == "skinny":
        gemm_skinny(x, w, out, bias, epilogue)
    elif kind == "tc":
        gemm_tc(x, w, out, bias, epilogue)
    else:
        gemm_tc_pair(x, w, out, bias, epilogue)


def gemm_kernel(x: torch.Tensor, w: torch.Tensor, N: int, bias: Optional[torch.Tensor], epilogue: int, fast: bool = True) -> str:
    """Which kernel `gemm` runs this product on: "plain", "cols" (an output head at decode time: W streams once, as the
    M side of the product), "splitk" (few tiles and a long K, a down projection: clusters cut K among their blocks),
    "skinny" (few rows: W streams through registers), "tc" or "pair" (tcgen05 tiles on one SM, on pairs of SMs)."""
    if not (fast and gemm_skinny_supported(x, w)):
        return "plain"
    M, K = x.shape
    few_rows_tc = ((M > 16 and N >= TC_MIN_COLUMNS_FEW_ROWS) or (M > 8 and N >= TC_MIN_COLUMNS_VERY_FEW_ROWS)
                   or gemm_streams_better(w))
    if (N >= TC_MIN_COLUMNS_VERY_FEW_ROWS and bias is None and epilogue == EPI_NONE and M <= 64
            and gemm_tc_cols_supported(x, w)):
        return "cols"
    if (epilogue != EPI_SWIGLU and M <= SPLITK_MAX_ROWS and (M >= SPLITK_MIN_ROWS or K >= SPLITK_VERY_LONG_K)
            and (K >= SPLITK_LONG_K or 64 < M <= 128) and gemm_tc_splitk_split(M, N, K, epilogue) >= 2):
        return "splitk"
    if M <= SKINNY_MAX_ROWS and not few_rows_tc:
        return "skinny"
    return "tc" if M < PAIR_MIN_ROWS else "pair"


def gemm_on_pairs(x: torch.Tensor, w: torch.Tensor, N: int, epilogue: int, fast: bool = True) -> bool:
    """Whether `gemm` would run this product on pairs of SMs (`gemm_tc_pair`): the kernel whose epilogues can leave an
    RMS norm pending (`gemm_residual_norm`) and apply a pending one (`gemm_swiglu_scaled`, `qkv_rope_tc`)."""
    return gemm_kernel(x, w, N, None, epilogue, fast) == "pair"


SKINNY_LINK_MIN_ROWS = 2       # steps of this many rows ...
SKINNY_LINK_MAX_ROWS = 16      # ... to this many share a norm between two register-streaming products (measured at the 0.5B
                               # sizes: a decode step 2 % faster at 2 rows, 6 % at 4, 4 % at 8, 1 % at 16; 2 % slower at 1 row)
SKINNY_LINK_MAX_BLOCKS = 592   # column blocks of 16 up to which the linked kernel keeps two batches of loads in flight (with more it
                               # runs its lighter form, and the fused norm + product kernel is the faster: 3B sizes, 688 blocks, +5 %)


def gemm_skinny_links_norm(x: torch.Tensor, w: torch.Tensor, N: int, epilogue: int, fast: bool = True) -> bool:
    """Whether `gemm` would run this product on the register-streaming kernel at a row count where that kernel's
    epilogues begin an RMS norm (`gemm_skinny_residual_norm`) and finish one (`gemm_skinny_scaled`)."""
    return (SKINNY_LINK_MIN_ROWS <= x.shape[0] <= SKINNY_LINK_MAX_ROWS and -(-N // 16) <= SKINNY_LINK_MAX_BLOCKS
            and gemm_kernel(x, w, N, None, epilogue, fast) == "skinny")


def gemm_skinny_residual_norm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, norm_w: torch.Tensor):
    """out += x @ w.T (32-bit residual stream, in place) on the register-streaming kernel, and, for the RMS norm with
    weight `norm_w` that reads `out` next, (hw, ss): hw = bfloat16(out * norm_w), ss[m, :] = sums of squares of row m
    by block of 16 columns (what `gemm_residual_norm` gives on pairs of SMs, for decode steps)."""
    M, K = x.shape
    N = out.shape[1]
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", torch.float32, (M, N))
    _need(norm_w, "norm_w", None, (N,))
    parts = int(_lib().bl_gemm_skinny_norm_parts(N))
    hw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ss = torch.empty((M, parts), dtype=torch.float32, device=x.device)
    _call(_lib().bl_gemm_skinny_residual_norm, _p(x), _p(w), _p(out), M, N, K, _p(norm_w), _dt(norm_w), _p(hw), _p(ss), _stream())
    return hw, ss


def gemm_skinny_scaled(hw: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ss: torch.Tensor, eps: float,
                       bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE) -> None:
    """out = epilogue(r * (hw @ w.T)), r[m] = 1 / sqrt(ss[m].sum() / K + eps): the product of rows whose RMS norm
    `gemm_skinny_residual_norm` (or `gemm_residual_norm`) left pending. Epilogues: none, bias, SwiGLU."""
    M, K = hw.shape
    N = out.shape[1]
    _need(hw, "hw", torch.bfloat16); _need(w, "w", torch.bfloat16, ((2 * N if epilogue == EPI_SWIGLU else N), K))
    _need(out, "out", None, (M, N)); _need(ss, "ss", torch.float32)
    if ss.shape[0] != M:
        raise KernelError("gemm_skinny_scaled: ss and hw differ in rows")
    if bias is not None:
        _need_bias(bias, N, epilogue)
    _call(_lib().bl_gemm_skinny_scaled, _p(hw), _p(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), _dt(out),
          M, N, K, epilogue, _p(ss), ss.shape[1], ctypes.c_float(eps), _stream())


def gemm_residual_norm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, norm_w: torch.Tensor):
    """out += x @ w.T (32-bit residual stream, in place) on pairs of SMs, and, for the RMS norm with weight `norm_w`
    that reads `out` next, (hw, ss): hw = bfloat16(out * norm_w) and ss[m, :] = sums of squares of row m's columns by
    tile. A product that takes hw as its x and scales its rows by 1 / sqrt(ss[m].sum() / N + eps) computes what it would
    from the normed rows (`gemm_swiglu_scaled`, `qkv_rope_tc` with `row_sums`)."""
    M, K = x.shape
    N = out.shape[1]
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K)); _need(out, "out", torch.float32, (M, N))
    _need(norm_w, "norm_w", None, (N,))
    parts = int(_lib().bl_gemm_tc_pair_norm_parts(M, N))
    hw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ss = torch.empty((M, parts), dtype=torch.float32, device=x.device)
    _call(_lib().bl_gemm_tc_pair_residual_norm, _p(x), _p(w), _p(out), M, N, K, _p(norm_w), _dt(norm_w), _p(hw), _p(ss), _stream())
    return hw, ss


def gemm_swiglu_scaled(hw: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ss: torch.Tensor, eps: float) -> None:
    """out = silu(r g) * (r u), g and u the two halves of hw @ w.T, r[m] = 1 / sqrt(ss[m].sum() / K + eps): the SwiGLU
    product of rows whose RMS norm `gemm_residual_norm` left pending."""
    M, K = hw.shape
    N = out.shape[1]
    _need(hw, "hw", torch.bfloat16); _need(w, "w", torch.bfloat16, (2 * N, K)); _need(out, "out", torch.bfloat16, (M, N))
    _need(ss, "ss", torch.float32)
    if ss.shape[0] != M:
        raise KernelError("gemm_swiglu_scaled: ss and hw differ in rows")
    _call(_lib().bl_gemm_tc_pair_swiglu_scaled, _p(hw), _p(w), _p(out), M, N, K, _p(ss), ss.shape[1], ctypes.c_float(1.0 / K),
          ctypes.c_float(eps), _stream())


def check_status() -> None:
    """Raises if a tensor-core block gave up on one of its bounded waits since the last check. Synchronises."""
    for name, fn in (("bl_gemm_tc", _lib().bl_gemm_tc_status), ("bl_gemm_tc_pair", _lib().bl_gemm_tc_pair_status),
                     ("bl_attention_prefill_tc", _lib().bl_attention_prefill_tc_status),
                     ("bl_gemm_tc_cols", _lib().bl_gemm_tc_cols_status),
                     ("bl_gemm_tc_splitk", _lib().bl_gemm_tc_splitk_status),
                     ("bl_attention_decode_tma", _lib().bl_attention_decode_tma_status)):
        v = ctypes.c_int(0)
        _call(fn, ctypes.byref(v))
        if v.value != 0:
            who = {1: "the TMA loader", 2: "the MMA issuer", 3: "the epilogue"}.get(v.value, "a thread")
            raise KernelError(f"{name}: {who} gave up on a bounded wait (code {v.value}); results of that launch are invalid")


def norm_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the fused norm + product kernels take these operands (float32 rows, bfloat16 matrix)."""
    return (x.dtype == torch.float32 and w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and bool(library.load().bl_norm_gemm_supported(x.shape[1])))


def norm_gemm(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
              bias: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE,
              row_idx: Optional[torch.Tensor] = None) -> None:
    """out = epilogue(rmsnorm(x[row_idx]) @ w.T) in one launch, for few rows. EPI_NONE / EPI_BIAS write float32,
    EPI_SWIGLU (w with twice the rows) writes bfloat16."""
    K = x.shape[1]
    M, N = out.shape
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    _need(x, "x", torch.float32); _need(norm_w, "norm_w", None, (K,)); _need(w, "w", torch.bfloat16, (rows_w, K))
    _need(out, "out", torch.bfloat16 if epilogue == EPI_SWIGLU else torch.float32)
    if row_idx is not None:
        _need(row_idx, "row_idx", torch.int32, (M,))
    elif x.shape[0] != M:
        raise KernelError("norm_gemm: x and out differ in rows")
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_norm_gemm, _p(x), _p(row_idx), _p(norm_w), _dt(norm_w), ctypes.c_float(eps), _p(w), _p(bias),
          _dt(bias) if bias is not None else 0, _p(out), M, N, K, epilogue, _stream())


def norm_qkv_rope(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                  positions: torch.Tensor, tok_req: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor,
                  mscale: float, q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  H: int, KV: int, dh: int, pair_layout: int = 0) -> None:
    """rmsnorm -> joined q/k/v product (+ bias) -> rotation of q and k -> k, v into the pages, q out, in one launch."""
    M, K = x.shape
    _need(x, "x", torch.float32); _need(norm_w, "norm_w", None, (K,)); _need(w_qkv, "w_qkv", torch.bfloat16, ((H + 2 * KV) * dh, K))
    _need(positions, "positions", torch.int32, (M,)); _need(tok_req, "tok_req", torch.int32, (M,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32, (dh // 2,))
    _need(q_out, "q_out", torch.bfloat16, (M, H * dh))
    if bias is not None:
        _need(bias, "bias", None, ((H + 2 * KV) * dh,))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
        if k_cache.shape[1] != KV or k_cache.shape[3] != dh:
            raise KernelError(f"k_cache: shape {tuple(k_cache.shape)} does not hold {KV} heads of {dh}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_norm_qkv_rope, _p(x), _p(norm_w), _dt(norm_w), ctypes.c_float(eps), _p(w_qkv), _p(bias),
          _dt(bias) if bias is not None else 0, _p(positions), _p(tok_req), _p(block_table), block_table.shape[1],
          _p(inv_freq), ctypes.c_float(mscale), _p(q_out), _p(k_cache), _p(v_cache), M, K, H, KV, dh, page_size,
          pair_layout, _stream())


# ---- norms with bias, gated residuals, the average over the layers' streams ----------------------------------------
ACT_SILU, ACT_GELU_ERF, ACT_GELU_TANH = 0, 1, 2
GATE_SIGMOID, GATE_SILU = 0, 1
RULE_GLA, RULE_DELTA, RULE_BONUS = 0, 1, 2


def _rows32(t: torch.Tensor, name: str, rows: int, min_cols: int) -> int:
    """Checks 32-bit CUDA rows that may be a column range of a wider matrix; returns their row stride."""
    if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != rows or t.shape[1] < min_cols:
        raise KernelError(f"{name}: must be 32-bit CUDA rows [{rows}, >= {min_cols}] with contiguous rows, got {tuple(t.shape)} {t.dtype}")
    return t.stride(0)


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
              row_idx: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x[src] - mean) / sqrt(var + eps) * weight + bias, src = row_idx[r] if given else r; 32-bit statistics."""
    d = x.shape[1]
    rows = out.shape[0]
    _need(x, "x", torch.float32); _need(weight, "weight", None, (d,)); _need(out, "out", None, (rows, d))
    if bias is not None:
        _need(bias, "bias", None, (d,))
    if row_idx is not None:
        _need(row_idx, "row_idx", torch.int32, (rows,))
    elif x.shape[0] != rows:
        raise KernelError("layernorm: x and out differ in rows")
    _call(_lib().bl_layernorm, _p(x), _p(row_idx), _p(weight), _dt(weight), _p(bias), _dt(bias) if bias is not None else 0,
          _p(out), _dt(out), rows, d, ctypes.c_float(eps), _stream())


def gated_norm_residual(x: torch.Tensor, sub: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor,
                        bias: Optional[torch.Tensor], eps: float, gate_bias: Optional[torch.Tensor] = None) -> None:
    """x += layer norm(sub * sigmoid(gate + gate_bias)) * weight + bias, row by row, in 32-bit (gate None: no gate; it
    may be a range of columns of a wider matrix)."""
    rows, d = x.shape
    _need(x, "x", torch.float32); _need(sub, "sub", torch.float32, (rows, d)); _need(weight, "weight", None, (d,))
    if bias is not None:
        _need(bias, "bias", None, (d,))
    ld = _rows32(gate, "gate", rows, d) if gate is not None else 0
    if gate_bias is not None:
        _need(gate_bias, "gate_bias", None, (d,))
    _call(_lib().bl_gated_norm_residual, _p(x), _p(sub), _p(gate), ld, _p(gate_bias), _dt(gate_bias) if gate_bias is not None else 0,
          _p(weight), _dt(weight), _p(bias), _dt(bias) if bias is not None else 0, rows, d, ctypes.c_float(eps), _stream())


def depth_mix(streams: torch.Tensor, coeffs: torch.Tensor, n: int, out: torch.Tensor) -> None:
    """out = sum_{j < n} coeffs[j] * streams[j]; streams [>= n, T, d] 32-bit, out [T, d] (it may be a later stream)."""
    _need(streams, "streams", torch.float32); _need(out, "out", torch.float32, tuple(streams.shape[1:]))
    _need(coeffs, "coeffs")
    if not (0 < n <= streams.shape[0] and coeffs.numel() >= n):
        raise KernelError(f"depth_mix: {n} streams asked of {streams.shape[0]} with {coeffs.numel()} coefficients")
    _call(_lib().bl_depth_mix, _p(streams), ctypes.c_longlong(streams.stride(0)), _p(coeffs), _dt(coeffs), n, _p(out),
          ctypes.c_longlong(out.numel()), _stream())


def activation(x: torch.Tensor, out: torch.Tensor, act: int) -> None:
    """out = silu, the exact (erf) gelu or the tanh gelu of every element of x, evaluated in 32-bit (out may be x). x and
    out are matrices whose rows are contiguous (either may be a range of columns of a wider matrix)."""
    if x.dim() != 2 or out.shape != x.shape or x.stride(1) != 1 or out.stride(1) != 1 or not (x.is_cuda and out.is_cuda):
        raise KernelError("activation: x and out must be CUDA matrices of one shape with contiguous rows")
    _call(_lib().bl_activation, _p(x), _dt(x), ctypes.c_longlong(x.stride(0)), _p(out), _dt(out), ctypes.c_longlong(out.stride(0)),
          x.shape[0], x.shape[1], act, _stream())


def qk_norm_rope_write(proj: torch.Tensor, off_k: int, off_v: int, q_norm_w: Optional[torch.Tensor],
                       k_norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor, tok_req: torch.Tensor,
                       block_table: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, pair_layout: int, q_out: torch.Tensor,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], H: int, KV: int, dk: int, dv: int) -> None:
    """From a token's joined projections (32-bit rows: q first, k from column off_k, v from off_v): RMS norm over the
    whole q row and the whole k row (weights None: no norm), rotation, q out, k and v into the request's pages."""
    T = proj.shape[0]
    ld = _rows32(proj, "proj", T, off_v + KV * dv)
    _need(positions, "positions", torch.int32, (T,)); _need(tok_req, "tok_req", torch.int32, (T,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rot_half:
        raise KernelError("inv_freq: fewer entries than rotated pairs")
    _need(q_out, "q_out", None, (T, H * dk))
    if q_norm_w is not None:
        _need(q_norm_w, "q_norm_w", None, (H * dk,))
    if k_norm_w is not None:
        _need(k_norm_w, "k_norm_w", None, (KV * dk,))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype)
        if tuple(k_cache.shape[1:]) != (KV, k_cache.shape[2], dk) or tuple(v_cache.shape) != (k_cache.shape[0], KV, k_cache.shape[2], dv):
            raise KernelError(f"caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not hold {KV} heads of {dk} / {dv}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_qk_norm_rope_write, _p(proj), ld, off_k, off_v, _p(q_norm_w), _dt(q_norm_w) if q_norm_w is not None else 0,
          _p(k_norm_w), _dt(k_norm_w) if k_norm_w is not None else 0, ctypes.c_float(eps), _p(positions), _p(tok_req),
          _p(block_table), block_table.shape[1], _p(inv_freq), rot_half, pair_layout, _p(q_out), _p(k_cache), _p(v_cache),
          _dt(q_out), T, H, KV, dk, dv, page_size, _stream())


def gemm_plain_decay(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], coef: torch.Tensor, group: int, sign: float,
                     out: torch.Tensor) -> None:
    """out[m, n] = exp(-coef[n // group] * softplus(sign * (x[m] . w[n] + bias[n]))), 32-bit: the decays of a linear
    recurrence as the epilogue of the product that makes their pre-activation (sign -1, coef 1 / tau: sigmoid(z)^(1 / tau)).
    x: 32-bit rows, possibly a column range of a wider matrix."""
    M, K = x.shape
    N = out.shape[1]
    ld = _rows32(x, "x", M, K)
    _need(w, "w", None, (N, K)); _need(out, "out", torch.float32, (M, N)); _need(coef, "coef", torch.float32, (N // group,))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_plain_decay, _p(x), ld, _p(w), _dt(w), _p(bias), _dt(bias) if bias is not None else 0, _p(out), M, N, K,
          _p(coef), group, ctypes.c_float(sign), _stream())


SCAN_MAX_PARTS = 16               # most parts a long portion of a request is cut into
SCAN_PART_MIN_TOKENS = 256        # requests with fewer tokens in a step are walked in one piece (the kernel's own rule)
SCAN_BLOCKS_PER_SM = 2            # blocks of the scan kernel that an SM holds (its registers)


def recurrent_scan_parts(rule: int, H: int, dk: int, dv: int, n_long: int) -> int:
    """How many parts `recurrent_scan` should cut the portions of a step's `n_long` long requests into (1: none). Cutting
    runs every token twice, on `parts` times the blocks: time goes as (2 / parts) x rounds of blocks, against 1 x rounds in
    one piece. It pays while a request's blocks leave most of the device idle (heads x value columns / 32 blocks: 28 for 7
    heads of 64 x 128, where 10 parts take 0.2 of the time; 128 blocks for 8 heads of 128 x 256, where no cut gains). The
    delta rule's first pass has as many columns more as the key size (its transition over a part is a matrix)."""
    if n_long <= 0:
        return 1
    blocks = int(library.load().bl_recurrent_scan_can_split(rule, H, dk, dv)) * n_long
    if blocks <= 0:
        return 1
    room = SCAN_BLOCKS_PER_SM * _sms()
    rounds = lambda b: -(-b // room)
    best = min(range(2, SCAN_MAX_PARTS + 1), key=lambda p: (2.0 / p * rounds(blocks * p), p))
    return best if 2.0 / best * rounds(blocks * best) <= 0.7 * rounds(blocks) else 1


def recurrent_scan(rule: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: Optional[torch.Tensor],
                   q_scale: float, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, out: torch.Tensor,
                   H: int, G: int, dk: int, dv: int, parts: int = 1) -> None:
    """A linear recurrence over a matrix state per head and request (`RULE_GLA`, `RULE_DELTA`, `RULE_BONUS`, whose beta is
    a given number per token and head, see `bonus_dot`; see `bl_recurrent_scan`).
    q, k [T, G * dk], v [T, H * dv], decay [T, H * dk] (in (0, 1], see `gemm_plain_decay`), beta [T, H] (logits): 32-bit
    rows, possibly column ranges of a wider matrix. state: [slots, >= H * dk * dv] 32-bit, the matrix state first in each
    slot. out [T, H * dv] 32-bit, already times q_scale. `parts` > 1 (`recurrent_scan_parts`): portions of 256 tokens and
    more are cut into that many parts, which run side by side (twice the arithmetic on `parts` times the blocks; the
    results differ from the walk in one piece by rounding only)."""
    T = out.shape[0]
    R = cu_q.shape[0] - 1
    ldq, ldk, ldv, ldz = (_rows32(q, "q", T, G * dk), _rows32(k, "k", T, G * dk), _rows32(v, "v", T, H * dv),
                          _rows32(decay, "decay", T, H * dk))
    ldb = _rows32(beta, "beta", T, H) if beta is not None else 0
    _need(slots, "slots", torch.int32); _need(cu_q, "cu_q", torch.int32)
    _need(out, "out", torch.float32, (T, H * dv))
    if not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * dk * dv:
        raise KernelError("state: must be 32-bit [slots, >= H * dk * dv] with contiguous rows")
    if parts > 1:
        lib = _lib()
        lib.bl_recurrent_scan_parts_scratch.restype = ctypes.c_longlong
        scratch = torch.empty(int(lib.bl_recurrent_scan_parts_scratch(rule, R, parts, H, dk, dv)), dtype=torch.float32, device=out.device)
        _call(_lib().bl_recurrent_scan_parts, rule, _p(q), ldq, _p(k), ldk, _p(v), ldv, _p(decay), ldz, _p(beta), ldb,
              ctypes.c_float(q_scale), _p(state), ctypes.c_longlong(state.stride(0)), _p(slots), _p(cu_q), R,
              _p(out), H, G, dk, dv, parts, _p(scratch), _stream())
        return
    _call(_lib().bl_recurrent_scan, rule, _p(q), ldq, _p(k), ldk, _p(v), ldv, _p(decay), ldz, _p(beta), ldb,
          ctypes.c_float(q_scale), _p(state), ctypes.c_longlong(state.stride(0)), _p(slots), _p(cu_q), R,
          _p(out), H, G, dk, dv, _stream())


def head_norm_gate(o: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], gate_kind: int, eps: float,
                   out: torch.Tensor, H: int, dv: int) -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * g(gate[t, h]), g = sigmoid or silu (gate None: 1)."""
    T = o.shape[0]
    _need(o, "o", torch.float32, (T, H * dv)); _need(out, "out", None, (T, H * dv))
    if weight is not None:                   # None: the norm has no weight
        _need(weight, "weight", None, (dv,))
    ld = _rows32(gate, "gate", T, H * dv) if gate is not None else 0
    _call(_lib().bl_head_norm_gate, _p(o), _p(weight), _vec_dt(weight), _p(gate), ld, gate_kind, _p(out), _dt(out), T, H, dv,
          ctypes.c_float(eps), _stream())


def conv_silu_unit(x: torch.Tensor, taps: torch.Tensor, tail: torch.Tensor, slots: torch.Tensor, tok_req: torch.Tensor,
                   cu_q: torch.Tensor, out: torch.Tensor, unit_heads: int, scaled_heads: int, dk: int, q_scale: float,
                   unit_eps: float, bias: Optional[torch.Tensor] = None) -> None:
    """out = silu(short causal convolution of x over a request's tokens, per channel), then the first `unit_heads` heads
    of dk columns made unit vectors (the first `scaled_heads` times q_scale). x: 32-bit rows [T, >= C]; taps [C, n]
    32-bit (the last column is the current token's); tail: [slots, >= (n - 1) * C] 32-bit rows (a column range of the
    state slots), each slot holding its request's last n - 1 inputs, oldest first."""
    T, C = out.shape
    n_taps = taps.shape[1]
    ld = _rows32(x, "x", T, C)
    _need(taps, "taps", torch.float32, (C, n_taps)); _need(out, "out", torch.float32)
    _need(slots, "slots", torch.int32); _need(tok_req, "tok_req", torch.int32, (T,)); _need(cu_q, "cu_q", torch.int32)
    if not tail.is_cuda or tail.dtype != torch.float32 or tail.stride(1) != 1 or tail.shape[1] < (n_taps - 1) * C:
        raise KernelError("tail: must be 32-bit [slots, >= (taps - 1) * C] with contiguous rows")
    if bias is not None:                     # a bias per channel that the convolution's sum starts from
        _need(bias, "bias", None, (C,))
    _call(_lib().bl_conv_silu_unit_bias, _p(x), ld, _p(taps), n_taps, _p(tail), ctypes.c_longlong(tail.stride(0)), _p(slots),
          _p(tok_req), _p(cu_q), _p(out), T, C, unit_heads, scaled_heads, dk, ctypes.c_float(q_scale), ctypes.c_float(unit_eps),
          _p(bias), _vec_dt(bias), _stream())


def conv_tail_update(x: torch.Tensor, n_taps: int, tail: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, C: int) -> None:
    """After `conv_silu_unit`: every request with tokens in this step keeps its last n_taps - 1 inputs in its slot."""
    ld = _rows32(x, "x", x.shape[0], C)
    _need(slots, "slots", torch.int32); _need(cu_q, "cu_q", torch.int32)
    _call(_lib().bl_conv_tail_update, _p(x), ld, n_taps, _p(tail), ctypes.c_longlong(tail.stride(0)), _p(slots), _p(cu_q),
          cu_q.shape[0] - 1, C, _stream())


def linear_act(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: int, fast: bool = True):
    """out = act((x @ w.T)[:, :N]), N = out's columns, the activation evaluated in 32-bit on the product's 32-bit sums.
    w may have more rows than out has columns: the sums of those further rows are returned as they are (a 32-bit view
    [M, rows - N]; None when there are none)."""
    M, N = out.shape
    rows_w = w.shape[0]
    if rows_w < N:
        raise KernelError("linear_act: w has fewer rows than out has columns")
    sums = torch.empty((M, rows_w), dtype=torch.float32, device=x.device)
    gemm(x, w, sums, None, EPI_NONE, fast=fast)
    activation(sums[:, :N], out, act)
    return sums[:, N:] if rows_w > N else None


NORM_CHAIN_MAX_STREAMS = 512      # streams that `norm_chain` averages in its launch


def norm_chain_supported(x: torch.Tensor, gate: Optional[torch.Tensor]) -> bool:
    """Whether `norm_chain` takes rows of this width (a multiple of 4, up to 4,096) with this gate (rows 16-byte aligned)."""
    ld = gate.stride(0) if gate is not None else 0
    return (x.data_ptr() % 16 == 0 and (gate is None or gate.data_ptr() % 16 == 0)
            and bool(library.load().bl_norm_chain_supported(x.shape[1], ld)))


def norm_chain(x: torch.Tensor, sub: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
               gate_bias: Optional[torch.Tensor] = None, post=None, streams: Optional[torch.Tensor] = None,
               coeffs: Optional[torch.Tensor] = None, n: int = 0, mix_out: Optional[torch.Tensor] = None, then=None,
               y: Optional[torch.Tensor] = None) -> None:
    """Up to three row-wise steps on the 32-bit rows x in one launch (what `gated_norm_residual`, `depth_mix` and
    `layernorm` do one after the other, bit for bit): with `sub`, x += layer norm(sub * sigmoid(gate + gate_bias)) with
    the norm `post` = (weight, bias, eps); with `streams` [>= n, T, d] (x being stream n - 1), mix_out = sum_{j < n}
    coeffs[j] * streams[j]; with `then` = (weight, bias, eps), y = layer norm(that row)."""
    rows, d = x.shape
    _need(x, "x", torch.float32)
    pw = pb = tw = tb = None
    peps = teps = 0.0
    ld = 0
    if sub is not None:
        _need(sub, "sub", torch.float32, (rows, d))
        pw, pb, peps = post
        _need(pw, "post weight", None, (d,))
        if gate is not None:
            ld = _rows32(gate, "gate", rows, d)
    stride = 0
    if streams is not None:
        _need(streams, "streams", torch.float32); _need(mix_out, "mix_out", torch.float32, (rows, d)); _need(coeffs, "coeffs")
        if not (0 < n <= streams.shape[0] and coeffs.numel() >= n and tuple(streams.shape[1:]) == (rows, d)
                and x.data_ptr() == streams[n - 1].data_ptr()):
            raise KernelError("norm_chain: x must be stream n - 1 of the streams it is averaged with")
        stride = streams.stride(0)
    if then is not None:
        tw, tb, teps = then
        _need(tw, "then weight", None, (d,)); _need(y, "y", None, (rows, d))
    dt = lambda t: _dt(t) if t is not None else 0
    _call(_lib().bl_norm_chain, _p(x), _p(sub), _p(gate), ld, _p(gate_bias), dt(gate_bias), _p(pw), dt(pw), _p(pb), dt(pb),
          ctypes.c_float(peps), _p(streams), ctypes.c_longlong(stride), _p(coeffs), dt(coeffs), n, _p(mix_out), _p(tw), dt(tw),
          _p(tb), dt(tb), ctypes.c_float(teps), _p(y), dt(y) if y is not None else 0, rows, d, _stream())


# ---- layers with the norm behind the sublayer; mixers and feed-forwards of newer designs -----------------------------

def _vec_dt(t: Optional[torch.Tensor]) -> int:
    return _dt(t) if t is not None else 0


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (32-bit, contiguous) in out's dtype."""
    _need(x, "x", torch.float32); _need(out, "out", None, tuple(x.shape))
    _call(_lib().bl_cast_rows, _p(x), _p(out), _dt(out), ctypes.c_longlong(x.numel()), _stream())


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap), in place (32-bit)."""
    _need(x, "x", torch.float32)
    _call(_lib().bl_softcap, _p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream())


def post_norm_residual(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float, y: Optional[torch.Tensor] = None,
                       b: Optional[torch.Tensor] = None, wa: Optional[torch.Tensor] = None, wb: Optional[torch.Tensor] = None,
                       rms_eps: float = 0.0) -> None:
    """x += LN(s) * weight (layer norm without bias) with s = a, or, with b, s = (rms_norm(a) * wa + rms_norm(b) * wb) / 2;
    y (optional): the new rows of x in y's dtype as well (what the next sublayer's products read)."""
    rows, d = x.shape
    _need(x, "x", torch.float32); _need(a, "a", torch.float32, (rows, d)); _need(weight, "weight", None, (d,))
    if b is not None:
        _need(b, "b", torch.float32, (rows, d)); _need(wa, "wa", None, (d,)); _need(wb, "wb", None, (d,))
    if y is not None:
        _need(y, "y", None, (rows, d))
    _call(_lib().bl_post_norm_residual, _p(x), _p(a), _p(wa), _vec_dt(wa), _p(b), _p(wb), _vec_dt(wb), ctypes.c_float(rms_eps),
          _p(weight), _dt(weight), ctypes.c_float(eps), _p(y), _dt(y) if y is not None else 0, rows, d, _stream())


def pair_rms_mean(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, rms_eps: float, out: torch.Tensor) -> None:
    """out = (rms_norm(a) * wa + rms_norm(b) * wb) / 2, row by row, 32-bit."""
    rows, d = a.shape
    _need(a, "a", torch.float32); _need(b, "b", torch.float32, (rows, d)); _need(out, "out", torch.float32, (rows, d))
    _need(wa, "wa", None, (d,)); _need(wb, "wb", None, (d,))
    _call(_lib().bl_pair_rms_mean, _p(a), _p(wa), _dt(wa), _p(b), _p(wb), _dt(wb), ctypes.c_float(rms_eps), _p(out), rows, d, _stream())


def qk_head_norm_rope_write(proj: torch.Tensor, off_k: int, off_v: int, q_norm_w: Optional[torch.Tensor],
                            k_norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor, tok_req: torch.Tensor,
                            block_table: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, pair_layout: int, q_out: torch.Tensor,
                            k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], H: int, KV: int, dk: int, dv: int,
                            q_head_scale: Optional[torch.Tensor] = None) -> None:
    """`qk_norm_rope_write` with an RMS norm over each HEAD of q and of k (weights [dk], shared by the heads), and an optional
    factor per head on q (32-bit [H]), applied as q is written."""
    T = proj.shape[0]
    ld = _rows32(proj, "proj", T, off_v + KV * dv)
    _need(positions, "positions", torch.int32, (T,)); _need(tok_req, "tok_req", torch.int32, (T,))
    _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rot_half:
        raise KernelError("inv_freq: fewer entries than rotated pairs")
    _need(q_out, "q_out", None, (T, H * dk))
    for w, name in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w")):
        if w is not None:
            _need(w, name, None, (dk,))
    if q_head_scale is not None:
        _need(q_head_scale, "q_head_scale", torch.float32, (H,))
    page_size = 1
    if k_cache is not None:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype)
        if tuple(k_cache.shape[1:]) != (KV, k_cache.shape[2], dk) or tuple(v_cache.shape) != (k_cache.shape[0], KV, k_cache.shape[2], dv):
            raise KernelError(f"caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not hold {KV} heads of {dk} / {dv}")
        page_size = k_cache.shape[2]
    _call(_lib().bl_qk_norm_rope_write_scope, _p(proj), ld, off_k, off_v, _p(q_norm_w), _vec_dt(q_norm_w), _p(k_norm_w),
          _vec_dt(k_norm_w), ctypes.c_float(eps), 1, _p(positions), _p(tok_req), _p(block_table), block_table.shape[1],
          _p(inv_freq), rot_half, pair_layout, _p(q_out), _p(k_cache), _p(v_cache), _dt(q_out), T, H, KV, dk, dv, page_size,
          _p(q_head_scale), _stream())


def attention_talk_plain(q, k_cache, v_cache, tok_req, cu_q, ctx_len, block_table, A: torch.Tensor, H: int, chunk: int, window: int,
                         scale: float, head_scale: Optional[torch.Tensor]) -> None:
    """A[t, g, c] = sum_j softmax_j(q_g . k_kv(g)(j) * scale * head_scale[g]) v_c(j) over the keys of the query's chunk
    (positions [i - i % chunk, i]; chunk 0: all before it; window > 0: also the last `window` only): every head's softmax
    applied to the values of every key/value head. A: 32-bit [T, H, KV, dv]."""
    T = q.shape[0]
    KV, page_size, dh = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    dv = v_cache.shape[3]
    _need(q, "q", None, (T, H * dh)); _need(k_cache, "k_cache", q.dtype); _need(v_cache, "v_cache", q.dtype)
    _need(A, "A", torch.float32, (T, H, KV, dv)); _need(block_table, "block_table", torch.int32)
    if head_scale is not None:
        _need(head_scale, "head_scale", None, (H,))
    _call(_lib().bl_attention_talk_plain, _p(q), _p(k_cache), _p(v_cache), _dt(q), _p(tok_req), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(A), T, H, KV, dh, dv, page_size, chunk, window, ctypes.c_float(scale), _p(head_scale),
          _vec_dt(head_scale), _stream())


def talk_mix(A: torch.Tensor, talk: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h] = sum_g talk[h, g] * A[t, g, kv(h)]: the heads' softmax weights mixed, applied to each head's own values."""
    T, H, KV, dv = A.shape
    _need(A, "A"); _need(talk, "talk", None, (H, H)); _need(out, "out", None, (T, H * dv))
    _call(_lib().bl_talk_mix, _p(A), _dt(A), _p(talk), _dt(talk), _p(out), _dt(out), T, H, KV, dv, _stream())


def attention_prefill_talk(q, k_cache, v_cache, cu_q, ctx_len, block_table, tiles, A: torch.Tensor, H: int, chunk: int, window: int,
                           scale: float, head_scale: Optional[torch.Tensor]) -> None:
    """`attention_talk_plain` on tensor cores for the requests with several new tokens (tiles as `attention_prefill`);
    A: bfloat16 [T, H, KV, dh]; head_scale 32-bit and positive."""
    KV, dh = k_cache.shape[1], k_cache.shape[3]
    _need(q, "q", torch.bfloat16); _need(A, "A", torch.bfloat16, (q.shape[0], H, KV, dh)); _need(tiles, "tiles", torch.int32)
    if head_scale is not None:
        _need(head_scale, "head_scale", torch.float32, (H,))
    _call(_lib().bl_attention_prefill_talk, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table), block_table.shape[1],
          _p(tiles), tiles.shape[0], _p(A), H, KV, dh, k_cache.shape[2], chunk, window, ctypes.c_float(scale), _p(head_scale), _stream())


def attention_decode_talk(q, k_cache, v_cache, cu_q, ctx_len, block_table, reqs, n_splits: int, A: torch.Tensor, H: int, chunk: int,
                          window: int, scale: float, head_scale: Optional[torch.Tensor]) -> None:
    """The same for the requests with a single new token (reqs, slices as `attention_decode` without scratch)."""
    KV, dh = k_cache.shape[1], k_cache.shape[3]
    _need(q, "q", torch.bfloat16); _need(A, "A", torch.bfloat16, (q.shape[0], H, KV, dh)); _need(reqs, "reqs", torch.int32)
    if head_scale is not None:
        _need(head_scale, "head_scale", torch.float32, (H,))
    _call(_lib().bl_attention_decode_talk, _p(q), _p(k_cache), _p(v_cache), _p(cu_q), _p(ctx_len), _p(block_table), block_table.shape[1],
          _p(reqs), reqs.shape[0], n_splits, _p(A), H, KV, dh, k_cache.shape[2], chunk, window, ctypes.c_float(scale), _p(head_scale),
          _stream())


def gemm_plain_decay_exp(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, x_tanh: bool = False) -> None:
    """out[m, n] = exp(-exp(u[m] . w[n] + bias[n])), u = tanh(x) with `x_tanh`, 32-bit: decays in (0, 1) from a product in
    two factors (x: the first factor's 32-bit sums, possibly a column range of a wider matrix)."""
    M, K = x.shape
    N = out.shape[1]
    ld = _rows32(x, "x", M, K)
    _need(w, "w", None, (N, K)); _need(out, "out", torch.float32, (M, N))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    _call(_lib().bl_gemm_plain_decay_exp, _p(x), ld, 1 if x_tanh else 0, _p(w), _dt(w), _p(bias), _vec_dt(bias), _p(out), M, N, K, _stream())


def _slot_rows(state: torch.Tensor, name: str, min_cols: int) -> None:
    if not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < min_cols:
        raise KernelError(f"{name}: must be 32-bit [slots, >= {min_cols}] with contiguous rows")


def memory_gates(proj: torch.Tensor, off_k: int, off_v: int, off_i: int, off_f: int, bias_i: torch.Tensor, bias_f: torch.Tensor,
                 cap: float, state: torch.Tensor, off_m: int, slots: torch.Tensor, cu_q: torch.Tensor, H: int, dk: int, dv: int):
    """The gates of a matrix memory with exponential gating held against a running maximum (see `bl_memory_gates`): from
    the joined projections, what the scan reads, (decay [T, H * dk], keys times their input weight [T, H * dk], values with
    a last column of ones [T, H * (dv + 1)]), and the floor e^(-m) of the read-out's denominator [T, H]. The running maximum
    [H] is kept in the request's slot at `off_m`; the normaliser is the state's last value column."""
    T = proj.shape[0]
    ld = _rows32(proj, "proj", T, 1)
    _slot_rows(state, "state", off_m + H)
    _need(bias_i, "bias_i", None, (H,)); _need(bias_f, "bias_f", None, (H,))
    _need(slots, "slots", torch.int32); _need(cu_q, "cu_q", torch.int32)
    f32 = dict(dtype=torch.float32, device=proj.device)
    gates = torch.empty((3, T, H), **f32)
    decay, keys, values = torch.empty((T, H * dk), **f32), torch.empty((T, H * dk), **f32), torch.empty((T, H * (dv + 1)), **f32)
    _call(_lib().bl_memory_gates, _p(proj), ld, off_k, off_v, off_i, off_f, _p(bias_i), _dt(bias_i), _p(bias_f), _dt(bias_f),
          ctypes.c_float(cap), _p(state), ctypes.c_longlong(state.stride(0)), ctypes.c_longlong(off_m), _p(slots), _p(cu_q),
          cu_q.shape[0] - 1, T, _p(gates), _p(decay), _p(keys), _p(values), H, dk, dv, _stream())
    return decay, keys, values, gates[2]


def head_norm_gate_ext(o: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], gate_kind: int, eps: float,
                       out: torch.Tensor, H: int, dv: int, floor: Optional[torch.Tensor] = None) -> None:
    """`head_norm_gate` with a weight per head and channel when `weight` has H * dv values; with `floor` [T, H], o has
    dv + 1 columns a head, and o[t, h, :dv] is divided by max(|o[t, h, dv]|, floor[t, h]) + 1e-6 before the norm."""
    T = o.shape[0]
    stride = dv + 1 if floor is not None else dv
    _need(o, "o", torch.float32, (T, H * stride)); _need(out, "out", None, (T, H * dv))
    per_head = weight.numel() == H * dv and H > 1
    _need(weight, "weight", None, (H * dv,) if per_head else (dv,))
    if floor is not None:
        _need(floor, "floor", torch.float32, (T, H))
    ld = _rows32(gate, "gate", T, H * dv) if gate is not None else 0
    _call(_lib().bl_head_norm_gate_ext, _p(o), stride, _p(weight), _dt(weight), 1 if per_head else 0, _p(floor), _p(gate), ld, gate_kind,
          _p(out), _dt(out), T, H, dv, ctypes.c_float(eps), _stream())


def shift_mix(x: torch.Tensor, mu: torch.Tensor, prev: torch.Tensor, slots: torch.Tensor, tok_req: torch.Tensor, cu_q: torch.Tensor,
              out: torch.Tensor) -> None:
    """out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] within each request; the row before a step's first token of a request is
    its slot's `prev` [slots, >= d] (keep it with `conv_tail_update(x, 2, prev, ...)` after this call)."""
    T, d = x.shape
    n_mix = mu.shape[0]
    ld = _rows32(x, "x", T, d)
    _need(mu, "mu", torch.float32, (n_mix, d)); _need(out, "out", None, (n_mix, T, d)); _slot_rows(prev, "prev", d)
    _need(slots, "slots", torch.int32); _need(tok_req, "tok_req", torch.int32, (T,)); _need(cu_q, "cu_q", torch.int32)
    _call(_lib().bl_shift_mix, _p(x), ld, _p(mu), n_mix, _p(prev), ctypes.c_longlong(prev.stride(0)), _p(slots), _p(tok_req),
          _p(cu_q), _p(out), _dt(out), T, d, _stream())


def bonus_dot(q: torch.Tensor, k: torch.Tensor, u: torch.Tensor, out: torch.Tensor, H: int, dk: int) -> None:
    """out[t, h] = sum_c u[h, c] * k[t, h, c] * q[t, h, c]: the beta of `RULE_BONUS` for a bonus per head and key channel."""
    T = out.shape[0]
    ldq, ldk = _rows32(q, "q", T, H * dk), _rows32(k, "k", T, H * dk)
    _need(u, "u", None, (H, dk)); _need(out, "out", torch.float32, (T, H))
    _call(_lib().bl_bonus_dot, _p(q), ldq, _p(k), ldk, _p(u), _dt(u), _p(out), T, H, dk, _stream())


SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1


def moe_route(z: torch.Tensor, correction: Optional[torch.Tensor], top: int, n_groups: int, keep: int, ids: torch.Tensor,
              wts: torch.Tensor, score: int = SCORE_SIGMOID, group_top: int = 2) -> None:
    """The experts of each token and their weights from the router's 32-bit logits z [T, E] (see `bl_moe_route`). `score`:
    sigmoid of each logit, or the softmax over all E; `group_top`: a group's score is the sum of its two largest choice
    scores (2) or its largest (1)."""
    T, E = z.shape
    ld = _rows32(z, "z", T, E)
    if correction is not None:
        _need(correction, "correction", None, (E,))
    _need(ids, "ids", torch.int32, (T, top)); _need(wts, "wts", torch.float32, (T, top))
    _call(_lib().bl_moe_route_ext, _p(z), ld, _p(correction), _vec_dt(correction), T, E, top, n_groups, keep, _p(ids), _p(wts),
          score, group_top, _stream())


def expert_gemm_plain(x: torch.Tensor, x_div: int, w: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                      act: Optional[torch.Tensor] = None) -> None:
    """out[p] = epilogue(x[p // x_div] @ w[ids[p]].T): rows that each use the matrix of their own expert. w [E, N, K]
    ([E, 2N, K], gate rows then up rows, for EPI_SWIGLU). `act`: the gated activation of EPI_SWIGLU when it is not SiLU
    (`glu_args`)."""
    if act is not None:
        if epilogue != EPI_SWIGLU:
            raise KernelError("an activation goes with the gated epilogue only")
        _need(act, "act", torch.float32, (2,))
    P, N = out.shape
    K = x.shape[1]
    _need(x, "x"); _need(w, "w", x.dtype); _need(out, "out"); _need(ids, "ids", torch.int32)
    rows_w = 2 * N if epilogue == EPI_SWIGLU else N
    if w.dim() != 3 or w.shape[1] != rows_w or w.shape[2] != K or ids.numel() != P or x.shape[0] * x_div != P:
        raise KernelError(f"expert_gemm_plain: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, {ids.numel()} ids do not fit")
    # (ids beyond w's experts are identity experts: their rows are skipped)
    _call(_lib().bl_expert_gemm_plain_some, _p(x), _dt(x), x_div, _p(w), _dt(w), ctypes.c_longlong(w.stride(0)), _p(ids), _p(out), _dt(out),
          P, N, K, epilogue, _p(act), w.shape[0], _stream())


def moe_combine(y: torch.Tensor, wts: torch.Tensor, out: torch.Tensor, add: bool = False, ids: Optional[torch.Tensor] = None,
                n_real: int = 0, x: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k wts[t, k] * y[t * top + k], k ascending (32-bit); with `add` the sum is added to out. With `ids`, a pair
    whose expert number is `n_real` or more is an identity expert and contributes x[t] (the token's input row) instead."""
    T, top = wts.shape
    d = out.shape[1]
    _need(y, "y", torch.float32, (T * top, d)); _need(wts, "wts", torch.float32); _need(out, "out", torch.float32, (T, d))
    if ids is not None:
        _need(ids, "ids", torch.int32, (T, top)); _need(x, "x", None, (T, d))
    _call(_lib().bl_moe_combine_some, _p(y), _p(wts), _p(out), T, top, d, 1 if add else 0, _p(ids), n_real, _p(x),
          _dt(x) if x is not None else 0, _stream())


GROUPED_TILE = 128         # rows of a tile of the grouped tensor-core product (every expert's rows start a new tile)


def grouped_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `moe_grouped` takes these operands: bfloat16, inner sizes that are multiples of 8, 16-byte alignment."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.shape[2] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_plan(ids: torch.Tensor, n_experts: int):
    """The layout of the pairs (token, chosen expert) for the grouped product: (pos [P] the row of each pair, row_src
    [rows] the pair of each row or -1, tile_expert [tiles] the expert of each tile of 128 rows or -1). The number of
    rows depends on the number of pairs and experts only (every expert may leave one tile partly empty). Pairs whose expert
    number is `n_experts` or more (identity experts) get no row: their pos is -1."""
    P = ids.numel()
    tiles = -(-P // GROUPED_TILE) + n_experts
    _need(ids, "ids", torch.int32)
    pos = torch.empty(P, dtype=torch.int32, device=ids.device)
    row_src = torch.empty(tiles * GROUPED_TILE, dtype=torch.int32, device=ids.device)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=ids.device)
    _call(_lib().bl_moe_plan, _p(ids), P, n_experts, GROUPED_TILE, tiles, _p(pos), _p(row_src), _p(tile_expert), _stream())
    return pos, row_src, tile_expert


def gather_rows(x: torch.Tensor, row_src: torch.Tensor, div: int, out: torch.Tensor) -> None:
    """out[row] = x[row_src[row] // div] (zeros where row_src is negative); bfloat16 rows of a multiple of 8 values."""
    _need(x, "x", torch.bfloat16); _need(out, "out", torch.bfloat16, (row_src.numel(), x.shape[1])); _need(row_src, "row_src", torch.int32)
    _call(_lib().bl_gather_rows, _p(x), _p(row_src), div, _p(out), out.shape[0], x.shape[1], _stream())


def gemm_grouped(x: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                 act: Optional[torch.Tensor] = None) -> None:
    """out = epilogue(x @ w[expert of the row's tile].T) on tcgen05: x [tiles * 128, K] bfloat16 in tiles of 128 rows, w
    [E, N, K] ([E, 2N, K], gate rows then up rows, for EPI_SWIGLU), tile_expert [tiles] (negative: an empty tile). `act`:
    the gated activation of EPI_SWIGLU when it is not SiLU (`glu_args`)."""
    if act is not None:
        if epilogue != EPI_SWIGLU:
            raise KernelError("an activation goes with the gated epilogue only")
        _need(act, "act", torch.float32, (2,))
    M, K = x.shape
    N = out.shape[1]
    E = w.shape[0]
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16, (E, 2 * N if epilogue == EPI_SWIGLU else N, K))
    _need(out, "out", None, (M, N)); _need(tile_expert, "tile_expert", torch.int32, (M // GROUPED_TILE,))
    _call(_lib().bl_gemm_tc_grouped, _p(x), _p(w), _p(out), _dt(out), M, N, K, epilogue, E, _p(tile_expert), _p(act), _stream())


def moe_combine_rows(y: torch.Tensor, pos: torch.Tensor, wts: torch.Tensor, out: torch.Tensor, add: bool = False,
                     x: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k wts[t, k] * y[pos[t * top + k]], k ascending (32-bit); with `add` the sum is added to out. A pair without
    a row (pos < 0: an identity expert, see `moe_plan`) contributes x[t], the token's input row."""
    T, top = wts.shape
    d = out.shape[1]
    _need(y, "y", torch.float32); _need(pos, "pos", torch.int32, (T * top,)); _need(wts, "wts", torch.float32); _need(out, "out", torch.float32, (T, d))
    if y.shape[1] != d:
        raise KernelError("moe_combine_rows: y and out differ in width")
    if x is not None:
        _need(x, "x", None, (T, d))
    _call(_lib().bl_moe_combine_rows_some, _p(y), _p(pos), _p(wts), _p(out), T, top, d, 1 if add else 0, _p(x),
          _dt(x) if x is not None else 0, _stream())


GLU_SILU, GLU_GELU_TANH, GLU_CLAMPED = 0, 1, 2


def glu_act(sums: torch.Tensor, out: torch.Tensor, kind: int, limit: float = 0.0) -> None:
    """out[r, c] = glu(sums[r, c], sums[r, N + c]) on the 32-bit sums of a joined gate | up product (N = out's columns):
    GLU_SILU silu(g) u; GLU_GELU_TANH gelu_tanh(g) u; GLU_CLAMPED g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit)
    and u' = clamp(u, -limit, limit). Evaluated in 32-bit."""
    M, N = out.shape
    ld = _rows32(sums, "sums", M, 2 * N)
    if out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("glu_act: out must be a CUDA matrix with contiguous rows")
    _call(_lib().bl_glu_act, _p(sums), ctypes.c_longlong(ld), _p(out), _dt(out), ctypes.c_longlong(out.stride(0)), M, N, kind,
          ctypes.c_float(limit), _stream())


def table_route(table: torch.Tensor, tokens: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor) -> None:
    """ids[t] = table[tokens[t]] (table [vocabulary, top] int32), wts[t, :] = 1 / top."""
    T = tokens.shape[0]
    top = table.shape[1]
    _need(table, "table", torch.int32); _need(tokens, "tokens", torch.int32, (T,))
    _need(ids, "ids", torch.int32, (T, top)); _need(wts, "wts", torch.float32, (T, top))
    _call(_lib().bl_table_route, _p(table), _p(tokens), T, top, _p(ids), _p(wts), _stream())


def latent_prep(proj: torch.Tensor, off_q: int, q_rank: int, off_kv: int, rank: int, rot_dim: int, rot_half: int,
                q_norm_w: Optional[torch.Tensor], kv_norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
                tok_req: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor, mscale: float,
                cq: Optional[torch.Tensor], cache: Optional[torch.Tensor]) -> None:
    """From the 32-bit sums `proj` of a mixer's joined first product: cq [T, q_rank] = RMS norm of the query latent times
    its weight (None: skipped), and into each token's page the row [RMS norm of the key/value latent times its weight |
    the shared key part of rot_dim values, its first 2 * rot_half rotated by the token's position] (`cache` [pages, 1, page,
    rank + rot_dim]; None: skipped)."""
    T = proj.shape[0]
    ld = _rows32(proj, "proj", T, 1)
    dtype = cq.dtype if cq is not None else cache.dtype
    page_size = 1
    if cq is not None:
        _need(cq, "cq", None, (T, q_rank)); _need(q_norm_w, "q_norm_w", None, (q_rank,))
    if cache is not None:
        _need(cache, "cache", dtype); _need(kv_norm_w, "kv_norm_w", None, (rank,))
        if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != rank + rot_dim:
            raise KernelError(f"latent_prep: cache {tuple(cache.shape)} does not hold rows of {rank} + {rot_dim}")
        page_size = cache.shape[2]
        _need(block_table, "block_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _call(_lib().bl_latent_prep, _p(proj), ld, off_q, q_rank, off_kv, rank, rot_dim, rot_half, _p(q_norm_w), _vec_dt(q_norm_w), _p(kv_norm_w),
          _vec_dt(kv_norm_w), ctypes.c_float(eps), _p(positions), _p(tok_req), _p(block_table), block_table.shape[1], page_size,
          _p(inv_freq), ctypes.c_float(mscale), _p(cq), _p(cache), _dt(cq if cq is not None else cache), T, _stream())


def _head_view(t: torch.Tensor, name: str, T: int, H: int, n: int):
    """(row stride, head stride) of a [T, H, >= n] view whose last dimension is contiguous."""
    if not t.is_cuda or t.dim() != 3 or t.shape[0] != T or t.shape[1] != H or t.shape[2] < n or t.stride(2) != 1:
        raise KernelError(f"{name}: must be CUDA [T={T}, H={H}, >= {n}] with a contiguous last dimension, got {tuple(t.shape)}")
    return t.stride(0), t.stride(1)


def head_gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """out[t, h, n] = sum_k x[t, h, k] * w[h, n, k] (times sigmoid(gate[t, h * N + n]) if given): a product per head on
    CUDA cores, one FMA chain per output in ascending k. x [T, H, K] and out [T, H, N] are views with a contiguous last
    dimension (32-bit or bfloat16), w [H, N, K] a view with any strides; gate 32-bit rows [T, >= H * N]."""
    T, H, K = x.shape
    N = w.shape[1]
    ldx, xh = _head_view(x, "x", T, H, K)
    ldo, oh = _head_view(out, "out", T, H, N)
    if w.dim() != 3 or w.shape[0] != H or w.shape[2] != K or not w.is_cuda:
        raise KernelError(f"head_gemm_plain: w {tuple(w.shape)} does not fit x {tuple(x.shape)}")
    ld_gate = _rows32(gate, "gate", T, H * N) if gate is not None else 0
    _call(_lib().bl_head_gemm_plain, _p(x), _dt(x), ctypes.c_longlong(ldx), ctypes.c_longlong(xh), _p(w), _dt(w),
          ctypes.c_longlong(w.stride(0)), ctypes.c_longlong(w.stride(1)), ctypes.c_longlong(w.stride(2)), _p(out), _dt(out),
          ctypes.c_longlong(ldo), ctypes.c_longlong(oh), T, H, N, K, _p(gate), ctypes.c_longlong(ld_gate), _stream())


def rope_heads(q: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rot_half: int, mscale: float,
               out: torch.Tensor, lead: Optional[torch.Tensor] = None, lead_out: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = q[t, h, :] with its first 2 * rot_half values rotated in pairs (j, j + rot_half) by
    float(position[t]) * inv_freq[j], cos and sin times mscale. q: 32-bit view [T, H, n], out a view of the same shape, last
    dimensions contiguous. `lead` / `lead_out`: in the same launch, another slice of the same rows (a view [T, H, m] with q's
    strides: the part of a head that is not rotated) cast into a tensor of its own, of out's dtype."""
    T, H, n = q.shape
    if n < 2 * rot_half or q.dtype != torch.float32:
        raise KernelError("rope_heads: q must be a 32-bit view [T, H, >= 2 * rot_half]")
    ldq, qh = _head_view(q, "q", T, H, n)
    ldo, oh = _head_view(out, "out", T, H, n)
    _need(positions, "positions", torch.int32, (T,)); _need(inv_freq, "inv_freq", torch.float32)
    m, ldl, lh = 0, 0, 0
    if lead is not None:
        m = lead.shape[2]
        if lead.dtype != torch.float32 or _head_view(lead, "lead", T, H, m) != (ldq, qh) or lead_out is None or lead_out.dtype != out.dtype:
            raise KernelError("rope_heads: the second slice must be a 32-bit view with q's strides, its result of out's dtype")
        ldl, lh = _head_view(lead_out, "lead_out", T, H, m)
    _call(_lib().bl_rope_heads, _p(q), ctypes.c_longlong(ldq), ctypes.c_longlong(qh), 0, _p(positions), _p(inv_freq), n, rot_half,
          ctypes.c_float(mscale), _p(out), _dt(out), ctypes.c_longlong(ldo), ctypes.c_longlong(oh), 0, T, H,
          _p(lead), m, _p(lead_out), ctypes.c_longlong(ldl), ctypes.c_longlong(lh), _stream())


def latent_attention_plain(q: torch.Tensor, cache: torch.Tensor, tok_req: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor,
                           block_table: torch.Tensor, out: torch.Tensor, window: int, scale: float,
                           sinks: Optional[torch.Tensor] = None) -> None:
    """Causal attention of q [T, H, dk] over cached rows of dk values (cache [pages, 1, page, dk]) whose first dv values
    are also the values: out [T, H, dv]. One warp per (token, head); `window` 0 sees every earlier row; `sinks` [H] joins
    each head's softmax denominator once."""
    T, H, dk = q.shape
    dv = out.shape[2]
    _need(q, "q", cache.dtype); _need(cache, "cache"); _need(out, "out", q.dtype, (T, H, dv))
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != dk:
        raise KernelError(f"latent_attention_plain: cache {tuple(cache.shape)} does not hold rows of {dk}")
    _need(tok_req, "tok_req", torch.int32, (T,)); _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if sinks is not None:
        _need(sinks, "sinks", None, (H,))
    _call(_lib().bl_latent_attention_plain, _p(q), _p(cache), _dt(q), _p(tok_req), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(out), T, H, dk, dv, cache.shape[2], window, ctypes.c_float(scale), _p(sinks), _vec_dt(sinks),
          _stream())


def latent_attention_mma_supported(dtype: torch.dtype, rank: int, rot: int, page_size: int) -> bool:
    """Whether the tensor-core kernel takes cached rows of rank + rot values: bfloat16, pages of 16, both parts multiples
    of 8, values of at most 512, operands that fit shared memory."""
    return dtype == torch.bfloat16 and bool(_lib().bl_latent_attention_mma_supported(rank, rot, page_size))


def latent_attention_mma(q_lat: torch.Tensor, q_rot: Optional[torch.Tensor], cache: torch.Tensor, cu_q: torch.Tensor,
                         ctx_len: torch.Tensor, block_table: torch.Tensor, work: torch.Tensor, single: bool, out: torch.Tensor,
                         window: int, scale: float, sinks: Optional[torch.Tensor] = None, n_splits: int = 1) -> None:
    """Causal attention over cached rows [latent | rotated part] on tensor cores. q_lat [H, Tp, rank], q_rot [H, Tp, rot]
    (None when rot is 0) and out [H, Tp, rank] lie head-major (row h * Tp + t is token t of the step, head h), bfloat16;
    cache [pages, 1, 16, rank + rot]. `work`: the step's 64-token tiles [n, 2] of requests with several new tokens, or,
    with `single`, the requests [n] with one, whose keys `n_splits` blocks may share (slices merged by a second kernel: long
    contexts in small batches). `window` 0 sees every earlier row; `sinks` [H] joins each head's denominator."""
    H, Tp, rank = q_lat.shape
    rot = cache.shape[3] - rank
    _need(q_lat, "q_lat", torch.bfloat16); _need(cache, "cache", torch.bfloat16); _need(out, "out", torch.bfloat16, (H, Tp, rank))
    if cache.dim() != 4 or cache.shape[1] != 1 or rot < 0:
        raise KernelError(f"latent_attention_mma: cache {tuple(cache.shape)} does not hold rows of {rank} and more")
    if rot:
        _need(q_rot, "q_rot", torch.bfloat16, (H, Tp, rot))
    _need(cu_q, "cu_q", torch.int32); _need(ctx_len, "ctx_len", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(work, "work", torch.int32)
    if sinks is not None:
        _need(sinks, "sinks", None, (H,))
    n_splits = max(1, int(n_splits)) if single else 1
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((work.shape[0] * H, n_splits, rank), dtype=torch.float32, device=out.device)
        part_ml = torch.empty((work.shape[0] * H, n_splits, 2), dtype=torch.float32, device=out.device)
    _call(_lib().bl_latent_attention_mma, _p(q_lat), _p(q_rot if rot else None), _p(cache), _p(cu_q), _p(ctx_len), _p(block_table),
          block_table.shape[1], _p(work), work.shape[0], 1 if single else 0, _p(out), H, Tp, rank, rot, cache.shape[2], window,
          ctypes.c_float(scale), _p(sinks), _vec_dt(sinks), n_splits, _p(part_o), _p(part_ml), _stream())


LATENT_ROWS = 32               # rows of a block of the latent attention kernel (heads of a single token)
LATENT_RESIDENT = 2 * 148      # its blocks that the device holds at once (two an SM up to 256 latent values)
LATENT_MAX_SPLITS = 16


def latent_attention_splits(n_single: int, H: int, longest: int) -> int:
    """Into how many slices the keys of requests with a single token are cut: as many as fill the device once, one key
    block of 64 each at least."""
    units = max(1, n_single * (-(-H // LATENT_ROWS)))
    return max(1, min(-(-longest // 64), LATENT_RESIDENT // units, LATENT_MAX_SPLITS))


def head_tiles(n_heads: int, per: int, device) -> torch.Tensor:
    """[n_heads * per] int32: tile i of a head-major matrix [n_heads, per * 128, .] belongs to head i // per."""
    tile = torch.empty(n_heads * per, dtype=torch.int32, device=device)
    _call(_lib().bl_head_tiles, _p(tile), n_heads, per, _stream())
    return tile


def heads_gate_rows(hv: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t, h * N + n] = hv[h, t, n] (* sigmoid(gate[t, h * N + n])): head-major 32-bit sums hv [H, Tp, N] back to the
    step's token rows out [T, H * N]; gate 32-bit rows [T, >= H * N] that may be a column range of a wider matrix."""
    H, Tp, N = hv.shape
    T = out.shape[0]
    _need(hv, "hv", torch.float32); _need(out, "out", None, (T, H * N))
    ld = _rows32(gate, "gate", T, H * N) if gate is not None else 0
    _call(_lib().bl_heads_gate_rows, _p(hv), _p(gate), ctypes.c_longlong(ld), _p(out), _dt(out), T, H, N, Tp, _stream())


def rope_decay_prep(proj: torch.Tensor, off_k: int, positions: torch.Tensor, inv_freq: torch.Tensor, rot_half: int,
                    head_decay: torch.Tensor, k_scale: float, H: int, dk: int):
    """In front of a recurrence with a fixed decay per head: (q, k, decay), each 32-bit [T, H * dk], from the joined
    projections (q first, k from column off_k): q and k rotated by position (pairs (i, i + rot_half) of each head's first
    2 * rot_half values, 32-bit angles), k times k_scale, decay[t, h, :] = head_decay[h]."""
    T = proj.shape[0]
    ld = _rows32(proj, "proj", T, off_k + H * dk)
    _need(positions, "positions", torch.int32, (T,)); _need(inv_freq, "inv_freq", torch.float32); _need(head_decay, "head_decay", torch.float32, (H,))
    if inv_freq.numel() < rot_half:
        raise KernelError("inv_freq: fewer entries than rotated pairs")
    q, k, decay = (torch.empty((T, H * dk), dtype=torch.float32, device=proj.device) for _ in range(3))
    _call(_lib().bl_rope_decay_prep, _p(proj), ld, off_k, _p(positions), _p(inv_freq), rot_half, _p(head_decay), ctypes.c_float(k_scale),
          _p(q), _p(k), _p(decay), T, H, dk, _stream())
    return q, k, decay


def ssd_prep(raw: torch.Tensor, dt_bias: torch.Tensor, rate: torch.Tensor, x: torch.Tensor, H: int, n_state: int, dv: int):
    """In front of a selective state-space recurrence: dt = softplus(raw + dt_bias) per (token, head), 32-bit; returns
    (decay [T, H * n_state] = exp(-rate[h] * dt) for every key channel, v [T, H * dv] = dt * x). raw [T, >= H] and x
    [T, >= H * dv] are 32-bit rows, possibly column ranges of wider matrices."""
    T = raw.shape[0]
    ld_raw, ld_x = _rows32(raw, "raw", T, H), _rows32(x, "x", T, H * dv)
    _need(dt_bias, "dt_bias", None, (H,)); _need(rate, "rate", torch.float32, (H,))
    decay = torch.empty((T, H * n_state), dtype=torch.float32, device=raw.device)
    v = torch.empty((T, H * dv), dtype=torch.float32, device=raw.device)
    _call(_lib().bl_ssd_prep, _p(raw), ld_raw, _p(dt_bias), _dt(dt_bias), _p(rate), _p(x), ld_x, _p(decay), _p(v), T, H, n_state, dv, _stream())
    return decay, v


def gated_group_norm(o: torch.Tensor, x: Optional[torch.Tensor], skip: Optional[torch.Tensor], dv: int, z: Optional[torch.Tensor],
                     weight: Optional[torch.Tensor], n_parts: int, eps: float, out: torch.Tensor) -> None:
    """out = rms_norm_in_parts((o + skip[c // dv] * x) * silu(z)) * weight: the gate stands IN FRONT of the norm, and each of
    `n_parts` equal parts of a row is normed by its own root mean square. o [T, width] 32-bit; x, z: 32-bit rows (column
    ranges allowed); x with skip, z and weight may each be None."""
    T, width = o.shape
    _need(o, "o", torch.float32); _need(out, "out", None, (T, width))
    ld_x = _rows32(x, "x", T, width) if x is not None else 0
    ld_z = _rows32(z, "z", T, width) if z is not None else 0
    if x is not None:
        _need(skip, "skip", None, (width // dv,))
    if weight is not None:
        _need(weight, "weight", None, (width,))
    _call(_lib().bl_gated_group_norm, _p(o), _p(x), ld_x, _p(skip), _vec_dt(skip), dv, _p(z), ld_z, _p(weight), _vec_dt(weight),
          _p(out), _dt(out), T, width, n_parts, ctypes.c_float(eps), _stream())


def add_scaled_pair(x: torch.Tensor, a: torch.Tensor, ca: float, b: torch.Tensor, cb: float) -> None:
    """x += ca * a + cb * b (32-bit): two sublayer results that join the stream with a constant factor each."""
    _need(x, "x", torch.float32); _need(a, "a", torch.float32, tuple(x.shape)); _need(b, "b", torch.float32, tuple(x.shape))
    _call(_lib().bl_add_scaled_pair, _p(x), _p(a), ctypes.c_float(ca), _p(b), ctypes.c_float(cb), ctypes.c_longlong(x.numel()), _stream())


def add_row_gated(x: torch.Tensor, a: torch.Tensor, gate: torch.Tensor) -> None:
    """x[r] += sigmoid(gate[r, 0]) * a[r] (32-bit; gate: rows of a 32-bit matrix, its first column the logit)."""
    rows, d = x.shape
    _need(x, "x", torch.float32); _need(a, "a", torch.float32, (rows, d))
    ld = _rows32(gate, "gate", rows, 1)
    _call(_lib().bl_add_row_gated, _p(x), _p(a), _p(gate), ctypes.c_longlong(ld), rows, d, _stream())


def xielu_args(p: float, q: float, device) -> torch.Tensor:
    """The two numbers the xIELU kernel reads, from the learned p and q: {softplus(p), 1/2 + softplus(q)}, 32-bit."""
    sp = lambda v: float(torch.nn.functional.softplus(torch.tensor(v, dtype=torch.float64)))
    return torch.tensor([sp(p), 0.5 + sp(q)], dtype=torch.float32, device=device)


def xielu(x: torch.Tensor, out: torch.Tensor, args: torch.Tensor) -> None:
    """out = xIELU(x) on 32-bit sums (rows contiguous; column ranges allowed): v > 0: args[0] v^2 + v / 2, else
    args[1] (e^v - 1 - v) + v / 2."""
    rows, cols = out.shape
    ld = _rows32(x, "x", rows, cols)
    _need(args, "args", torch.float32, (2,))
    if out.stride(1) != 1:
        raise KernelError("xielu: out must have contiguous rows")
    _call(_lib().bl_xielu, _p(x), ctypes.c_longlong(ld), _p(out), _dt(out), ctypes.c_longlong(out.stride(0)), rows, cols, _p(args), _stream())
