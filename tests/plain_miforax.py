"""A plain, slow implementation of the Miforax decoder: whole sequences, no cache, no batching, one function for each
mechanism, float64. It shares no code with the engine and is what the engine's Miforax results are compared with.

The design in this file's notation (x: residual stream [T, d]):

    embedding:  x = table[token] * s
    layer:      x <- x + mixer(N1(x));   x <- x + ff(N2(x))     (N: RMS norm with a weight; a layer may have no ff)
    mixer:      attention whose keys and values are made from ONE small vector per token (the latent c, kv_rank wide)
                and one rotated key part that all heads share; queries pass through a latent of their own; a window,
                a sink per head in the softmax's denominator, a sigmoid gate per channel on the heads' outputs.
                A layer may read the latent and rotated key part of an earlier layer instead of making its own.
    ff:         dense (act(gate) * up with the tanh form of GELU), or experts that a table picks by TOKEN ID, each
                with weight 1 / top, plus an optional expert that every token uses
    output:     RMS norm, head
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------------------------ rotation
def yarn_frequencies(n, base, scaling):
    """(f [n / 2], m): the angle per position of each of the n / 2 pairs and the factor on cos and sin.
    Without `scaling`: f_i = base^(-2i / n), m = 1. With (factor, original, fast, slow): pairs that turn fast keep
    f_i, pairs that turn slowly get f_i / factor, a linear ramp between the two over the pair index."""
    half = n // 2
    f = torch.tensor([base ** (-2.0 * i / n) for i in range(half)], dtype=F64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):                       # the (fractional) pair index that makes `turns` turns over `original` positions
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), n - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x, positions, freqs, m):
    """x [..., T, n] with n >= 2 * len(freqs): the first 2 * len(freqs) values are rotated in pairs (u, v) = (x_i, x_(i + half))
    -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i, cos and sin both times m; the rest pass unchanged."""
    half = freqs.shape[0]
    a = positions.to(F64)[:, None] * freqs[None, :]
    c, s = torch.cos(a) * m, torch.sin(a) * m
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


def rotation_of(c):
    """(f, m) of a mixer: its rot.dims rotated values (rot_dim of them when the key is absent), stretched if it says so."""
    return yarn_frequencies(c["rot"].get("dims", c["rot_dim"]), c["rot"]["base"], c["rot"].get("scaling"))


# ------------------------------------------------------------------------------------------------ attention
def window_mask(T, size):
    """[T, T] bool: row i sees column j with 0 <= i - j < size (size 0 or None: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def sink_softmax_attention(q, k, v, scale, sinks, mask):
    """q [H, T, dq], k [H, T, dq], v [H, T, dv], sinks [H] or None. Weights e^(s_ij) / (sum_j e^(s_ij) + e^(sink)),
    s = q . k * scale on the visible keys; the sink is not scaled and has no value. Returns [H, T, dv]."""
    s = torch.einsum("hid,hjd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sinks is not None:
        m = torch.maximum(m, sinks[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sinks is not None:
        den = den + torch.exp(sinks[:, None, None] - m)
    return torch.einsum("hij,hjd->hid", e / den, v)


def latent_and_rotated_key(h, w, c, eps, positions):
    """What a layer caches: (latent [T, kv_rank], rotated key part [T, rot_dim]) of the rows h."""
    r = c["kv_rank"]
    z = h @ w["dkv"].T
    lat = rms_norm(z[:, :r], w["dkv.norm"], eps)
    f, m = rotation_of(c)
    return lat, rotate_halves(z[:, r:], positions, f, m)


def latent_attention_mixer(h, w, c, eps, positions, shared=None):
    """The mixer's result [T, d] and what it caches. `shared`: (latent, rotated key part) of the layer it reads from."""
    T = h.shape[0]
    H, dn, dr, dv = c["heads"], c["dim"], c["rot_dim"], c["vdim"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, dn + dr)
    f, m = rotation_of(c)
    q_rot = rotate_halves(q[:, :, dn:].permute(1, 0, 2), positions, f, m)            # [H, T, dr]
    lat, k_rot = shared if shared is not None else latent_and_rotated_key(h, w, c, eps, positions)
    k_nope = (lat @ w["uk"].T).view(T, H, dn).permute(1, 0, 2)
    val = (lat @ w["uv"].T).view(T, H, dv).permute(1, 0, 2)
    qq = torch.cat([q[:, :, :dn].permute(1, 0, 2), q_rot], dim=-1)
    kk = torch.cat([k_nope, k_rot[None].expand(H, T, dr)], dim=-1)
    size = (c.get("mask") or {}).get("size", 0)
    o = sink_softmax_attention(qq, kk, val, c["scale"], w.get("sink"), window_mask(T, size))
    o = o.permute(1, 0, 2).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T, (lat, k_rot)


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def table_experts(h, tokens, w, c):
    """Each token's experts come from a table by its id; each weighs 1 / top; a shared expert is added if there is one."""
    top = c["router"]["top"]
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t, tok in enumerate(tokens):
        for e in w["table"][tok].tolist():
            out[t] += clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], c["expert"]["limit"])[0] / top
    if c.get("shared"):
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], c["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ the model
def _sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, streams: bool = False):
    """Logits [T, vocab] of one sequence from its start (float64). `streams`: also the stream behind every layer."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = tensors["embed"].to(F64)[torch.tensor(tokens)] * config["embedding"]["scale"]
    kept, cached = [], {}
    for i, layer in enumerate(config["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        c = layer["mixer"]
        w = _sub(tensors, f"l{i}.mix.")
        h = rms_norm(x, tensors[f"l{i}.norm1"].to(F64), eps)
        src = c.get("kv_from")
        y, cached[i] = latent_attention_mixer(h, w, c, eps, positions, cached[src] if src is not None else None)
        x = x + y
        m = layer.get("mlp")
        if m is not None:
            h = rms_norm(x, tensors[f"l{i}.norm2"].to(F64), eps)
            wf = _sub(tensors, f"l{i}.mlp.")
            if m["kind"] == "dense":
                x = x + dense_ff(h, wf)
            elif m["kind"] == "moe":
                x = x + table_experts(h, tokens, wf, m)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward {m['kind']!r}")
        kept.append(x.clone())
    logits = rms_norm(x, tensors["final.norm"].to(F64), eps) @ tensors["head"].to(F64).T
    return (logits, kept) if streams else logits
