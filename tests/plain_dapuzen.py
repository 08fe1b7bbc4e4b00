"""A plain, slow implementation of the Dapuzen decoder: whole sequences, no cache, no batching, one function for each
mechanism, float64. It shares no code with the engine and is what the engine's Dapuzen results are compared with.

The design in this file's notation (x: residual stream [T, d]):

    embedding:  x = table[token] * s
    layer:      h = N(x);  x <- x + mixer(h) + ff(h)        (ONE norm, both sublayers read it; N: RMS norm times one number)
    mixer:      'attention'  grouped queries, rotation in halves, a window, a sigmoid gate per head on the head's output
                'retention'  per head S <- c_h S + k v^T, o = S^T q with a fixed c_h, rotation, unit RMS per head, SiLU gate
                'parallel'   a * left + b * right of  left:  windowed attention with biases, no rotation, capped scores
                                                      right: a selective state space (scalar decay per head and token)
    ff:         dense with the xIELU activation, or routed experts (softmax scores, groups, identity experts, a gated
                shared expert), or none
    a layer may run with ANOTHER layer's tensors ('weights_of') while keeping a cache of its own
    output:     N(x) head^T
"""
import math

import torch

F64 = torch.float64


def scalar_rms_norm(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * g with g ONE number."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap = softplus(torch.as_tensor(p, dtype=F64))
    an = 0.5 + softplus(torch.as_tensor(q, dtype=F64))
    zn = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.exp(zn) - 1.0 - zn) + 0.5 * z)


# ------------------------------------------------------------------------------------------------ rotation, masks
def rotate_halves(x, positions, base, n_rot):
    """x [..., T, n]: of the first n_rot values, value i is paired with i + n_rot / 2; (u, v) -> (u cos a - v sin a,
    v cos a + u sin a), a = position * base^(-2i / n_rot). The rest pass unchanged."""
    if not n_rot:
        return x
    half = n_rot // 2
    f = torch.tensor([base ** (-2.0 * i / n_rot) for i in range(half)], dtype=F64)
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:n_rot]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., n_rot:]], dim=-1)


def window_mask(T, size):
    """[T, T] bool: row i sees column j with 0 <= i - j < size (no size: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def softmax_attention(q, k, v, scale, mask, softcap=0.0):
    """q [H, T, dk], k [G, T, dk], v [G, T, dv]; query head h reads key/value head h // (H / G).
    s = q . k * scale, then, with a cap c, s <- c tanh(s / c); softmax over the visible keys. Returns [H, T, dv]."""
    H, G = q.shape[0], k.shape[0]
    rep = H // G
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    s = torch.einsum("hid,hjd->hij", q, k) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask[None], -math.inf)
    return torch.einsum("hij,hjd->hid", torch.softmax(s, dim=-1), v)


def _heads(x, n, d):
    """[T, n * d] -> [n, T, d]."""
    return x.reshape(x.shape[0], n, d).permute(1, 0, 2)


def _join(x):
    """[n, T, d] -> [T, n * d]."""
    return x.permute(1, 0, 2).reshape(x.shape[1], -1)


# ------------------------------------------------------------------------------------------------ mixers
def gated_attention_mixer(h, w, c, positions):
    """'attention': no biases, rotation of q and k, window, softmax, head h's output times sigmoid(g h)_h, then Wo."""
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    rot = c.get("rot") or {}
    q = rotate_halves(_heads(h @ w["q"].T, H, dk), positions, rot.get("base", 1.0), rot.get("dims", 0))
    k = rotate_halves(_heads(h @ w["k"].T, G, dk), positions, rot.get("base", 1.0), rot.get("dims", 0))
    v = _heads(h @ w["v"].T, G, dv)
    o = softmax_attention(q, k, v, c["scale"], window_mask(h.shape[0], (c.get("mask") or {}).get("size", 0)))
    gate = torch.sigmoid(h @ w["g"].T)                                   # [T, H]
    o = o * gate.T[:, :, None]
    return _join(o) @ w["o"].T


def capped_attention_mixer(h, w, c):
    """The left half of 'parallel': biases on q, k, v and the output, no rotation, capped scores, window."""
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = _heads(h @ w["q"].T + w["q.b"], H, dk)
    k = _heads(h @ w["k"].T + w["k.b"], G, dk)
    v = _heads(h @ w["v"].T + w["v.b"], G, dv)
    o = softmax_attention(q, k, v, c["scale"], window_mask(h.shape[0], (c.get("mask") or {}).get("size", 0)),
                          softcap=c.get("softcap", 0.0))
    return _join(o) @ w["o"].T + w["o.b"]


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, n] (the last column is the current token's), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    pad = torch.cat([torch.zeros((n - 1, x.shape[1]), dtype=x.dtype), x], dim=0)
    out = bias[None, :].expand(T, -1).clone()
    for j in range(n):
        out = out + pad[j:j + T] * taps[:, j][None, :]
    return out


def decayed_outer_recurrence(q, k, v, a, S0=None):
    """Per head: S_t = a_t S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [H, T, N], v [H, T, P], a [H, T] -> o [H, T, P]."""
    H, T, N = k.shape
    P = v.shape[2]
    S = torch.zeros((H, N, P), dtype=F64) if S0 is None else S0.clone()
    o = torch.zeros((H, T, P), dtype=F64)
    for t in range(T):
        S = a[:, t, None, None] * S + k[:, t, :, None] * v[:, t, None, :]
        o[:, t] = torch.einsum("hnp,hn->hp", S, q[:, t])
    return o


def state_space_mixer(h, w, c, eps):
    """The right half of 'parallel' (state-space duality). W_in h = [z | x | B | C | dt]; x, B, C pass a causal convolution
    per channel and a SiLU; dt <- softplus(dt + dt_bias); per head S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D x_t; y * silu(z), RMS norm in `norm_groups` parts times a weight, Wo."""
    T = h.shape[0]
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * P
    u = h @ w["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = _heads(xbc[:, :inner], H, P)                                     # [H, T, P]
    B = _heads(xbc[:, inner:inner + G * N], G, N).repeat_interleave(H // G, dim=0)
    C = _heads(xbc[:, inner + G * N:], G, N).repeat_interleave(H // G, dim=0)
    dt = softplus(dt + w["dt_bias"]).T                                   # [H, T]
    a = torch.exp(-torch.exp(w["A_log"])[:, None] * dt)
    y = decayed_outer_recurrence(C, B, x * dt[:, :, None], a) + w["D"][:, None, None] * x
    y = _join(y) * silu(z)
    parts = c["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def parallel_mixer(h, w, c, eps):
    left = capped_attention_mixer(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, c["left"])
    right = state_space_mixer(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def retention_mixer(h, w, c, eps, positions):
    """Rotation on q and k, k / sqrt(dim) after it, S_t = c_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, each head's o divided
    by its root mean square, heads joined, times silu(Wg h), Wo."""
    H, dk, dv = c["heads"], c["dim"], c["vdim"]
    rot = c.get("rot") or {}
    q = rotate_halves(_heads(h @ w["q"].T, H, dk), positions, rot.get("base", 1.0), rot.get("dims", 0))
    k = rotate_halves(_heads(h @ w["k"].T, H, dk), positions, rot.get("base", 1.0), rot.get("dims", 0)) * dk ** -0.5
    v = _heads(h @ w["v"].T, H, dv)
    a = torch.tensor(c["decay"], dtype=F64)[:, None].expand(H, h.shape[0])
    o = unit_rms(decayed_outer_recurrence(q, k, v, a), eps)
    return (_join(o) * silu(h @ w["g"].T)) @ w["o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


def glu_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def choose_experts(scores, correction, top, groups, keep):
    """scores [T, E] -> ids [T, top]: choice = scores + correction; a group's score is its largest choice score; experts
    outside the `keep` best groups count as minus infinity; the `top` largest remain (lower index first on a tie)."""
    T, E = scores.shape
    choice = scores + correction
    per = E // groups
    gs = choice.reshape(T, groups, per).max(dim=-1).values
    ids = torch.zeros((T, top), dtype=torch.int64)
    for t in range(T):
        order = sorted(range(groups), key=lambda g: (-float(gs[t, g]), g))[:keep]
        open_ = [e for g in sorted(order) for e in range(g * per, (g + 1) * per)]
        best = sorted(open_, key=lambda e: (-float(choice[t, e]), e))[:top]
        ids[t] = torch.tensor(best)
    return ids


def routed_experts(h, w, c, forced=None, info=None):
    """Softmax scores over experts + identity experts; choice with correction and groups; the weights are the chosen
    scores as they are; an identity expert returns h; the shared expert is added times sigmoid(w_sg . h)."""
    r = c["router"]
    E, n_id, top = r["experts"], r.get("identity", 0), r["top"]
    g = r.get("groups") or {}
    z = h @ w["router"].T
    s = torch.softmax(z, dim=-1)
    corr = w["correction"] if "correction" in w else torch.zeros(E + n_id, dtype=F64)
    own = choose_experts(s, corr, top, g.get("count", 1), g.get("keep", 1))
    ids = own if forced is None else forced.to(torch.int64)
    if info is not None:
        info.append({"scores": s, "choice": s + corr, "own": own, "groups": g.get("count", 1)})
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in ids[t].tolist():
            y = h[t] if e >= E else glu_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            out[t] = out[t] + s[t, e] * y
    if c.get("shared"):
        sh = glu_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * sh
    return out


# ------------------------------------------------------------------------------------------------ the model
def _sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, streams: bool = False, forced=None, info=None):
    """Logits [T, vocab] of one sequence (and, with `streams`, the residual stream behind every layer). `forced`:
    {layer: ids [T, top]} takes the experts from outside; `info` (a dict) receives each routed layer's scores."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    T = tokens.shape[0]
    positions = torch.arange(T)
    x = tensors["embed"].to(F64)[tokens] * (config.get("embedding") or {}).get("scale", 1.0)
    kept = []
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        h = scalar_rms_norm(x, tensors[p + "norm1"].to(F64), eps)
        w, c = _sub(tensors, p + "mix."), layer["mixer"]
        if layer["type"] == "attention":
            m = gated_attention_mixer(h, w, c, positions)
        elif layer["type"] == "retention":
            m = retention_mixer(h, w, c, eps, positions)
        elif layer["type"] == "parallel":
            m = parallel_mixer(h, w, c, eps)
        else:
            raise ValueError(layer["type"])
        f = 0.0
        mlp = layer.get("mlp")
        if mlp is not None:
            wf = _sub(tensors, p + "mlp.")
            if mlp["kind"] == "dense":
                f = dense_ff(h, wf)
            else:
                rec = [] if info is not None else None
                f = routed_experts(h, wf, mlp, forced=None if forced is None else forced.get(i), info=rec)
                if info is not None:
                    info[i] = rec[0]
        x = x + (m + f)
        kept.append(x.clone())
    logits = scalar_rms_norm(x, tensors["final.norm"].to(F64), eps) @ tensors["head"].to(F64).T
    return (logits, kept) if streams else logits
