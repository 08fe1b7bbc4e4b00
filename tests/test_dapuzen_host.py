"""The Dapuzen design without a GPU: configuration keys and their errors, the declared tensors, the run order and cache
layers of layers that run with another layer's tensors, and the plain implementation against closed forms."""
import math

import pytest
import torch

import plain_dapuzen as pd

F64 = torch.float64


def small_config():
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 9}, "rot": {"base": 100.0, "dims": 4}}
    ret = {"heads": 3, "dim": 8, "vdim": 6, "decay": [0.5, 0.9, 1.0], "rot": {"base": 50.0, "dims": 8}}
    par = {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.5, "softcap": 3.0, "mask": {"size": 5}},
           "right": {"heads": 4, "vdim": 6, "state": 5, "groups": 2, "conv": 3, "norm_groups": 3},
           "left_scale": 0.25, "right_scale": 2.0}
    moe = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 4, "top": 2, "identity": 2, "groups": {"count": 3, "keep": 2}},
           "shared": {"ff": 14}}
    return {"architecture": "Dapuzen", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "layers": [{"type": "parallel", "mixer": par, "mlp": {"kind": "dense", "ff": 20}},
                       {"type": "retention", "mixer": ret, "mlp": moe},
                       {"type": "attention", "mixer": att, "mlp": None},
                       {"type": "parallel", "mixer": par, "mlp": {"kind": "dense", "ff": 20}, "weights_of": 0},
                       {"type": "retention", "mixer": ret, "mlp": moe, "weights_of": 1}]}


def test_configuration_round_trip_and_fields():
    from boring_llm_b200 import DapuzenConfig
    cfg = DapuzenConfig.from_dict(small_config())
    assert DapuzenConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.embedding_scale == 2.0 and cfg.layers[3].weights_of == 0 and cfg.layers[0].weights_of is None
    par, ret, att = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[2].mixer
    assert (par.left.softcap, par.left.window, par.left_scale, par.right_scale) == (3.0, 5, 0.25, 2.0)
    assert (par.right.state, par.right.groups, par.right.conv, par.right.norm_groups) == (5, 2, 3, 3)
    assert ret.decay == (0.5, 0.9, 1.0) and (att.rot_dims, att.rot_base, att.window, att.scale) == (4, 100.0, 9, 0.3)
    moe = cfg.layers[1].mlp
    assert (moe.experts, moe.identity, moe.top, moe.groups, moe.keep, moe.shared_ff) == (4, 2, 2, 3, 2, 14)


@pytest.mark.parametrize("edit,needle", [
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9]), "decay"),
    (lambda c: c["layers"][2]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("norm_groups", 5), "parts"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "router"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "router"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 3), "weights_of"),
    (lambda c: c["layers"][4].__setitem__("weights_of", 3), "no tensors of its own"),
    (lambda c: c["layers"][3]["mlp"].__setitem__("ff", 24), "differs"),
    (lambda c: c["layers"][0].__setitem__("type", "mlstm"), "unknown layer type"),
])
def test_configuration_errors_name_the_key(edit, needle):
    import copy
    from boring_llm_b200 import ConfigError, DapuzenConfig
    c = copy.deepcopy(small_config())
    edit(c)
    with pytest.raises(ConfigError) as e:
        DapuzenConfig.from_dict(c)
    assert needle in str(e.value)


def test_declared_tensors_run_order_and_cache_layers():
    from boring_llm_b200 import DapuzenConfig, build_model
    from boring_llm_b200.cache import PagedKVSpec, StateSpec
    model = build_model(DapuzenConfig.from_dict(small_config()))
    specs = {k: tuple(v.shape) for k, v in model.tensor_specs().items()}
    assert not any(k.startswith(("l3.", "l4.")) for k in specs)          # layers that run with another's tensors declare none
    assert specs["l0.norm1"] == () and specs["final.norm"] == ()
    assert specs["l0.mix.left.q"] == (16, 24) and specs["l0.mix.left.v.b"] == (4,) and specs["l0.mix.left.o"] == (24, 8)
    assert specs["l0.mix.right.in"] == (2 * 24 + 2 * 2 * 5 + 4, 24) and specs["l0.mix.right.conv"] == (24 + 20, 3)
    assert specs["l0.mix.right.norm"] == (24,) and specs["l0.mix.right.A_log"] == (4,) and specs["l0.mlp.act"] == (2,)
    assert specs["l1.mix.g"] == (18, 24) and specs["l1.mlp.router"] == (6, 24) and specs["l1.mlp.correction"] == (6,)
    assert specs["l1.mlp.shared.sg"] == (1, 24) and "l1.mlp.e4.gate" not in specs and specs["l1.mlp.e3.down"] == (24, 10)
    assert specs["l2.mix.g"] == (4, 24) and "l2.mlp.up" not in specs
    order = [(c.block, c.cache) for c in model.schedule]
    assert order == [(0, (0, 1)), (1, 2), (2, 3), (0, (4, 5)), (1, 6)]
    cs = model.cache_specs()
    assert isinstance(cs[0], PagedKVSpec) and (cs[0].n_kv_heads, cs[0].head_dim, cs[0].window, cs[0].v_head_dim) == (1, 8, 5, 4)
    assert cs[1] == StateSpec((4 * 5 * 6 + 2 * (24 + 20),), "float32") and cs[1] == cs[5] and cs[0] == cs[4]
    assert cs[2] == StateSpec((3 * 8 * 6,), "float32") and cs[2] == cs[6]


def test_random_weights_of_the_design(tmp_path):
    from boring_llm_b200 import DapuzenConfig, write_random_model
    import plain_model as plain
    write_random_model(str(tmp_path), DapuzenConfig.from_dict(small_config()), 3, "bfloat16", 0.2)
    cfg, W = plain.read_model_folder(str(tmp_path))
    assert W["l0.norm1"].shape == () and abs(float(W["l0.norm1"]) - 1.0) < 1.0
    logits, streams = pd.forward(cfg, W, [1, 5, 7, 7, 2, 40, 3], streams=True)
    assert logits.shape == (7, 50) and len(streams) == 5 and bool(torch.isfinite(logits).all())


# ---- the plain implementation against closed forms ---------------------------------------------------------------------
def test_norm_with_one_number():
    x = torch.tensor([[3.0, -3.0, 3.0, -3.0]], dtype=F64)
    assert torch.allclose(pd.scalar_rms_norm(x, torch.tensor(2.0, dtype=F64), 0.0), torch.tensor([[2.0, -2.0, 2.0, -2.0]], dtype=F64))


def test_window_counts_and_capped_scores():
    m = pd.window_mask(6, 3)
    assert m.sum(1).tolist() == [1, 2, 3, 3, 3, 3] and bool(m[5, 3]) and not bool(m[5, 2])
    # scores far beyond the cap all become the cap: the visible values' mean
    T = 5
    q = torch.full((1, T, 2), 100.0, dtype=F64)
    k = torch.arange(1, T + 1, dtype=F64).reshape(1, T, 1).expand(1, T, 2).contiguous()
    v = torch.arange(T, dtype=F64).reshape(1, T, 1)
    o = pd.softmax_attention(q, k, v, 1.0, pd.window_mask(T, 2), softcap=1.0)
    assert torch.allclose(o[0, :, 0], torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5], dtype=F64), atol=1e-9)
    sharp = pd.softmax_attention(q, k, v, 1.0, pd.window_mask(T, 2))
    assert torch.allclose(sharp[0, :, 0], torch.tensor([0.0, 1.0, 2.0, 3.0, 4.0], dtype=F64), atol=1e-9)


def test_rotation_pairs_halves_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64)
    y = pd.rotate_halves(x, torch.tensor([3]), 10.0, 4)
    a0, a1 = 3.0, 3.0 * 10.0 ** -0.5
    want = [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(y[0, 0], torch.tensor(want, dtype=F64), atol=1e-12)
    assert torch.equal(pd.rotate_halves(x, torch.tensor([0]), 10.0, 4), x)


def test_recurrence_against_its_unrolled_sum():
    g = torch.Generator().manual_seed(0)
    H, T, N, P = 2, 7, 3, 4
    q, k, v = (torch.randn(H, T, n, generator=g, dtype=F64) for n in (N, N, P))
    a = torch.rand(H, T, generator=g, dtype=F64)
    o = pd.decayed_outer_recurrence(q, k, v, a)
    for h in range(H):
        for t in range(T):
            want = sum(torch.prod(a[h, j + 1:t + 1]) * (q[h, t] @ k[h, j]) * v[h, j] for j in range(t + 1))
            assert torch.allclose(o[h, t], want, atol=1e-12)


def test_convolution_last_tap_is_now_and_starts_from_zeros():
    x = torch.arange(1.0, 6.0, dtype=F64).reshape(5, 1)
    y = pd.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=F64), torch.tensor([0.5], dtype=F64))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]


def test_xielu_both_sides():
    z = torch.tensor([-2.0, 0.0, 1.5], dtype=F64)
    p, q = 0.3, -0.7
    ap, an = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
    y = pd.xielu(z, p, q)
    assert abs(float(y[0]) - (an * (math.exp(-2.0) + 1.0) - 1.0)) < 1e-12 and float(y[1]) == 0.0
    assert abs(float(y[2]) - (ap * 2.25 + 0.75)) < 1e-12
    e = 1e-6                                             # the slope at zero is 1 / 2 from both sides
    assert abs(float(pd.xielu(torch.tensor([e], dtype=F64), p, q)) / e - 0.5) < 1e-5
    assert abs(float(pd.xielu(torch.tensor([-e], dtype=F64), p, q)) / -e - 0.5) < 1e-5


def test_choice_of_experts():
    # six router outputs in three groups of two; choice scores may be negative: a closed group is minus infinity, not zero
    s = torch.tensor([[0.05, 0.10, 0.40, 0.05, 0.30, 0.10]], dtype=F64)
    corr = torch.tensor([-1.0, -1.0, -1.0, -3.0, -2.0, -2.5], dtype=F64)
    # group scores (the largest choice score): -0.90, -0.60, -1.70 -> groups 1 and 0 are kept
    ids = pd.choose_experts(s, corr, 3, 3, 2)
    assert ids.tolist() == [[2, 1, 0]]                   # -0.60, -0.90, -0.95; expert 3 (-2.95) loses; group 2 is closed
    # the correction moves the choice, not the weights
    assert pd.choose_experts(s, torch.zeros(6, dtype=F64), 2, 1, 1).tolist() == [[2, 4]]
    assert pd.choose_experts(s, torch.tensor([0, 0, -1.0, 0, 0, 0.3], dtype=F64), 2, 1, 1).tolist() == [[5, 4]]


def test_identity_experts_and_the_gated_shared_expert():
    g = torch.Generator().manual_seed(1)
    d, ff = 6, 4
    h = torch.randn(3, d, generator=g, dtype=F64)
    w = {"router": torch.zeros(4, d, dtype=F64), "correction": torch.tensor([0.0, 0.0, 5.0, 4.0], dtype=F64)}
    for e in range(2):
        for n, shape in (("gate", (ff, d)), ("up", (ff, d)), ("down", (d, ff))):
            w[f"e{e}.{n}"] = torch.randn(*shape, generator=g, dtype=F64)
    c = {"router": {"experts": 2, "top": 2, "identity": 2}}
    out = pd.routed_experts(h, w, c)                     # equal scores of 1 / 4, both identity experts chosen
    assert torch.allclose(out, 0.5 * h, atol=1e-12)
    w["correction"] = torch.tensor([5.0, 0.0, 4.0, 0.0], dtype=F64)
    out = pd.routed_experts(h, w, c)
    assert torch.allclose(out, 0.25 * (pd.glu_expert(h, w["e0.gate"], w["e0.up"], w["e0.down"]) + h), atol=1e-12)
    for n, shape in (("shared.gate", (ff, d)), ("shared.up", (ff, d)), ("shared.down", (d, ff))):
        w[n] = torch.randn(*shape, generator=g, dtype=F64)
    w["shared.sg"] = torch.zeros(1, d, dtype=F64)
    with_shared = pd.routed_experts(h, w, dict(c, shared={"ff": ff}))
    assert torch.allclose(with_shared - out, 0.5 * pd.glu_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"]), atol=1e-12)


def test_state_space_head_groups_and_gate_before_the_norm():
    """With the skip term alone (A large: no memory; B = 0 through a zero input matrix) y = D x; the gate multiplies before
    each part of the row is normed by its own root mean square."""
    g = torch.Generator().manual_seed(2)
    d, H, P, N, G = 5, 2, 3, 2, 1
    inner = H * P
    c = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": 1, "norm_groups": 2}
    h = torch.randn(4, d, generator=g, dtype=F64)
    w_in = torch.randn(2 * inner + 2 * G * N + H, d, generator=g, dtype=F64)
    w_in[2 * inner:2 * inner + 2 * G * N] = 0                       # B and C are silu(0 + 0) = 0
    w = {"in": w_in, "conv": torch.ones(inner + 2 * G * N, 1, dtype=F64), "conv.b": torch.zeros(inner + 2 * G * N, dtype=F64),
         "dt_bias": torch.zeros(H, dtype=F64), "A_log": torch.zeros(H, dtype=F64), "D": torch.tensor([2.0, -1.0], dtype=F64),
         "norm": torch.ones(inner, dtype=F64), "o": torch.eye(inner, dtype=F64)[:d]}
    y = pd.state_space_mixer(h, w, c, 0.0)
    u = h @ w_in.T
    x = pd.silu(u[:, inner:2 * inner])
    t = torch.cat([2.0 * x[:, :P], -1.0 * x[:, P:]], dim=1) * pd.silu(u[:, :inner])
    want = torch.cat([pd.unit_rms(t[:, :P], 0.0), pd.unit_rms(t[:, P:], 0.0)], dim=1)[:, :d]
    assert torch.allclose(y, want, atol=1e-12)
