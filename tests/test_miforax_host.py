"""Miforax without a GPU: configuration keys and errors, declared tensors, the run order of layers that read another
layer's cached rows, what the cache keeps for them, the stretched rotation angles, the random table of experts, and the
plain implementation against closed forms."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_miforax as pm
from boring_llm_b200 import ConfigError, MiforaxConfig
from boring_llm_b200.cache import CacheManager
from boring_llm_b200.models import build_model
from boring_llm_b200.models.miforax import cache_windows
from boring_llm_b200.parts import RotaryTable
from boring_llm_b200.weights import TensorSpec, INT_TABLE
from boring_llm_b200.weights.random_init import random_tensor

SC = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def mixer(window, kv_from=None, heads=2, scaling=SC):
    m = {"heads": heads, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3,
         "rot": {"base": 1000.0, "dims": 4, "scaling": scaling}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CFG = {"architecture": "Miforax", "vocab": 90, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.5}, "layers": [
    {"type": "latent_attention", "mixer": mixer(24), "mlp": {"kind": "dense", "ff": 40}},
    {"type": "latent_attention", "mixer": mixer(9, kv_from=0, heads=3),
     "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 1.25}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 20, "limit": 2.0}}},
    {"type": "latent_attention", "mixer": mixer(30), "mlp": None},
    {"type": "latent_attention", "mixer": mixer(0, kv_from=2), "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0},
                                                                      "router": {"experts": 3, "top": 1}}}]}


def test_config_round_trip_and_fields():
    cfg = MiforaxConfig.from_dict(CFG)
    assert cfg.to_dict() == CFG
    assert cfg.embedding_scale == 5.5 and cfg.norm_eps == 1e-5
    m = cfg.layers[1].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, m.window, m.kv_from) == (3, 8, 4, 6, 10, 12, 0.3, 9, 0)
    assert (m.scaling.factor, m.scaling.original, m.scaling.fast, m.scaling.slow) == (4.0, 64.0, 8.0, 1.0)
    f = cfg.layers[1].mlp
    assert (f.ff, f.limit, f.experts, f.top, f.shared_ff, f.shared_limit) == (16, 1.25, 6, 2, 20, 2.0)
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.shared_ff == 0 and cfg.layers[3].mixer.window == 0


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "attention", "unknown layer type"),
    (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("layers", 0, "mixer", "rot", "base"), 1.0, "rot.base"),
    (("layers", 1, "mixer", "kv_from"), 1, "earlier layer"),
    (("layers", 3, "mixer", "kv_from"), 1, "no rows of its own"),
    (("layers", 1, "mixer", "kv_rank"), 16, "differ"),
    (("layers", 1, "mlp", "router", "top"), 7, "out of 6"),
    (("layers", 1, "mlp", "expert", "limit"), 0.0, "limit"),
    (("layers", 0, "mlp", "kind"), "swiglu", "not supported"),
    (("layers", 0, "mixer", "mask", "size"), -1, "mask.size"),
    (("norm", "eps"), 0.0, "norm.eps"),
])
def test_config_errors_name_the_key(path, value, word):
    d = copy.deepcopy(CFG)
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        MiforaxConfig.from_dict(d)


def test_declared_tensors_run_order_and_caches():
    cfg = MiforaxConfig.from_dict(CFG)
    model = build_model(cfg)
    specs = model.tensor_specs()
    for name, shape in {"embed": (90, 32), "head": (90, 32), "final.norm": (32,), "l0.norm1": (32,), "l0.norm2": (32,),
                        "l0.mix.dq": (10, 32), "l0.mix.dq.norm": (10,), "l0.mix.uq": (24, 10), "l0.mix.dkv": (16, 32),
                        "l0.mix.dkv.norm": (12,), "l0.mix.uk": (16, 12), "l0.mix.uv": (12, 12), "l0.mix.sink": (2,),
                        "l0.mix.g": (12, 32), "l0.mix.o": (32, 12), "l0.mlp.gate": (40, 32), "l0.mlp.down": (32, 40),
                        "l1.mix.uq": (36, 10), "l1.mix.uk": (24, 12), "l1.mix.sink": (3,), "l1.mlp.table": (90, 2),
                        "l1.mlp.e5.up": (16, 32), "l1.mlp.shared.down": (32, 20), "l3.mlp.table": (90, 1), "l3.mlp.e2.gate": (8, 32)}.items():
        assert tuple(specs[name].shape) == shape, name
    for absent in ("l1.mix.dkv", "l1.mix.dkv.norm", "l3.mix.dkv", "l2.norm2", "l3.mlp.shared.gate", "l0.mlp.table"):
        assert absent not in specs
    # layers 1 and 3 read the rows of layers 0 and 2: two cache layers, the readers do not write
    assert [(c.block, c.cache, c.write_cache) for c in model.schedule] == [(0, 0, True), (1, 0, False), (2, 1, True), (3, 1, False)]
    # a cache layer keeps the widest window among its layers, everything if one of them sees everything
    assert cache_windows(cfg) == {0: 24, 2: 0}
    s0, s1 = model.cache_specs()
    assert (s0.n_kv_heads, s0.head_dim, s0.value_dim, s0.window, s0.values_in_keys) == (1, 16, 12, 24, True) and s1.window == 0
    mgr = CacheManager(model.cache_specs(), page_size=16, capacity_tokens=160, max_requests=2)
    mgr.add_request("a")
    mgr.reserve("a", 100)
    mgr.commit("a", 100)
    held = [sum(1 for p in t if p >= 0) for t in mgr._requests["a"].tables]
    assert sorted(held) == [3, 7], held           # a window of 24 before position 100 begins at 77: pages 4 to 6; all seven pages without


def test_stretched_angles_against_the_closed_form():
    """Pairs below `lo` keep base^(-2i/n); pairs above `hi` get it divided by the factor; between, the ramp."""
    n, base = 16, 500000.0
    sc = {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}
    table = RotaryTable.yarn(n, base, n, sc["factor"], sc["original"], sc["fast"], sc["slow"])
    f, m = pm.yarn_frequencies(n, base, sc)
    assert np.allclose(table.inv_freq_host[: n // 2], f.numpy(), rtol=1e-6) and abs(table.mscale - m) < 1e-12
    assert abs(m - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    plain_f = np.array([base ** (-2.0 * i / n) for i in range(n // 2)])
    lo = max(math.floor(n * math.log(512 / (2 * math.pi * 32.0)) / (2 * math.log(base))), 0)
    hi = min(math.ceil(n * math.log(512 / (2 * math.pi * 1.0)) / (2 * math.log(base))), n - 1)
    assert 0 <= lo < hi < n // 2                      # this choice of constants has all three regimes
    assert np.allclose(f.numpy()[: lo + 1], plain_f[: lo + 1]) and np.allclose(f.numpy()[hi:], plain_f[hi:] / 8.0)
    assert all(plain_f[i] / 8.0 < f[i] < plain_f[i] for i in range(lo + 1, hi))
    # tables with different stretching do not share a step's memo entry
    other = RotaryTable.yarn(n, base, n, 4.0, sc["original"], sc["fast"], sc["slow"])
    assert table.variant != other.variant and RotaryTable(n, base).variant is None


def test_random_table_of_experts_has_rows_of_different_numbers():
    t = random_tensor("l1.mlp.table", TensorSpec((200, 3), INT_TABLE, high=5), seed=3)
    assert t.dtype == torch.int32 and int(t.min()) >= 0 and int(t.max()) < 5
    assert all(len(set(row)) == 3 for row in t.tolist()) and len({row[0] for row in t.tolist()}) == 5


def test_plain_attention_closed_forms():
    # a window of one: every token sees itself only, so the weights are e^s / (e^s + e^sink)
    q, k, v = torch.ones(1, 4, 3, dtype=pm.F64), torch.ones(1, 4, 3, dtype=pm.F64), torch.arange(8.0, dtype=pm.F64).view(1, 4, 2)
    sink = torch.tensor([0.7], dtype=pm.F64)
    out = pm.sink_softmax_attention(q, k, v, 0.5, sink, pm.window_mask(4, 1))
    w = math.exp(1.5) / (math.exp(1.5) + math.exp(0.7))
    assert torch.allclose(out, v * w)
    # without a sink and with equal scores: the mean of the visible values; a window of 2 sees one token back
    out = pm.sink_softmax_attention(q, k, v, 0.5, None, pm.window_mask(4, 2))
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], (v[0, 2] + v[0, 3]) / 2)
    assert pm.window_mask(5, 3).int().sum(1).tolist() == [1, 2, 3, 3, 3] and pm.window_mask(3, 0).int().sum(1).tolist() == [1, 2, 3]
    # the clamped expert: the gate is cut above only, the up value on both sides, and one is added to it
    h = torch.tensor([[1.0]], dtype=pm.F64)
    one = lambda g, u: pm.clamped_expert(h, torch.tensor([[g]], dtype=pm.F64), torch.tensor([[u]], dtype=pm.F64),
                                         torch.ones(1, 1, dtype=pm.F64), 2.0).item()
    assert abs(one(5.0, 0.0) - 2.0 / (1 + math.exp(-3.404))) < 1e-12
    assert abs(one(-5.0, 9.0) - (-5.0 / (1 + math.exp(8.51)) * 3.0)) < 1e-12
    assert abs(one(1.0, -9.0) - (1.0 / (1 + math.exp(-1.702)) * -1.0)) < 1e-12
