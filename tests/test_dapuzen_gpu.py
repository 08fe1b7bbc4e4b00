"""The Dapuzen decoder on the GPU against the plain float64 implementation in `plain_dapuzen`: each mechanism alone through its
kernels and parts, then whole models of several small shapes through the runner (prompts whole, tails token by token,
portions down to two tokens, mixed batches with pages and slots used again, long decoding), and greedy generation through
`Engine`. The test models are random; where random weights would hide a fault the inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_dapuzen as pd
import plain_model as plain
from part_harness import run_portions, runner_for

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


# ---- small shapes -----------------------------------------------------------------------------------------------------
def att(heads, kv, dim, vdim, window, scale, base=10000.0, dims=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if dims != 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
    return m


def ret(heads, dim, vdim, decay, base=10000.0, dims=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if dims != 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
    return m


def par(left, right, ls, rs, softcap):
    l = {k: v for k, v in left.items() if k != "rot"}
    if softcap:
        l["softcap"] = softcap
    return {"left": l, "right": right, "left_scale": ls, "right_scale": rs}


def ssd(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity=0, groups=1, keep=1, shared=0):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity,
                                                           "groups": {"count": groups, "keep": keep}}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(kind, mixer, mlp=None, weights_of=None):
    d = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def model(vocab, width, eps, scale, layers):
    return {"architecture": "Dapuzen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


_PA = par(att(4, 2, 16, 24, 21, 0.2), ssd(4, 12, 8, 2, 4, 3), 0.7, 1.3, 5.0)
_RA = ret(3, 16, 8, [0.9, 0.99, 0.75], dims=8)
_MA = moe(16, 4, 2, identity=2, groups=3, keep=2, shared=24)
_AA = att(4, 1, 16, 16, 13, 0.25, base=500.0)
SHAPES = {
    # every mixer and feed-forward; windows that are no multiple of the page; values wider than keys; partial rotation;
    # groups of two over experts and identity experts together; layers that run with another's tensors; a layer without
    # feed-forward
    "A": model(97, 64, 1e-5, 2.5, [
        layer("parallel", _PA, dense(48)), layer("retention", _RA, _MA), layer("attention", _AA),
        layer("parallel", _PA, dense(48), weights_of=0), layer("attention", _AA, weights_of=2),
        layer("retention", _RA, _MA, weights_of=1),
        layer("attention", att(2, 2, 24, 8, 30, 0.2, dims=12), moe(24, 3, 1))]),
    # sizes that are 1 or equal, and no multiple of 8 anywhere: one head, a window of one position and of two, a decay of
    # one (nothing is forgotten) and of zero (nothing is kept), one tap, one part of the norm, one expert, every expert taken,
    # no rotation
    "B": model(61, 40, 1e-6, 1.0, [
        layer("retention", ret(2, 6, 6, [1.0, 0.0], dims=0), moe(12, 1, 1)),
        layer("parallel", par(att(1, 1, 6, 10, 1, 0.4), ssd(1, 5, 5, 1, 1, 1), 1.0, 1.0, 0.0), moe(20, 2, 3, identity=1, shared=12)),
        layer("attention", att(1, 1, 6, 6, 2, 0.4, base=100.0, dims=2), dense(30)),
        layer("parallel", par(att(3, 3, 10, 4, 5, 0.3), ssd(6, 3, 7, 3, 2, 2), -0.5, 2.0, 1.5), None)]),
    # head size 64 with values of the keys' size, a window wider than two key blocks: prompts of a few hundred tokens send
    # the products, the gated attention and the capped attention through the tensor-core kernels, and the scans are cut
    "C": model(300, 128, 1e-6, 11.3, [
        layer("parallel", par(att(4, 2, 64, 64, 150, 0.11), ssd(4, 32, 64, 2, 4, 2), 0.8, 0.6, 30.0), dense(256)),
        layer("attention", att(6, 2, 64, 64, 70, 0.12, base=500000.0, dims=32), moe(64, 8, 3, identity=2, groups=2, keep=1, shared=96)),
        layer("retention", ret(2, 64, 64, [0.95, 0.998], base=5e5), dense(192))]),
}
SEEDS = {"A": 41, "B": 42, "C": 43}
BF16_TOL = 6e-2


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from boring_llm_b200 import DapuzenConfig, write_random_model
    made = {}

    def get(name, std=0.25):
        key = (name, std)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"dap_{name}"))
            write_random_model(d, DapuzenConfig.from_dict(SHAPES[name]), SEEDS[name], "bfloat16", std)
            made[key] = d
        return made[key]
    return get


def std_for(dtype):
    return 0.25 if dtype == "float32" else 0.1


def plain_logits(folder, tokens):
    cfg, W = plain.read_model_folder(folder)
    return pd.forward(cfg, W, tokens).numpy()


def experts_of(block):
    from boring_llm_b200.parts import RoutedExperts, SumFeedForward
    f = block.ffn
    if isinstance(f, SumFeedForward):
        f = f.parts[0]
    return f if isinstance(f, RoutedExperts) else None


def run_recording(folder, dtype, steps, max_tokens, debug_poison=False):
    """`helpers.run_inprocess` with kernels launched singly, which also returns the experts every routed layer chose:
    {layer: {(request, position): experts}}. A block that several entries of the run order name records once per entry."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    cfg, model = load_model(folder, dtype, DEV)
    cap = -(-max_tokens // 16) * 16
    runner = ModelRunner(model, EngineOptions(dtype=dtype, page_size=16, max_tokens=cap, ctx_size=cap, max_num_seqs=8,
                                              cuda_graphs=False, debug_poison=debug_poison))
    parts = [experts_of(b) for b in model.blocks]
    for p in parts:
        if p is not None:
            p.record = []
    routed = [i for i, call in enumerate(model.schedule) if parts[call.block] is not None]
    outputs, chosen, at = {}, {i: {} for i in routed}, {}
    for s in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits.shape[0]:
            outputs[s["step"]] = logits.float().cpu().numpy()
        for i in routed:                                 # the entries of the run order recorded in order
            ids = parts[model.schedule[i].block].record.pop(0).cpu()
            t = 0
            for e in s["entries"]:
                for j in range(len(e["tokens"])):
                    chosen[i][(e["id"], at.get(e["id"], 0) + j)] = ids[t]
                    t += 1
        assert all(p is None or not p.record for p in parts)
        for e in s["entries"]:
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
        for rid in s["end"]:
            runner.free_request(rid)
            at.pop(rid, None)
    runner.cache.check()
    return outputs, runner, chosen


def check_trace(folder, dtype, reqs, steps, max_tokens, what, **kw):
    """float32: the engine against the plain implementation, experts and all. bfloat16: rounding may turn a close choice
    between two experts the other way, so the plain implementation is told which experts the engine took, and the engine's
    choice must be the plain one wherever that is not close."""
    if dtype == "float32":
        outputs, runner = helpers.run_inprocess(folder, dtype, steps, max_tokens, **kw)
        chosen = None
    else:
        outputs, runner, chosen = run_recording(folder, dtype, steps, max_tokens, **kw)
    rows = helpers.collect_rows(steps, outputs)
    cfg, W = plain.read_model_folder(folder)
    errors, scale = [], 1e-6
    for rid, toks in reqs.items():
        forced = None if chosen is None else {i: torch.stack([c[(rid, p)] for p in range(len(toks))]) for i, c in chosen.items()}
        info = {}
        want = pd.forward(cfg, W, toks, forced=forced, info=info).numpy()
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        assert np.isfinite(got).all(), f"{what} {rid}: non-finite logits"
        if dtype == "float32":
            helpers.assert_close(got, want, dtype, f"{what} {rid}")
            continue
        errors.append(np.abs(got - want).max(-1))
        scale = max(scale, np.abs(want).max())
        for i, rec in info.items():
            # the engine's choice is the plain one wherever no two choice scores and no two group scores lie close together
            c, n_groups = rec["choice"], rec["groups"]
            gaps = lambda v: (torch.sort(v, dim=-1).values.diff(dim=-1).min(-1).values if v.shape[1] > 1 else torch.ones(v.shape[0], dtype=F64))
            clear = (gaps(c) > 0.03) & (gaps(c.reshape(c.shape[0], n_groups, -1).max(-1).values) > 0.03)
            same = (rec["own"].sort(-1).values == forced[i].long().sort(-1).values).all(-1)
            assert bool((same | ~clear).all()), f"{what} {rid}: layer {i} chose other experts where the choice is clear"
    if errors:
        e = np.concatenate(errors) / scale
        over = int((e > BF16_TOL).sum())
        assert over <= max(1, int(0.04 * e.size)), f"{what}: {over} of {e.size} positions differ by more than {BF16_TOL} (worst {e.max():.3f})"
        assert np.median(e) <= BF16_TOL / 4, f"{what}: median difference {np.median(e):.4f}"
    return runner


def solo_steps(reqs, cut):
    steps, n0 = [], 0
    for i, (rid, toks) in enumerate(reqs.items()):
        s = helpers.solo_trace(rid, toks, cut(toks, i), n0)
        steps += s
        n0 += len(s)
    return steps


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_whole_tails_singly_and_portions(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"r{i}": helpers.random_tokens(vocab, n, 100 + i) for i, n in enumerate([1, 2, 19, 75, 130])}
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256, f"{name} whole")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 45)), 256, f"{name} tail")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_varying(t, i)), 256, f"{name} portions")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: [2] * (len(t) // 2) + [1] * (len(t) % 2)), 256, f"{name} pairs")


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"m{i}": helpers.random_tokens(vocab, n, 200 + i) for i, n in enumerate([33, 7, 90, 41, 2, 64, 17, 58])}
    steps, peak = helpers.mixed_trace(reqs, seed=5, max_live=3)
    runner = check_trace(folder, dtype, reqs, steps, peak, f"{name} mixed", debug_poison=True)
    assert all(hw <= runner.cache.num_pages for hw in runner.cache.stats()["pages_high_water"])
    # every entry of the run order has cache layers of its own, also the entries that run with another layer's tensors
    n_paged = sum(1 for l in SHAPES[name]["layers"] if l["type"] in ("attention", "parallel"))
    n_state = sum(1 for l in SHAPES[name]["layers"] if l["type"] in ("retention", "parallel"))
    assert sum(len(g.cache_layers) for g in runner.cache.paged_groups) == n_paged
    assert sum(len(g.cache_layers) for g in runner.cache.state_groups) == n_state


def test_float32_does_not_depend_on_the_cut_or_the_batch(folders):
    folder = folders("A")
    reqs = {f"c{i}": helpers.random_tokens(97, n, 300 + i) for i, n in enumerate([50, 21, 77])}
    a, _ = helpers.run_inprocess(folder, "float32", solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256)
    whole = helpers.collect_rows(solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), a)
    steps, peak = helpers.mixed_trace(reqs, seed=9, max_live=3)
    b, _ = helpers.run_inprocess(folder, "float32", steps, peak)
    mixed = helpers.collect_rows(steps, b)
    for key, row in whole.items():
        assert np.abs(row - mixed[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_windows(folders, dtype):
    """300 tokens decoded one by one: the windows (21, 13 and 30 positions) pass over decoded tokens and page edges, the
    pages behind them go back while the request runs, and the states carry the first tokens on."""
    folder = folders("A", std_for(dtype))
    toks = helpers.random_tokens(97, 330, 7)
    steps = helpers.solo_trace("long", toks, [30] + [1] * 300)
    runner = check_trace(folder, dtype, {"long": toks}, steps, 384, "long decoding")
    assert max(runner.cache.stats()["pages_high_water"]) <= 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_shape_on_the_tensor_core_kernels(folders, dtype):
    """Prompts of 300 and 90 tokens: in bfloat16 the products run on tcgen05, the gated attention on the tcgen05 and TMA-fed
    kernels, the capped attention on the `mma.sync` kernels, the experts as grouped products, the scans of the long prompt
    in parts, and decode steps replay captured graphs."""
    folder = folders("C", 0.25 if dtype == "float32" else 0.06)
    reqs = {"w0": helpers.random_tokens(300, 300, 1), "w1": helpers.random_tokens(300, 90, 2)}
    steps = solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 24))
    check_trace(folder, dtype, reqs, steps, 512, "wide tail").check_kernels()
    steps, peak = helpers.mixed_trace(reqs, seed=3, max_live=2)
    check_trace(folder, dtype, reqs, steps, peak, "wide mixed").check_kernels()


def test_captured_steps_replay_the_same_bits(folders):
    folder = folders("A", 0.1)
    reqs = {f"g{i}": helpers.random_tokens(97, n, 400 + i) for i, n in enumerate([40, 23, 31])}
    steps, peak = helpers.mixed_trace(reqs, seed=4, max_live=3)
    twice = steps + [dict(s, step=s["step"] + len(steps)) for s in steps]
    out, runner = helpers.run_inprocess(folder, "bfloat16", twice, peak, step_graph_after=1)
    assert runner.graph_steps > 0
    for s in steps:
        if s["step"] in out:
            np.testing.assert_array_equal(out[s["step"]], out[s["step"] + len(steps)])


def test_greedy_generation_through_the_engine(folders):
    import boring_llm_b200 as b
    for name, dtype, std in (("A", "float32", 0.25), ("B", "float32", 0.25), ("A", "bfloat16", 0.1)):
        folder = folders(name, std)
        vocab = SHAPES[name]["vocab"]
        prompts = [helpers.random_tokens(vocab, n, 500 + n) for n in (5, 26, 61)]
        eng = b.Engine(folder, dtype=dtype, ctx_size=128, max_num_seqs=2, max_tokens=192, prefill_chunk=16)
        outs = eng.generate(prompts, n_predict=12, ignore_eos=True)
        for p, o in zip(prompts, outs):
            assert len(o) == 12
            logits = plain_logits(folder, p + o)
            for i, tok in enumerate(o):
                row = logits[len(p) - 1 + i]
                gap = row.max() - row[tok]
                assert gap <= (1e-4 if dtype == "float32" else 0.05) * np.abs(logits).max(), (name, i, gap)


def test_layer_streams_one_by_one(folders):
    """float32: the residual stream behind every entry of the run order against the plain implementation's."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    for name in ("A", "B"):
        folder = folders(name)
        toks = helpers.random_tokens(SHAPES[name]["vocab"], 70, 3)
        cfg, W = plain.read_model_folder(folder)
        _, want = pd.forward(cfg, W, toks, streams=True)
        _, model = load_model(folder, "float32", DEV)
        runner = ModelRunner(model, EngineOptions(dtype="float32", max_tokens=128, ctx_size=128, max_num_seqs=2, cuda_graphs=False))
        model.keep_streams = []
        runner.step([StepEntry("s", toks, [])])
        assert len(model.keep_streams) == len(cfg["layers"])
        for i, got in enumerate(model.keep_streams):
            w = want[i].numpy()
            assert np.abs(got.cpu().numpy() - w).max() <= 1e-4 * np.abs(w).max(), (name, i)


def test_the_trace_program_on_a_model_folder(folders, tmp_path):
    reqs = {f"t{i}": helpers.random_tokens(97, n, 600 + i) for i, n in enumerate([30, 12, 45])}
    steps, peak = helpers.mixed_trace(reqs, seed=2, max_live=2)
    outputs = helpers.run_trace_program(folders("A"), "float32", steps, peak, str(tmp_path / "out"), 97)
    rows = helpers.collect_rows(steps, outputs)
    for rid, t in reqs.items():
        helpers.assert_close(np.stack([rows[(rid, i)] for i in range(len(t))]), plain_logits(folders("A"), t), "float32", rid)


# ---- mechanisms alone --------------------------------------------------------------------------------------------------
def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=F64) * scale


def dev(t, dtype=torch.float32):
    return t.to(dtype).to(DEV).contiguous()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def paged(x, page, n_pages, order):
    """x [T, G, d] of one request -> (cache [n_pages + 1, G, page, d] filled with NaN elsewhere, block table row)."""
    T, G, d = x.shape
    cache = torch.full((n_pages + 1, G, page, d), float("nan"), dtype=torch.float32)
    table = []
    for i in range(-(-T // page)):
        p = order[i]
        table.append(p)
        n = min(page, T - i * page)
        cache[p, :, :n] = x[i * page:i * page + n].permute(1, 0, 2).float()
        cache[p, :, n:] = 0.0
    return cache, table


def attention_oracle(q, k, v, scale, window, cap):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]."""
    o = pd.softmax_attention(q.permute(1, 0, 2), k.permute(1, 0, 2), v.permute(1, 0, 2), scale, pd.window_mask(q.shape[0], window), cap)
    return o.permute(1, 0, 2)


@pytest.mark.parametrize("H,G,dk,dv,window,cap", [(4, 2, 16, 16, 0, 4.0), (3, 1, 24, 8, 21, 2.0), (2, 2, 8, 40, 16, 0.0), (1, 1, 32, 32, 1, 7.0)])
def test_capped_attention_kernel_with_planted_keys(H, G, dk, dv, window, cap):
    """Keys at chosen distances get a score far beyond the cap: just inside and just outside the window, at page borders,
    the first token, far back. With the cap their weight is bounded by e^cap against e^score; a kernel without the cap, or
    one that caps after the mask, gives other rows. Pages are scattered and the unused rest of the pool is NaN."""
    from boring_llm_b200.kernels import ops
    T, page = 150, 16
    q, k, v = rnd(T, H, dk, seed=1), rnd(T, G, dk, seed=2), rnd(T, G, dv, seed=3)
    for qi, kj in ((149, 0), (149, 149 - (window or 100) + 1), (149, 149 - (window or 100)), (100, 96), (100, 95), (64, 63),
                   (64, 48), (64, 47), (33, 32), (16, 15), (16, 0)):
        kj = max(0, kj)
        k[kj] = k[kj] * 0 + q[qi, 0] / q[qi, 0].norm() * 9.0
    want = attention_oracle(q, k, v, 0.7, window, cap)
    if cap and window != 1:
        assert (attention_oracle(q, k, v, 0.7, window, 0.0) - want).abs().max() > 1e-2
    order = list(np.random.default_rng(0).permutation(12))
    kc, table = paged(k, page, 12, order)
    vc, _ = paged(v, page, 12, order)
    out = torch.empty(T, H * dv, device=DEV)
    at = 0
    tb = i32([table + [-1] * (16 - len(table))])
    for n in [90, 50] + [1] * 10:                        # two portions, then token by token
        sl = slice(at, at + n)
        o = torch.empty(n, H * dv, device=DEV)
        ops.attention_plain(dev(q[sl].reshape(n, H * dk)), kc.to(DEV), vc.to(DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                            i32([0, n]), i32([at + n]), tb, o, H, window, 0.7, None, None, softcap=cap)
        out[sl] = o
        at += n
    got = out.cpu().numpy().reshape(T, H, dv)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want.numpy(), atol=3e-5, rtol=2e-4)


@pytest.mark.parametrize("dh,H,G,window,cap", [(64, 4, 2, 0, 3.0), (32, 2, 2, 40, 1.5), (96, 4, 1, 150, 6.0), (128, 2, 1, 0, 2.0)])
def test_capped_scores_in_the_tensor_core_attention_kernels(dh, H, G, window, cap):
    """The bfloat16 tensor-core kernels (prompt tiles on `mma.sync` and, at head sizes 64 and 128, on tcgen05; single tokens
    in one slice, in a cluster's slices, merged through scratch, and fed by TMA) with a cap well below the raw scores' spread, so that a
    kernel without the cap gives visibly other rows."""
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts.attention import attention_plan
    T, page = 300, 16
    bf = lambda x: x.to(torch.bfloat16).to(F64)
    q, k, v = bf(rnd(T, H, dh, seed=1)), bf(rnd(T, G, dh, seed=2)), bf(rnd(T, G, dh, seed=3))
    scale = 2.0 * dh ** -0.5
    want = attention_oracle(q, k, v, scale, window, cap).reshape(T, H * dh)
    assert (attention_oracle(q, k, v, scale, window, 0.0).reshape(T, H * dh) - want).abs().max() > 0.2
    n_pages = 24
    order = list(np.random.default_rng(1).permutation(n_pages))
    kc, table = paged(k, page, n_pages, order)
    vc, _ = paged(v, page, n_pages, order)
    kc, vc = torch.nan_to_num(kc, nan=0.0).to(torch.bfloat16).to(DEV), torch.nan_to_num(vc, nan=0.0).to(torch.bfloat16).to(DEV)
    qg = q.reshape(T, H * dh).to(torch.bfloat16).to(DEV).contiguous()
    tol = dict(atol=2e-2 * float(want.abs().max()), rtol=2e-2)
    plan = attention_plan([T], [T])
    tb = i32([table + [-1] * (32 - len(table))])
    out = torch.zeros(T, H * dh, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill(qg, kc, vc, i32([0, T]), i32([T]), tb, i32(plan.arrays["tiles64"]), out, H, window, scale, softcap=cap)
    np.testing.assert_allclose(out.float().cpu().numpy(), want.numpy(), **tol)
    if ops.attention_prefill_tc_supported(torch.bfloat16, dh, page):
        out = torch.zeros(T, H * dh, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(qg, kc, vc, i32([0, T]), i32([T]), tb, i32(plan.arrays["tiles128"]), out, H, window, scale, softcap=cap)
        ops.check_status()
        np.testing.assert_allclose(out.float().cpu().numpy(), want.numpy(), err_msg="tcgen05", **tol)
    ctxs = [300, 170, 33]
    rows = [c - 1 for c in ctxs]
    qd = qg[rows].contiguous()
    tb3 = tb.repeat(3, 1).contiguous()
    for splits, scratch in ((1, False), (4, False), (5, True)):
        out = torch.zeros(3, H * dh, dtype=torch.bfloat16, device=DEV)
        sc = torch.empty(ops.attention_decode_scratch(3, H, dh, splits), device=DEV) if scratch else None
        ops.attention_decode(qd, kc, vc, i32([0, 1, 2, 3]), i32(ctxs), tb3, i32([0, 1, 2]), splits, out, H, window, scale, sc, softcap=cap)
        np.testing.assert_allclose(out.float().cpu().numpy(), want[rows].numpy(), err_msg=f"decode, {splits} slices", **tol)
    if ops.attention_decode_tma_supported(torch.bfloat16, dh, page):
        for splits in (1, 3):
            out = torch.zeros(3, H * dh, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_tma(qd, kc, vc, i32([0, 1, 2, 3]), i32(ctxs), tb3, i32([0, 1, 2]), splits, out, H, window, scale, softcap=cap)
            ops.check_status()
            np.testing.assert_allclose(out.float().cpu().numpy(), want[rows].numpy(), err_msg=f"TMA decode, {splits} slices", **tol)


def load_part(part, W, dtype):
    part.load({part.names[k]: v for k, v in W.items()}, dtype, DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,n_rot,decay", [(2, 16, 8, 8, [0.9, 1.0]), (3, 20, 9, 20, [0.5, 0.99, 0.0]), (1, 64, 40, 0, [0.97])])
def test_retention_part_whole_in_portions_and_with_a_far_first_token(dtype, H, dk, dv, n_rot, decay):
    """The retention mixer through the runner: whole, then in portions down to single tokens in a slot that another request
    left dirty. With a decay of one the first token, whose key and value are made large, still stands in every later
    row; rotation of the first n_rot values only."""
    from boring_llm_b200.parts import Retention, RotaryTable
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, n, eps = 40, 90, 1e-5
    names = {k: k for k in ("wq", "wk", "wv", "wg", "wo")}
    part = Retention(d, H, dk, dv, decay, RotaryTable(dk, 300.0, n_rot=n_rot) if n_rot else None, eps, names)
    W = {"wq": rnd(H * dk, d, seed=1, scale=0.3), "wk": rnd(H * dk, d, seed=2, scale=0.3), "wv": rnd(H * dv, d, seed=3, scale=0.3),
         "wg": rnd(H * dv, d, seed=4, scale=0.3), "wo": rnd(d, H * dv, seed=5, scale=0.3)}
    W = {k: v.to(tdt) for k, v in W.items()}
    load_part(part, W, tdt)
    x = rnd(n, d, seed=9)
    x[0] *= 4.0                                           # the first token: a large key and value
    x = x.to(tdt)
    cfg = {"heads": H, "dim": dk, "vdim": dv, "decay": decay}
    if n_rot:
        cfg["rot"] = {"base": 300.0, "dims": n_rot}
    want = pd.retention_mixer(x.double(), {k[1:]: v.double() for k, v in W.items()}, cfg, eps, torch.arange(n))
    lost = pd.retention_mixer(torch.cat([x[:1].double() * 0, x[1:].double()]), {k[1:]: v.double() for k, v in W.items()}, cfg, eps, torch.arange(n))
    if decay[-1] == 1.0:
        assert (lost[-1] - want[-1]).abs().max() > 1e-2 * want[-1].abs().max()       # losing the first token would show at the end

    def body(ctx, h):
        res = torch.zeros((h.shape[0], d), dtype=torch.float32, device=DEV)
        part.forward(ctx, h.to(tdt), res, 0, True)
        return res

    r = runner_for(x.to(DEV), body, [part.cache_spec()], dtype=dtype, max_tokens=128)
    tol = 2e-4 if dtype == "float32" else 4e-2
    whole = run_portions(r, "a", n, [n])
    assert (whole.double().cpu() - want).abs().max() <= tol * want.abs().max(), "whole"
    cut = run_portions(r, "b", n, [2, 31, 1, 17, 2, 1, 1, 35])            # the slot of request a is used again
    assert (cut.double().cpu() - want).abs().max() <= tol * want.abs().max(), "portions"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,P,N,G,taps,parts", [(4, 12, 8, 2, 4, 3), (1, 5, 5, 1, 1, 1), (6, 4, 20, 3, 2, 8), (2, 64, 64, 1, 3, 2)])
def test_state_space_part_whole_and_in_portions_shorter_than_the_taps(dtype, H, P, N, G, taps, parts):
    """The state-space mixer through the runner: whole, then in portions of one and two tokens (shorter than the
    convolution's taps, so its inputs come from the slot), in a slot that another request left dirty."""
    from boring_llm_b200.parts import StateSpaceDuality
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, n, eps = 48, 80, 1e-5
    inner, C = H * P, H * P + 2 * G * N
    names = {k: k for k in ("w_in", "conv", "conv_bias", "dt_bias", "a_log", "skip", "norm", "wo")}
    part = StateSpaceDuality(d, H, P, N, G, taps, parts, eps, names)
    W = {"w_in": rnd(2 * inner + 2 * G * N + H, d, seed=1, scale=0.25), "conv": rnd(C, taps, seed=2, scale=0.6),
         "conv_bias": rnd(C, seed=3, scale=0.3), "dt_bias": rnd(H, seed=4), "a_log": rnd(H, seed=5) - 1.0,
         "skip": rnd(H, seed=6), "norm": rnd(inner, seed=7, scale=0.3) + 1.0, "wo": rnd(d, inner, seed=8, scale=0.3)}
    W = {k: v.to(tdt) for k, v in W.items()}
    load_part(part, W, tdt)
    x = rnd(n, d, seed=9).to(tdt)
    cfg = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": parts}
    pw = {"in": W["w_in"], "conv": W["conv"], "conv.b": W["conv_bias"], "dt_bias": W["dt_bias"], "A_log": W["a_log"], "D": W["skip"],
          "norm": W["norm"], "o": W["wo"]}
    want = pd.state_space_mixer(x.double(), {k: v.double() for k, v in pw.items()}, cfg, eps)

    def body(ctx, h):
        res = torch.zeros((h.shape[0], d), dtype=torch.float32, device=DEV)
        part.forward(ctx, h.to(tdt), res, 0, True)
        return res

    r = runner_for(x.to(DEV), body, [part.cache_spec()], dtype=dtype, max_tokens=128)
    tol = 3e-4 if dtype == "float32" else 5e-2
    whole = run_portions(r, "a", n, [n])
    assert (whole.double().cpu() - want).abs().max() <= tol * want.abs().max(), "whole"
    cut = run_portions(r, "b", n, [1, 2, 1, 1, 30, 2, 1, 17, 1, 24])
    assert (cut.double().cpu() - want).abs().max() <= tol * want.abs().max(), "portions"


def test_long_portions_of_both_recurrences_cut_into_parts():
    """A portion of 600 tokens behind 40 cached ones: the scan cuts it into parts that run side by side; the result and
    the state it leaves are those of the walk in one piece."""
    from boring_llm_b200.kernels import ops
    H, G, dk, dv, T0, T1 = 4, 2, 32, 16, 40, 600
    T = T0 + T1
    q, k, v = rnd(T, G * dk, seed=1, scale=0.3), rnd(T, G * dk, seed=2, scale=0.3), rnd(T, H * dv, seed=3)
    a = torch.rand(T, H, generator=torch.Generator().manual_seed(4), dtype=F64) * 0.2 + 0.8
    want = pd.decayed_outer_recurrence(q.reshape(T, G, dk).permute(1, 0, 2).repeat_interleave(H // G, 0),
                                       k.reshape(T, G, dk).permute(1, 0, 2).repeat_interleave(H // G, 0),
                                       v.reshape(T, H, dv).permute(1, 0, 2), a.T)
    want = want.permute(1, 0, 2).reshape(T, H * dv)
    decay = dev(a[:, :, None].expand(T, H, dk).reshape(T, H * dk))
    for parts in (1, 5):
        state = torch.zeros((2, H * dk * dv), device=DEV)
        out = torch.empty((T, H * dv), device=DEV)
        for lo, hi, p in ((0, T0, 1), (T0, T, parts)):
            ops.recurrent_scan(ops.RULE_GLA, dev(q[lo:hi]), dev(k[lo:hi]), dev(v[lo:hi]), decay[lo:hi].contiguous(), None, 1.0, state,
                               i32([1]), i32([0, hi - lo]), out[lo:hi], H, G, dk, dv, parts=p)
        assert (out.double().cpu() - want).abs().max() <= 2e-4 * want.abs().max(), parts


def test_prep_and_finish_kernels_of_the_recurrences():
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts import RotaryTable
    # rotation of the first values of each head, the key's factor, the heads' decays
    T, H, dk, n_rot = 5, 3, 10, 6
    proj = rnd(T, 2 * H * dk + 7, seed=1)
    positions = [37, 5, 16, 0, 1000]
    rt = RotaryTable(dk, 200.0, n_rot=n_rot).to(DEV)
    q, k, decay = ops.rope_decay_prep(dev(proj), H * dk, i32(positions), rt.inv_freq, rt.rot_half, dev(torch.tensor([0.5, 0.25, 1.0], dtype=F64)),
                                      0.3, H, dk)
    pos = torch.tensor(positions)
    wq = pd.rotate_halves(proj[:, :H * dk].reshape(T, H, dk).permute(1, 0, 2), pos, 200.0, n_rot).permute(1, 0, 2).reshape(T, -1)
    wk = pd.rotate_halves(proj[:, H * dk:2 * H * dk].reshape(T, H, dk).permute(1, 0, 2), pos, 200.0, n_rot).permute(1, 0, 2).reshape(T, -1) * 0.3
    assert (q.double().cpu() - wq).abs().max() <= 2e-4 and (k.double().cpu() - wk).abs().max() <= 1e-4
    assert decay.cpu().reshape(T, H, dk)[2, :, 3].tolist() == [0.5, 0.25, 1.0]
    # step sizes, decays and scaled inputs of the state-space recurrence; pre-activations far out on both sides
    H, N, dv = 3, 4, 5
    raw = torch.tensor([[-30.0, 0.0, 50.0], [1.0, -2.0, 3.0]], dtype=F64)
    bias, a_log, x = rnd(H, seed=2), rnd(H, seed=3), rnd(2, H * dv + 3, seed=4)
    decay, v = ops.ssd_prep(dev(raw), dev(bias), dev(torch.exp(a_log)), dev(x)[:, :H * dv], H, N, dv)
    dt = pd.softplus(raw + bias)
    assert torch.allclose(decay.double().cpu().reshape(2, H, N)[:, :, 1], torch.exp(-torch.exp(a_log) * dt), rtol=1e-5, atol=1e-7)
    assert torch.allclose(v.double().cpu().reshape(2, H, dv), dt[:, :, None] * x[:, :H * dv].reshape(2, H, dv), rtol=1e-5, atol=1e-6)
    # the gate in front of the norm, the norm in parts that span heads or cut them, the skip term
    T, Hh, dv, parts = 4, 4, 6, 3
    width = Hh * dv
    o, xx, z, w, skip = rnd(T, width, seed=5), rnd(T, width + 2, seed=6), rnd(T, width + 1, seed=7), rnd(width, seed=8) + 1.0, rnd(Hh, seed=9)
    u = (o + skip.repeat_interleave(dv) * xx[:, :width]) * pd.silu(z[:, :width])
    want = pd.unit_rms(u.reshape(T, parts, width // parts), 1e-5).reshape(T, width) * w
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        y = torch.empty((T, width), dtype=dtype, device=DEV)
        ops.gated_group_norm(dev(o), dev(xx)[:, :width], dev(skip), dv, dev(z)[:, :width], dev(w), parts, 1e-5, y)
        assert (y.double().cpu() - want).abs().max() <= tol * want.abs().max(), dtype
    gated_after = pd.unit_rms((o + skip.repeat_interleave(dv) * xx[:, :width]).reshape(T, parts, -1), 1e-5).reshape(T, width) * w * pd.silu(z[:, :width])
    assert (gated_after - want).abs().max() > 0.1          # the other order would show
    # the unit RMS per head without a weight, times a SiLU gate
    y = torch.empty((T, width), device=DEV)
    ops.head_norm_gate(dev(o), None, dev(z)[:, :width], ops.GATE_SILU, 1e-5, y, Hh, dv)
    want = pd.unit_rms(o.reshape(T, Hh, dv), 1e-5).reshape(T, width) * pd.silu(z[:, :width])
    assert (y.double().cpu() - want).abs().max() <= 1e-5 * want.abs().max()


def test_xielu_pair_sum_and_row_gate():
    from boring_llm_b200.kernels import ops
    p, q = 0.4, -1.1
    args = ops.xielu_args(p, q, DEV)
    for n in (13, 24):
        z = rnd(7, n + 3, seed=n, scale=3.0)
        want = pd.xielu(z[:, :n], p, q)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            out = torch.empty((7, n), dtype=dtype, device=DEV)
            ops.xielu(dev(z)[:, :n], out, args)
            assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max(), (n, dtype)
    x, a, b = rnd(5, 12, seed=1), rnd(5, 12, seed=2), rnd(5, 12, seed=3)
    xs = dev(x)
    ops.add_scaled_pair(xs, dev(a), 0.8, dev(b), -0.5)
    assert (xs.double().cpu() - (x + 0.8 * a - 0.5 * b)).abs().max() <= 1e-5
    g = rnd(5, 3, seed=4, scale=2.0)
    xs = dev(x)
    ops.add_row_gated(xs, dev(a), dev(g)[:, 1:2])
    assert (xs.double().cpu() - (x + torch.sigmoid(g[:, 1:2]) * a)).abs().max() <= 1e-5


def test_scalar_norm_part():
    from boring_llm_b200.parts import RMSNorm
    for d in (40, 41):
        part = RMSNorm(d, 1e-5, {"weight": "w"}, scalar_weight=True)
        assert part.local_specs()["weight"].shape == ()
        part.load({"w": torch.tensor(1.75, dtype=torch.bfloat16)}, torch.float32, DEV)
        x = rnd(6, d, seed=d)
        r = runner_for(x.float().to(DEV), lambda ctx, h: part.forward(ctx, h), dtype="float32")
        got = run_portions(r, "a", 6, [6])
        assert (got.double().cpu() - pd.scalar_rms_norm(x.float().double(), torch.tensor(1.75, dtype=F64), 1e-5)).abs().max() <= 1e-5


@pytest.mark.parametrize("E,n_id,top,groups,keep", [(4, 2, 2, 3, 2), (8, 2, 4, 2, 1), (1, 0, 1, 1, 1), (3, 3, 6, 1, 1), (5, 1, 3, 6, 4)])
def test_softmax_routing_with_groups_and_identity_experts(E, n_id, top, groups, keep):
    """The choice against the plain one on logits whose choice scores are well apart (negative ones included, so that a
    closed group counted as zero would win), and the weights: the softmax over ALL router outputs, not renormalised."""
    from boring_llm_b200.kernels import ops
    T, n = 64, E + n_id
    z = rnd(T, n + 2, seed=E * 10 + n_id, scale=2.0)
    corr = rnd(n, seed=5, scale=0.5) - 1.0                   # choice scores are negative
    s = torch.softmax(z[:, :n].float().double(), dim=-1)
    want = pd.choose_experts(s, corr.float().double(), top, groups, keep)
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((T, top), dtype=torch.float32, device=DEV)
    ops.moe_route(dev(z)[:, :n], dev(corr), top, groups, keep, ids, wts, ops.SCORE_SOFTMAX, 1)
    c = s + corr.float().double()
    srt = torch.sort(c, dim=-1, descending=True).values
    clear = (srt[:, :-1] - srt[:, 1:]).min(-1).values > 1e-5 if n > 1 else torch.ones(T, dtype=torch.bool)
    assert clear.sum() > T // 2
    assert torch.equal(ids.cpu().long()[clear], want[clear])
    assert torch.allclose(wts.double().cpu()[clear], torch.gather(s, 1, want)[clear], rtol=1e-5, atol=1e-7)
    if (groups, keep) == (2, 1):                               # with every group open the choice would differ somewhere
        assert not torch.equal(pd.choose_experts(s, corr.float().double(), top, 1, 1), want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_part_with_identity_experts_and_a_gated_shared_expert(dtype):
    """The feed-forward alone with the choice given to the plain implementation: rows of real experts, rows that are the
    input itself, and the shared expert behind its gate; 200 rows send bfloat16 through the grouped tensor-core products."""
    from boring_llm_b200.parts import GluMLP, RoutedExperts, RowGatedFeedForward, SumFeedForward
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, ff, E, n_id, top, sff = 64, 24, 3, 2, 3, 40
    names = {"router": "router", "correction": "correction", "gate": "shared.sg"}
    W = {"router": rnd(E + n_id, d, seed=1, scale=0.3), "correction": rnd(E + n_id, seed=2, scale=0.1),
         "shared.gate": rnd(sff, d, seed=3, scale=0.2), "shared.up": rnd(sff, d, seed=4, scale=0.2), "shared.down": rnd(d, sff, seed=5, scale=0.2),
         "shared.sg": rnd(1, d, seed=6, scale=0.3)}
    for e in range(E):
        names.update({f"gate{e}": f"e{e}.gate", f"up{e}": f"e{e}.up", f"down{e}": f"e{e}.down"})
        W.update({f"e{e}.gate": rnd(ff, d, seed=10 + e, scale=0.2), f"e{e}.up": rnd(ff, d, seed=20 + e, scale=0.2),
                  f"e{e}.down": rnd(d, ff, seed=30 + e, scale=0.2)})
    W = {k: v.to(tdt) for k, v in W.items()}
    experts = RoutedExperts(d, ff, E, top, {k: v for k, v in names.items() if k != "gate"}, score="softmax", group_score="max", n_identity=n_id)
    shared = RowGatedFeedForward(d, GluMLP(d, sff, {"w_gate": "shared.gate", "w_up": "shared.up", "w_down": "shared.down"}), {"gate": "shared.sg"})
    part = SumFeedForward([experts, shared])
    part.load(W, tdt, DEV)
    experts.record = []
    for n in (9, 200):
        x = rnd(n, d, seed=40 + n).to(tdt)

        def body(ctx, h):
            res = torch.zeros((h.shape[0], d), dtype=torch.float32, device=DEV)
            part.forward(ctx, h.to(tdt), res)
            return res

        r = runner_for(x.to(DEV), body, dtype=dtype, max_tokens=256)
        got = run_portions(r, "a", n, [n])
        ids = experts.record.pop().cpu()
        assert int((ids >= E).sum()) > 0 and int((ids < E).sum()) > 0
        cfg = {"router": {"experts": E, "top": top, "identity": n_id}, "shared": {"ff": sff}}
        want = pd.routed_experts(x.double(), {k: v.double() for k, v in W.items()}, cfg, forced=ids)
        tol = 1e-4 if dtype == "float32" else 4e-2
        assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max(), n
