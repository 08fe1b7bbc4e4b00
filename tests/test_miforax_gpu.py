"""The Miforax decoder on the GPU against the plain float64 implementation in `plain_miforax`: each mechanism alone through
its kernels (the plain ones and the tensor-core ones), then whole models of several small shapes through the runner (prompts
whole, tails token by token, portions down to two tokens, mixed batches with pages used again), and greedy generation
through `Engine`. The test models are random; where random weights would hide a fault the inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_miforax as pm
import plain_model as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


# ---- small shapes -----------------------------------------------------------------------------------------------------
def mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base=10000.0, dims=None, scaling=None, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(m, mlp=None):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def model(vocab, width, eps, scale, layers):
    return {"architecture": "Miforax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


SHAPES = {
    # sizes in multiples of 8 (bfloat16 runs head-major on the tensor cores); windows that are no multiple of the page and
    # differ between a layer and the layer whose rows it reads; a layer that sees everything; a layer without feed-forward;
    # two and one expert a token, with and without the expert that every token uses
    "A": model(101, 64, 1e-5, 3.0, [
        layer(mixer(4, 16, 8, 24, 24, 32, 20, scaling=YARN), dense(48)),
        layer(mixer(2, 24, 8, 8, 16, 32, 13, scaling=YARN, kv_from=0), moe(24, 1.0, 5, 2, (40, 2.0))),
        layer(mixer(3, 8, 16, 16, 32, 48, 0, base=500.0, dims=8)),
        layer(mixer(5, 8, 16, 8, 8, 48, 37, base=500.0, dims=8, kv_from=2), moe(16, 0.5, 3, 1))]),
    # sizes that are 1 or equal, and no multiple of 8 anywhere (plain kernels in both dtypes): one head, a window of one
    # position (a token sees itself only) and of two, every expert taken, one expert
    "B": model(61, 40, 1e-6, 1.0, [
        layer(mixer(1, 6, 4, 6, 6, 12, 1, base=100.0), moe(12, 1.5, 2, 2, (12, 1.5))),
        layer(mixer(1, 6, 4, 10, 5, 12, 2, base=100.0, kv_from=0), moe(20, 3.0, 1, 1)),
        layer(mixer(3, 4, 2, 5, 7, 9, 5, base=50.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0}), dense(30))]),
    # wider rows and 160 latent values (eight value tiles a warp): prompts of a few hundred tokens send the joined products
    # through the tcgen05 kernels; a window wider than two key blocks
    "C": model(300, 128, 1e-6, 11.3, [
        layer(mixer(6, 64, 32, 40, 48, 160, 150, base=500000.0, dims=16, scaling={"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0},
                    scale=0.1), moe(64, 1.5, 8, 2, (96, 1.5))),
        layer(mixer(6, 32, 32, 64, 64, 160, 70, base=500000.0, dims=16, scaling={"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0},
                    scale=0.12, kv_from=0), dense(256))]),
    # 272 latent values (sixteen value tiles a warp), more heads than a block has rows, no stretching of the angles
    "D": model(83, 96, 1e-5, 2.0, [
        layer(mixer(35, 8, 8, 8, 40, 272, 45), dense(64)),
        layer(mixer(3, 16, 8, 24, 40, 272, 0, kv_from=0), moe(32, 1.0, 4, 3))]),
}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from boring_llm_b200 import MiforaxConfig, write_random_model
    made = {}

    def get(name, std=0.25):
        key = (name, std)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"mif_{name}"))
            write_random_model(d, MiforaxConfig.from_dict(SHAPES[name]), SEEDS[name], "bfloat16", std)
            made[key] = d
        return made[key]
    return get


def plain_logits(folder, tokens):
    cfg, W = plain.read_model_folder(folder)
    return pm.forward(cfg, W, tokens).numpy()


def check_trace(folder, dtype, reqs, steps, max_tokens, what, **kw):
    outputs, runner = helpers.run_inprocess(folder, dtype, steps, max_tokens, **kw)
    rows = helpers.collect_rows(steps, outputs)
    for rid, toks in reqs.items():
        want = plain_logits(folder, toks)
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        if dtype == "float32":
            helpers.assert_close(got, want, dtype, f"{what} {rid}")
        else:
            # bfloat16 against pure float64: a few positions of a random model amplify rounding; a fault moves most of them
            assert np.isfinite(got).all(), f"{what} {rid}: non-finite logits"
            e = np.abs(got - want).max(-1) / max(np.abs(want).max(), 1e-6)
            assert int((e > BF16_TOL).sum()) <= max(1, int(0.04 * e.size)), f"{what} {rid}: worst {e.max():.3f}, {int((e > BF16_TOL).sum())} of {e.size} over"
            assert np.median(e) <= BF16_TOL / 4, f"{what} {rid}: median difference {np.median(e):.4f}"
    return runner


def solo_steps(reqs, cut):
    steps, n0 = [], 0
    for i, (rid, toks) in enumerate(reqs.items()):
        s = helpers.solo_trace(rid, toks, cut(toks, i), n0)
        steps += s
        n0 += len(s)
    return steps


BF16_TOL = 6e-2


def std_for(dtype):
    return 0.25 if dtype == "float32" else 0.1


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_whole_tails_singly_and_portions(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"r{i}": helpers.random_tokens(vocab, n, 100 + i) for i, n in enumerate([1, 2, 19, 75, 130])}
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256, f"{name} whole")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 45)), 256, f"{name} tail")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_varying(t, i)), 256, f"{name} portions")
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: [2] * (len(t) // 2) + [1] * (len(t) % 2)), 256, f"{name} pairs")


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"m{i}": helpers.random_tokens(vocab, n, 200 + i) for i, n in enumerate([33, 7, 90, 41, 2, 64, 17, 58])}
    steps, peak = helpers.mixed_trace(reqs, seed=5, max_live=3)
    runner = check_trace(folder, dtype, reqs, steps, peak, f"{name} mixed", debug_poison=True)
    assert all(hw <= runner.cache.num_pages for hw in runner.cache.stats()["pages_high_water"])
    # one cache layer for each layer with rows of its own: the layers that read another's rows keep nothing
    own = sum(1 for l in SHAPES[name]["layers"] if "kv_from" not in l["mixer"])
    assert sum(len(g.cache_layers) for g in runner.cache.paged_groups) == own


def test_float32_does_not_depend_on_the_cut_or_the_batch(folders):
    folder = folders("A")
    reqs = {f"c{i}": helpers.random_tokens(101, n, 300 + i) for i, n in enumerate([50, 21, 77])}
    a, _ = helpers.run_inprocess(folder, "float32", solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256)
    whole = helpers.collect_rows(solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), a)
    steps, peak = helpers.mixed_trace(reqs, seed=9, max_live=3)
    b, _ = helpers.run_inprocess(folder, "float32", steps, peak)
    mixed = helpers.collect_rows(steps, b)
    for key, row in whole.items():
        assert np.abs(row - mixed[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_the_windows(folders, dtype):
    """300 tokens decoded one by one: the windows (20 and 13 positions over the first layer's rows, 37 over the third's, which
    the third layer itself reads without a window) pass over decoded tokens and page edges."""
    folder = folders("A", std_for(dtype))
    toks = helpers.random_tokens(101, 330, 7)
    steps = helpers.solo_trace("long", toks, [30] + [1] * 300)
    runner = check_trace(folder, dtype, {"long": toks}, steps, 384, "long decoding")
    # the first group's rows (windows of 20 and 13) went back while the request was running; the second group (a layer that
    # sees everything) kept all 21 pages
    hw = sorted(runner.cache.stats()["pages_high_water"])
    assert hw[0] <= 4 and hw[-1] == 21, hw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_shape_on_the_tensor_core_products(folders, dtype):
    """Prompts of 300 and 90 tokens: in bfloat16 the joined products run on tcgen05 and the per-head products as grouped
    products over three tiles a head, decode steps replay captured graphs; a window wider than two key blocks."""
    folder = folders("C", 0.25 if dtype == "float32" else 0.06)
    reqs = {"w0": helpers.random_tokens(300, 300, 1), "w1": helpers.random_tokens(300, 90, 2)}
    steps = solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 24))
    check_trace(folder, dtype, reqs, steps, 512, "wide tail").check_kernels()
    steps, peak = helpers.mixed_trace(reqs, seed=3, max_live=2)
    check_trace(folder, dtype, reqs, steps, peak, "wide mixed").check_kernels()


def test_captured_steps_replay_the_same_bits(folders):
    folder = folders("A", 0.1)
    reqs = {f"g{i}": helpers.random_tokens(101, n, 400 + i) for i, n in enumerate([40, 23, 31])}
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
    """float32: the residual stream behind every layer against the plain implementation's."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    folder = folders("A")
    toks = helpers.random_tokens(101, 70, 3)
    cfg, W = plain.read_model_folder(folder)
    _, want = pm.forward(cfg, W, toks, streams=True)
    _, model = load_model(folder, "float32", DEV)
    runner = ModelRunner(model, EngineOptions(dtype="float32", max_tokens=128, ctx_size=128, max_num_seqs=2, cuda_graphs=False))
    model.keep_streams = []
    runner.step([StepEntry("s", toks, [])])
    assert len(model.keep_streams) == len(cfg["layers"])
    for i, got in enumerate(model.keep_streams):
        w = want[i].numpy()
        assert np.abs(got.cpu().numpy() - w).max() <= 1e-4 * np.abs(w).max(), i


# ---- mechanisms alone --------------------------------------------------------------------------------------------------
def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


def dev(t, dtype=torch.float32):
    return t.to(dtype).to(DEV).contiguous()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def paged_rows(rows_by_request, dk, dtype, seed):
    """A cache [pages, 1, 16, dk] holding each request's rows on scattered pages, everything else NaN; the block table."""
    n_pages = sum(-(-len(r) // 16) for r in rows_by_request) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    cache = torch.full((n_pages, 1, 16, dk), float("nan"), dtype=torch.float64)
    width = max(-(-len(r) // 16) for r in rows_by_request)
    table = torch.full((len(rows_by_request), width), -1, dtype=torch.int32)
    for r, rows in enumerate(rows_by_request):
        for j in range(len(rows)):
            if j % 16 == 0:
                table[r, j // 16] = order.pop()
            cache[table[r, j // 16], 0, j % 16] = rows[j]
    return dev(cache, dtype), table.to(DEV)


def attention_case(H, rank, rot, window, seed):
    """Three requests in one step: a portion of 70 tokens behind 130 cached ones, a single token at position 149, a prompt of
    5 tokens. One score per query stands out: the key just inside the window (or the first key) is planted along the query,
    the key just outside it twice as strongly, so a mask that is one position off changes the result completely; the same
    at the page and key-block borders before a query."""
    dk = rank + rot
    ctx, q_lens = [200, 150, 5], [70, 1, 5]
    rows = [rnd(n, dk, seed=seed + r, scale=0.5) for r, n in enumerate(ctx)]
    qs, where = [], []
    for r, (n, ql) in enumerate(zip(ctx, q_lens)):
        q = rnd(ql, H, dk, seed=seed + 10 + r, scale=0.5)
        for t in range(ql):
            pos = n - ql + t
            edge = max(0, pos - window + 1) if window else (pos // 16) * 16        # the first visible key / the page's first
            a = (t * 7 + r) % dk
            q[t, :, a] += 6.0
            rows[r][edge, a] += 6.0
            if edge > 0:
                rows[r][edge - 1, a] += 12.0 if window else 3.0
            where.append((r, pos))
        qs.append(q)
    return ctx, q_lens, rows, torch.cat(qs), where


def attention_oracle(ctx, q_lens, rows, q, rank, window, scale, sinks):
    out, t0 = [], 0
    for r, (n, ql) in enumerate(zip(ctx, q_lens)):
        qq = q[t0:t0 + ql].permute(1, 0, 2)
        i = torch.arange(n - ql, n)[:, None]
        j = torch.arange(n)[None, :]
        mask = (j <= i) & ((i - j < window) if window else (j >= 0))
        H = qq.shape[0]
        k = rows[r][None].expand(H, n, rows[r].shape[1])
        out.append(pm.sink_softmax_attention(qq, k, k[:, :, :rank], scale, sinks, mask).permute(1, 0, 2))
        t0 += ql
    return torch.cat(out)


@pytest.mark.parametrize("H,rank,rot,window", [(4, 32, 8, 20), (3, 96, 16, 64), (35, 160, 32, 0), (2, 272, 8, 17), (16, 512, 64, 130), (3, 520, 24, 75)])
def test_latent_attention_kernels(H, rank, rot, window):
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts.attention import attention_plan
    scale = 0.4
    ctx, q_lens, rows, q, _ = attention_case(H, rank, rot, window, seed=H)
    sinks = rnd(H, seed=99, scale=2.0)
    want = attention_oracle(ctx, q_lens, rows, q, rank, window, scale, sinks)
    T = q.shape[0]
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    tok_req = i32([r for r, n in enumerate(q_lens) for _ in range(n)])
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        # the rows as the dtype stores them are the oracle's inputs as well
        rows_d = [r.to(dtype).to(torch.float64) for r in rows]
        q_d = q.to(dtype).to(torch.float64)
        want = attention_oracle(ctx, q_lens, rows_d, q_d, rank, window, scale, sinks)
        cache, table = paged_rows(rows_d, rank + rot, dtype, seed=5)
        out = torch.full((T, H, rank), float("nan"), dtype=dtype, device=DEV)
        ops.latent_attention_plain(dev(q_d, dtype), cache, tok_req, i32(cu), i32(ctx), table, out, window, scale, dev(sinks))
        err = (out.double().cpu() - want).abs().max().item()
        assert err <= tol * want.abs().max().item(), ("plain", dtype, err)
        if dtype != torch.bfloat16 or not ops.latent_attention_mma_supported(dtype, rank, rot, 16):
            continue
        Tp = 128
        plan = attention_plan(q_lens, ctx)
        q_lat = torch.full((H, Tp, rank), float("nan"), dtype=dtype, device=DEV)
        q_rot = torch.full((H, Tp, rot), float("nan"), dtype=dtype, device=DEV)
        q_lat[:, :T] = dev(q_d[:, :, :rank], dtype).transpose(0, 1)
        q_rot[:, :T] = dev(q_d[:, :, rank:], dtype).transpose(0, 1)
        lat = torch.full((H, Tp, rank), float("nan"), dtype=dtype, device=DEV)
        for splits in (1, 2, 5):                                   # the single token's keys in one block, in slices, in more slices than key blocks
            lat.fill_(float("nan"))
            for name, single in (("tiles64", False), ("singles", True)):
                work = torch.from_numpy(plan.arrays[name]).to(DEV)
                ops.latent_attention_mma(q_lat, q_rot, cache, i32(cu), i32(ctx), table, work, single, lat, window, scale, dev(sinks),
                                         splits)
            got = lat[:, :T].transpose(0, 1).double().cpu()
            assert torch.isfinite(got).all()
            err = (got - want).abs().max().item()
            assert err <= tol * want.abs().max().item(), ("tensor cores", splits, err)
            assert torch.isnan(lat[:, T:].float()).all()           # rows that are no token of the step are not written


def test_latent_prep_norms_rotation_and_cache_rows():
    """The kernel behind the mixer's first product: both RMS norms, the stretched rotation of the shared key part (the first
    `dims` of its values, in halves), rows written where the block table says."""
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts import RotaryTable
    q_rank, rank, rot_dim, dims, eps = 10, 12, 8, 6, 1e-5
    sc = {"factor": 3.0, "original": 32, "fast": 4.0, "slow": 1.0}
    table_part = RotaryTable.yarn(rot_dim, 300.0, dims, sc["factor"], sc["original"], sc["fast"], sc["slow"]).to(DEV)
    positions = [37, 5, 16, 0, 15]
    T = len(positions)
    proj = rnd(T, 40, seed=1)
    qw, kw = rnd(q_rank, seed=2) + 1.0, rnd(rank, seed=3) + 1.0
    cache = torch.full((9, 1, 16, rank + rot_dim), float("nan"), dtype=torch.float32, device=DEV)
    block_table = i32([[4, 7, 2], [6, 1, 0], [3, 5, 8]])
    tok_req = i32([0, 1, 2, 2, 2])
    cq = torch.empty((T, q_rank), dtype=torch.float32, device=DEV)
    ops.latent_prep(dev(proj), 0, q_rank, 16, rank, rot_dim, table_part.rot_half, dev(qw), dev(kw), eps, i32(positions), tok_req,
                    block_table, table_part.inv_freq, table_part.mscale, cq, cache)
    want_q = pm.rms_norm(proj[:, :q_rank], qw, eps)
    assert (cq.double().cpu() - want_q).abs().max() <= 1e-5
    f, m = pm.yarn_frequencies(dims, 300.0, sc)
    z = proj[:, 16:16 + rank + rot_dim]
    lat = pm.rms_norm(z[:, :rank], kw, eps)
    turned = pm.rotate_halves(z[:, rank:rank + dims], torch.tensor(positions), f, m)
    want = torch.cat([lat, turned, z[:, rank + dims:]], dim=1)
    pages = block_table.cpu()
    for t, (pos, r) in enumerate(zip(positions, tok_req.tolist())):
        got = cache[pages[r, pos // 16], 0, pos % 16].double().cpu()
        assert (got - want[t]).abs().max() <= 2e-5, (t, (got - want[t]).abs().max())
    assert int(torch.isfinite(cache).all(-1).sum()) == T          # no other row was touched


def test_gated_activations_and_the_table_of_experts():
    from boring_llm_b200.kernels import ops
    for n in (13, 24):                                   # a value a thread; four values a thread
        sums = rnd(7, 2 * n, seed=4, scale=2.0)
        g, u = sums[:, :n], sums[:, n:]
        gc = torch.clamp(g, max=0.8)
        for kind, want in ((ops.GLU_GELU_TANH, pm.gelu_tanh(g) * u),
                           (ops.GLU_CLAMPED, gc * torch.sigmoid(1.702 * gc) * (torch.clamp(u, -0.8, 0.8) + 1.0)),
                           (ops.GLU_SILU, g * torch.sigmoid(g) * u)):
            for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
                out = torch.empty((7, n), dtype=dtype, device=DEV)
                ops.glu_act(dev(sums), out, kind, 0.8)
                assert (out.double().cpu() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (kind, n, dtype)
    table = torch.tensor([[2, 0], [1, 3], [4, 1], [0, 2]], dtype=torch.int32, device=DEV)
    tokens = i32([3, 3, 0, 2, 1])
    ids = torch.empty((5, 2), dtype=torch.int32, device=DEV)
    wts = torch.empty((5, 2), dtype=torch.float32, device=DEV)
    ops.table_route(table, tokens, ids, wts)
    assert ids.tolist() == [[0, 2], [0, 2], [2, 0], [4, 1], [1, 3]] and bool((wts == 0.5).all())
    emb = rnd(6, 8, seed=6)
    out = torch.empty((5, 8), dtype=torch.float32, device=DEV)
    ops.embed(dev(emb), tokens, out, 2.5)
    assert (out.double().cpu() - emb[tokens.cpu().long()].float().double() * 2.5).abs().max() <= 1e-5


def gated(kind, g, u, limit):
    from boring_llm_b200.kernels import ops
    if kind == ops.GLU_GELU_TANH:
        return pm.gelu_tanh(g) * u
    if kind == ops.GLU_CLAMPED:
        gc = torch.clamp(g, max=limit)
        return gc * torch.sigmoid(1.702 * gc) * (torch.clamp(u, -limit, limit) + 1.0)
    return g * torch.sigmoid(g) * u


def test_gated_activations_in_the_epilogue_of_every_product():
    """The joined gate/up product with the activation in its epilogue, on every kernel the row count can send it to (few
    rows: W through registers; tcgen05 tiles on one SM; on pairs of SMs; CUDA cores in 32-bit), the grouped product and the
    plain product over rows with a matrix each: against float64 on the same bfloat16 roundings."""
    from boring_llm_b200.kernels import ops
    K, N, limit = 256, 192, 0.7
    seen = set()
    for kind in (ops.GLU_SILU, ops.GLU_GELU_TANH, ops.GLU_CLAMPED):
        args = ops.glu_args(kind, limit, DEV)
        assert (args is None) == (kind == ops.GLU_SILU)
        for M in (3, 16, 40, 130, 600):
            x = rnd(M, K, seed=M, scale=0.5).bfloat16().double()
            w = rnd(2 * N, K, seed=M + 1, scale=0.2).bfloat16().double()
            want = gated(kind, x @ w[:N].T, x @ w[N:].T, limit)
            for dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-5)):
                out = torch.empty((M, N), dtype=dtype, device=DEV)
                seen.add(ops.gemm_kernel(dev(x, dtype), dev(w, dtype), N, args, ops.EPI_SWIGLU))
                ops.gemm(dev(x, dtype), dev(w, dtype), out, args, ops.EPI_SWIGLU)
                assert (out.double().cpu() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (kind, M, dtype)
        # three matrices; rows with a matrix each (plain), and the same rows in tiles of 128 behind the plan (grouped)
        E, T, top = 3, 50, 2
        x = rnd(T, K, seed=9, scale=0.5).bfloat16().double()
        w = rnd(E, 2 * N, K, seed=10, scale=0.2).bfloat16().double()
        ids = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(t))[:top] for t in range(T)]).int()
        want = torch.stack([gated(kind, x[t] @ w[e, :N].T, x[t] @ w[e, N:].T, limit) for t in range(T) for e in ids[t].tolist()])
        for dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-5)):
            out = torch.empty((T * top, N), dtype=dtype, device=DEV)
            ops.expert_gemm_plain(dev(x, dtype), top, dev(w, dtype), ids.to(DEV), out, ops.EPI_SWIGLU, args)
            assert (out.double().cpu() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (kind, "rows", dtype)
        pos, row_src, tile_expert = ops.moe_plan(ids.to(DEV), E)
        rows = torch.zeros((row_src.numel(), K), dtype=torch.bfloat16, device=DEV)
        ops.gather_rows(dev(x, torch.bfloat16), row_src, top, rows)
        out = torch.empty((row_src.numel(), N), dtype=torch.bfloat16, device=DEV)
        ops.gemm_grouped(rows, dev(w, torch.bfloat16), tile_expert, out, ops.EPI_SWIGLU, args)
        got = out[pos.long()].double().cpu()
        assert (got - want).abs().max() <= 2e-2 * max(1.0, want.abs().max().item()), (kind, "grouped")
    assert {"plain", "skinny", "tc", "pair"} <= seen, seen


def test_the_command_line_and_the_trace_program_on_a_model_folder(folders, tmp_path):
    """`bin/boring-llm` generates what the plain implementation's arg-max gives, and `bin/trace_run`, started as a user
    would start it, writes the logits of a mixed trace (float32, and bfloat16 on poisoned pools)."""
    import os
    import subprocess
    import sys
    folder = folders("A")
    exe = [sys.executable, os.path.join(helpers.ROOT, "bin", "boring-llm")]
    prompt = helpers.random_tokens(101, 9, 3)
    p = subprocess.run(exe + ["--model", folder, "--prompt-tokens", ",".join(map(str, prompt)), "--n-predict", "6", "--dtype", "f32",
                              "--ctx-size", "64", "--ignore-eos"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(plain_logits(folder, toks)[-1].argmax()))
    assert p.stdout.strip().splitlines()[-1] == "generated: " + ",".join(map(str, toks[9:]))
    reqs = {f"t{i}": helpers.random_tokens(101, n, 600 + i) for i, n in enumerate([30, 12, 45])}
    steps, peak = helpers.mixed_trace(reqs, seed=2, max_live=2)
    outputs = helpers.run_trace_program(folder, "float32", steps, peak, str(tmp_path / "out"), 101)
    rows = helpers.collect_rows(steps, outputs)
    for rid, t in reqs.items():
        helpers.assert_close(np.stack([rows[(rid, i)] for i in range(len(t))]), plain_logits(folder, t), "float32", rid)
    outputs = helpers.run_trace_program(folders("A", 0.1), "bfloat16", steps, peak, str(tmp_path / "out16"), 101, extra=["--poison"])
    rows = helpers.collect_rows(steps, outputs)
    for rid, t in reqs.items():
        got = np.stack([rows[(rid, i)] for i in range(len(t))])
        want = plain_logits(folders("A", 0.1), t)
        assert np.isfinite(got).all() and np.median(np.abs(got - want).max(-1)) <= BF16_TOL / 4 * np.abs(want).max(), rid
