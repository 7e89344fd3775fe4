"""Kagorax on the GPU against the plain implementation: every mechanism alone, whole prompts,
the same requests cut in different ways, long decoding, reused pages, and greedy generation
through the entry point.  float32 is the sharp comparison (2e-5 of the largest logit); in
bfloat16 a router's choice between two near-equal experts may fall the other way for a token,
so a tenth of the rows may exceed the bound there."""
import copy
import math
import os
from types import SimpleNamespace

import pytest
import torch

import plain_kagorax as plain
import traces
from kagorax_util import SMALL, make_model, write_model
from util import FP32_RTOL, assert_close_logits, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"A": [70, 45, 120, 33, 17, 2, 64], "B": [40, 9, 65, 1], "C": [200, 33, 130, 64, 95, 17],
           "D": [420, 140, 33, 300, 129], "E": [150, 70, 9, 260, 66]}


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.kernels import cuda_ops
    return cuda_ops(DEV)


def _requests(name):
    vocab = SMALL[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=300 + i) for i, n in enumerate(LENGTHS[name])}


_PLAIN = {}


def _plain(model_dir, name):
    if name not in _PLAIN:
        cfg, w = plain.load_folder(model_dir)
        _PLAIN[name] = {r: plain.forward(cfg, w, t) for r, t in _requests(name).items()}
    return _PLAIN[name]


def _run(model_dir, dtype, steps, max_tokens, page_size=16, max_requests=4):
    from tinyinfer_b200 import Engine, StepEntry
    eng = Engine(model_dir, dtype=dtype, page_size=page_size, num_pages=-(-max_tokens // page_size),
                 max_requests=max_requests)
    outputs = {}
    for s in steps:
        outputs[s["step"]] = eng.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).cpu()
        for r in s["end"]:
            eng.finish(r)
        eng.cache.check()
    eng.ops.check_status()
    assert eng.cache.free_pages() == [g.pool.count for g in eng.cache.groups], "pages were lost"
    return outputs


def _compare(steps, outputs, want, dtype, what):
    rows = traces.collect(steps, outputs)
    worst = 0.0
    for r, got in rows.items():
        pos = [p for p, _ in got]
        g = torch.stack([x for _, x in got])
        ref = want[r][pos]
        if dtype == "float32":
            worst = max(worst, assert_close_logits(g, ref, FP32_RTOL, f"{what} {r}"))
        else:
            err = (g.double() - ref).abs().max(dim=-1).values / ref.abs().max()
            assert torch.isfinite(g).all()
            bound = torch.quantile(err, 0.9) if len(err) >= 10 else err.median()
            assert bound < 3e-2, f"{what} {r}: rows off by {err.topk(min(5, len(err))).values.tolist()}"
    return worst


# ---- mechanisms alone ------------------------------------------------------------------------
def test_embedding_with_scale_and_position_wave(ops):
    g = torch.Generator().manual_seed(0)
    table = torch.randn((50, 37), generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 50, (9,), generator=g)
    pos = torch.tensor([0, 1, 2, 63, 64, 500, 5000, 17, 3])
    i = torch.arange(19, dtype=torch.float64)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / 37).float().to(DEV)
    out = torch.empty((9, 37), dtype=torch.float32, device=DEV)
    ops.embed_sinusoid(table.to(DEV), ids.int().to(DEV), pos.int().to(DEV), freq, 3.25, out)
    want = table.double()[ids] * 3.25 + torch.cat(
        [plain.sinusoid_rows([int(p)], 37, torch.float64) for p in pos])
    assert (out.cpu().double() - want).abs().max() < 5e-4          # float32 angle at position 5000
    assert (out.cpu().double() - want)[:5].abs().max() < 2e-6


def _attention_case(heads, kv, dk, dv, page_size, ctx_lens, q_lens, dtype, seed=0, scramble=True):
    """Requests with ``ctx_lens[r]`` tokens of which the last ``q_lens[r]`` are new; a page holds
    its keys and then its values."""
    n = len(ctx_lens)
    blocks = [-(-c // page_size) for c in ctx_lens]
    num_pages = sum(blocks) + 2
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist() if scramble \
        else list(range(num_pages))
    bt = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    it = iter(perm)
    for i, b in enumerate(blocks):
        bt[i, :b] = torch.tensor([next(it) for _ in range(b)], dtype=torch.int32)
    g = torch.Generator().manual_seed(seed + 1)
    keys = [torch.randn((c, kv, dk), generator=g) for c in ctx_lens]
    values = [torch.randn((c, kv, dv), generator=g) for c in ctx_lens]
    positions, req_of_tok = [], []
    for i, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        positions += list(range(c - ql, c))
        req_of_tok += [i] * ql
    q = torch.randn((len(positions), heads, dk), generator=g)
    ti = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    # the lists the kernel set asks of a step (single-token rows, portions cut into its tiles)
    from tinyinfer_b200.engine.batch import build_lists
    from tinyinfer_b200.kernels import cuda_ops
    lists = build_lists(cuda_ops(DEV).step_lists(torch.bfloat16), list(q_lens),
                        [c - n for c, n in zip(ctx_lens, q_lens)])
    step = SimpleNamespace(positions=ti(positions), req_of_tok=ti(req_of_tok), scratch={},
                           lists={k: torch.from_numpy(a).to(torch.int32).to(DEV) for k, a in lists.items()},
                           max_position=max(ctx_lens), max_ctx_len=max(ctx_lens))
    pages = torch.zeros((num_pages, kv * page_size * (dk + dv)), dtype=dtype, device=DEV)
    cache = SimpleNamespace(pages=pages, block_table=bt.to(DEV), page_size=page_size, writes=True)
    return step, cache, q, keys, values, bt


def _fill_pages(cache, bt, keys, values, kv, dk, dv):
    ps = cache.page_size
    for r, (k, v) in enumerate(zip(keys, values)):
        for p in range(k.shape[0]):
            page = cache.pages[int(bt[r, p // ps])]
            kpart = page[: kv * ps * dk].view(kv, ps, dk)
            vpart = page[kv * ps * dk:].view(kv, ps, dv)
            kpart[:, p % ps] = k[p].to(page.dtype)
            vpart[:, p % ps] = v[p].to(page.dtype)


@pytest.mark.parametrize("geom", [(4, 2, 16, 24, 16), (6, 1, 32, 32, 8), (1, 1, 8, 8, 16), (8, 2, 64, 64, 64),
                                  (4, 4, 128, 128, 32), (3, 1, 48, 48, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_bias_unit_norm_store_and_attention(ops, geom, dtype):
    heads, kv, dk, dv, ps = geom
    ctx, ql = [90, 41, 7, 130, 300], [90, 1, 3, 2, 150]
    window, keep, far, rows = 20, 3, 40, 8
    step, cache, _, keys, values, bt = _attention_case(heads, kv, dk, dv, ps, ctx, ql, dtype, seed=2)
    _fill_pages(cache, bt, keys, values, kv, dk, dv)          # the context that earlier steps left
    g = torch.Generator().manual_seed(9)
    t = sum(ql)
    ncol = heads * dk + kv * (dk + dv) + heads * dv
    proj = torch.randn((t, ncol), generator=g)
    bias = torch.randn((heads * dk + kv * (dk + dv),), generator=g)
    rel = torch.randn((rows, heads), generator=g)
    eps, scale = 1e-5, 0.3
    from tinyinfer_b200.parts.gated_attention import distance_rows
    dist = rel[torch.tensor(distance_rows(rows, far))].t().contiguous().to(DEV)
    q_out = torch.empty((t, heads * dk), dtype=dtype, device=DEV)
    proj_d = proj.to(DEV)
    ops.qkv_bias_norm_store(proj_d, bias.to(DEV), None, None, eps, step, cache, q_out, heads, kv, dk, dv)
    out = torch.empty((t, heads * dv), dtype=dtype, device=DEV)
    gate = proj_d[:, ncol - heads * dv:]
    ops.biased_attention(q_out, step, cache, out, heads, kv, dk, dv, window, keep, scale, dist, gate)
    ops.check_status()
    # the plain statement: new keys and values replace the ends of the contexts
    pb = (proj[:, : bias.shape[0]] + bias).double()
    nq, nk = heads * dk, kv * dk
    row = 0
    for r, (c, n) in enumerate(zip(ctx, ql)):
        mine = pb[row:row + n]
        k_all, v_all = keys[r].double().clone(), values[r].double().clone()
        if dtype == torch.bfloat16:
            k_all, v_all = k_all.bfloat16().double(), v_all.bfloat16().double()
        k_new = plain.unit_rms(mine[:, nq:nq + nk].view(n, kv, dk), eps)
        v_new = mine[:, nq + nk:].view(n, kv, dv)
        q = plain.unit_rms(mine[:, :nq].view(n, heads, dk), eps)
        if dtype == torch.bfloat16:
            k_new, v_new, q = (x.bfloat16().double() for x in (k_new, v_new, q))
        k_all[c - n:], v_all[c - n:] = k_new, v_new
        want = plain.attend(q, k_all, v_all, rel.double(), heads // kv, scale, window, keep, far, c - n)
        want = want.reshape(n, heads * dv) * torch.sigmoid(proj[row:row + n, ncol - heads * dv:].double())
        got = out[row:row + n].cpu().double()
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max()), f"request {r}"
        row += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", ["decoded", "portion", "long portion"])
def test_one_key_carries_the_weight_at_every_edge(ops, where, dtype):
    """One key stands out by a scaled query and key: its value comes back exactly when the mask
    lets it through, far back among hundreds, at a page's border, just inside and just outside
    the window, and among the kept first tokens."""
    heads, kv, dk, dv, ps = 2, 1, 16, (8 if dtype == torch.float32 else 16), 16
    if dtype == torch.bfloat16 and where == "long portion":
        dk = dv = 128                                      # the tcgen05 kernel's head size
    window, keep = 48, 5
    ctx = 400
    n_new = {"decoded": 1, "portion": 3, "long portion": 170}[where]
    last = ctx - 1
    cases = [(last - window + 1, True), (last - window, False), (keep - 1, True), (keep, False), (0, True),
             (last - 1, True), (last - 15, True), (last - 16, True), (352, True), (351, False), (200, False)]
    for target, seen in cases:
        step, cache, q, keys, values, bt = _attention_case(heads, kv, dk, dv, ps, [ctx], [n_new], dtype, seed=4)
        keys[0].mul_(0.01)
        keys[0][target] = 3.0 if dk == 16 else 1.0
        values[0][target] = torch.arange(1, dv + 1, dtype=torch.float32)
        _fill_pages(cache, bt, keys, values, kv, dk, dv)
        q.fill_(3.0 if dk == 16 else 1.0)
        qd = q.reshape(n_new, heads * dk).to(DEV).to(dtype)
        out = torch.empty((n_new, heads * dv), dtype=dtype, device=DEV)
        dist = torch.zeros((heads, 9), dtype=torch.float32, device=DEV)
        ops.biased_attention(qd, step, cache, out, heads, kv, dk, dv, window, keep, 1.0, dist, None)
        got = out[-1].float().cpu().view(heads, dv)               # the last row sits at position ctx - 1
        hit = (got - torch.arange(1, dv + 1)).abs().max() < (1e-3 if dtype == torch.float32 else 0.1)
        assert bool(hit) == seen, f"key {target} seen from {last}: expected {'visible' if seen else 'hidden'}"


@pytest.mark.parametrize("window, keep", [(0, 0), (2500, 7), (1000, 40)])
def test_single_rows_with_their_keys_cut_into_runs(ops, window, keep):
    """Few single-token rows with thousands of keys: the walk over the keys is cut into runs, a
    block each, and a second launch adds them."""
    heads, kv, d, ps = 8, 2, 64, 16
    ctx = [3000, 777, 2049]
    rows, far = 16, 600
    from tinyinfer_b200.parts.gated_attention import distance_rows
    step, cache, q, keys, values, bt = _attention_case(heads, kv, d, d, ps, ctx, [1, 1, 1], torch.bfloat16, seed=8)
    _fill_pages(cache, bt, keys, values, kv, d, d)
    rel = torch.randn((rows, heads), generator=torch.Generator().manual_seed(2))
    dist = rel[torch.tensor(distance_rows(rows, far))].t().contiguous().to(DEV)
    gate = torch.randn((3, heads * d), generator=torch.Generator().manual_seed(3)).to(DEV)
    out = torch.empty((3, heads * d), dtype=torch.bfloat16, device=DEV)
    qd = q.reshape(3, heads * d).to(torch.bfloat16).to(DEV)
    ops.biased_attention(qd, step, cache, out, heads, kv, d, d, window or None, keep, 0.2, dist, gate)
    ops.check_status()
    for r, c in enumerate(ctx):
        want = plain.attend(q[r:r + 1].bfloat16().double(), keys[r].bfloat16().double(), values[r].bfloat16().double(),
                            rel.double(), heads // kv, 0.2, window or 10 ** 9, keep, far, c - 1)
        want = want.reshape(1, heads * d) * torch.sigmoid(gate[r:r + 1].cpu().double())
        assert (out[r:r + 1].cpu().double() - want).abs().max() < 2e-2 * max(1.0, want.abs().max()), f"row {r}"


def test_distance_bias_reaches_the_scores(ops):
    """With equal keys the weights are the softmax of the bias alone: the row of every distance,
    below half the table, in the logarithmic part and beyond the far end."""
    heads, kv, dk, dv, ps = 3, 1, 8, 4, 16
    rows, far, ctx = 6, 20, 60
    from tinyinfer_b200.parts.gated_attention import distance_rows
    step, cache, q, keys, values, bt = _attention_case(heads, kv, dk, dv, ps, [ctx], [1], torch.float32, seed=6)
    keys[0].fill_(0.25)
    _fill_pages(cache, bt, keys, values, kv, dk, dv)
    rel = torch.randn((rows, heads), generator=torch.Generator().manual_seed(1)) * 2
    dist = rel[torch.tensor(distance_rows(rows, far))].t().contiguous().to(DEV)
    out = torch.empty((1, heads * dv), dtype=torch.float32, device=DEV)
    ops.biased_attention(q.reshape(1, -1).to(DEV), step, cache, out, heads, kv, dk, dv, 1000, 0, 0.5, dist, None)
    want = plain.attend(q.double(), keys[0].double(), values[0].double(), rel.double(), heads, 0.5, 1000, 0, far, ctx - 1)
    assert (out.cpu().double().view(1, heads, dv) - want).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(7, 3, 40, 24, 24, 37), (4, 4, 32, 16, None, 37), (9, 1, 64, 32, 16, 37),
                                   (8, 2, 64, 96, 32, 301), (5, 5, 96, 32, None, 130), (16, 1, 128, 160, None, 700)])
def test_router_and_experts(ops, dtype, sizes):
    experts, top, width, ff, shared, t = sizes
    g = torch.Generator().manual_seed(experts)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    w = {"router": (torch.randn((experts, width), generator=g) * 0.5).to(torch.bfloat16)}
    for e in range(experts):
        for kind, shape in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
            w[f"e{e}.{kind}"] = (torch.randn(shape, generator=g) / shape[1] ** 0.5).to(torch.bfloat16)
    if shared:
        mlp["shared"] = {"ff": shared}
        for kind, shape in (("gate", (shared, width)), ("up", (shared, width)), ("down", (width, shared)), ("sg", (1, width))):
            w[f"shared.{kind}"] = (torch.randn(shape, generator=g) / shape[1] ** 0.5).to(torch.bfloat16)
    from tinyinfer_b200.parts.moe import RoutedExperts
    part = RoutedExperts(width, experts, top, ff, shared)
    part.load_weights({k: v.to(DEV) for k, v in w.items()}, ops)
    h = torch.randn((t, width), generator=g).to(dtype)
    residual = torch.randn((t, width), generator=g)
    res_d = residual.to(DEV)
    part.forward(ops, h.to(DEV), res_d, None)
    want = residual.double() + plain.routed_experts(h.double(), {k: v.double() for k, v in w.items()}, "", mlp)
    err = (res_d.cpu().double() - want).abs().max(dim=1).values / want.abs().max()
    if dtype == torch.float32:
        assert err.max() < 2e-5
    else:
        assert torch.quantile(err, 0.9) < 2e-2
    # the choice itself: ids in the order of the scores, ties to the lower index
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0, 0.1, 0.0, 3.0]], device=DEV)
    ids = torch.empty((1, 4), dtype=torch.int32, device=DEV)
    wts = torch.empty((1, 4), dtype=torch.float32, device=DEV)
    sg = torch.empty((1,), dtype=torch.float32, device=DEV)
    ops.router_topk(logits, 7, 4, ids, wts, sg)
    assert ids.cpu().tolist() == [[1, 2, 4, 0]]
    assert torch.allclose(wts.cpu(), torch.sigmoid(torch.tensor([[2.0, 2.0, 2.0, 0.5]])), atol=1e-6)
    assert abs(float(sg[0]) - 1 / (1 + math.exp(-3.0))) < 1e-6


# ---- the model through the engine ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts(tmp_path_factory, name, dtype):
    d = make_model(tmp_path_factory.getbasetemp(), name)
    steps = traces.whole(_requests(name))
    out = _run(d, dtype, steps, traces.max_live_tokens(steps))
    _compare(steps, out, _plain(d, name), dtype, f"{name} whole")


@pytest.mark.parametrize("name, family, dtype", [
    ("A", "tail", "float32"), ("A", "portions", "float32"), ("A", "mixed", "float32"), ("A", "mixed", "bfloat16"),
    ("B", "portions", "float32"), ("B", "mixed", "float32"),
    ("C", "tail", "float32"), ("C", "portions", "bfloat16"), ("C", "mixed", "float32"), ("C", "mixed", "bfloat16"),
    ("D", "long portions", "bfloat16"), ("D", "long portions", "float32"), ("D", "mixed", "bfloat16"),
    ("E", "long portions", "bfloat16"), ("E", "mixed", "float32"), ("E", "mixed", "bfloat16"), ("E", "tail", "bfloat16")])
def test_cuttings_agree_with_the_plain_implementation(tmp_path_factory, name, family, dtype):
    """Prefill against token-by-token decoding, portions down to two tokens, and up to four live
    requests of unequal length in a pool so small that pages and slots are used again."""
    d = make_model(tmp_path_factory.getbasetemp(), name)
    reqs = _requests(name)
    steps = {"tail": lambda: traces.tail_decoded(reqs, tail=40), "portions": lambda: traces.portions(reqs),
             "long portions": lambda: traces.portions(reqs, sizes=(150, 2, 131, 70, 128, 3)),
             "mixed": lambda: traces.mixed(reqs, seed=5)}[family]()
    out = _run(d, dtype, steps, traces.max_live_tokens(steps))
    _compare(steps, out, _plain(d, name), dtype, f"{name} {family}")


def test_float32_cuttings_give_the_same_bits(tmp_path_factory):
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    reqs = _requests("A")
    seen = {}
    for family in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, seed=2)):
        out = _run(d, "float32", family, traces.max_live_tokens(family))
        for r, rows in traces.collect(family, out).items():
            for p, x in rows:
                if (r, p) in seen:
                    assert torch.equal(seen[(r, p)], x), f"request {r} position {p}"
                seen[(r, p)] = x


def test_long_decoding_passes_every_window_and_gives_pages_back(tmp_path_factory):
    from tinyinfer_b200 import Engine, StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    tokens = random_tokens(SMALL["A"][0]["vocab"], 170, seed=77)
    cfg, w = plain.load_folder(d)
    want = plain.forward(cfg, w, tokens)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=6, max_requests=2)   # 96 tokens of room for 170
    got = [eng.step([StepEntry("x", tokens[:4], [3])])[0].cpu()]
    for p in range(4, len(tokens)):
        got.append(eng.decode_step([StepEntry("x", [tokens[p]], [0])])[0].cpu().clone())
        eng.cache.check()
    assert_close_logits(torch.stack(got), want[3:], FP32_RTOL, "long decoding")
    eng.finish("x")
    assert eng.cache.free_pages() == [6, 6]


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, graphs):
    from tinyinfer_b200 import LLM, SamplingParams
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(cfg["vocab"], n, seed=n) for n in (5, 31, 12)]
    llm = LLM(d, dtype="float32", max_seq=128, max_num_seqs=2, max_batched_tokens=24, page_size=16,
              cuda_graph=graphs)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8))
    for prompt, out in zip(prompts, outs):
        assert out.tokens == plain.greedy(cfg, w, prompt, 8), f"prompt of {len(prompt)} tokens"


def test_random_weights_from_a_configuration(tmp_path):
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    cfg = copy.deepcopy(SMALL["C"][0])
    for layer, rows in zip(cfg["layers"], SMALL["C"][1]):
        layer["mixer"]["bias_rows"] = rows                  # no stored table to tell its size
    tokens = random_tokens(cfg["vocab"], 90, seed=1)
    a = Engine(config=cfg, seed=5, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    la = a.step([StepEntry("a", tokens, [0, 50, 89])])
    d = os.path.join(str(tmp_path), "written")
    write_random_model(d, cfg, seed=5)
    b = Engine(d, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    lb = b.step([StepEntry("a", tokens, [0, 50, 89])])
    assert torch.isfinite(la).all() and torch.equal(la, lb)


def test_command_line_with_token_ids(tmp_path_factory, capsys):
    from tinyinfer_b200 import cli
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    cfg, w = plain.load_folder(d)
    prompt = random_tokens(cfg["vocab"], 9, seed=4)
    rc = cli.main(["-m", d, "--tokens", "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                   "--max-seq", "64", "--max-num-seqs", "2", "--page-size", "16"])
    assert rc == 0
    out = capsys.readouterr().out
    line = [ln for ln in out.splitlines() if ln.startswith("[output]")][0]
    assert [int(x) for x in line.split()[1:]] == plain.greedy(cfg, w, prompt, 6)
