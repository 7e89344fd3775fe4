"""Ruvuvik on the GPU against the plain implementation: every mechanism alone (also with one key
carrying all the weight at every edge), each mixer alone over requests cut into portions, whole
prompts, the same requests cut in different ways, long decoding, reused pages and state slots, and
greedy generation through the entry point.  float32 is the sharp comparison (2e-5 of the largest
logit); in bfloat16 the bound is 3e-2 for nine rows out of ten."""
import copy
import math
import os
from types import SimpleNamespace

import pytest
import torch

import plain_ruvuvik as plain
import traces
from ruvuvik_util import SMALL, make_model, mixer_weights
from util import FP32_RTOL, assert_close_logits, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LENGTHS = {"A": [70, 45, 120, 33, 17, 2, 64, 1], "B": [40, 9, 130, 1], "C": [300, 33, 150, 64, 217, 17]}


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.kernels import cuda_ops
    return cuda_ops(DEV)


def _requests(name):
    vocab = SMALL[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=500 + i) for i, n in enumerate(LENGTHS[name])}


_PLAIN = {}


def _plain(model_dir, name):
    if name not in _PLAIN:
        cfg, w = plain.load_folder(model_dir)
        _PLAIN[name] = {r: plain.forward(cfg, w, t)[0] for r, t in _requests(name).items()}
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
    for r, got in traces.collect(steps, outputs).items():
        pos = [p for p, _ in got]
        g = torch.stack([x for _, x in got])
        ref = want[r][pos]
        if dtype == "float32":
            assert_close_logits(g, ref, FP32_RTOL, f"{what} {r}")
        else:
            err = (g.double() - ref).abs().max(dim=-1).values / ref.abs().max()
            assert torch.isfinite(g).all()
            bound = torch.quantile(err, 0.9) if len(err) >= 10 else err.median()
            assert bound < 3e-2, f"{what} {r}: rows off by {err.topk(min(5, len(err))).values.tolist()}"


# ---- kernels alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(ops, dtype):
    z = torch.cat([torch.linspace(-12, 12, 1001), torch.tensor([0.0, -1e-4, 1e-4])]).view(4, -1).contiguous()
    out = torch.empty(z.shape, dtype=dtype, device=DEV)
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    for p, q in ((0.3, -0.7), (-2.0, 1.5)):
        ops.xielu_rows(z.to(DEV), plain.softplus(p), 0.5 + plain.softplus(q), out)
        want = plain.xielu(z.double(), p, q)
        assert ((out.cpu().double() - want).abs() / (1 + want.abs())).max() < tol
    ops.tanh_rows(z.to(DEV), out)
    assert (out.cpu().double() - torch.tanh(z.double())).abs().max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(1, 96, 64), (8, 288, 256), (33, 130, 64), (64, 256, 96), (200, 192, 128), (5, 40, 24)])
def test_product_with_activation(ops, sizes, dtype):
    """Few rows take the product whose epilogue applies the activation, many rows (and sizes that
    product does not take) the product followed by the row-wise kernel: the same numbers."""
    m, n, k = sizes
    g = torch.Generator().manual_seed(m)
    h = torch.randn((m, k), generator=g).to(dtype)
    w = (torch.randn((n, k), generator=g) * 2 / k ** 0.5).to(torch.bfloat16)
    out = torch.empty((m, n), dtype=dtype, device=DEV)
    ops.linear_xielu(h.to(DEV), w.to(DEV), plain.softplus(0.4), 0.5 + plain.softplus(-0.3), out)
    want = plain.xielu(h.double() @ w.double().T, 0.4, -0.3)
    err = ((out.cpu().double() - want).abs() / (1 + want.abs())).max()
    assert err < (2e-5 if dtype == torch.float32 else 1e-2), err


def _paged(ctx_lens, q_lens, page_size, row_elems, dtype, seed=0):
    """A step of requests with ``ctx_lens[r]`` tokens of which the last ``q_lens[r]`` are new, over
    scrambled pages of ``row_elems`` elements per token."""
    n = len(ctx_lens)
    blocks = [-(-c // page_size) for c in ctx_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    bt = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    it = iter(perm)
    for i, b in enumerate(blocks):
        bt[i, :b] = torch.tensor([next(it) for _ in range(b)], dtype=torch.int32)
    positions, req_of_tok = [], []
    for i, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        positions += list(range(c - ql, c))
        req_of_tok += [i] * ql
    ti = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    # the tile lists that the tensor-core kernel walks, for every number of heads per kv head
    from tinyinfer_b200.kernels.step_lists import row_tiles
    lists = {f"row_tiles_{n}": ti(row_tiles(list(q_lens), [c - n_ for c, n_ in zip(ctx_lens, q_lens)], n).tolist()).view(-1, 3)
             for n in (1, 2, 4, 8, 16, 32, 64)}
    step = SimpleNamespace(positions=ti(positions), req_of_tok=ti(req_of_tok), scratch={}, lists=lists,
                           max_position=max(ctx_lens), max_ctx_len=max(ctx_lens), max_q_len=max(q_lens))
    pages = torch.zeros((num_pages, page_size * row_elems), dtype=dtype, device=DEV)
    cache = SimpleNamespace(pages=pages, block_table=bt.to(DEV), page_size=page_size, writes=True)
    return step, cache, bt, positions, req_of_tok


def _fill(cache, bt, keys, values, kv, dk, dv):
    """keys[r] [ctx, kv, dk] and values[r] [ctx, kv, dv] into the pages: a page's keys, then its values."""
    ps = cache.page_size
    for r, (k, v) in enumerate(zip(keys, values)):
        for p in range(k.shape[0]):
            page = cache.pages[int(bt[r, p // ps])]
            page[: kv * ps * dk].view(kv, ps, dk)[:, p % ps] = k[p].to(page.dtype)
            if dv:
                page[kv * ps * dk:].view(kv, ps, dv)[:, p % ps] = v[p].to(page.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geom", [(4, 2, 12, 8, 6, 8), (1, 1, 16, 16, 16, 16), (6, 3, 10, 24, 0, 16), (2, 1, 64, 64, 32, 64)])
def test_row_norm_rotation_and_store(ops, geom, dtype):
    heads, kv, dk, dv, rot, ps = geom
    ctx, ql = [37, 5, 300], [9, 5, 1]
    step, cache, bt, positions, req = _paged(ctx, ql, ps, kv * (dk + dv), dtype)
    g = torch.Generator().manual_seed(3)
    t = len(positions)
    nq, nk, nv = heads * dk, kv * dk, kv * dv
    proj = torch.randn((t, nq + nk + nv + 5), generator=g)
    qw, kw = 1 + 0.3 * torch.randn((nq,), generator=g), 1 + 0.3 * torch.randn((nk,), generator=g)
    from tinyinfer_b200.parts.rope import RopeInterleaved, NoPosition
    rotation = (RopeInterleaved(dk, 777.0, rot) if rot else NoPosition()).rotation(DEV)
    q_out = torch.empty((t, nq), dtype=dtype, device=DEV)
    ops.qk_rownorm_rope_store(proj.to(DEV), qw.to(DEV), kw.to(DEV), 1e-5, rotation, step, cache, q_out, heads, kv, dk, dv)
    p64 = proj.double()
    q_want = plain.rotate_pairs(plain.norm_plain(p64[:, :nq], qw.double(), 1e-5).view(t, heads, dk), positions, rot, 777.0)
    k_want = plain.rotate_pairs(plain.norm_plain(p64[:, nq:nq + nk], kw.double(), 1e-5).view(t, kv, dk), positions, rot, 777.0)
    v_want = p64[:, nq + nk:nq + nk + nv].view(t, kv, dv)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (q_out.cpu().double().view(t, heads, dk) - q_want).abs().max() < tol
    for i, (p, r) in enumerate(zip(positions, req)):
        page = cache.pages[int(bt[r, p // ps])].cpu().double()
        assert (page[: kv * ps * dk].view(kv, ps, dk)[:, p % ps] - k_want[i]).abs().max() < tol
        assert (page[kv * ps * dk:].view(kv, ps, dv)[:, p % ps] - v_want[i]).abs().max() < tol


OPTIONS = [dict(chunk=7, cap=3.0, head_scale=True), dict(chunk=64, cap=None, head_scale=False, gate="head"),
           dict(chunk=None, cap=None, sink=True), dict(chunk=20, cap=1.5, head_scale=True, sink=True, gate="element"),
           dict(chunk=None, cap=None)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "bfloat16 on CUDA cores"])
@pytest.mark.parametrize("opt", OPTIONS)
@pytest.mark.parametrize("geom", [(4, 2, 12, 8, 8), (1, 1, 16, 16, 16), (6, 1, 40, 24, 16), (8, 2, 64, 64, 64), (2, 2, 160, 130, 16),
                                  (12, 4, 96, 48, 32), (16, 2, 128, 128, 16), (5, 1, 32, 80, 16), (70, 1, 48, 16, 16)])
@pytest.mark.parametrize("shape", ["mixed", "decoding"])
def test_attention_with_options(ops, geom, opt, dtype, shape, monkeypatch):
    heads, kv, dk, dv, ps = geom
    if dtype == "bfloat16 on CUDA cores":
        if dk % 16 or dv % 16 or ps % 16:
            pytest.skip("these sizes run on the CUDA cores anyway")
        dtype = torch.bfloat16
        monkeypatch.setattr(ops, "use_tc_attention_options", False)
    ctx, ql = ([70, 9, 129, 40, 1, 300], [70, 1, 30, 2, 1, 1]) if shape == "mixed" else ([700, 9, 129, 1], [1, 1, 1, 1])
    step, cache, bt, positions, req = _paged(ctx, ql, ps, kv * (dk + dv), dtype, seed=dk)
    g = torch.Generator().manual_seed(dv)
    keys = [torch.randn((c, kv, dk), generator=g) for c in ctx]
    values = [torch.randn((c, kv, dv), generator=g) for c in ctx]
    _fill(cache, bt, keys, values, kv, dk, dv)
    t = len(positions)
    q = torch.randn((t, heads, dk), generator=g)
    hs = (1 + torch.rand((heads,), generator=g)) if opt.get("head_scale") else None
    sink = torch.randn((heads,), generator=g) + 1.0 if opt.get("sink") else None
    gate = None
    if opt.get("gate"):
        gate = torch.randn((t, heads if opt["gate"] == "head" else heads * dv), generator=g)
    out = torch.empty((t, heads * dv), dtype=dtype, device=DEV)
    dev = lambda x: None if x is None else x.to(DEV)
    ops.attention_options(q.reshape(t, -1).to(dtype).to(DEV), step, cache, out, heads, kv, dk, dv, 0.3,
                          chunk=opt["chunk"], softcap=opt["cap"], head_scale=dev(hs), sink=dev(sink),
                          gate=dev(gate), gate_per_head=opt.get("gate") == "head")
    rd = lambda x: x.to(dtype).double()              # what the kernel reads
    at = 0
    for r, (c, n) in enumerate(zip(ctx, ql)):
        want = plain.attend(rd(q[at:at + n]), rd(keys[r]), rd(values[r]), positions[at:at + n], 0.3, opt["chunk"],
                            opt["cap"], None if hs is None else hs.double(), None if sink is None else sink.double())
        if gate is not None:
            want = want * torch.sigmoid(gate[at:at + n].double()).view(n, heads, -1)
        got = out[at:at + n].cpu().double().view(n, heads, dv)
        assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2), f"request {r}"
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
def test_one_key_stands_out_at_every_edge(ops, decoded, dtype):
    """The query points at one key, whose value is a one-hot row: the output says which keys were
    seen.  Targets: the last key before the query's chunk (must not be seen), the chunk's first
    key, keys on both sides of page borders, a key hundreds of positions back, the query's own."""
    heads, kv, dk, dv, ps, chunk = 2, 1, 16, 32, 16, 150
    for pos, targets in ((415, [299, 300, 301, 415, 303, 304]), (149, [0, 15, 16, 149, 100]), (150, [149, 150]),
                         (640, [599, 600, 639, 640]), (15, [0, 15])):
        ctx = pos + 1
        for target in targets:
            step, cache, bt, positions, req = _paged([ctx], [1 if decoded else min(ctx, 40)], ps, kv * (dk + dv), dtype, seed=pos)
            g = torch.Generator().manual_seed(target)
            keys = torch.randn((ctx, kv, dk), generator=g) * 0.1
            values = torch.zeros((ctx, kv, dv))
            values[:, 0, 1] = 1.0
            values[target, 0, :2] = torch.tensor([1.0, 0.0])
            direction = torch.nn.functional.normalize(torch.randn((dk,), generator=g), dim=0)
            keys[target, 0] = direction * 8
            _fill(cache, bt, [keys], [values], kv, dk, dv)
            t = len(positions)
            q = torch.randn((t, heads, dk), generator=g) * 0.1
            q[-1] = direction * 8
            out = torch.empty((t, heads * dv), dtype=dtype, device=DEV)
            ops.attention_options(q.reshape(t, -1).to(dtype).to(DEV), step, cache, out, heads, kv, dk, dv, 1.0, chunk=chunk)
            seen = float(out[-1, 0])
            visible = target // chunk == pos // chunk
            assert (seen > 0.99) == visible and (visible or seen < 0.01), f"query {pos}, key {target}: {seen}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_and_shared_rows(ops, dtype):
    """One shared row per token is key and (its first elements) value; a large sink empties the output,
    a very negative one changes nothing."""
    heads, dk, dv, ps = 3, 24, 20, 8
    ctx, ql = [50, 9], [12, 1]
    step, cache, bt, positions, req = _paged(ctx, ql, ps, dk, dtype)
    g = torch.Generator().manual_seed(9)
    rows = [torch.randn((c, 1, dk), generator=g) for c in ctx]
    _fill(cache, bt, rows, rows, 1, dk, 0)
    t = len(positions)
    q = torch.randn((t, heads, dk), generator=g)
    rd = lambda x: x.to(dtype).double()
    for sink in (torch.tensor([0.5, -1.0, 2.0]), torch.tensor([60.0, -60.0, 0.0])):
        out = torch.empty((t, heads * dv), dtype=dtype, device=DEV)
        ops.attention_options(q.reshape(t, -1).to(dtype).to(DEV), step, cache, out, heads, 1, dk, dv, 0.2,
                              sink=sink.to(DEV), shared_rows=True)
        at = 0
        for r, (c, n) in enumerate(zip(ctx, ql)):
            want = plain.attend(rd(q[at:at + n]), rd(rows[r]), rd(rows[r])[:, :, :dv], positions[at:at + n], 0.2,
                                sink=sink.double())
            got = out[at:at + n].cpu().double().view(n, heads, dv)
            assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)
            at += n
    assert out.view(t, heads, dv)[:, 0].abs().max() < 1e-6          # the sink of 60 took everything


@pytest.mark.parametrize("q_lens", [[1, 1, 1], [70, 2, 40]])
@pytest.mark.parametrize("heads", [16, 24, 40])
def test_wide_shared_rows_with_many_heads(ops, heads, q_lens):
    """Single tokens and portions over shared rows wide enough for several slices of value columns,
    with as many heads as one block takes and more."""
    dk, dv, ps = 288, 256, 16
    ctx = [70, 9, 300]
    step, cache, bt, positions, req = _paged(ctx, q_lens, ps, dk, torch.bfloat16, seed=heads)
    g = torch.Generator().manual_seed(heads)
    rows = [torch.randn((c, 1, dk), generator=g) * 0.5 for c in ctx]
    _fill(cache, bt, rows, rows, 1, dk, 0)
    t = len(positions)
    q = torch.randn((t, heads, dk), generator=g) * 0.3
    sink = torch.randn((heads,), generator=g)
    out = torch.empty((t, heads * dv), dtype=torch.bfloat16, device=DEV)
    ops.attention_options(q.reshape(t, -1).bfloat16().to(DEV), step, cache, out, heads, 1, dk, dv, 0.1,
                          sink=sink.to(DEV), shared_rows=True)
    rd = lambda x: x.bfloat16().double()
    at = 0
    for r, n in enumerate(q_lens):
        want = plain.attend(rd(q[at:at + n]), rd(rows[r]), rd(rows[r])[:, :, :dv], positions[at:at + n], 0.1,
                            sink=sink.double())
        assert (out[at:at + n].cpu().double().view(n, heads, dv) - want).abs().max() < 2e-2
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 8, 20, 11, 3), (1, 16, 16, 1, 3), (4, 64, 96, 70, 3), (2, 130, 12, 9, 3),
                                   (3, 128, 512, 200, 8), (2, 80, 24, 130, 8), (16, 512, 128, 70, 8), (2, 48, 136, 65, 0)])
def test_head_project(ops, sizes, dtype):
    """Few tokens, many tokens, and (bfloat16, rows that start on 16 bytes) many tokens on the tensor cores."""
    heads, n_in, n_out, t, pad = sizes
    g = torch.Generator().manual_seed(n_in)
    x = torch.randn((t, heads, n_in + pad), generator=g).to(dtype)
    w = torch.randn((heads, n_in, n_out), generator=g).to(torch.bfloat16)
    out = torch.zeros((t, heads, n_out + 5), dtype=dtype, device=DEV)
    ops.head_project(x.to(DEV)[:, :, :n_in], w.to(DEV), out[:, :, 2:2 + n_out])
    want = torch.einsum("thk,hkn->thn", x[:, :, :n_in].double(), w.double())
    assert (out[:, :, 2:2 + n_out].cpu().double() - want).abs().max() < (2e-5 * n_in ** 0.5 if dtype == torch.float32 else 0.3)
    assert out[:, :, :2].abs().max() == 0 and out[:, :, 2 + n_out:].abs().max() == 0


# ---- mixers alone ----------------------------------------------------------------------------
def _run_mixer(ops, part, inputs, cuts, dtype, page_size=16):
    """Run a mixer part over requests whose rows ``inputs[r]`` [T_r, width] arrive cut as ``cuts``
    (a list of steps, each a list of (request, count)); returns its output rows per request."""
    from tinyinfer_b200.cache import CacheManager
    from tinyinfer_b200.engine.batch import StepEntry, build_step_batch
    width = next(iter(inputs.values())).shape[1]
    cm = CacheManager([part.cache_spec()], page_size=page_size,
                      num_pages=sum(-(-x.shape[0] // page_size) for x in inputs.values()) + 2,
                      max_requests=3, kv_dtype=dtype, device=DEV)
    at = {r: 0 for r in inputs}
    got = {r: [] for r in inputs}
    for step_cuts in cuts:
        entries = [StepEntry(r, [0] * n, []) for r, n in step_cuts]
        starts = cm.reserve_step([(r, n) for r, n in step_cuts])
        tables = [[cm.block_table(g, r) for r, _ in step_cuts] for g in range(len(cm.groups))]
        batch = build_step_batch(entries, starts, tables, [cm.state_slot(r) for r, _ in step_cuts], dtype, DEV,
                                 lists=ops.step_lists(dtype))
        h = torch.cat([inputs[r][at[r]:at[r] + n] for r, n in step_cuts]).to(dtype).to(DEV)
        residual = torch.zeros((h.shape[0], width), dtype=torch.float32, device=DEV)
        part.forward(ops, h, residual, batch, cm.view(0, True, batch.block_tables, batch.state_slots))
        ops.flush()
        o = 0
        for r, n in step_cuts:
            got[r].append(residual[o:o + n].cpu())
            at[r] += n
            o += n
            cm.release_passed(r)
    ops.check_status()
    return {r: torch.cat(v) for r, v in got.items()}


CUTS = [[("a", 30), ("b", 1)], [("b", 2), ("c", 5)], [("a", 1), ("b", 30), ("c", 1)], [("a", 2), ("c", 1)],
        [("a", 17), ("b", 7), ("c", 33)], [("a", 1)], [("a", 1), ("c", 2)]]
TOTAL = {"a": 52, "b": 40, "c": 42}

MIXER_CASES = [
    ("attention", dict(heads=4, kv_heads=2, dim=12, vdim=8, mask={"size": 7}, rot={"dims": 6, "base": 1000.0}, scale=0.29, softcap=5.0)),
    ("attention", dict(heads=2, kv_heads=2, dim=64, vdim=64, mask={"size": 19}, rot={"dims": 64, "base": 1e5}, scale=0.12, softcap=20.0)),
    ("latent_attention", dict(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, rot={"dims": 4, "base": 10000.0}, scale=0.3)),
    ("latent_attention", dict(heads=2, dim=32, rot_dim=16, vdim=24, kv_rank=64, rot={"dims": 16, "base": 50.0}, scale=0.11)),
    ("wkv", dict(heads=2, dim=12)), ("wkv", dict(heads=1, dim=64)), ("wkv", dict(heads=3, dim=40)),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,m", MIXER_CASES)
def test_each_mixer_alone_in_portions(ops, kind, m, dtype):
    from tinyinfer_b200.config import ruvuvik
    width = 48
    g = torch.Generator().manual_seed(m["heads"] * 100 + m["dim"])
    w = mixer_weights(kind, m, width, g, decay_rank=5)
    cfg = ruvuvik.RuvuvikConfig.from_dict({"vocab": 8, "width": width, "norm": {"eps": 1e-5},
                                           "layers": [{"type": kind, "mixer": m, "mlp": None}]})
    from tinyinfer_b200.parts.base import build_part
    part = build_part("mixer", ruvuvik.build_plan(cfg).layers[0].mixer)
    part.load_weights({k: v.to(DEV) for k, v in w.items()}, ops)
    inputs = {r: torch.randn((n, width), generator=g) for r, n in TOTAL.items()}
    got = _run_mixer(ops, part, inputs, CUTS, dtype)
    fn = {"attention": plain.chunked_attention, "latent_attention": plain.latent_attention, "wkv": plain.wkv}[kind]
    w64 = {"x." + k: v.double() for k, v in w.items()}
    for r, x in inputs.items():
        want = fn(x.to(dtype).double(), w64, "x.", m, 1e-5)[0]
        err = (got[r].double() - want).abs().max() / want.abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 3e-2), f"{kind} request {r}: {err}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", [dict(heads=2, dim=12), dict(heads=1, dim=64), dict(heads=3, dim=40), dict(heads=1, dim=128)])
def test_recurrence_over_long_portions(ops, m, dtype):
    """Portions long enough that a head's state columns are cut over several blocks, between portions
    that are not: the state passes from one form of the kernel to the other."""
    from tinyinfer_b200.parts.wkv import WkvMixer
    width = 64
    g = torch.Generator().manual_seed(m["dim"])
    w = mixer_weights("wkv", m, width, g, decay_rank=6)
    part = WkvMixer(width, m["heads"], m["dim"], 1e-5)
    part.load_weights({k: v.to(DEV) for k, v in w.items()}, ops)
    inputs = {"a": torch.randn((203, width), generator=g), "b": torch.randn((72, width), generator=g)}
    cuts = [[("a", 3)], [("a", 130)], [("a", 1), ("b", 70)], [("a", 69), ("b", 2)]]
    got = _run_mixer(ops, part, inputs, cuts, dtype)
    w64 = {"x." + k: v.double() for k, v in w.items()}
    for r, x in inputs.items():
        want = plain.wkv(x.to(dtype).double(), w64, "x.", m, 1e-5)[0]
        err = (got[r].double() - want).abs().max() / want.abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 3e-2), f"request {r}: {err}"


# ---- the model through the engine ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts(tmp_path_factory, name, dtype):
    d = make_model(tmp_path_factory.getbasetemp(), name)
    steps = traces.whole(_requests(name))
    out = _run(d, dtype, steps, traces.max_live_tokens(steps))
    _compare(steps, out, _plain(d, name), dtype, f"{name} whole")


@pytest.mark.parametrize("name, family, dtype", [
    ("A", "tail", "float32"), ("A", "portions", "float32"), ("A", "mixed", "float32"), ("A", "mixed", "bfloat16"),
    ("B", "portions", "float32"), ("B", "mixed", "float32"), ("B", "tail", "bfloat16"),
    ("C", "tail", "float32"), ("C", "portions", "bfloat16"), ("C", "mixed", "float32"), ("C", "mixed", "bfloat16"),
    ("C", "long portions", "bfloat16"), ("C", "long portions", "float32")])
def test_cuttings_agree_with_the_plain_implementation(tmp_path_factory, name, family, dtype):
    """Prefill against token-by-token decoding, portions down to two tokens, and up to four live
    requests of unequal length in a pool so small that pages and state slots are used again."""
    d = make_model(tmp_path_factory.getbasetemp(), name)
    reqs = _requests(name)
    steps = {"tail": lambda: traces.tail_decoded(reqs, tail=40), "portions": lambda: traces.portions(reqs),
             "long portions": lambda: traces.portions(reqs, sizes=(150, 2, 71, 70, 128, 3)),
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


def test_long_decoding_passes_chunks_and_gives_pages_back(tmp_path_factory):
    from tinyinfer_b200 import Engine, StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    tokens = random_tokens(SMALL["A"][0]["vocab"], 170, seed=77)
    cfg, w = plain.load_folder(d)
    want = plain.forward(cfg, w, tokens)[0]
    eng = Engine(d, dtype="float32", page_size=16, num_pages=11, max_requests=2)
    got = [eng.step([StepEntry("x", tokens[:4], [3])])[0].cpu()]
    for p in range(4, len(tokens)):
        got.append(eng.decode_step([StepEntry("x", [tokens[p]], [0])])[0].cpu().clone())
        eng.cache.check()
    assert_close_logits(torch.stack(got), want[3:], FP32_RTOL, "long decoding")
    # the chunked layers hold one page (a chunk of 7 positions), the latent layers all eleven
    assert sorted(eng.cache.free_pages()) == [0, 10] or sorted(eng.cache.free_pages()) == [0, 9]
    eng.finish("x")
    assert eng.cache.free_pages() == [11, 11]


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
    for layer in cfg["layers"]:
        if layer["type"] == "wkv":
            layer["mixer"]["decay_rank"] = 24               # no stored tensor to tell its size
    tokens = random_tokens(cfg["vocab"], 90, seed=1)
    a = Engine(config=cfg, seed=5, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    la = a.step([StepEntry("a", tokens, [0, 50, 89])])
    d = os.path.join(str(tmp_path), "written")
    write_random_model(d, cfg, seed=5)
    b = Engine(d, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    lb = b.step([StepEntry("a", tokens, [0, 50, 89])])
    assert torch.isfinite(la).all() and torch.equal(la, lb)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(tmp_path_factory, tmp_path, dtype):
    """The replay program as a user starts it: steps on standard input, logits in files."""
    import json
    import subprocess
    import sys
    import numpy as np
    d = make_model(tmp_path_factory.getbasetemp(), "C")
    steps = traces.mixed(_requests("C"), seed=9)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
         "--max-tokens", str(traces.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = SMALL["C"][0]["vocab"]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            data = np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4")
            outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, vocab).copy())
    _compare(steps, outputs, _plain(d, "C"), dtype, f"replay {dtype}")


def test_command_line_with_token_ids(tmp_path_factory, capsys):
    from tinyinfer_b200 import cli
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    cfg, w = plain.load_folder(d)
    prompt = random_tokens(cfg["vocab"], 9, seed=4)
    rc = cli.main(["-m", d, "--tokens", "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                   "--max-seq", "64", "--max-num-seqs", "2", "--page-size", "16"])
    assert rc == 0
    out = capsys.readouterr().out
    line = [ln for ln in out.splitlines() if ln.startswith("[output]")][0]
    assert [int(x) for x in line.split()[1:]] == plain.greedy(cfg, w, prompt, 6)
