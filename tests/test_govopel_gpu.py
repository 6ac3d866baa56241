"""Govopel through the engine against the plain implementation (tests/plain_govopel.py, float64).

Each mechanism's kernel alone against its plain function; whole prompts against token-by-token
decoding; portions down to two tokens; batches of unequal requests against each alone with pages
used again; keys just inside and just outside a run of the chunked mask, at page borders and far
back (with sharp attention and a check that an off-by-one mask or a lost key would show); the first
tokens of a sequence; long decoding through CUDA-graph replay; sizes the kernels' fast paths do not
take; greedy generation through ``LLM.generate`` and the scheduler; ``bin/trace_run``.  The
configurations and weights are made in tests/govopel_cases.py.
"""
import json
import math

import pytest
import torch

import govopel_cases as gc
import plain_govopel as pg
from govopel_cases import CASES, row_error

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a logits row (means taken off).  float32: the engine sums in
# another order than the float64 plain implementation.  bfloat16: weights, the operands of every product
# and the cache are rounded to 8 bits of mantissa (an off-by-one mask or a lost key moves rows by 0.1 to 1).
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
DEV = "cuda:0"


def stored(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def run(engine, steps):
    """`steps`: list of (entries, end); an entry is (request, tokens, want).  Returns {(request, position): row}."""
    from rllm_b200.engine import StepItem
    pos, out = {}, {}
    for entries, end in steps:
        logits = engine.step([StepItem(r, toks, want) for r, toks, want in entries])
        row = 0
        for r, toks, want in entries:
            start = pos.get(r, 0)
            for w in want:
                out[(r, start + w)] = logits[row].detach().float().cpu()
                row += 1
            pos[r] = start + len(toks)
        for r in end:
            engine.finish(r)
            pos.pop(r, None)
    engine.check_device_errors()
    return out


def compare(out, refs, dtype, what, tol=None):
    tol = tol or TOL[dtype]
    assert out, what
    for (r, p), row in out.items():
        e = row_error(row, refs[r][p])
        assert e <= tol, f"{what}: request {r} position {p}: error {e:.3e} > {tol}"


def cut(tokens, sizes):
    """Portions of the given sizes in turn (the last size repeats), every position wanted."""
    out, at, i = [], 0, 0
    while at < len(tokens):
        k = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        out.append((tokens[at:at + k], list(range(k))))
        at, i = at + k, i + 1
    return out


def one_by_one(r, toks, lo=0):
    return [([(r, [t], [0])], []) for t in toks[lo:]]


# ---------------------------------------------------------------- each kernel alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_rows_kernel(dtype):
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    y = torch.randn(9, 70, generator=g).to(DEV)
    w = (1 + 0.3 * torch.randn(50, generator=g)).to(DEV)
    x = torch.randn(9, 50, generator=g).to(DEV)
    want = x.double() + pg.rms_norm(y[:, 5:55].double(), w.double(), 1e-4)
    low = torch.zeros((9, 64), dtype=dtype, device=DEV)
    x2 = x.clone()
    ops.norm_rows(y[:, 5:55], w, 1e-4, x=x2, add=True, low=low[:, :50])
    assert torch.allclose(x2.double(), want, atol=1e-5)
    assert torch.allclose(low[:, :50].double(), want, atol=1e-5 if dtype == torch.float32 else 3e-2)
    assert float(low[:, 50:].abs().max()) == 0.0
    x3 = x.clone()
    ops.norm_rows(x3, None, 1e-4, x=x3)                       # in place, no weight, nothing added
    assert torch.allclose(x3.double(), pg.rms_unit(x.double(), 1e-4), atol=1e-5)


@pytest.mark.parametrize("rot,scaling", [(6, None), (10, (4.0, 16, 8.0, 2.0)), (0, None)])
def test_rotate_then_unit_norm_kernel(rot, scaling):
    from rllm_b200.csrc import ops
    from rllm_b200.parts import Runtime, part_class
    H, G, d, bs, n = 5, 2, 10, 4, 7
    g = torch.Generator().manual_seed(2)
    rows = torch.randn(n, (H + G) * d + 3, generator=g).to(DEV)
    positions = torch.tensor([0, 1, 2, 40, 41, 300, 7], dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 0, 5, -1, 9, 11, 6], dtype=torch.int32, device=DEV)
    q = torch.empty((n, H * d), device=DEV)
    kc, vc = torch.zeros((3, G, bs, d), device=DEV), torch.zeros((3, G, bs, d), device=DEV)
    cs, mult = None, 1.0
    rspec = gc.rot(max(rot, 2), 300.0, scaling)
    if rot:
        part = part_class("position", "rotary_scaled")({"dims": rot, "base": 300.0, "scaling": rspec.get("scaling")}, "",
                                                       Runtime(torch.device(DEV), torch.float32))
        cs, mult = ops.rope_table(positions, part.table()), part.mult
    ops.rope_unitnorm_store(rows[:, :(H + G) * d], cs, rot, mult, slots, q, kc, vc, H, G, d, bs, 1e-5)
    heads = rows[:, :(H + G) * d].double().cpu().view(n, H + G, d)
    turned = pg.rotate(heads, positions.tolist(), rspec) if rot else heads
    want = pg.rms_unit(turned, 1e-5)
    assert torch.allclose(q.double().cpu().view(n, H, d), want[:, :H], atol=2e-5)
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.allclose(kc[s // bs, :, s % bs].double().cpu(), want[t, H:], atol=2e-5)
        assert torch.equal(vc[s // bs, :, s % bs].cpu(), rows[t, H * d:(H + G) * d].cpu().view(G, d))
    assert float(kc[0, :, 1].abs().max()) == 0.0 and float(kc[0, :, 2].abs().max()) == 0.0     # slots nobody named


def test_latent_store_kernel_and_head_products():
    from rllm_b200.csrc import ops
    from rllm_b200.parts import Runtime, part_class
    H, dq, r, rank, bs, n = 3, 5, 6, 9, 4, 6
    g = torch.Generator().manual_seed(3)
    q = torch.randn(n, H * (dq + r), generator=g).to(DEV)
    kv = torch.randn(n, rank + r + 2, generator=g).to(DEV)
    w = (1 + 0.2 * torch.randn(rank, generator=g)).to(DEV)
    positions = torch.tensor([0, 5, 6, 100, 2, 3], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 7, 2, 5, -1, 4], dtype=torch.int32, device=DEV)
    part = part_class("position", "rotary_scaled")({"dims": r, "base": 77.0, "scaling": None}, "",
                                                   Runtime(torch.device(DEV), torch.float32))
    cache = torch.zeros((2, 1, bs, rank + r), device=DEV)
    q_att = torch.zeros((n, H * (rank + r)), device=DEV)
    ops.latent_rope_store(q, kv[:, :rank + r], w, ops.rope_table(positions, part.table()), part.mult, slots, q_att,
                          cache, H, dq, r, rank, bs, 1e-5)
    rspec = gc.rot(r, 77.0)
    q_rot = pg.rotate(q.double().cpu().view(n, H, dq + r)[:, :, dq:], positions.tolist(), rspec)
    assert torch.allclose(q_att.double().cpu().view(n, H, rank + r)[:, :, rank:], q_rot, atol=1e-5)
    assert float(q_att.view(n, H, rank + r)[:, :, :rank].abs().max()) == 0.0
    c = pg.rms_norm(kv[:, :rank].double().cpu(), w.double().cpu(), 1e-5)
    kr = pg.rotate(kv[:, rank:rank + r].double().cpu().view(n, 1, r), positions.tolist(), rspec)[:, 0]
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.allclose(cache[s // bs, 0, s % bs].double().cpu(), torch.cat([c[t], kr[t]]), atol=1e-5)
    # one product per head, operands and results as columns of wider rows
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        for k, m in ((5, 9), (16, 24)):
            a = torch.randn(n, H, k + 8, generator=g).to(DEV, dtype)
            wh = torch.randn(H, m, k, generator=g).to(DEV, dtype)
            out = torch.zeros((n, H, m + 8), device=DEV, dtype=dtype)
            ops.head_linear(a[:, :, :k], wh, out[:, :, :m])
            want = torch.einsum("nhk,hmk->nhm", a[:, :, :k].double(), wh.double())
            assert torch.allclose(out[:, :, :m].double(), want, atol=tol * float(want.abs().max()))
            assert float(out[:, :, m:].abs().max()) == 0.0


def test_clamped_glu_and_softcap_kernels():
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    gu = (3 * torch.randn(5, 2 * 13, generator=g)).to(DEV)
    out = torch.empty((5, 13), device=DEV)
    ops.glu_clamped(gu, out, 2.0, 1.702, 1.0)
    eye = torch.eye(13, dtype=torch.float64)
    gate, up = gu[:, :13].double().cpu(), gu[:, 13:].double().cpu()
    want = torch.clamp(gate, max=2.0) * torch.sigmoid(1.702 * torch.clamp(gate, max=2.0)) * (torch.clamp(up, -2.0, 2.0) + 1.0)
    assert torch.allclose(out.double().cpu(), want @ eye, atol=1e-5)
    assert float((gate > 2.0).sum()) > 0 and float((up < -2.0).sum()) > 0
    x = (40 * torch.randn(3, 11, generator=g)).to(DEV)
    want = 30.0 * torch.tanh(x.double() / 30.0)
    ops.softcap_rows(x, 30.0)
    assert torch.allclose(x.double(), want, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_attention_kernel_chunk_cap_and_values_in_keys(dtype):
    """The plain attention kernel with a chunked mask, capped scores and the values read from the key
    rows, against the formula written with torch; pages in a scrambled order."""
    from rllm_b200.csrc import ops
    H, hd, hdv, bs, T, chunk, cap, scale = 3, 12, 8, 4, 23, 6, 4.0, 0.9
    g = torch.Generator().manual_seed(5)
    keys = torch.randn(T, hd, generator=g).to(dtype)
    q = torch.randn(T, H * hd, generator=g).to(dtype)
    pages = torch.randperm(8, generator=g)[:6]
    cache = torch.zeros((8, 1, bs, hd), dtype=dtype)
    for p in range(T):
        cache[pages[p // bs], 0, p % bs] = keys[p]
    out = torch.empty((T, H * hdv), dtype=dtype, device=DEV)
    cache = cache.to(DEV)
    ops.paged_attention_generic(q.to(DEV), cache, cache, out, torch.arange(T, dtype=torch.int32, device=DEV),
                                torch.zeros(T, dtype=torch.int32, device=DEV), pages.to(torch.int32).view(1, -1).to(DEV),
                                H, 1, hd, bs, scale, v_head_dim=hdv, chunk=chunk, softcap=cap)
    vis = pg.chunk_mask(T, chunk)
    for h in range(H):
        s = q.double().view(T, H, hd)[:, h] @ keys.double().T * scale
        want = pg.softmax_rows(cap * torch.tanh(s / cap), vis) @ keys.double()[:, :hdv]
        got = out.double().cpu().view(T, H, hdv)[:, h]
        assert torch.allclose(got, want, atol=1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("H,W,V,cap", [(40, 144, 128, 0.0), (8, 576, 512, 20.0), (3, 80, 64, 0.0)])
def test_latent_decode_kernel_against_the_plain_kernel(H, W, V, cap):
    """The tensor-core decode kernel of attention over one shared key/value head (head chunks that are
    not full, several splits, contexts that end inside a tile, a split and a page; scrambled pages)
    gives what the plain kernel gives from the same cache."""
    from rllm_b200.csrc import ops
    bs, lens = 16, [1, 33, 128, 129, 300, 517]
    g = torch.Generator().manual_seed(6)
    n_pages = sum(-(-L // bs) for L in lens)
    order = torch.randperm(n_pages + 3, generator=g).tolist()
    cache = torch.randn(n_pages + 3, 1, bs, W, generator=g).to(DEV, torch.bfloat16)
    table = torch.zeros((len(lens), -(-max(lens) // bs)), dtype=torch.int32)
    for r, L in enumerate(lens):
        for b in range(-(-L // bs)):
            table[r, b] = order.pop()
    # two tokens of the longest request, one of each other
    seq = torch.tensor([0, 1, 2, 3, 4, 5, 5], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 32, 127, 128, 299, 515, 516], dtype=torch.int32, device=DEV)
    q = torch.randn(7, H * W, generator=g).to(DEV, torch.bfloat16)
    want = torch.empty((7, H * V), dtype=torch.bfloat16, device=DEV)
    got = torch.zeros_like(want)
    scale = 1.0 / math.sqrt(W)
    ops.paged_attention_generic(q, cache, cache, want, pos, seq, table.to(DEV), H, 1, W, bs, scale, v_head_dim=V,
                                softcap=cap)
    ops.latent_decode_attention(q, cache, got, pos, seq, table.to(DEV), H, W, V, bs, scale, cap, max(lens))
    ops.check_device_errors(DEV)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), float((got.float() - want.float()).abs().max())
    assert torch.equal(got[0].view(H, V), cache[table[0, 0], 0, 0, :V].expand(H, V))       # one key: the value itself


# ---------------------------------------------------------------- each configuration, each way of cutting

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompt(name, dtype):
    cfg = CASES[name]
    w = gc.make_weights(cfg, 3, stored(dtype))
    toks = gc.tokens_for(cfg, 45, 1)
    ref = gc.oracle(cfg, w, toks)
    eng = gc.build_engine(cfg, w, dtype, max_tokens=64)
    out = run(eng, [([("a", toks, list(range(len(toks))))], ["a"])])
    compare(out, {"a": ref}, dtype, f"{name} whole")
    if dtype == "float32":
        assert all(int(out["a", p].argmax()) == int(ref[p].argmax()) for p in range(len(toks)))


def test_stream_after_every_layer():
    """The residual stream itself, layer by layer, in float32."""
    cfg = CASES["stack"]
    w = gc.make_weights(cfg, 8)
    toks = gc.tokens_for(cfg, 21, 9)
    want = []
    gc.oracle(cfg, w, toks, want)
    eng = gc.build_engine(cfg, w, "float32", max_tokens=32)
    seen = []
    for block in eng.model.blocks:
        inner = block.forward

        def spy(x, pending, ctx, cache, _inner=inner):
            out = _inner(x, pending, ctx, cache)
            seen.append(x.detach().double().cpu().clone())
            return out
        block.forward = spy
    run(eng, [([("a", toks, [20])], ["a"])])
    assert len(seen) == len(want) == 4
    for got, ref in zip(seen, want):
        assert float((got - ref).abs().max()) < 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_token_by_token_and_portions(name, dtype):
    """The same prompt decoded one token a step from the first token on, and in portions of 2, 3, 2,
    17, 5, 2, 2, ... tokens: every row as the plain implementation has it."""
    cfg = CASES[name]
    w = gc.make_weights(cfg, 4, stored(dtype))
    toks = gc.tokens_for(cfg, 52, 2)
    ref = {"a": gc.oracle(cfg, w, toks)}
    eng = gc.build_engine(cfg, w, dtype, max_tokens=128)
    steps = one_by_one("a", toks)
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), ref, dtype, f"{name} one by one")
    steps = [([("a", p, want)], []) for p, want in cut(toks, [2, 3, 2, 17, 5, 2, 2, 9, 1, 1, 2])]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), ref, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["stack", "stack_attention_first", "latent_odd", "chunked", "heads64", "heads128"])
def test_unequal_requests_in_one_batch_with_reuse(name, dtype):
    """Four requests of 61, 9, 33 and 2 tokens come and go in a pool of two request slots and few
    pages: portions of some beside single tokens of others; pages that a finished request gave back
    go to the next one.  Every row equals the request alone."""
    cfg = CASES[name]
    w = gc.make_weights(cfg, 5, stored(dtype))
    lens = {"a": 61, "b": 9, "c": 33, "d": 2}
    toks = {r: gc.tokens_for(cfg, n, 10 + i) for i, (r, n) in enumerate(lens.items())}
    refs = {r: gc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = gc.build_engine(cfg, w, dtype, max_tokens=96, block_size=8, max_requests=2)
    at = {r: 0 for r in toks}
    plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 5)], [("a", 16), ("b", 1)], [("a", 1), ("b", 1)],      # b ends
            [("a", 3), ("c", 9)], [("a", 1), ("c", 1)], [("a", 2), ("c", 17)], [("a", 30), ("c", 1)],     # a ends
            [("c", 1), ("d", 2)],                                                                         # d ends
            [("c", 4)]]
    steps = []
    for st in plan:
        entries = []
        for r, k in st:
            lo = at[r]
            at[r] = lo + k
            entries.append((r, toks[r][lo:lo + k], list(range(k))))
        steps.append((entries, [r for r, _ in st if at[r] == len(toks[r])]))
    assert all(at[r] == len(toks[r]) for r in toks)
    compare(run(eng, steps), refs, dtype, f"{name} mixed")
    eng.cache.check_invariants()
    assert not eng.cache.requests


def test_pages_used_again_give_the_same_bits():
    """A request that runs on pages another request just left has the bits it has in a fresh engine."""
    cfg = CASES["stack"]
    w = gc.make_weights(cfg, 6)
    a, b = gc.tokens_for(cfg, 40, 20), gc.tokens_for(cfg, 37, 21)
    sched = [([("b", b[:20], [19])], []), ([("b", b[20:], list(range(17)))], ["b"])]
    fresh = run(gc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1), sched)
    eng = gc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1)
    run(eng, [([("a", a, [39])], ["a"])])
    again = run(eng, sched)
    for key, row in fresh.items():
        assert torch.equal(row, again[key]), key


# ---------------------------------------------------------------- edges of the chunked mask, far keys

ASK, TARGET = 5, 6         # the asking token's queries are turned towards the target token's keys


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunk_edges_to_the_token(dtype):
    """Runs of 21 positions on pages of 8 (run borders fall inside pages), sharp attention, and pairs of
    (target, asker) tokens: 2 apart inside a run, 2 apart across a run's border (the asker is the first
    or second position of the next run), and at the two ends of one run.  First a test of the test:
    with runs one position longer or shorter the rows of askers near a border move by far more than
    the tolerance.  Then the engine has the true rows in a whole prompt, in portions cut inside runs
    and pages, and in single-token steps."""
    cfg = gc.config([gc.att(4, 2, 16, 4, 21, scale=1.6, softcap=40.0, ff=48), gc.lat(2, 8, 4, 8, 12, 10)],
                    width=32, vocab=67)
    w = gc.marked_attention(cfg, gc.make_weights(cfg, 7, stored(dtype)), ASK, TARGET)
    toks = gc.tokens_for(cfg, 110, 3, avoid=(ASK, TARGET))
    pairs = [(8, 10), (19, 21), (20, 22), (41, 42), (42, 62), (63, 83), (82, 84), (83, 85), (100, 104)]
    for t, a in pairs:
        toks[t], toks[a] = TARGET, ASK
    ref = gc.oracle(cfg, w, toks)
    tol = TOL[dtype]
    for delta in (1, -1):
        other = gc.oracle(gc.with_chunk(cfg, delta), w, toks)
        moved = {p for p in range(len(toks)) if row_error(other[p], ref[p]) > 3 * tol}
        assert {21, 22, 42} & moved and len(moved & {a for _, a in pairs}) >= 4, (delta, sorted(moved))
    eng = gc.build_engine(cfg, w, dtype, max_tokens=128, block_size=8)
    whole = run(eng, [([("a", toks, list(range(len(toks))))], ["a"])])
    compare(whole, {"a": ref}, dtype, "whole")
    steps = [([("a", p, want)], []) for p, want in cut(toks, [20, 2, 19, 3, 2, 37, 2, 2, 5])]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), {"a": ref}, dtype, "portions")
    steps = [([("a", toks[:17], list(range(17)))], [])] + one_by_one("a", toks, 17)
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), {"a": ref}, dtype, "single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(dtype):
    """Attention through the latent, sharp: askers at places 300 to 420 hang on one target key at
    place 3 (its page is the first of fourteen and more; pages of 32), in a long portion, in short
    ones and decoded alone.  Without the target the rows are others."""
    cfg = gc.config([gc.lat(3, 16, 4, 12, 24, 24, scale=1.5, ff=40), gc.att(2, 1, 8, 4, 50)], width=40, vocab=73)
    w = gc.marked_latent(cfg, gc.make_weights(cfg, 9, stored(dtype)), ASK, TARGET)
    toks = gc.tokens_for(cfg, 430, 4, avoid=(ASK, TARGET))
    askers = [300, 333, 352, 383, 384, 401, 419, 420, 429]
    toks[3] = TARGET
    for a in askers:
        toks[a] = ASK
    ref = gc.oracle(cfg, w, toks)
    blind = gc.oracle(cfg, w, [7 if t == TARGET else t for t in toks])
    assert all(row_error(blind[a], ref[a]) > 3 * TOL[dtype] for a in askers)
    eng = gc.build_engine(cfg, w, dtype, max_tokens=448, block_size=32)
    steps = [([("a", toks[:340], [0, 3, 300, 333, 339])], []), ([("a", toks[340:353], [12])], []),
             ([("a", toks[353:355], [0, 1])], []), ([("a", toks[355:400], [28, 29])], [])]
    steps += one_by_one("a", toks, 400)
    compare(run(eng, steps), {"a": ref}, dtype, "far key")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """200 single-token steps of two requests behind short prompts (graphs captured per context
    bucket, padded to a power of two of requests), every tenth row against the plain implementation;
    in float32 the replayed steps give what eager steps give."""
    cfg = CASES["stack"]
    w = gc.make_weights(cfg, 10, stored(dtype))
    reqs = {"a": gc.tokens_for(cfg, 215, 30), "b": gc.tokens_for(cfg, 203, 31), "c": gc.tokens_for(cfg, 206, 32)}
    refs = {r: gc.oracle(cfg, w, t) for r, t in reqs.items()}
    outs = []
    for graphs in ((True, False) if dtype == "float32" else (True,)):
        eng = gc.build_engine(cfg, w, dtype, max_tokens=768, block_size=16, use_graphs=graphs)
        steps = [([("a", reqs["a"][:15], [14]), ("b", reqs["b"][:3], [2]), ("c", reqs["c"][:6], [5])], [])]
        for i in range(200):
            steps.append(([(r, [t[len(t) - 200 + i]], [0] if i % 10 == 9 else []) for r, t in reqs.items()], []))
        outs.append(run(eng, steps))
        if graphs:
            assert eng.stats["graph_replays"] > 150
    compare(outs[0], refs, dtype, "long decoding")
    if len(outs) == 2:
        for key, row in outs[0].items():
            assert row_error(row, outs[1][key]) < 1e-6, key


REAL = gc.config([gc.lat(8, 128, 64, 128, 512, 384, ff=1536), gc.att(8, 2, 128, 64, 100, softcap=50.0, ff=1024),
                  gc.att(16, 4, 64, 64, 160, scaling=(4.0, 128, 32.0, 1.0), ff=2048)], width=1024, vocab=1531,
                 logit_softcap=30.0)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_a_real_model(dtype):
    """Width 1,024 and layers of real sizes (a latent of 512 + 64 entries under 8 heads; heads of 128
    and 64 with runs of 100 and 160 positions): the products take the library, the tcgen05 and the
    weight-streaming kernels.  A prompt of 300 tokens, a portion of 40 beside another request's 20,
    then single tokens of both."""
    cfg = REAL
    w = gc.make_weights(cfg, 16, stored(dtype), gain=1.0)
    toks = {"a": gc.tokens_for(cfg, 352, 70), "b": gc.tokens_for(cfg, 32, 71)}
    refs = {r: gc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = gc.build_engine(cfg, w, dtype, max_tokens=512, block_size=32, max_requests=2)
    steps = [([("a", toks["a"][:300], list(range(0, 300, 23)) + [99, 100, 159, 160, 299])], []),
             ([("a", toks["a"][300:340], list(range(40))), ("b", toks["b"][:20], [0, 19])], [])]
    steps += [([("a", [toks["a"][340 + i]], [0]), ("b", [toks["b"][20 + i]], [0])], []) for i in range(12)]
    compare(run(eng, steps), refs, dtype, "real layer sizes")


# ---------------------------------------------------------------- the entry points a user calls

def write_folder(path, cfg, w):
    from rllm_b200.weights.safetensors_io import write_safetensors
    path.mkdir(exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", w)
    return path


def test_greedy_generation_through_the_scheduler(tmp_path):
    """LLM.generate (scheduler, continuous batching, prompts cut into portions of 16, device sampler)
    on a folder written in the stored format: the greedy continuation of each prompt is the plain
    implementation's."""
    from rllm_b200.llm import LLM
    cfg = CASES["stack"]
    w = gc.make_weights(cfg, 11)
    write_folder(tmp_path, cfg, w)
    prompts = [gc.tokens_for(cfg, n, 40 + i) for i, n in enumerate((37, 3, 21, 50, 9))]
    llm16 = LLM(str(tmp_path), dtype="bfloat16", ctx=128, block_size=8, prefill_chunk=16, parallel=3)
    got16 = llm16.generate(prompts, max_tokens=12, temperature=0.7, top_k=20, seed=5)
    assert all(len(g) == 12 and all(0 <= t < cfg["vocab"] for t in g) for g in got16)
    assert not llm16.engine.cache.requests
    del llm16
    llm = LLM(str(tmp_path), dtype="float32", ctx=128, block_size=8, prefill_chunk=16, parallel=3)
    got = llm.generate(prompts, max_tokens=12)
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = gc.oracle(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-4:       # a tie at float32 precision decides nothing
                break
            assert int(logits.argmax()) == tok
            seq.append(tok)
    assert all(len(g) == 12 for g in got)
    assert not llm.engine.cache.requests


def test_trace_replay_program_chooses_the_model_by_its_config(tmp_path):
    """bin/trace_run on a Govopel folder: steps from standard input, rows out as little-endian float32."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    cfg = CASES["stack_attention_first"]
    w = gc.make_weights(cfg, 12, torch.bfloat16)
    model = write_folder(tmp_path / "model", cfg, w)
    toks = gc.tokens_for(cfg, 30, 6)
    lines = [json.dumps({"step": 0, "entries": [{"id": "x", "tokens": toks[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "x", "tokens": toks[20:], "want": []}], "end": ["x"]})]
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "64"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    rows = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    ref = gc.oracle(cfg, w, toks)
    assert row_error(rows[0], ref[0]) < TOL["float32"] and row_error(rows[1], ref[19]) < TOL["float32"]
    assert not (tmp_path / "out" / "1.f32").exists()


def test_random_weights_mode_writes_a_folder_the_engine_loads(tmp_path):
    """The package's own random-weights mode knows the design's tensors."""
    from rllm_b200.config import config_from_dict
    from rllm_b200.models.model import load_model
    from rllm_b200.weights import write_random_model
    write_random_model(config_from_dict(CASES["stack"]), tmp_path, seed=3, dtype=torch.bfloat16)
    cfg, model = load_model(tmp_path, "bfloat16", DEV)
    assert cfg.to_dict() == CASES["stack"] and model.loaded
