"""Falalix through the engine against the plain implementation (tests/plain_falalix.py, float64).

Each mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, batches of unequal requests against each alone, pages and state slots that are freed and
used again, keys at page borders and just inside and outside the window and the kept first keys
(with sharp attention and a check that an off-by-one mask would show), the first tokens of a
sequence, long decoding, CUDA-graph replay against eager steps, and greedy generation through
``LLM.generate`` and the scheduler.  The configurations and weights are made in
tests/falalix_cases.py.
"""
import json

import pytest
import torch

import falalix_cases as fc
from falalix_cases import CASES, row_error

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a logits row (means taken off).  float32: the engine sums
# in another order than the float64 plain implementation; measured worst 4e-6.  bfloat16: weights
# and the activations handed between kernels are rounded to 8 bits of mantissa; measured worst
# 2.5e-2 at these sizes (an off-by-one window or a lost state moves rows by 0.1 to 1).
TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def stored(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def run(engine, steps):
    """`steps`: list of (entries, end); an entry is (request, tokens, want).  Returns {(request, position): row}."""
    from rllm_b200.engine import StepItem
    pos, out = {}, {}
    for entries, end in steps:
        items = [StepItem(r, toks, want) for r, toks, want in entries]
        logits = engine.step(items)
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


# ---------------------------------------------------------------- each mechanism, each way of cutting

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompt(name, dtype):
    cfg = CASES[name]
    w = fc.make_weights(cfg, 3, stored(dtype))
    toks = fc.tokens_for(cfg, 45, 1)
    ref = fc.oracle(cfg, w, toks)
    eng = fc.build_engine(cfg, w, dtype, max_tokens=64)
    out = run(eng, [([("a", toks, list(range(len(toks))))], ["a"])])
    compare(out, {"a": ref}, dtype, f"{name} whole")
    if dtype == "float32":
        assert all(int(out["a", p].argmax()) == int(ref[p].argmax()) for p in range(len(toks)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_token_by_token_and_portions(name, dtype):
    """The same prompt decoded one token a step from the first token on, and in portions of 2, 3, 2,
    17, 5, 2, 2, ... tokens: every row as the plain implementation has it."""
    cfg = CASES[name]
    w = fc.make_weights(cfg, 4, stored(dtype))
    toks = fc.tokens_for(cfg, 52, 2)
    ref = {"a": fc.oracle(cfg, w, toks)}
    eng = fc.build_engine(cfg, w, dtype, max_tokens=128)
    steps = [([("a", [t], [0])], []) for t in toks]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), ref, dtype, f"{name} one by one")
    parts = cut(toks, [2, 3, 2, 17, 5, 2, 2, 9, 1, 1, 2])
    steps = [([("a", p, want)], []) for p, want in parts]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), ref, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["loop3_from_0", "loop1_tail", "no_loop", "mamba", "time_mix"])
def test_unequal_requests_in_one_batch_with_reuse(name, dtype):
    """Four requests of 61, 9, 33 and 2 tokens come and go in a pool of two state slots and few
    pages: portions of some beside single tokens of others; a slot and pages that a finished
    request gave back go to the next one.  Every row equals the request alone."""
    cfg = CASES[name]
    w = fc.make_weights(cfg, 5, stored(dtype))
    lens = {"a": 61, "b": 9, "c": 33, "d": 2}
    toks = {r: fc.tokens_for(cfg, n, 10 + i) for i, (r, n) in enumerate(lens.items())}
    refs = {r: fc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = fc.build_engine(cfg, w, dtype, max_tokens=96, block_size=8, max_requests=2)
    at = {r: 0 for r in toks}

    def take(r, k):
        lo = at[r]
        k = min(k, len(toks[r]) - lo)
        at[r] = lo + k
        return (r, toks[r][lo:lo + k], list(range(k)))

    def done():
        return [r for r in toks if at[r] == len(toks[r]) and r in live]

    steps, live = [], set()
    plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 5)], [("a", 16), ("b", 1)], [("a", 1), ("b", 1)],      # b ends
            [("a", 3), ("c", 9)], [("a", 1), ("c", 1)], [("a", 2), ("c", 17)], [("a", 30), ("c", 1)],     # a ends
            [("c", 1), ("d", 2)],                                                                         # d ends
            [("c", 4)]]
    for st in plan:
        entries = []
        for r, k in st:
            live.add(r)
            entries.append(take(r, k))
        end = done()
        live -= set(end)
        steps.append((entries, end))
    assert all(at[r] == len(toks[r]) for r in toks)
    out = run(eng, steps)
    compare(out, refs, dtype, f"{name} mixed")
    eng.cache.check_invariants()
    assert not eng.cache.requests


def test_slot_and_pages_used_again_give_the_same_bits():
    """A request that runs in a slot and on pages another request just left has the bits it has in a
    fresh engine: nothing of the earlier request's state or keys is seen."""
    cfg = CASES["loop1_tail"]
    w = fc.make_weights(cfg, 6)
    a, b = fc.tokens_for(cfg, 40, 20), fc.tokens_for(cfg, 37, 21)
    fresh = run(fc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1),
                [([("b", b[:20], [19])], []), ([("b", b[20:], list(range(17)))], ["b"])])
    eng = fc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1)
    run(eng, [([("a", a, [39])], ["a"])])
    again = run(eng, [([("b", b[:20], [19])], []), ([("b", b[20:], list(range(17)))], ["b"])])
    for key, row in fresh.items():
        assert torch.equal(row, again[key]), key


# ---------------------------------------------------------------- edges of the window and of the kept keys

EDGE = fc.config([fc.parallel(fc.att(4, 2, 16, 24, 21, 10, scale=6.0), 2, 16, 4, ls=1.0, rs=0.3, ff=48),
                  fc.mamba(32, 6, 2, 3)], width=32, vocab=67, mult=0.8)
MARK = 5          # the token whose key every query of layer 0 is turned towards


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layout", ["window", "kept", "not_kept"])
def test_window_and_kept_keys_to_the_token(layout, dtype):
    """A window of 21 keys and 10 kept first keys on pages of 8 (the kept keys span two pages, the
    window's edge crosses page borders as the request grows), and marked keys that decide a row when
    they are visible.  `window`: marked keys 25 apart, so that a query sees at most one: the query 20
    behind it does, the query 21 behind it does not.  `kept`: one marked key at place 9, the last kept
    one, which every later query sees.  `not_kept`: at place 10, the first that is not kept, which
    queries from 31 on do not see.  First a test of the test: with a window one key longer or shorter
    (one kept key more or fewer) exactly those rows move by far more than the tolerance.  Then the
    engine has the true rows in a whole prompt, in portions cut inside pages and windows, and in
    single-token steps."""
    cfg = EDGE
    w = fc.marked(cfg, fc.make_weights(cfg, 7, stored(dtype)), MARK)
    toks = [t if t != MARK else MARK + 1 for t in fc.tokens_for(cfg, 122, 3)]
    marks, variants = {"window": ((25, 50, 75, 100), ((1, 0), (-1, 0))), "kept": ((9,), ((0, -1),)),
                       "not_kept": ((10,), ((0, 1),))}[layout]
    for p in marks:
        toks[p] = MARK
    ref = fc.oracle(cfg, w, toks)
    tol = TOL[dtype]
    for d_size, d_keep in variants:
        other = fc.oracle(fc.with_mask(cfg, d_size, d_keep), w, toks)
        moved = {p for p in range(len(toks)) if row_error(other[p], ref[p]) > 3 * tol}
        if layout == "window":
            edge = {p + 21 for p in marks} if d_size > 0 else {p + 20 for p in marks}
            assert edge <= moved, f"a window off by {d_size} would not show at rows {sorted(edge - moved)}"
        else:
            assert len(moved) >= 50, f"{d_keep} kept keys more would move only {len(moved)} rows"
    eng = fc.build_engine(cfg, w, dtype, max_tokens=128, block_size=8)
    allw = list(range(len(toks)))
    compare(run(eng, [([("a", toks, allw)], ["a"])]), {"a": ref}, dtype, "edges, whole")
    steps = [([("a", p, want)], []) for p, want in cut(toks, [5, 2, 11, 3, 8, 2, 21, 1, 1, 1, 7])]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), {"a": ref}, dtype, "edges, portions")
    steps = [([("a", toks[:12], list(range(12)))], [])] + [([("a", [t], [0])], []) for t in toks[12:]]
    steps[-1] = (steps[-1][0], ["a"])
    compare(run(eng, steps), {"a": ref}, dtype, "edges, decoded")


@pytest.mark.parametrize("dim,window,keep,heads,kv", [(64, 150, 70, 4, 2), (128, 200, 3, 4, 2), (64, 64, 64, 4, 1),
                                                      (128, 130, 129, 3, 3), (64, 100, 17, 8, 1)])
def test_tensor_core_attention_with_kept_keys(dim, window, keep, heads, kv):
    """bfloat16 with head sizes the mma kernels take, windows and kept keys longer than their key
    tiles (64 keys in prompt portions, 16 in decode steps, splits of 128).  Two requests side by
    side, with marked keys as above: `edge` has them window + 5 apart behind the kept keys (the query
    window - 1 behind one sees it, the next does not), `kept` has one at the last kept place.  Whole
    prompts of 300 tokens, portions (more than 8 tokens take the prefill shape, fewer the decode
    shape), then 130 single-token steps for both at once."""
    cfg = fc.config([fc.parallel(fc.att(heads, kv, dim, dim, window, keep, scale=96.0 / dim), 2, 16, 4, ls=1.0, rs=0.2,
                                 ff=48)], width=48, vocab=97, mult=0.9)
    w = fc.marked(cfg, fc.make_weights(cfg, 13, torch.bfloat16), MARK)
    base = [t if t != MARK else MARK + 1 for t in fc.tokens_for(cfg, 430, 7)]
    toks = {"edge": list(base), "kept": list(base)}
    marks = list(range(keep + 20, 430 - window, window + 5))
    for p in marks:
        toks["edge"][p] = MARK
    toks["kept"][keep - 1] = MARK
    ref = {r: fc.oracle(cfg, w, t) for r, t in toks.items()}
    tol = TOL["bfloat16"]
    longer = fc.oracle(fc.with_mask(cfg, 1, 0), w, toks["edge"])
    assert all(row_error(longer[p + window], ref["edge"][p + window]) > 3 * tol for p in marks), "blind to the window's edge"
    fewer = fc.oracle(fc.with_mask(cfg, 0, -1), w, toks["kept"])
    assert sum(row_error(fewer[p], ref["kept"][p]) > 3 * tol for p in range(430)) >= 100, "blind to the kept keys"
    eng = fc.build_engine(cfg, w, "bfloat16", max_tokens=960, block_size=16)
    from rllm_b200.csrc import ops
    calls = []
    real = ops.paged_attention_generic
    ops.paged_attention_generic = lambda *a, **k: calls.append(1) or real(*a, **k)
    try:
        want = list(range(300))
        compare(run(eng, [([(r, t[:300], want)], [r]) for r, t in toks.items()]), ref, "bfloat16", "kept keys, whole")
        parts = {r: cut(t[:300], [70, 3, 90, 8, 9, 64, 2, 54]) for r, t in toks.items()}
        steps = [([(r, parts[r][i][0], parts[r][i][1]) for r in toks], []) for i in range(len(parts["edge"]))]
        steps += [([(r, [t[i]], [0]) for r, t in toks.items()], []) for i in range(300, 430)]
        compare(run(eng, steps), ref, "bfloat16", "kept keys, portions and decoding")
    finally:
        ops.paged_attention_generic = real
    assert not calls, "the plain attention kernel ran where the tensor-core kernels should"


def test_pages_behind_the_window_go_back_and_kept_pages_stay():
    """A request far longer than window + kept keys in a pool that could not hold it whole: the pages
    between the kept first keys and the window are given back while it grows, the kept ones stay, and
    every row is still right."""
    cfg = fc.config([fc.parallel(fc.att(2, 1, 16, 8, 40, 5, scale=2.0), 1, 16, 3, ff=32)], width=24, vocab=41)
    w = fc.make_weights(cfg, 8)
    toks = fc.tokens_for(cfg, 700, 4)
    ref = fc.oracle(cfg, w, toks)
    eng = fc.build_engine(cfg, w, "float32", max_tokens=448, block_size=8, max_requests=1)
    want = [0, 1, 4, 5, 6, 39, 40, 41, 44, 45, 46, 127, 128, 300, 301, 511, 512, 513, 698, 699]
    steps, at = [], 0
    for k in [130, 2, 64, 200, 1, 1, 1, 190, 100, 11]:
        steps.append(([("a", toks[at:at + k], [p - at for p in want if at <= p < at + k])], []))
        at += k
    assert at == 700
    out = run(eng, steps)
    compare(out, {"a": ref}, "float32", "long windowed request")
    table = eng.cache.block_table("a", 0, raw=True)
    assert table[0] is not None and all(b is None for b in table[1:60]), "kept page stays, passed pages go back"
    assert eng.cache.n_free_pages(0) > 56 - 12
    eng.finish("a")
    eng.cache.check_invariants()


# ---------------------------------------------------------------- far back through the states, long decoding

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_then_long_decoding(dtype):
    """600 tokens in portions of 97, then 150 single-token steps (replayed from CUDA graphs, through
    several context buckets): what the early tokens left in the states and the kept keys still
    shapes the last rows, and the rows stay right all the way."""
    cfg = CASES["loop1_tail"]
    w = fc.make_weights(cfg, 9, stored(dtype))
    toks = fc.tokens_for(cfg, 750, 5)
    ref = fc.oracle(cfg, w, toks)
    # the early tokens matter: another first token moves the last row
    other = fc.oracle(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert row_error(other[-1], ref[-1]) > 1e-4
    eng = fc.build_engine(cfg, w, dtype, max_tokens=768, block_size=16)
    steps = [([("a", p, [len(p) - 1])], []) for p, _ in cut(toks[:600], [97])]
    steps += [([("a", [t], [0])], []) for t in toks[600:]]
    out = run(eng, steps)
    assert eng.stats["graph_replays"] >= 140
    compare(out, {"a": ref}, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["time_mix", "time_mix_one_head", "mamba", "mamba_wide_state", "loop1_tail"])
def test_long_portions_cut_along_time(name, dtype):
    """Portions of 256 tokens and more are cut into segments that the recurrent kernels work through
    side by side (local end states, a combine step, then the outputs).  Requests of 700 and 300 tokens
    in one step beside one of 5; then the rest of the first in a portion of 257 beside single tokens
    of the others; then single tokens: every row and the states left behind are the plain ones."""
    from rllm_b200.csrc import ops
    cfg = CASES[name]
    w = fc.make_weights(cfg, 14, stored(dtype))
    toks = {"a": fc.tokens_for(cfg, 970, 50), "b": fc.tokens_for(cfg, 310, 51), "c": fc.tokens_for(cfg, 15, 52)}
    refs = {r: fc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = fc.build_engine(cfg, w, dtype, max_tokens=1400, block_size=16, max_requests=3)
    made = []
    real = ops.TimeSegments.__init__
    ops.TimeSegments.__init__ = lambda self, *a, **k: made.append(1) or real(self, *a, **k)
    try:
        sample = lambda lo, hi: sorted(set(range(lo, hi, 37)) | {hi - 1, lo})
        steps = [([("a", toks["a"][:700], sample(0, 700)), ("b", toks["b"][:300], sample(0, 300)),
                   ("c", toks["c"][:5], [0, 4])], []),
                 ([("a", toks["a"][700:957], sample(0, 257)), ("b", [toks["b"][300]], [0]), ("c", [toks["c"][5]], [0])], [])]
        for i in range(9):
            steps.append(([("a", [toks["a"][957 + i]], [0]), ("b", [toks["b"][301 + i]], [0]),
                           ("c", [toks["c"][6 + i]], [0])], []))
        out = run(eng, steps)
    finally:
        ops.TimeSegments.__init__ = real
    assert len(made) == 2, "the two steps with long portions were not cut"
    compare(out, refs, dtype, f"{name}, long portions")


BIG = {
    # sizes that take the kernels' other instantiations: time-mixing heads of 96, 128 and 200 (tiles of 128 and
    # 256, more shared memory than the default), 70 and 200 states per channel, attention heads of 192 / 320
    "heads_96_128": fc.config([fc.parallel(fc.att(2, 1, 192, 320, 30, 2), 1, 128, 8, ff=64),
                               fc.parallel(fc.att(2, 2, 8, 16, 5, 1), 2, 96, 8)], width=64, vocab=67, mult=0.7),
    "head_200_states_70_200": fc.config([fc.parallel(fc.att(1, 1, 16, 16, 9, 0), 1, 200, 4, ls=0.3, rs=1.0),
                                         fc.mamba(40, 70, 3, 2), fc.mamba(24, 200, 2, 3, ff=32)], width=32, vocab=53,
                                        mult=0.8),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(BIG))
def test_large_heads_and_states(name, dtype):
    cfg = BIG[name]
    w = fc.make_weights(cfg, 15, stored(dtype))
    toks = fc.tokens_for(cfg, 300, 60)
    ref = {"a": fc.oracle(cfg, w, toks)}
    eng = fc.build_engine(cfg, w, dtype, max_tokens=320, block_size=16)
    steps = [([("a", toks[:270], list(range(0, 270, 9)) + [269])], []), ([("a", toks[270:290], list(range(20)))], [])]
    steps += [([("a", [t], [0])], []) for t in toks[290:]]
    compare(run(eng, steps), ref, dtype, name)


REAL = fc.config([fc.mamba(2048, 16, 64, 4), fc.parallel(fc.att(8, 2, 128, 128, 96, 4), 16, 64, 64, ls=0.7, rs=0.8, ff=3072),
                  fc.parallel(fc.att(8, 4, 64, 96, 80, 0), 8, 128, 32, ls=0.9, rs=0.6, ff=2048)],
                 width=1024, vocab=1531, loop=(0, 2, 2), mult=0.5)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_a_real_model(dtype):
    """Width 1,024, layers of real sizes (Mamba of 2,048 channels; attention heads of 128 with a window
    and kept keys beside 16 time-mixing heads of 64; heads of 64 / 96 beside time-mixing heads of 128), the
    first two layers run twice: the products then take the library, the tcgen05 and the weight-streaming
    kernels, the attention the mma kernels with kept keys, the recurrences their cut along time.  A
    prompt of 300 tokens, a portion of 40 beside another request's 20, then single tokens of both."""
    cfg = REAL
    w = fc.make_weights(cfg, 16, stored(dtype))
    toks = {"a": fc.tokens_for(cfg, 352, 70), "b": fc.tokens_for(cfg, 32, 71)}
    refs = {r: fc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = fc.build_engine(cfg, w, dtype, max_tokens=512, block_size=32, max_requests=2)
    steps = [([("a", toks["a"][:300], list(range(0, 300, 23)) + [299])], []),
             ([("a", toks["a"][300:340], list(range(40))), ("b", toks["b"][:20], [0, 19])], [])]
    steps += [([("a", [toks["a"][340 + i]], [0]), ("b", [toks["b"][20 + i]], [0])], []) for i in range(12)]
    compare(run(eng, steps), refs, dtype, "real layer sizes")


def test_graph_replay_equals_eager_steps():
    """Decode steps replayed from CUDA graphs (padded to four requests and a context bucket, the
    padding rows on the spare state slot) give what the same steps give launched one by one."""
    cfg = CASES["loop3_from_0"]
    w = fc.make_weights(cfg, 10)
    reqs = {r: fc.tokens_for(cfg, n, 30 + i) for i, (r, n) in enumerate({"a": 19, "b": 33, "c": 5}.items())}
    outs = []
    for graphs in (True, False):
        eng = fc.build_engine(cfg, w, "float32", max_tokens=256, use_graphs=graphs)
        steps = [([(r, t[:4], [3]) for r, t in reqs.items()], [])]
        for i in range(4, 19):
            steps.append(([(r, [t[min(i, len(t) - 1)]], [0]) for r, t in reqs.items()], []))
        outs.append(run(eng, steps))
        if graphs:
            assert eng.stats["graph_replays"] > 8
    for key, row in outs[0].items():
        assert row_error(row, outs[1][key]) < 1e-6, key


# ---------------------------------------------------------------- the entry point a user calls

def test_greedy_generation_through_the_scheduler(tmp_path):
    """LLM.generate (scheduler, continuous batching, prompts cut into portions of 16, device sampler)
    on a folder written in the stored format: the greedy continuation of each prompt is the plain
    implementation's."""
    from rllm_b200.llm import LLM
    from rllm_b200.weights.safetensors_io import write_safetensors
    cfg = CASES["loop3_from_0"]
    w = fc.make_weights(cfg, 11)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", w)
    prompts = [fc.tokens_for(cfg, n, 40 + i) for i, n in enumerate((37, 3, 21, 50, 9))]
    # bfloat16: the same path with the storage type a served model has; rounding may pick another token
    # where two logits are close, so only the shape of the answer is checked
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
            logits = fc.oracle(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-4:       # a tie at float32 precision decides nothing
                break
            assert int(logits.argmax()) == tok
            seq.append(tok)
    assert all(len(g) == 12 for g in got)
    assert not llm.engine.cache.requests


def test_trace_replay_program_chooses_the_model_by_its_config(tmp_path):
    """bin/trace_run on a Falalix folder: steps from standard input, rows out as little-endian float32."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from rllm_b200.weights.safetensors_io import write_safetensors
    cfg = CASES["no_loop"]
    w = fc.make_weights(cfg, 12, torch.bfloat16)
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(cfg))
    write_safetensors(model / "model.safetensors", w)
    toks = fc.tokens_for(cfg, 30, 6)
    lines = [json.dumps({"step": 0, "entries": [{"id": "x", "tokens": toks[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "x", "tokens": toks[20:], "want": []}], "end": ["x"]})]
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "64"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    rows = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    ref = fc.oracle(cfg, w, toks)
    assert row_error(rows[0], ref[0]) < TOL["float32"] and row_error(rows[1], ref[19]) < TOL["float32"]
    assert not (tmp_path / "out" / "1.f32").exists()
