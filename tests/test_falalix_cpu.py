"""Falalix without a GPU: the configuration and what it makes of a model, tensor names and shapes,
the cache manager with a mixer that needs several things, kept first keys when pages go back,
and the plain implementation's own pieces."""
import copy

import pytest
import torch

import falalix_cases as fc
import plain_falalix as pf
from rllm_b200.cache import CacheManager
from rllm_b200.cache.native import NativeCacheManager
from rllm_b200.config import ConfigError, FalalixConfig, config_from_dict
from rllm_b200.models.model import expected_tensors
from rllm_b200.parts import PagedKVNeed, StateNeed
from rllm_b200.weights.loader import shape_fits


def test_registry_reads_a_single_architecture_name():
    cfg = config_from_dict(fc.CASES["no_loop"])
    assert isinstance(cfg, FalalixConfig)
    assert config_from_dict(cfg.to_dict()) == cfg
    with pytest.raises(ConfigError, match="architecture"):
        config_from_dict({"vocab": 3})


@pytest.mark.parametrize("name", list(fc.CASES))
def test_tensor_names_and_shapes(name):
    """What the model asks of a weight file is what the layers' descriptions say, tensor by tensor."""
    cfg = fc.CASES[name]
    want = {n: s for n, (s, _) in fc.tensor_shapes(cfg).items()}
    got = {n: tuple(s) for n, (s, _) in expected_tensors(config_from_dict(cfg).model_spec()).items()}
    assert got == want


def test_decay_bottleneck_may_come_from_the_file():
    cfg = copy.deepcopy(fc.CASES["time_mix"])
    del cfg["layers"][0]["mixer"]["right"]["decay_rank"]
    got = expected_tensors(config_from_dict(cfg).model_spec())
    assert got["l0.mix.right.w1"][0] == (None, 36) and got["l0.mix.right.w2"][0] == (48, None)
    assert shape_fits((5, 36), (None, 36)) and not shape_fits((5, 35), (None, 36)) and not shape_fits((5,), (None, 36))


def test_run_order_of_loops():
    order = lambda name: [(e.layer, e.junction, e.junction_arg, e.cache_of)
                          for e in config_from_dict(fc.CASES[name]).model_spec().run_order]
    assert order("no_loop") == [(0, None, 0, None), (1, None, 0, None)]
    assert order("loop1_tail") == [(0, None, 0, None), (1, 0, 0, None), (2, None, 0, None)]
    assert order("loop3_from_0") == [(0, 0, 0, None), (1, None, 0, None), (0, 0, 1, None), (1, None, 1, None),
                                     (0, 0, 2, None), (1, None, 2, None), (2, None, 0, None), (3, None, 0, None)]
    assert [i for i, _ in pf.run_order(fc.CASES["loop3_from_0"])] == [0, 1, 0, 1, 0, 1, 2, 3]
    spec = config_from_dict(fc.CASES["loop3_from_0"]).model_spec()
    assert len(spec.junctions) == 1 and spec.residual_scale == 0.7 and spec.max_position == 0
    assert config_from_dict(fc.CASES["no_loop"]).model_spec().junctions == ()


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv2"), "conv2"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3, kv_heads=2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][1]["mixer"].update(state=0), "state"),
    (lambda c: c.update(loop={"start": 1, "stop": 5, "times": 2}), "loop"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "routed"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_name_the_key(edit, word):
    cfg = copy.deepcopy(fc.CASES["no_loop"])
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


@pytest.mark.parametrize("manager", [CacheManager, NativeCacheManager])
def test_a_mixer_with_several_needs_and_kept_first_keys(manager):
    """Run entries whose mixer is two mixers: a windowed attention that keeps 10 first keys (value
    heads of their own size) beside a state; a Mamba state between them.  Equal needs share a group
    whichever entry they come from; pages between the kept keys and the window go back, the kept
    pages never."""
    att = PagedKVNeed(2, 16, window=40, keep_first=10, v_head_dim=24)
    rw, mb = StateNeed((100,)), StateNeed((60,))
    cm = manager([mb, (att, rw), (att, rw), mb], [None] * 4, block_size=8, max_tokens=512, max_requests=2)
    assert len(cm.paged) == 1 and len(cm.stateful) == 2
    assert cm.entry_place == [("state", 0, 0), (("kv", 0, 0), ("state", 1, 0)), (("kv", 0, 1), ("state", 1, 1)),
                              ("state", 0, 1)]
    cm.allocate_device("cpu", torch.float32)
    k, v = cm.paged[0].planes(1)
    assert k.shape == (64, 2, 8, 16) and v.shape == (64, 2, 8, 24)
    assert cm.stateful[1].state.shape == (2, 3, 100)
    assert cm.bytes_per_token(2) == 2 * 2 * (16 + 24) * 2
    cm.append("r", 166)
    assert cm.release_passed("r") == 0                       # the next query still reads key 127
    cm.append("r", 1)
    assert cm.release_passed("r") == 14                      # keys 16..127; the two pages of the kept keys stay
    table = cm.block_table("r", 0, raw=True) if manager is NativeCacheManager else cm.requests["r"].tables[0]
    assert [b is None for b in table[:17]] == [False, False] + [True] * 14 + [False]
    cm.check_invariants()
    cm.free("r")
    assert cm.n_free_pages(0) == 64
    cm.check_invariants()
    with pytest.raises(ValueError):
        manager([(att, rw), (att, mb)], [None, 0], 8, 64, 2)   # reading a cache of another kind


def test_smaller_pool_for_a_window_counts_the_kept_pages():
    att = PagedKVNeed(1, 8, window=32, keep_first=20)
    cm = CacheManager([att], [None], block_size=8, max_tokens=4096, max_requests=2, max_step_tokens=16)
    assert cm.paged[0].n_blocks == 2 * (-(-(32 + 16 + 128) // 8) + 1 + 3)


# ---------------------------------------------------------------- the plain implementation's own pieces

def test_plain_mask():
    see = pf.visible(8, 3, 2)
    assert see[7].tolist() == [True, True, False, False, False, True, True, True]
    assert see[2].tolist() == [True, True, True, False, False, False, False, False]
    assert pf.visible(5, 9, 0).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()


def test_plain_recurrences_do_not_depend_on_later_tokens():
    """Causality of the plain implementation itself: a row depends on the tokens up to it."""
    for name in ("mamba", "time_mix", "loop3_from_0"):
        cfg = fc.CASES[name]
        w = fc.make_weights(cfg, 1)
        toks = fc.tokens_for(cfg, 20, 0)
        a = pf.forward(cfg, w, toks)
        b = pf.forward(cfg, w, toks[:11] + [(t + 1) % cfg["vocab"] for t in toks[11:]])
        assert torch.equal(a[:11], b[:11]) and not torch.allclose(a[11:], b[11:])
        # and on all of them: the first token still moves the last row
        c = pf.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
        assert not torch.allclose(a[-1], c[-1], rtol=0, atol=1e-9)


def test_random_weights_mode_makes_a_falalix_folder(tmp_path):
    from rllm_b200.weights import write_random_model
    from rllm_b200.weights.loader import load_checked
    cfg = config_from_dict(fc.CASES["loop1_tail"])
    write_random_model(cfg, tmp_path, seed=3)
    exp = {n: s for n, (s, _) in expected_tensors(cfg.model_spec()).items()}
    got = load_checked(tmp_path, exp)
    assert set(got) == set(exp)
    mu = got["l1.mix.right.mu.k"].float()
    assert 0 < float(mu.min()) and float(mu.max()) < 1
