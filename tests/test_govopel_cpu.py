"""Govopel without a GPU: the configuration reader, the model as data, tensor names and shapes, the
cache need of attention through a latent, and the plain implementation's own pieces."""
import copy
import math

import pytest
import torch

import govopel_cases as gc
import plain_govopel as pg
from govopel_cases import CASES


def test_registry_finds_the_configuration():
    from rllm_b200.config import GovopelConfig, config_from_dict, supported_architectures
    assert "Govopel" in supported_architectures()
    cfg = config_from_dict(CASES["stack"])
    assert isinstance(cfg, GovopelConfig)
    assert cfg.to_dict() == CASES["stack"]
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("name", list(CASES))
def test_tensor_names_and_shapes(name):
    from rllm_b200.config import config_from_dict
    from rllm_b200.models.model import expected_tensors
    exp = {n: tuple(s) for n, (s, _) in expected_tensors(config_from_dict(CASES[name]).model_spec()).items()}
    assert exp == {n: s for n, (s, _) in gc.tensor_shapes(CASES[name]).items()}


def test_model_as_data():
    from rllm_b200.config import config_from_dict
    spec = config_from_dict(CASES["stack"]).model_spec()
    assert [l.block for l in spec.layers] == ["post_norm"] * 4
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "chunked_attention", "chunked_attention",
                                                   "latent_attention"]
    assert spec.layers[1].mixer.params["chunk"] == 11 and spec.layers[1].mixer.params["softcap"] == 12.0
    assert spec.layers[2].mixer.params["softcap"] == 0.0 and spec.layers[2].position.params["scaling"]["factor"] == 2.0
    assert spec.layers[0].ffn.kind == "clamped_glu" and spec.layers[0].ffn.params["limit"] == 2.5
    assert spec.layers[2].ffn is None and "ffn" not in spec.layers[2].norms
    assert spec.lm_head.params["tied_to"] == "embed" and spec.lm_head.params["softcap"] == 30.0
    assert spec.embedding.params["norm"] == "embed.norm" and spec.max_position == 0


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "not supported"),
    (("layers", 1, "mixer", "kv_heads"), 4, "multiple"),
    (("layers", 1, "mixer", "vdim"), 16, "vdim"),
    (("layers", 1, "mixer", "rot", "dims"), 33, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 6, "rot_dim"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mlp", "kind"), "routed", "not supported"),
    (("layers", 0, "mlp", "limit"), -1.0, "limit"),
    (("norm", "eps"), 0.0, "eps"),
])
def test_config_errors_name_the_key(path, value, word):
    from rllm_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(CASES["stack"])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_latent_cache_need_has_no_value_pool():
    from rllm_b200.cache import CacheManager
    from rllm_b200.cache.native import NativeCacheManager
    from rllm_b200.parts import PagedKVNeed
    needs = [PagedKVNeed(1, 24, values_in_keys=20), PagedKVNeed(2, 16), PagedKVNeed(1, 24, values_in_keys=20)]
    for manager in (CacheManager, NativeCacheManager):
        m = manager(needs, [None] * 3, 8, 64, 2)
        assert len(m.paged) == 2 and m.paged[0].entries == [0, 2]
        assert m.bytes_per_token(2) == 2 * (2 * 24 + 2 * 2 * 16)
        m.allocate_device("cpu", torch.float32)
        k, v = m.paged[0].planes(1)
        assert k.shape == (8, 1, 8, 24) and v.data_ptr() == k.data_ptr() and m.paged[0].pool_v is None
        slots = m.append("a", 11)
        assert len(slots) == 2 and len(slots[0]) == 11
        m.free("a")
        m.check_invariants()


# ---------------------------------------------------------------- the plain implementation's own pieces

def test_plain_frequencies():
    f, m = pg.rotary_frequencies({"dims": 8, "base": 100.0})
    assert m == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64))
    # scaling: fast pairs keep their frequency, slow pairs are divided by the factor, cos and sin grow
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    g, m = pg.rotary_frequencies({"dims": 8, "base": 100.0, "scaling": sc})
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8)) / (2 * math.log(100))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1)) / (2 * math.log(100))), 7)
    assert (lo, hi) == (0, 3)
    assert m == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert g[0] == f[0] and g[3] == pytest.approx(float(f[3]) / 4.0)
    assert all(float(f[i]) / 4.0 < float(g[i]) < float(f[i]) for i in (1, 2))


def test_plain_rotation_keeps_lengths_and_the_tail():
    x = torch.randn(5, 2, 10, dtype=torch.float64)
    y = pg.rotate(x, [0, 1, 2, 50, 51], {"dims": 6, "base": 50.0})
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., :6].norm(dim=-1), x[..., :6].norm(dim=-1))
    assert not torch.allclose(y[3, :, :6], x[3, :, :6])


def test_plain_chunk_mask():
    vis = pg.chunk_mask(9, 4)
    assert vis[3, 0] and vis[3, 3] and not vis[4, 3] and vis[4, 4] and vis[7, 4] and not vis[8, 7] and not vis[2, 3]
    assert pg.chunk_mask(5, 0).sum() == 15 and pg.chunk_mask(5, 1).sum() == 5


def test_plain_feed_forward_clamps():
    w = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64),
         "down": torch.eye(3, dtype=torch.float64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    y = pg.dense_ff(h, {"limit": 2.0}, w)
    sig = lambda z: 1 / (1 + math.exp(-z))
    want = [2.0 * sig(1.702 * 2.0) * 3.0, -5.0 * sig(1.702 * -5.0) * (-2.0 + 1.0), 0.5 * sig(1.702 * 0.5) * 1.5]
    assert torch.allclose(y[0], torch.tensor(want, dtype=torch.float64))


def test_plain_latent_scores_ignore_distance_when_rotated_parts_are_silent():
    """The marked weights of the tests: a query of the asking token scores the target's key the same
    wherever the two stand."""
    cfg = gc.config([gc.lat(2, 8, 4, 6, 12, 12, scale=2.0)], width=24, vocab=31)
    w = gc.marked_latent(cfg, gc.make_weights(cfg, 1), asker=3, target=4)
    toks = [4, 7, 9, 3, 11, 12, 13, 3]
    rows = gc.oracle(cfg, w, toks)
    other = gc.oracle(cfg, w, [5] + toks[1:])
    assert gc.row_error(rows[3], other[3]) > 0.05 and gc.row_error(rows[7], other[7]) > 0.05
    assert gc.row_error(rows[2], other[2]) < gc.row_error(rows[3], other[3])
