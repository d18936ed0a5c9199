"""Movazen without a GPU: configuration, tensor names, cache specs and the cache manager's
kept first pages, and the plain implementation's mechanisms on hand-made cases."""

import copy
import math

import numpy as np
import pytest

import plain_movazen as PM
import tiny_movazen as M
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.config.model_config import ConfigError
from mini_llm_stack_b200.config.registry import build_model
from mini_llm_stack_b200.parts.base import FixedState, PagedKV, PagedWithState


@pytest.mark.parametrize("raw", [M.M_MIXED, M.M_PLAIN, M.M_WIDE])
def test_config_round_trip(raw):
    cfg = config_from_dict(raw)
    assert cfg.architecture == "Movazen"
    again = config_from_dict(cfg.to_dict())
    assert again == cfg
    assert cfg.side_dim == (raw.get("token_side") or {}).get("dim", 0)


def _broken(path, value):
    raw = copy.deepcopy(M.M_MIXED)
    node = raw
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 0, "mixer", "rot"), {"base": 1.0}, "does not know"),
    (("layers", 1, "mixer", "right", "decay"), [0.5], "one number a head"),
    (("layers", 1, "mixer", "left", "q_temp", "every"), 0, "every"),
    (("layers", 1, "mixer", "left_scale"), KeyError, "lacks"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "equal groups"),
    (("layers", 0, "mlp", "router", "top"), 5, "exceeds"),
    (("layers", 0, "mlp", "kind"), "dense", "moe"),
    (("layers", 0, "mlp", "expert", "limit"), KeyError, "lacks"),
    (("token_side", "dim"), 0, "token_side.dim"),
    (("norm",), {"eps": 1e-5, "kind": "layer"}, "does not know"),
])
def test_config_refusals_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as err:
        config_from_dict(_broken(path, value))
    assert word in str(err.value)


def test_tensor_names_and_shapes():
    model = build_model(config_from_dict(M.M_MIXED))
    specs = {n: tuple(s.shape) for n, s in model.tensor_specs().items()}
    assert specs["embed"] == (97, 40) and specs["head"] == (97, 40)
    assert specs["side.embed"] == (97, 4 * 6)
    assert specs["l0.mix.q"] == (4 * 12, 40) and specs["l0.mix.k"] == (2 * 12, 40)
    assert specs["l0.mix.v"] == (2 * 20, 40) and specs["l0.mix.g"] == (4 * 20, 40)
    assert specs["l0.mix.o"] == (40, 4 * 20)
    assert specs["l0.mix.q.norm"] == (12,) and specs["l0.mix.k.norm"] == (12,)
    assert specs["l1.mix.left.q.b"] == (2 * 16,) and specs["l1.mix.left.v.b"] == (8,)
    assert specs["l1.mix.left.o"] == (40, 2 * 8)
    assert specs["l1.mix.right.q"] == (3 * 8, 40) and specs["l1.mix.right.v"] == (3 * 12, 40)
    assert specs["l1.mix.right.norm"] == (36,) and specs["l1.mix.right.o"] == (40, 36)
    assert "l1.norm2" not in specs and "l1.mlp.router" not in specs
    assert specs["l0.mlp.router"] == (6, 40) and specs["l0.mlp.correction"] == (6,)
    assert specs["l0.mlp.e5.gate"] == (24, 40) and specs["l0.mlp.e5.down"] == (40, 24)
    assert specs["l0.mlp.shared.sg"] == (1, 40) and specs["l0.mlp.shared.up"] == (16, 40)
    assert "l2.mlp.shared.sg" not in specs
    assert specs["l3.side.gate"] == (6, 40) and specs["l3.side.proj"] == (40, 6)
    assert specs["l3.side.norm"] == (40,)
    plain = build_model(config_from_dict(M.M_PLAIN)).tensor_specs()
    assert not any(n.startswith("side") or ".side." in n for n in plain)


def test_cache_specs():
    specs = build_model(config_from_dict(M.M_MIXED)).cache_specs()
    assert specs[0] == PagedKV(2, 32, 21, keep_first=3)          # heads of 12 / 20 padded to 32
    assert specs[2] == PagedKV(3, 16, 40, keep_first=17)
    assert specs[1] == PagedWithState(PagedKV(1, 16, None), FixedState((3 * 8 * 12,)))
    assert specs[3] == PagedWithState(PagedKV(4, 32, None), FixedState((1 * 20 * 4,)))


def test_cache_manager_keeps_the_first_pages():
    spec = PagedKV(1, 16, window=10, keep_first=5)
    cm = CacheManager([spec, PagedKV(1, 16, window=10)], num_blocks=12, block_size=4,
                      max_requests=2, max_seq_len=64, allocate=False)
    cm.admit("a")
    assert cm.reserve("a", 30)
    cm.commit("a", 30)
    kept, plain = cm.pages_of("a", 0), cm.pages_of("a", 1)
    # keys before 30 - 10 + 1 = 21 are dead: pages 0..4; the first two pages hold kept tokens
    assert [p >= 0 for p in kept] == [True, True, False, False, False, True, True, True]
    assert [p >= 0 for p in plain] == [False] * 5 + [True] * 3
    cm.check()
    assert cm.reserve("a", 9)
    cm.commit("a", 9)
    assert [p >= 0 for p in cm.pages_of("a", 0)][:8] == [True, True] + [False] * 5 + [True]
    cm.check()
    free_before = cm.paged[0].pool.num_free
    cm.free("a")
    cm.check()
    assert cm.paged[0].pool.num_free == 12 and free_before < 12
    # the pages come back for the next request
    cm.admit("b")
    assert cm.reserve("b", 48)
    cm.commit("b", 48)
    cm.check()


# ------------------------------------------------------------- the plain mechanisms
def test_visibility():
    assert PM.visible(10, 10, 4, 2) and PM.visible(10, 7, 4, 2) and not PM.visible(10, 6, 4, 2)
    assert PM.visible(10, 1, 4, 2) and not PM.visible(10, 2, 4, 2)
    assert not PM.visible(3, 4, None, 0) and PM.visible(3, 0, None, 0)


def test_sink_and_slopes():
    q = np.ones((1, 1, 2)); k = np.zeros((1, 1, 2)); v = np.full((1, 1, 3), 6.0)
    assert np.allclose(PM.softmax_attention(q, k, v, 1.0, sink=True), 3.0)    # e^0 / (1 + e^0)
    assert np.allclose(PM.softmax_attention(q, k, v, 1.0), 6.0)
    assert PM.distance_slopes(8)[0] == 0.5 and PM.distance_slopes(8)[7] == 2.0 ** -8
    # two keys with equal scores: the nearer one gets e^slope times the weight of the other
    q = np.ones((2, 1, 1)); k = np.ones((2, 1, 1)); v = np.array([[[1.0]], [[0.0]]])
    out = PM.softmax_attention(q, k, v, 1.0, slopes=[math.log(3.0)])
    assert np.allclose(out[1, 0, 0], 0.25)


def test_query_temperature_steps():
    assert PM.query_temperature(0, 0.5, 4) == 1.0 and PM.query_temperature(2, 0.5, 4) == 1.0
    assert PM.query_temperature(3, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(2))
    assert PM.query_temperature(11, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(4))


def test_sinusoid():
    v = PM.sinusoid(3, 6)
    assert v[0] == pytest.approx(math.sin(3.0)) and v[1] == pytest.approx(math.cos(3.0))
    assert v[4] == pytest.approx(math.sin(3.0 * 10000 ** (-4 / 6)))


def test_grouped_choice():
    # group 1 holds the single best score, but group 0's two best sum higher
    c = [0.6, 0.5, 0.1, 0.9, 0.1, 0.0]
    assert PM.choose_experts(c, 2) == [3, 0]
    assert PM.choose_experts(c, 2, {"count": 2, "keep": 1}) == [0, 1]
    assert PM.choose_experts(c, 3, {"count": 3, "keep": 2}) == [3, 0, 1]
    # negative choice scores still beat experts outside the kept groups
    assert PM.choose_experts([-0.5, -0.6, -0.9, -0.9], 2, {"count": 2, "keep": 1}) == [0, 1]
    assert PM.choose_experts([0.3, 0.3, 0.3], 2) == [0, 1]


@pytest.mark.parametrize("change", ["window+1", "window-1", "keep+1", "keep-1", "no slopes",
                                    "no sink", "no groups", "no temperature", "no side"])
def test_the_oracle_feels_every_mechanism(tmp_path, change, monkeypatch):
    """What the GPU tests compare against moves, by far more than they tolerate, when a window
    is one token off, a kept token is lost or gained, or a mechanism is left out."""
    def sharp(w):
        for n in w:
            if n.endswith("mix.q.norm") or n.endswith("left.q") or n.endswith("left.q.b"):
                w[n] *= 6.0
    cfg, w = M.make_movazen(tmp_path / "m", M.M_MIXED, 5, "float32", patch=sharp)
    tokens = list(np.random.RandomState(1).randint(0, 97, 100))
    want = PM.forward(cfg, w, tokens)
    other = copy.deepcopy(cfg)
    if change.startswith("window"):
        other["layers"][0]["mixer"]["mask"]["size"] += 1 if change.endswith("+1") else -1
    elif change.startswith("keep"):
        other["layers"][2]["mixer"]["mask"]["keep_first"] += 1 if change.endswith("+1") else -1
    elif change == "no slopes":
        monkeypatch.setattr(PM, "distance_slopes", lambda n: [0.0] * n)
    elif change == "no sink":
        real = PM.softmax_attention
        monkeypatch.setattr(PM, "softmax_attention",
                            lambda *a, **k: real(*a, **dict(k, sink=False)))
    elif change == "no groups":
        del other["layers"][0]["mlp"]["router"]["groups"]
    elif change == "no temperature":
        del other["layers"][1]["mixer"]["left"]["q_temp"]
    elif change == "no side":
        del other["token_side"]
    got = PM.forward(other, w, tokens)
    moved = np.abs(got - want).max(axis=1) / np.abs(want).max()
    assert moved.max() > 2e-3, change
    if change == "window+1":
        assert moved[:21].max() < 1e-12          # rows inside the window see the same keys
