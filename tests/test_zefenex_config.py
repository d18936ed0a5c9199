"""Zefenex without a GPU: configuration, registry, tensor names, cache specs, which call fills
and which reads a cache slot, and the oracle on cases worked out by hand."""

import copy
import math

import pytest
import torch

import plain_zefenex as PZ
import tiny_zefenex as Z
from mini_llm_stack_b200.cache.manager import CacheManager
from mini_llm_stack_b200.config import build_model, config_from_dict, config_from_folder
from mini_llm_stack_b200.config.model_config import ConfigError
from mini_llm_stack_b200.parts.base import PagedKV
from mini_llm_stack_b200.weights import write_random_model


def test_config_round_trip_and_kept_windows():
    cfg = config_from_dict(Z.Z_MIXED)
    assert cfg.architecture == "Zefenex" and cfg.vocab_size == 97 and cfg.width == 40
    assert cfg.embedding_scale == 3.0 and cfg.logit_softcap == 6.0 and cfg.norm_eps == 1e-5
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.cache_readers(0) == [0, 1] and cfg.cache_readers(2) == [2, 3]
    # the cache keeps what its widest reader sees; a reader without a window keeps all
    assert cfg.kept_window(0) == 33 and cfg.kept_window(2) is None
    plain = config_from_dict(Z.Z_PLAIN)
    assert plain.embedding_scale == 1.0 and plain.logit_softcap == 0.0
    assert plain.kept_window(0) is None and plain.kept_window(1) is None
    wide = config_from_dict(Z.Z_WIDE)
    assert wide.kept_window(0) == 100 and wide.kept_window(2) == 16


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "does not know"),
    (lambda r: r["layers"][0]["mixer"].pop("vdim"), "lacks"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "rotated"),
    (lambda r: r["layers"][1]["mixer"].update(kv_from=1), "earlier"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=1), "no cache of its own"),
    (lambda r: r["layers"][1]["mixer"].update(kv_rank=24), "differs"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(base=9.0), "differs"),
    (lambda r: r["layers"][1].update(type="mamba"), "not known"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "not known"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=8), "exceeds"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(bias=True), "does not know"),
    (lambda r: r.update(rope=1), "does not know"),
    (lambda r: r.pop("norm"), "required"),
])
def test_config_refuses_what_it_does_not_know(change, word):
    raw = copy.deepcopy(Z.Z_MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_tensor_names_shapes_and_cache_specs():
    cfg = config_from_dict(Z.Z_MIXED)
    model = build_model(cfg)
    specs = model.tensor_specs()
    assert specs["embed"].shape == (97, 40) and specs["head"].shape == (97, 40)
    assert specs["final.norm"].shape == (40,) and specs["final.norm.alpha"].shape == ()
    assert specs["l0.mix.q"].shape == (3 * 20, 40) and specs["l0.mix.dkv"].shape == (28, 40)
    assert specs["l0.mix.dkv.norm"].shape == (20,) and specs["l0.mix.uk"].shape == (36, 20)
    assert specs["l0.mix.uv"].shape == (30, 20) and specs["l0.mix.sink"].shape == (3,)
    assert specs["l0.mix.g"].shape == (30, 40) and specs["l0.mix.o"].shape == (40, 30)
    assert specs["l0.mlp.up.b"].shape == (72,) and specs["l0.mlp.down.b"].shape == (40,)
    assert specs["l0.ls1"].shape == (40,) and specs["l0.norm2b.b"].shape == (40,)
    # a layer that reads another layer's cache has no down projection
    assert "l1.mix.dkv" not in specs and "l1.mix.dkv.norm" not in specs
    assert specs["l1.mix.uk"].shape == (12, 20) and specs["l1.mix.q"].shape == (2 * 14, 40)
    assert specs["l1.mlp.router"].shape == (7, 40) and specs["l1.mlp.correction"].shape == (7,)
    assert specs["l1.mlp.e4.gate"].shape == (24, 40) and "l1.mlp.e5.gate" not in specs
    assert specs["l1.mlp.shared.down"].shape == (40, 16)
    # no feed-forward: neither its norms nor its scale
    assert "l2.norm2" not in specs and "l2.ls2" not in specs and "l2.ls1" in specs
    assert "l3.mlp.shared.up" not in specs and specs["l3.mlp.router"].shape == (3, 40)
    assert model.tied_names() == {}
    cache = model.cache_specs()
    assert len(cache) == 2                                   # two layers fill a cache
    assert cache[0] == PagedKV(1, 32, 33, shared_kv=True)    # 20 + 8 -> 32, the wider window
    assert cache[1] == PagedKV(1, 16, None, shared_kv=True)
    calls = [(c.layer, c.cache_slot, c.writes) for c in model.calls]
    assert calls == [(0, 0, True), (1, 0, False), (2, 1, True), (3, 1, False)]


def test_cache_manager_keeps_one_pool_a_filling_layer():
    model = build_model(config_from_dict(Z.Z_MIXED))
    cm = CacheManager(model.cache_specs(), num_blocks=6, block_size=4, max_requests=2,
                      max_seq_len=64, device="cpu")
    handles = cm.handles()
    assert len(handles) == 2 and all(h.kind == "paged" for h in handles)
    assert handles[0].k_pool.shape == (1, 6, 4, 32) and handles[0].window == 33
    assert handles[1].k_pool.shape == (1, 6, 4, 16) and not handles[1].window
    # keys and values are the same rows
    assert handles[0].v_pool.data_ptr() == handles[0].k_pool.data_ptr()
    assert cm.admit("a") and cm.reserve("a", 9)
    cm.commit("a", 9)
    cm.free("a")
    cm.check()


def test_random_folder_round_trip(tmp_path):
    cfg = config_from_dict(dict(Z.Z_PLAIN, dtype="float32"))
    write_random_model(tmp_path / "m", cfg, 3)
    assert config_from_folder(tmp_path / "m") == cfg


def test_plain_mechanisms_on_hand_made_cases():
    """The oracle itself, on cases small enough to work out by hand."""
    f64 = torch.float64
    # a quarter turn at position 1 with base 1 (every frequency 1 would need pi/2: use
    # position pi/2 instead); entry i pairs with entry i + dims/2, the rest stay
    x = torch.tensor([[1.0, 5.0, 0.0, 0.0, 7.0]], dtype=f64)
    y = PZ.plain_rotate_half(x, [math.pi / 2], 4, 1.0)
    assert torch.allclose(y, torch.tensor([[0.0, 0.0, 1.0, 5.0, 7.0]], dtype=f64), atol=1e-12)
    assert torch.equal(PZ.plain_rotate_half(x, [3], 0, 10.0), x)
    # the sink: one visible key with score 0 and a sink of 0 halve the weight
    s = torch.zeros(1, 2, 2, dtype=f64)
    hidden = torch.tensor([[False, True], [False, False]])
    a = PZ.plain_sink_softmax(s, hidden, torch.zeros(1, dtype=f64))
    assert torch.allclose(a[0], torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=f64))
    far = PZ.plain_sink_softmax(s, hidden, torch.full((1,), -1e9, dtype=f64))
    assert torch.allclose(far[0], torch.tensor([[1.0, 0.0], [0.5, 0.5]], dtype=f64))
    # the norm without statistics
    w = {"n": torch.tensor([2.0, 3.0], dtype=f64), "n.b": torch.tensor([1.0, -1.0], dtype=f64),
         "n.alpha": torch.tensor(0.5, dtype=f64)}
    got = PZ.plain_tanh_norm(torch.tensor([[2.0, -2.0]], dtype=f64), w, "n")
    t1 = math.tanh(1.0)
    assert torch.allclose(got, torch.tensor([[2 * t1 + 1, -3 * t1 - 1]], dtype=f64))
    # routing: the correction moves the choice, not the weights; ties go to the lower index
    h = torch.eye(3, dtype=f64)
    wr = {"m.router": torch.tensor([[0.0, 0.0, 2.0], [0.0, 0.0, 1.0], [0.0, 0.0, 0.0]], dtype=f64),
          "m.correction": torch.tensor([0.0, 0.0, 0.5], dtype=f64)}
    idx, val = PZ.plain_route(h, wr, "m", {"top": 2, "experts": 3})
    assert idx[0].tolist() == [2, 0]                        # equal scores: 1/3 + 0.5 first, then 0
    sm = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=f64), 0)
    assert idx[2].tolist() == [0, 2] and torch.allclose(val[2], sm[[0, 2]] / (sm[0] + sm[2]))
    assert torch.allclose(val[0], torch.tensor([0.5, 0.5], dtype=f64))


def test_plain_model_identity_experts_and_shared_cache():
    """An expert that returns its input, and a layer that reads another layer's cache, in the
    oracle: with a router that always takes the identity output the routed part is h itself;
    the reading layer's keys come from the filling layer's latent."""
    f64 = torch.float64
    g = torch.Generator().manual_seed(1)
    h = torch.randn(4, 6, generator=g, dtype=f64)
    w = {"m.router": torch.zeros(2, 6, dtype=f64), "m.correction": torch.tensor([0.0, 1.0], dtype=f64),
         "m.e0.gate": torch.randn(3, 6, generator=g, dtype=f64),
         "m.e0.up": torch.randn(3, 6, generator=g, dtype=f64),
         "m.e0.down": torch.randn(6, 3, generator=g, dtype=f64)}
    mlp = {"kind": "moe", "expert": {"ff": 3}, "router": {"experts": 1, "top": 1, "identity": 1}}
    assert torch.allclose(PZ.plain_routed_experts(h, w, "m", mlp), h)
    w["m.correction"] = torch.tensor([1.0, 0.0], dtype=f64)
    assert torch.allclose(PZ.plain_routed_experts(h, w, "m", mlp), PZ.plain_silu_unit(h, w, "m.e0"))
