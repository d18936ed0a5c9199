"""Zefenex on the GPU against the plain implementation of ``plain_zefenex``.

Kernels alone (through ``Ops``), every mechanism as a one-layer model, then whole models:
prompts whole, decoded token by token, in portions down to two tokens, unequal requests in
one batch, pages used again, long decoding through CUDA graphs, greedy generation through
``LLM.generate`` and the trace program.  Where random weights would hide a fault the weights
are made to show it: the query projection is scaled up until every softmax is nearly one key
(any key the engine loses, far away, at a page's edge or at the window's, then changes the
logits); a window one token too long or too short, a sink left out or scaled like a score
and a router without its correction are shown to move the oracle far more than the engine
is allowed to differ.
"""

import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_zefenex as PZ
import tiny_zefenex as Z
from engine_helpers import Replayer, tokens_for

pytestmark = pytest.mark.gpu

# largest |engine - plain| as a fraction of the largest |logit|: float32 differs from the
# float64 oracle by the order of its sums; bfloat16 by the rounding of products and activations
TOL = {"float32": 5e-5, "bfloat16": 3e-2}
# A sharp softmax turns a small change into another key, so a row may also be off by NOISE
# times what rounding does to that row of the oracle itself (the oracle run again with its
# activations rounded to the engine's format, against its exact run in float64).
NOISE = 6.0
# A router whose last chosen output leads the next one by less than this is a close call:
# rounding decides it, so the oracle is also run with every close call taken the other way,
# and what that changes (in the row itself and in the later rows that see it) is slack too.
CLOSE_CALL = {"float32": 1e-6, "bfloat16": 2e-2}


def close(got, want, tol, what, slack=None):
    scale = want.abs().max().item()
    err = (got.double() - want.double()).abs().max(dim=1).values
    bound = tol * scale if slack is None else tol * scale + NOISE * slack
    bad = int((err > bound).sum())
    assert bad == 0, (
        f"{what}: {bad} rows of {len(err)} differ by more than {tol:.0e} * {scale:.3f} "
        f"(worst {err.max().item():.3e}); first wrong row {int((err > bound).nonzero()[0])}")


def sharp(factor):
    """Scale the query projections so that softmax picks nearly one key."""
    def patch(w):
        for n in w:
            if n.endswith(".mix.q"):
                w[n] *= factor
    return patch


def oracle(w, raw, tokens, **kw):
    return PZ.plain_zefenex(w, raw, tokens, **kw)


def check(got, w, raw, tokens, dtype, what):
    """The engine's rows against the oracle's, every row with its own slack."""
    want = oracle(w, raw, tokens)
    g = torch.Generator().manual_seed(0)
    if dtype == "float32":
        def rounded_to(t):
            return t.float().to(t.dtype)
        step = 2.0 ** -23
    else:
        rounded_to, step = PZ.to_bf16, 2.0 ** -8

    def nudged(t):
        return rounded_to(t * (1 + (torch.rand(t.shape, generator=g, dtype=t.dtype) - 0.5) * step))

    slack = torch.zeros(len(tokens), dtype=want.dtype)
    for rnd, flip in ((rounded_to, 0.0), (nudged, 0.0), (nudged, 0.0), (PZ.ident, CLOSE_CALL[dtype]),
                      (rounded_to, CLOSE_CALL[dtype] / 2)):
        rounded = oracle(w, raw, tokens, rnd=rnd, flip_below=flip)
        slack = torch.maximum(slack, (rounded - want).abs().max(dim=1).values)
    close(got, want, TOL[dtype], what, slack=slack)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zefenex")
    out = {}
    for key, raw, patch in (("mixed", Z.Z_MIXED, None), ("plain", Z.Z_PLAIN, None),
                            ("wide", Z.Z_WIDE, None), ("sharp", Z.Z_WIDE, sharp(6.0)),
                            ("sharp_mixed", Z.Z_MIXED, sharp(5.0))):
        for dtype in ("float32", "bfloat16"):
            folder = tmp / f"{key}_{dtype}"
            out[(key, dtype)] = (folder, raw, Z.make_zefenex(folder, raw, 11, dtype, patch=patch))
    return out


# ------------------------------------------------------------------ kernels alone
@pytest.fixture(scope="module")
def rt32():
    from mini_llm_stack_b200.ops.kernels import Runtime
    return Runtime("cuda:0", torch.float32)


def plain_dyt(v, alpha, w, b):
    return torch.tanh(alpha * v) * w + b


@pytest.mark.parametrize("d", [36, 40, 200])
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_tanh_norm_kernel_in_every_role(rt32, d, act):
    """x += scale * n_post(delta + bias); h = n(x): with and without the map behind the
    sublayer, the bias and the scale; picked rows leave the stream alone; the map alone."""
    g = torch.Generator().manual_seed(d)
    t = 9
    ops = rt32.ops
    ops.require_part("tanhnorm")
    vec = {k: (torch.randn(d, generator=g) * 0.7).to(act) for k in ("w", "b", "pw", "pb", "s", "bias")}
    dv = {k: v.double() for k, v in vec.items()}
    cu = {k: v.cuda() for k, v in vec.items()}
    a, pa = 0.8, 1.3
    x0 = torch.randn(t, d, generator=g)
    delta = (torch.randn(t, d, generator=g) * 2).to(act)
    for post, bias, scale in ((True, True, True), (True, False, False), (False, False, False),
                              (True, True, False)):
        x = x0.clone().cuda()
        h = torch.empty(t, d, dtype=act, device="cuda")
        p = (pa, cu["pw"], cu["pb"], cu["s"] if scale else None) if post else None
        ops.add_tanh_norm(x, delta.cuda(), (a, cu["w"], cu["b"]), h, post=p,
                          bias=cu["bias"] if bias else None)
        y = delta.double() + (dv["bias"] if bias else 0)
        if post:
            y = plain_dyt(y, pa, dv["pw"], dv["pb"]) * (dv["s"] if scale else 1)
        want_x = x0.double() + y
        assert torch.allclose(x.cpu().double(), want_x, atol=2e-6), (post, bias, scale)
        want_h = plain_dyt(want_x, a, dv["w"], dv["b"])
        tol = 2e-6 if act == torch.float32 else 2e-2
        assert (h.cpu().double() - want_h).abs().max().item() < tol * max(1, want_h.abs().max().item())
    # picked rows: the stream stays, the rows come out as if it had been added
    x = x0.clone().cuda()
    rows = torch.tensor([7, 2, 2, 0], dtype=torch.int32, device="cuda")
    h = torch.empty(3, d, dtype=act, device="cuda")
    ops.add_tanh_norm(x, delta.cuda(), (a, cu["w"], cu["b"]), h,
                      post=(pa, cu["pw"], cu["pb"], cu["s"]), rows=rows, n_rows=3)
    assert torch.equal(x.cpu(), x0)
    y = plain_dyt(delta.double(), pa, dv["pw"], dv["pb"]) * dv["s"]
    want_h = plain_dyt(x0.double() + y, a, dv["w"], dv["b"])[[7, 2, 2]]
    assert (h.cpu().double() - want_h).abs().max().item() < (2e-6 if act == torch.float32 else 2e-2) * 3
    # the map alone
    y_out = torch.empty(t, d, device="cuda")
    ops.add_tanh_norm(None, delta.cuda(), None, None, post=(pa, cu["pw"], cu["pb"], cu["s"]),
                      bias=cu["bias"], y_out=y_out)
    want = plain_dyt(delta.double() + dv["bias"], pa, dv["pw"], dv["pb"]) * dv["s"]
    assert torch.allclose(y_out.cpu().double(), want, atol=2e-6)
    ops.check_status()


@pytest.mark.parametrize("softmax,correction,identity", [(True, True, 2), (True, False, 0),
                                                         (False, True, 0), (True, True, 0)])
def test_route_kernel_scores_choice_and_weights(rt32, softmax, correction, identity):
    """The choice uses score + correction, the weights the score alone, renormalised with the
    small constant; outputs past the real experts are chosen like any other."""
    g = torch.Generator().manual_seed(3 + identity)
    ops = rt32.ops
    ops.require_part("experts")
    t, n_real, top = 37, 6, 3
    n_out = n_real + identity
    logits = torch.randn(t, n_out, generator=g) * 2
    corr = torch.randn(n_out, generator=g) * 0.4 if correction else None
    i32 = torch.int32
    tiles = ops.expert_max_tiles(t * top, n_real)

    def dev(n, dt):
        return torch.zeros(n, dtype=dt, device="cuda")
    work = {"idx": dev(t * top, i32), "weight": dev(t * top, torch.float32),
            "order": dev(t * top, i32), "offsets": dev(n_out + 1, i32), "cursor": dev(n_out, i32),
            "tile_expert": dev(tiles, i32), "tile_row0": dev(tiles, i32), "max_tiles": tiles}
    ops.route(logits.cuda(), top, True, work, softmax=softmax,
              correction=corr.cuda() if correction else None, renorm_eps=1e-20, n_real=n_real)
    s = torch.softmax(logits.double(), -1) if softmax else torch.sigmoid(logits.double())
    choice = s + (corr.double() if correction else 0)
    idx = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    val = torch.gather(s, 1, idx)
    val = val / (val.sum(-1, keepdim=True) + 1e-20)
    got_idx = work["idx"].cpu().view(t, top).long()
    got_w = work["weight"].cpu().view(t, top).double()
    # the same set, whatever the order inside a token's choices
    assert torch.equal(got_idx.sort(-1).values, idx.sort(-1).values)
    by_expert = torch.zeros(t, n_out, dtype=torch.float64).scatter_(1, got_idx, got_w)
    assert torch.allclose(by_expert, torch.zeros(t, n_out, dtype=torch.float64).scatter_(1, idx, val),
                          atol=1e-6)
    offsets = work["offsets"].cpu().tolist()
    counts = torch.bincount(idx.flatten(), minlength=n_out).tolist()
    assert [offsets[i + 1] - offsets[i] for i in range(n_out)] == counts
    ops.check_status()


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_gate_headwise_and_biased_relu_squared_kernels(rt32, act):
    g = torch.Generator().manual_seed(5)
    ops = rt32.ops
    ops.require_part("latent")
    t, heads, k, n = 11, 3, 10, 7
    # o *= sigmoid(proj[:, col:]) with the projection in float32
    o = torch.randn(t, heads * n, generator=g).to(act)
    proj = torch.randn(t, 5 + heads * n + 3, generator=g)
    od = o.clone().cuda()
    ops.sigmoid_gate(od, proj.cuda(), 5)
    want = o.double() * torch.sigmoid(proj[:, 5:5 + heads * n].double())
    assert (od.cpu().double() - want).abs().max().item() < (1e-6 if act == torch.float32 else 2e-2)
    # dst[t, h, :n] = w[h] @ src[t, h, :k], heads further apart than they are wide
    for rows in (t, 90):
        w = (torch.randn(heads, n, k, generator=g) * 0.5).to(act)
        src = torch.randn(rows, heads * 12 + 1, generator=g).to(act)
        dst = torch.zeros(rows, heads * 9 + 2, dtype=act, device="cuda")
        ops.headwise_linear(src.cuda(), 12, w.cuda(), dst, 9, rows)
        got = dst.cpu().double()
        for h in range(heads):
            want = src[:, h * 12:h * 12 + k].double() @ w[h].double().T
            assert (got[:, h * 9:h * 9 + n] - want).abs().max().item() < \
                (1e-5 if act == torch.float32 else 5e-2), (rows, h)
            assert got[:, h * 9 + n:(h + 1) * 9].abs().max().item() == 0
    # relu(z + b)^2 from a float32 product
    z = torch.randn(6, 33, generator=g)
    b = torch.randn(33, generator=g).to(act)
    out = torch.empty(6, 33, dtype=act, device="cuda")
    ops.relu_squared(z.cuda(), out, bias=b.cuda())
    want = (z.double() + b.double()).clamp(min=0) ** 2
    assert (out.cpu().double() - want).abs().max().item() < (1e-5 if act == torch.float32 else 5e-2)
    x = (torch.randn(4, 50, generator=g) * 9).cuda()
    before = x.clone()
    ops.softcap_(x, 4.0)
    assert torch.allclose(x, 4.0 * torch.tanh(before / 4.0), atol=1e-6)
    ops.check_status()


# ------------------------------------------------------- mechanisms as one-layer models
ONE_LAYER = {
    # latent + rotated part on (32) and off (15 -> 16, 38 -> 48) the attention kernels' sizes
    "attention_window": Z.one_layer(Z.latent(3, 12, 8, 10, 24, 0.4, window=19, base=300.0)),
    "attention_no_window": Z.one_layer(Z.latent(2, 10, 6, 5, 9, 0.5, base=10000.0)),
    "attention_window_of_a_page": Z.one_layer(Z.latent(4, 8, 4, 8, 34, 0.5, window=16, base=50.0)),
    "attention_window1": Z.one_layer(Z.latent(2, 16, 2, 6, 14, 0.5, window=1, base=20.0)),
    "attention_one_head": Z.one_layer(Z.latent(1, 24, 16, 40, 16, 0.3, window=40, base=1e6),
                                      width=36),
    # 80 + 16 = 96 and 96 + 32 = 128: the tensor-core kernels in bfloat16
    "attention_pool_96": Z.one_layer(Z.latent(2, 32, 16, 24, 80, 0.15, window=33, base=1e4),
                                     width=64),
    "attention_pool_128": Z.one_layer(Z.latent(3, 64, 32, 80, 96, 0.1, window=50, base=1e6),
                                      width=96),
    "attention_pool_272": Z.one_layer(Z.latent(2, 16, 16, 8, 256, 0.2, window=25, base=100.0),
                                      width=48),
    "attention_pool_240": Z.one_layer(Z.latent(3, 24, 32, 16, 200, 0.1, window=37, base=1e4),
                                      width=56),
    # 44 heads of 240 turned entries: more than the preparation kernel holds in shared memory,
    # so it reads every entry where it is used
    "attention_long_rows": Z.one_layer(Z.latent(44, 4, 240, 4, 16, 0.06, window=30, base=1e5),
                                       width=32),
    "dense": Z.one_layer(Z.latent(1, 8, 2, 8, 6, 0.5, base=10.0), Z.dense(56)),
    "dense_wide": Z.one_layer(Z.latent(1, 8, 8, 8, 8, 0.5, base=10.0), Z.dense(200), width=64),
    "moe_identity_shared": Z.one_layer(Z.latent(1, 8, 2, 8, 6, 0.5, base=10.0),
                                       Z.moe(6, 3, 24, identity=3, shared=20)),
    "moe_top1_bare": Z.one_layer(Z.latent(1, 8, 2, 8, 6, 0.5, base=10.0), Z.moe(4, 1, 12)),
    "moe_one_expert": Z.one_layer(Z.latent(1, 8, 2, 8, 6, 0.5, base=10.0),
                                  Z.moe(1, 1, 16, identity=1, shared=8)),
    "moe_wide": Z.one_layer(Z.latent(2, 16, 16, 16, 48, 0.2, window=9, base=10.0),
                            Z.moe(8, 2, 64, identity=1, shared=128), width=128,
                            logit_softcap=5.0, embedding={"scale": 4.0}),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mechanism_alone(tmp_path, name, dtype):
    raw = ONE_LAYER[name]
    w = Z.make_zefenex(tmp_path / name, raw, 5, dtype, std=0.15,
                       patch=sharp(3.0) if name.startswith("attention") else None)
    toks = {0: tokens_for(raw["vocab"], 70, 3), 1: tokens_for(raw["vocab"], 45, 4)}
    rp = Replayer(tmp_path / name, dtype, num_blocks=8, max_requests=2)
    rp.step([(0, 70)], toks, end=[0])                       # whole
    rp.step([(1, 1)], toks)                                 # the first token alone
    rp.step([(1, 16)], toks)                                # portions, then token by token
    rp.step([(1, 2)], toks)
    for _ in range(26):
        rp.step([(1, 1)], toks)
    for i in toks:
        check(rp.logits(i), w, raw, toks[i], dtype, f"{name} {dtype} request {i}")


def _moved(wrong, want, rows):
    return (wrong - want).abs().max(dim=1).values[rows]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [15, 16, 17, 40])
def test_a_window_one_token_off_would_show(tmp_path, window, dtype):
    """Sharp attention behind a window: the engine agrees with the oracle of that window,
    and the oracles of a window one token longer or shorter are far away, in a prompt and
    in decoded tokens, with windows that end at, before and behind a page's edge."""
    raw = Z.one_layer(Z.latent(2, 16, 8, 12, 24, 1.0, window=window, base=100.0))
    w = Z.make_zefenex(tmp_path / "m", raw, 9, dtype, std=0.2, patch=sharp(3.0))
    n = 100
    toks = {0: tokens_for(raw["vocab"], n, 1), 1: tokens_for(raw["vocab"], n, 1)}
    rp = Replayer(tmp_path / "m", dtype, num_blocks=8, max_requests=1)
    rp.step([(0, n)], toks, end=[0])
    rp.step([(1, 37)], toks)
    for _ in range(n - 37):
        rp.step([(1, 1)], toks)
    want = oracle(w, raw, toks[0])
    for off in (-1, 1):
        wrong_raw = copy.deepcopy(raw)
        wrong_raw["layers"][0]["mixer"]["mask"]["size"] = window + off
        moved = _moved(oracle(w, wrong_raw, toks[0]), want, slice(window, None))
        for i in (0, 1):
            err = (rp.logits(i).double() - want).abs().max(dim=1).values[window:]
            if dtype == "float32":
                assert (moved > 20 * err).sum() >= 10, (window, off, i)
            else:
                assert (moved > 4 * err).sum() >= 3, (window, off, i)
    for i in (0, 1):
        check(rp.logits(i), w, raw, toks[i], dtype, f"window {window} {dtype} run {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_or_a_router_got_wrong_would_show(tmp_path, dtype):
    """The oracle with the sink left out, with the sink scaled like a score, and with other
    router scores: each moves the logits far more than the engine differs from the oracle
    as it is, in a prompt and in decoded tokens."""
    raw = Z.one_layer(Z.latent(3, 8, 8, 10, 16, 0.5, window=30, base=30.0),
                      Z.moe(5, 2, 16, identity=2, shared=12))

    def big_sinks(w):
        w["l0.mix.sink"] = w["l0.mix.sink"].abs() + 1.0      # a sink that takes a good share

    w = Z.make_zefenex(tmp_path / "m", raw, 13, dtype, std=0.2, patch=big_sinks)
    n_tok = 60
    toks = {0: tokens_for(raw["vocab"], n_tok, 2), 1: tokens_for(raw["vocab"], n_tok, 2)}
    rp = Replayer(tmp_path / "m", dtype, num_blocks=8, max_requests=1)
    rp.step([(0, n_tok)], toks, end=[0])
    rp.step([(1, 20)], toks)
    for _ in range(n_tok - 20):
        rp.step([(1, 1)], toks)
    want = oracle(w, raw, toks[0])
    err = max((rp.logits(i).double() - want).abs().max().item() for i in (0, 1))

    def no_sink(w2):
        w2["l0.mix.sink"] = torch.full_like(w2["l0.mix.sink"], -1e4)

    def scaled_sink(w2):
        w2["l0.mix.sink"] = w2["l0.mix.sink"] * raw["layers"][0]["mixer"]["scale"]

    def no_correction(w2):
        w2["l0.mlp.correction"] = torch.zeros_like(w2["l0.mlp.correction"])

    for name, change in (("no sink", no_sink), ("scaled sink", scaled_sink),
                         ("no correction", no_correction)):
        w2 = {k: v.clone() for k, v in w.items()}
        change(w2)
        moved = (oracle(w2, raw, toks[0]) - want).abs().max().item()
        assert moved > (50 if dtype == "float32" else 3) * err, (name, moved, err)
    for i in (0, 1):
        check(rp.logits(i), w, raw, toks[i], dtype, f"sink and routing {dtype} run {i}")


# ------------------------------------------------------------------- whole models
LENGTHS = {"mixed": [1, 2, 19, 150], "plain": [1, 33, 97], "wide": [3, 64, 260],
           "sharp": [5, 300], "sharp_mixed": [7, 210]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", sorted(LENGTHS))
def test_whole_prompts_and_decoding_agree_with_the_plain_model(models, key, dtype):
    folder, raw, w = models[(key, dtype)]
    rp = Replayer(folder, dtype, num_blocks=24, max_requests=2)
    for i, n in enumerate(LENGTHS[key]):
        toks = {i: tokens_for(raw["vocab"], n, 40 + i), ("d", i): tokens_for(raw["vocab"], n, 40 + i)}
        rp.step([(i, n)], toks, end=[i])
        check(rp.logits(i), w, raw, toks[i], dtype, f"{key} {dtype} whole prompt of {n}")
        # the same tokens: most at once, the last ones (up to 40, over page edges) one by one
        tail = min(40, n - 1)
        if tail:
            rp.step([(("d", i), n - tail)], toks)
            for _ in range(tail):
                rp.step([(("d", i), 1)], toks)
            rp.runner.release(("d", i))
            check(rp.logits(("d", i)), w, raw, toks[i], dtype, f"{key} {dtype} decoded tail of {n}")


def test_the_residual_stream_after_every_layer(models):
    """float32: the stream after each layer against the oracle's, layer by layer."""
    from mini_llm_stack_b200.engine.batch import Entry
    from mini_llm_stack_b200.engine.runner import ModelRunner, load_model
    folder, raw, w = models[("mixed", "float32")]
    toks = tokens_for(raw["vocab"], 50, 77)
    trace = []
    oracle(w, raw, toks, trace=trace)
    model = load_model(folder, dtype="float32")
    runner = ModelRunner(model, num_blocks=8, block_size=16, max_requests=1, cuda_graphs=False)
    seen = []
    for block in model.blocks:
        def forward(stream, step, cache, _inner=block.forward):
            _inner(stream, step, cache)
            # what waits on the stream still has to pass the norm behind the sublayer
            waiting = stream.take_pending()
            y = waiting.resolve().clone() if hasattr(waiting, "resolve") else waiting.float()
            seen.append((stream.x + y).cpu().double())
            stream.push(y)
        block.forward = forward
    entries = [Entry("r", toks, [49])]
    runner.reserve(entries)
    runner.step(entries)
    model.runtime.ops.check_status()
    assert len(seen) == len(trace)
    for i, (got, want) in enumerate(zip(seen, trace)):
        scale = want.abs().max().item()
        assert (got - want).abs().max().item() < 2e-5 * scale, f"layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "sharp", "sharp_mixed"])
def test_portions_of_every_size_do_not_change_the_logits(models, key, dtype):
    folder, raw, w = models[(key, dtype)]
    n = 231
    toks = {"r": tokens_for(raw["vocab"], n, 9), "w": tokens_for(raw["vocab"], n, 9)}
    rp = Replayer(folder, dtype, num_blocks=16, max_requests=1)
    fed = 0
    for size in [2, 3, 11, 16, 1, 1, 2, 47, 17, 64, 5, 2, 33]:      # cuts inside pages and at their edges
        rp.step([("r", size)], toks)
        fed += size
    while fed < n:
        rp.step([("r", 1)], toks)
        fed += 1
    rp.runner.release("r")
    check(rp.logits("r"), w, raw, toks["r"], dtype, f"{key} {dtype} portions")
    if dtype == "float32":
        rp.step([("w", n)], toks, end=["w"])
        assert torch.equal(rp.logits("r"), rp.logits("w")), "the cut changes float32 bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "wide", "plain"])
def test_unequal_requests_in_one_batch_with_pages_used_again(models, key, dtype):
    """Five requests over three request slots and so few pages that a finished request's
    pages go to the next one at once; every request must come out as alone."""
    folder, raw, w = models[(key, dtype)]
    lens = {0: 90, 1: 37, 2: 61, 3: 120, 4: 2}
    toks = {i: tokens_for(raw["vocab"], n, 70 + i) for i, n in lens.items()}
    rp = Replayer(folder, dtype, num_blocks=18, max_requests=3)
    rp.step([(0, 40), (1, 2)], toks)
    rp.step([(0, 1), (1, 35), (2, 30)], toks, end=[1])
    rp.step([(0, 17), (2, 1), (3, 50)], toks)                 # 3 takes the slot and pages of 1
    rp.step([(0, 32), (2, 30), (3, 2)], toks, end=[0, 2])
    rp.step([(3, 1), (4, 2)], toks, end=[4])                  # 4 starts from a slot 0 or 2 left
    rp.step([(3, 67)], toks, end=[3])
    assert rp.runner.cache.slots.num_free == 3
    for i in lens:
        check(rp.logits(i), w, raw, toks[i], dtype, f"{key} {dtype} request {i}")
    if dtype == "float32":
        # a token's logits do not depend on its batch: bit for bit the run of each alone
        for i in (1, 3):
            alone = Replayer(folder, dtype, num_blocks=18, max_requests=1)
            alone.step([(i, lens[i])], toks, end=[i])
            assert torch.equal(alone.logits(i), rp.logits(i)), f"request {i} depends on its batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs_and_sees_far_keys(models, dtype):
    """Two requests decode side by side for 160 steps; the third layer's window is a page,
    the second layer reads the first layer's cache 100 tokens back, softmaxes are sharp."""
    folder, raw, w = models[("sharp", dtype)]
    n = 190
    toks = {"a": tokens_for(raw["vocab"], n, 23), "b": tokens_for(raw["vocab"], n - 30, 24)}
    rp = Replayer(folder, dtype, num_blocks=32, max_requests=2)
    rp.step([("a", 10), ("b", 3)], toks)
    for _ in range(n - 30 - 3):                               # both decode, one token a step
        rp.step([("a", 1), ("b", 1)], toks)
    rp.runner.release("b")
    for _ in range(n - 10 - (n - 33)):
        rp.step([("a", 1)], toks)
    assert any(isinstance(v, tuple) for k, v in rp.runner._graphs.items() if k != "moved"), \
        "no decode step was replayed from a graph"
    for r in toks:
        check(rp.logits(r), w, raw, toks[r], dtype, f"long decoding {r} {dtype}")


def test_far_keys_without_a_window(tmp_path):
    """No window, hundreds of tokens, a sharp softmax: a key 500 tokens back decides."""
    raw = Z.one_layer(Z.latent(2, 16, 8, 12, 24, 1.0, base=1e4))
    for dtype in ("float32", "bfloat16"):
        w = Z.make_zefenex(tmp_path / dtype, raw, 21, dtype, std=0.2, patch=sharp(4.0))
        n = 600
        toks = {0: tokens_for(raw["vocab"], n, 5)}
        rp = Replayer(tmp_path / dtype, dtype, num_blocks=40, max_requests=1)
        rp.step([(0, 570)], toks)
        for _ in range(n - 570):
            rp.step([(0, 1)], toks)
        check(rp.logits(0), w, raw, toks[0], dtype, f"far keys {dtype}")
        # the far keys matter: a window of 300 moves the oracle's late rows
        short = copy.deepcopy(raw)
        short["layers"][0]["mixer"]["mask"] = {"size": 300}
        want = oracle(w, raw, toks[0])
        assert (oracle(w, short, toks[0]) - want).abs().max(dim=1).values[300:].max().item() > \
            0.05 * want.abs().max().item()


def test_greedy_generation_through_the_scheduler(models):
    from mini_llm_stack_b200.engine.llm import LLM
    folder, raw, w = models[("mixed", "float32")]
    prompts = [tokens_for(raw["vocab"], n, 300 + n) for n in (3, 41, 18, 1)]
    # three at a time, portions of at most 16 tokens, so few pages that requests wait
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=14, block_size=8, max_batch=3,
                          max_tokens_per_step=24, chunk_size=16)
    got = llm.generate(prompts, max_new_tokens=10)
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            row = oracle(w, raw, seq)[-1]
            assert row[tok] >= row.max() - 1e-4 * row.abs().max(), (len(p), len(seq), tok)
            seq.append(tok)
        assert len(g) == 10
    llm.engine.cache.check()
    assert llm.engine.cache.slots.num_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_replays_a_folder(models, tmp_path, dtype):
    """``bin/trace_run`` picks the model class by config.json; two requests, portions beside
    single tokens, a pool of two requests' worth of tokens."""
    folder, raw, w = models[("mixed", dtype)]
    a, b = tokens_for(raw["vocab"], 50, 1), tokens_for(raw["vocab"], 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:48], "want": []},
                                     {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[48:49], "want": [0]},
                                     {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[49:], "want": [0]}], "end": ["a"]}]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder),
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == \
        [f"done {i}" for i in range(4)]
    la, lb = oracle(w, raw, a), oracle(w, raw, b)
    want = {0: la[[0, 29]], 1: lb[[7]], 2: torch.stack([la[48], lb[8]]), 3: la[[49]]}
    for i, rows in want.items():
        got = torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32)
        got = got.view(-1, raw["vocab"]).double()
        tol = 5e-5 if dtype == "float32" else 6e-2
        assert (got - rows).abs().max().item() < tol * rows.abs().max().item(), i
