"""Zededra on the GPU against the plain implementation of ``plain_zededra``.

Mechanisms alone (kernels through ``Ops``, mixers and feed-forwards as one-layer
models), then whole models: prompts whole, decoded token by token, in portions down to
two tokens, unequal requests in one batch, pages and state slots used again, long
decoding through CUDA graphs, and greedy generation through ``LLM.generate``.  Where
random weights would hide a fault the weights are made to show it: queries and keys
scaled up until every softmax is nearly one key (any key the engine loses, far away or
at a page's edge, then changes the logits), forget gates near one so that the first
tokens of a sequence still matter hundreds of tokens later.
"""

import copy

import pytest
import torch

import plain_zededra as PZ
import tiny_zededra as Z
from engine_helpers import Replayer, tokens_for

pytestmark = pytest.mark.gpu

# largest |engine - plain| as a fraction of the largest |logit|: float32 differs from the
# float64 oracle by the order of its sums; bfloat16 by the rounding of weights' products
# and activations (the oracle rounds nothing), measured at 1-2 % on these models
TOL = {"float32": 5e-5, "bfloat16": 3e-2}
# Some rows are ill-conditioned: the mLSTM divides by |n . q|, which passes near zero, and
# a sharp softmax turns a small change of a score into another key.  There rounding alone
# moves the logits by more than any fixed bound, so a row may also be off by NOISE times
# what rounding does to that row of the oracle itself: the oracle run again with its
# activations rounded to the engine's format, against its exact run in float64.
NOISE = 6.0
# In bfloat16 a router whose best scores nearly tie may choose another expert than the
# oracle, which rounds nothing (with random inputs a few tokens in a hundred tie within
# bfloat16's rounding); such a token then differs by a whole expert, and through attention
# and the recurrent state so do the tokens after it.  Which experts are chosen is therefore
# tested in float32, where no row may be off; the bfloat16 models route every token to all
# of their experts (``no_choice``: the same kernels, sort and sums, nothing to tie), and the
# one bfloat16 case with a choice (a single layer, so nothing spreads) may have FLIPS of
# its rows off.
FLIPS = 0.06


def no_choice(raw):
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def close(got, want, tol, what, flips=False, slack=None):
    scale = want.abs().max().item()
    err = (got.double() - want.double()).abs().max(dim=1).values
    bound = tol * scale if slack is None else tol * scale + NOISE * slack
    bad = int((err > bound).sum())
    allowed = -(-int(FLIPS * 1000) * len(err) // 1000) if flips else 0
    assert bad <= allowed, (
        f"{what}: {bad} rows of {len(err)} differ by more than {tol:.0e} * {scale:.3f} "
        f"(worst {err.max().item():.3e}); first wrong row {int((err > bound).nonzero()[0])}")


def sharp(factor):
    """Scale every query and key projection so that softmax picks nearly one key."""
    def patch(w):
        for n in w:
            if n.endswith(".mix.uq") or n.endswith(".mix.uk"):
                w[n] *= factor
    return patch


def long_memory(w):
    """Forget gates near one, input gates spread out: early tokens stay in the memory."""
    for n in w:
        if n.endswith(".mix.f.b"):
            w[n] = w[n] * 0.3 + 4.0
        if n.endswith(".mix.i"):
            w[n] *= 4.0


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zededra")
    out = {}
    for key, raw, patch in (("mixed", Z.Z_MIXED, None), ("plain", Z.Z_PLAIN, None),
                            ("wide", Z.Z_WIDE, None),
                            ("sharp", Z.Z_WIDE, lambda w: (sharp(5.0)(w), long_memory(w)))):
        for dtype in ("float32", "bfloat16"):
            folder = tmp / f"{key}_{dtype}"
            used = no_choice(raw) if dtype == "bfloat16" else raw
            out[(key, dtype)] = (folder, used, Z.make_zededra(folder, used, 11, dtype, patch=patch))
    return out


def oracle(w, raw, tokens):
    return PZ.plain_zededra(w, raw, tokens)


def check(got, w, raw, tokens, dtype, what, flips=False):
    """The engine's rows against the oracle's, every row with its own slack."""
    want = oracle(w, raw, tokens)
    # several realisations of the rounding (values nudged by under half a step of the format
    # before they are rounded to it): one alone may happen to leave an ill-conditioned row still
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
    for rnd in (rounded_to, nudged, nudged, nudged):
        rounded = PZ.plain_zededra(w, raw, tokens, rnd=rnd)
        slack = torch.maximum(slack, (rounded - want).abs().max(dim=1).values)
    close(got, want, TOL[dtype], what, flips=flips, slack=slack)


# ------------------------------------------------------------------ kernels alone
@pytest.fixture(scope="module")
def rt32():
    from mini_llm_stack_b200.ops.kernels import Runtime
    return Runtime("cuda:0", torch.float32)


def test_layernorm_kernel_with_every_addend(rt32):
    g = torch.Generator().manual_seed(0)
    for d in (36, 320, 1000):
        x = torch.randn(9, d, generator=g) * 3 + 1
        delta, rows, vec = torch.randn(9, d, generator=g), torch.randn(9, d, generator=g), \
            torch.randn(d, generator=g)
        w = torch.randn(d, generator=g)
        xd = x.cuda()
        h = torch.empty(9, d, device="cuda")
        rt32.ops.add_layernorm(xd, delta.cuda(), w.cuda(), 1e-5, h, more_rows=rows.cuda(),
                               more_vec=vec.cuda())
        v = (x + delta + rows + vec).double()
        assert torch.allclose(xd.cpu().double(), v, atol=1e-6)
        assert torch.allclose(h.cpu().double(), PZ.plain_layernorm(v, w.double(), 1e-5), atol=2e-5)
        pick = torch.tensor([7, 2, 2], dtype=torch.int32, device="cuda")
        h3 = torch.empty(3, d, device="cuda")
        before = xd.clone()
        rt32.ops.add_layernorm(xd, None, w.cuda(), 1e-5, h3, rows=pick, n_rows=3)
        assert torch.equal(xd, before)
        assert torch.allclose(h3.cpu().double(), PZ.plain_layernorm(v[[7, 2, 2]], w.double(), 1e-5),
                              atol=2e-5)


def test_residual_add_kernel(rt32):
    """What a norm of another kind uses to settle a pass's addends."""
    g = torch.Generator().manual_seed(5)
    x, rows, vec = torch.randn(7, 52, generator=g), torch.randn(7, 52, generator=g), \
        torch.randn(52, generator=g)
    xd = x.cuda()
    rt32.ops.residual_add(xd, rows.cuda(), vec.cuda())
    assert torch.allclose(xd.cpu(), x + rows + vec, atol=1e-6)
    rt32.ops.residual_add(xd, None, vec.cuda().bfloat16())
    assert torch.allclose(xd.cpu(), x + rows + vec + vec.bfloat16().float(), atol=1e-6)


def test_clamped_glu_kernel(rt32):
    g = torch.Generator().manual_seed(1)
    gu = (torch.randn(5, 2 * 37, generator=g) * 3).cuda()
    out = torch.empty(5, 37, device="cuda")
    rt32.ops.clamped_glu(gu, out, 1.702, 1.25)
    gate, up = gu[:, :37].double().cpu(), gu[:, 37:].double().cpu()
    gate, up = gate.clamp(max=1.25), up.clamp(-1.25, 1.25)
    assert torch.allclose(out.cpu().double(), gate * torch.sigmoid(1.702 * gate) * (up + 1), atol=1e-6)


def test_fused_clamped_glu_product(rt32):
    """Gate-up product with the clamped unit in its epilogue (bfloat16, tcgen05): few rows
    (weight-major, K cut in parts), a prompt's rows on one CTA and on pairs of CTAs."""
    from mini_llm_stack_b200.ops.kernels import Runtime
    ops = Runtime("cuda:0", torch.bfloat16).ops
    g = torch.Generator().manual_seed(3)
    d, inter = 256, 96
    wg = (torch.randn(inter, d, generator=g) * 0.2).bfloat16().cuda()
    wu = (torch.randn(inter, d, generator=g) * 0.2).bfloat16().cuda()
    assert ops.can_fuse_swiglu(d, inter)
    w = ops.prepare_weight(ops.interleave_gate_up(wg, wu))
    for m in (3, 40, 100, 300):
        a = torch.randn(m, d, generator=g).bfloat16().cuda()
        out = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
        ops.linear_clamped_glu(a, w, out, 1.702, 0.8)
        gate = (a.double() @ wg.double().T).clamp(max=0.8)
        up = (a.double() @ wu.double().T).clamp(-0.8, 0.8)
        want = gate * torch.sigmoid(1.702 * gate) * (up + 1)
        assert (out.double() - want).abs().max().item() < 1e-2 * want.abs().max().item(), m
    ops.check_status()


def test_router_picks_lowest_index_on_ties_and_can_renormalise(rt32):
    z = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0], [3.0, -3.0, 0.0, 3.0, 1.0]]).cuda()
    fns = rt32.ops._part_lib("experts")
    idx = torch.empty(6, dtype=torch.int32, device="cuda")
    wt = torch.empty(6, device="cuda")
    for renorm in (0, 1):
        # rows of five logits; sigmoid scores, no correction, nothing added to the sum of the
        # chosen scores, one group
        fns["topk"](z.data_ptr(), 5, 2, 5, 3, renorm, 0, None, 0.0, 1, 1, idx.data_ptr(),
                    wt.data_ptr(), rt32.ops._stream())
        assert idx.tolist() == [1, 2, 4, 0, 3, 4]
        want = torch.sigmoid(torch.tensor([[2.0, 2.0, 2.0], [3.0, 3.0, 1.0]]))
        if renorm:
            want = want / want.sum(-1, keepdim=True)
        assert torch.allclose(wt.cpu().view(2, 3), want, atol=1e-6)


# ------------------------------------------------------- mechanisms as one-layer models
ONE_LAYER = {
    "latent": {"type": "latent_attention", "mixer": Z.latent(3, 8, 24, 40, 12, 0.6), "mlp": None},
    "latent_one_head": {"type": "latent_attention", "mixer": Z.latent(1, 16, 8, 16, 16, 0.5),
                        "mlp": None},
    # a latent beyond the tensor-core kernels' head sizes
    "latent_wide": {"type": "latent_attention", "mixer": Z.latent(2, 16, 24, 300, 40, 0.1),
                    "mlp": None},
    "mlstm": {"type": "mlstm", "mixer": Z.mlstm(2, 12, 20, 6.0), "mlp": None},
    "mlstm_many_columns": {"type": "mlstm", "mixer": Z.mlstm(1, 40, 150, 20.0), "mlp": None},
    "dense": {"type": "latent_attention", "mixer": Z.latent(1, 8, 8, 16, 8, 0.5),
              "mlp": Z.dense(56, 0.4)},
    "experts_top1": {"type": "latent_attention", "mixer": Z.latent(1, 8, 8, 16, 8, 0.5),
                     "mlp": Z.moe(7, 1, 20)},
    "experts_top3_shared": {"type": "latent_attention", "mixer": Z.latent(1, 8, 8, 16, 8, 0.5),
                            "mlp": Z.moe(4, 3, 36, shared=24)},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mechanism_alone(tmp_path, name, dtype):
    raw = Z.one_layer(ONE_LAYER[name])
    patch = long_memory if name.startswith("mlstm") else sharp(3.0)
    w = Z.make_zededra(tmp_path / name, raw, 5, dtype, std=0.15, patch=patch)
    toks = {0: tokens_for(raw["vocab"], 70, 3), 1: tokens_for(raw["vocab"], 45, 4)}
    rp = Replayer(tmp_path / name, dtype, num_blocks=8, max_requests=2)
    rp.step([(0, 70)], toks, end=[0])                       # whole
    rp.step([(1, 17)], toks)                                # portions, then token by token
    rp.step([(1, 2)], toks)
    for _ in range(26):
        rp.step([(1, 1)], toks)
    for i in toks:
        check(rp.logits(i), w, raw, toks[i], dtype, f"{name} {dtype} request {i}",
              flips=dtype == "bfloat16" and name == "experts_top1")


# ------------------------------------------------------------------- whole models
LENGTHS = {"mixed": [1, 2, 19, 150], "plain": [1, 33, 97], "wide": [3, 64, 260], "sharp": [5, 300]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "plain", "wide", "sharp"])
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "sharp"])
def test_portions_of_every_size_do_not_change_the_logits(models, key, dtype):
    folder, raw, w = models[(key, dtype)]
    n = 231
    toks = {"r": tokens_for(raw["vocab"], n, 9)}
    rp = Replayer(folder, dtype, num_blocks=16, max_requests=1)
    fed = 0
    for size in [2, 3, 11, 16, 1, 1, 2, 47, 17, 64, 5, 2, 33]:      # cuts inside pages and at their edges
        rp.step([("r", size)], toks)
        fed += size
    while fed < n:
        rp.step([("r", 1)], toks)
        fed += 1
    check(rp.logits("r"), w, raw, toks["r"], dtype, f"{key} {dtype} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "wide"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, key, dtype):
    """Four requests over three state slots and so few pages that a finished request's
    pages and slot go to the next one at once; every request must come out as alone."""
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


def test_long_decoding_replays_graphs_and_keeps_the_state(models):
    folder, raw, w = models[("sharp", "float32")]
    n = 190
    toks = {"a": tokens_for(raw["vocab"], n, 21), "b": tokens_for(raw["vocab"], n - 30, 22)}
    rp = Replayer(folder, "float32", num_blocks=32, max_requests=2)
    rp.step([("a", 10), ("b", 3)], toks)
    for _ in range(n - 30 - 3):                               # both decode, one token a step
        rp.step([("a", 1), ("b", 1)], toks)
    rp.runner.release("b")
    for _ in range(n - 10 - (n - 33)):
        rp.step([("a", 1)], toks)
    assert any(isinstance(v, tuple) for k, v in rp.runner._graphs.items() if k != "moved"), \
        "no decode step was replayed from a graph"
    for r in toks:
        close(rp.logits(r), oracle(w, raw, toks[r]), TOL["float32"], f"long decoding {r}")


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
