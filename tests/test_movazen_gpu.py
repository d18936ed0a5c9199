"""Movazen on the GPU against the plain implementation of ``plain_movazen``.

Kernels alone (through ``Ops``), then whole models: prompts whole, decoded token by token, in
portions down to two tokens, unequal requests in one batch on few pages and fewer state slots
than requests, long decoding through CUDA graphs, greedy generation through ``LLM.generate``
and the trace program.  Where random weights would hide a fault the weights are made to show
it: queries are scaled up until every softmax is nearly one key, so a key the engine loses (far
away, at a page's edge, at the window's, among the kept first tokens) changes the logits.
"""

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_movazen as PM
import tiny_movazen as M
from engine_helpers import Replayer, tokens_for

pytestmark = pytest.mark.gpu

# largest |engine - plain| of a row as a fraction of the largest |logit|: float32 differs from
# the float64 oracle by the order of its sums, bfloat16 by the rounding of products and
# activations.  A router's close call could fall the other way in a bfloat16 run, so the models
# of the bfloat16 runs have routers whose choices rest on their corrections (``decisive_routers``:
# clear margins, the weights still follow the tokens); the float32 runs keep routers that choose
# by the token.  A row in a hundred of a bfloat16 run may still differ by more.
TOL = {"float32": 5e-5, "bfloat16": 4e-2}
LOOSE_ROWS = {"float32": 0.0, "bfloat16": 0.02}


def close(got, want, dtype, what, tol=None):
    want = torch.as_tensor(np.asarray(want)).double()
    got = got.double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = want.abs().max().item()
    err = (got - want).abs().max(dim=1).values / scale
    tol = tol or TOL[dtype]
    bad = int((err > tol).sum())
    assert bad <= LOOSE_ROWS[dtype] * len(err), (
        f"{what}: {bad} rows of {len(err)} differ by more than {tol:.0e} of the largest logit "
        f"(worst {err.max().item():.3e}); first wrong row {int((err > tol).nonzero()[0])}")
    assert err.max().item() < 20 * tol, f"{what}: worst row off by {err.max().item():.3e}"


def sharp(factor):
    """Scale the queries so that softmax picks nearly one key (the attention mixer's queries are
    normalised, so there the norm's weight is scaled)."""
    def patch(w):
        for n in w:
            if n.endswith("mix.q.norm") or n.endswith("left.q") or n.endswith("left.q.b"):
                w[n] *= factor
    return patch


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("movazen")
    out = {}
    for key, raw, patch in (("mixed", M.M_MIXED, None), ("plain", M.M_PLAIN, None),
                            ("wide", M.M_WIDE, None), ("sharp", M.M_MIXED, sharp(6.0)),
                            ("sharp_wide", M.M_WIDE, sharp(5.0))):
        for dtype in ("float32", "bfloat16"):
            folder = tmp / f"{key}_{dtype}"

            def both(w, patch=patch, dtype=dtype, raw=raw):
                if patch:
                    patch(w)
                if dtype == "bfloat16":
                    M.decisive_routers(w, raw)
            cfg, w = M.make_movazen(folder, raw, 11, dtype, patch=both)
            out[(key, dtype)] = (folder, cfg, w)
    return out


# ------------------------------------------------------------------ kernels alone
@pytest.fixture(scope="module")
def rt32():
    from mini_llm_stack_b200.ops.kernels import Runtime
    return Runtime("cuda:0", torch.float32)


def fake_step(positions, slots, block_size):
    from mini_llm_stack_b200.parts.base import GroupView, StepContext
    t = len(positions)
    i32 = dict(dtype=torch.int32, device="cuda")
    return StepContext(
        n_tokens=t, n_requests=1, token_ids=torch.zeros(t, **i32),
        positions=torch.tensor(positions, **i32), req_of_token=torch.zeros(t, **i32),
        cu_q=torch.tensor([0, t], **i32), ctx_len=torch.tensor([t, t], **i32),
        state_slot=torch.zeros(1, **i32), out_rows=torch.zeros(1, **i32), n_out=0,
        groups={0: GroupView(torch.zeros((1, 8), **i32), torch.tensor(slots, **i32),
                             block_size, 8)})


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("options", ["norms", "biases and temperature", "bare"])
def test_head_preparation_kernel(rt32, act, options):
    """Biases, per-head norms with one weight for all heads, the query's temperature, the
    values' scale, zero padding to the kernels' head size, and the cleared rest of a page."""
    from mini_llm_stack_b200.parts.base import CacheHandle
    g = torch.Generator().manual_seed(3)
    nh, nkv, e, f, hd, bs, t = 3, 2, 12, 20, 32, 4, 6
    positions = [10, 11, 12, 13, 14, 15]
    slots = [6, 7, 20, 21, 22, 40]            # two tokens end an old page, then a new page, then one more
    width = 5 + nh * e + nkv * e + nkv * f
    proj = torch.randn(t, width, generator=g)
    cols = (5, 5 + nh * e, 5 + nh * e + nkv * e)
    biases = norms = temp = None
    if options == "norms":
        norms = tuple(torch.randn(e, generator=g).cuda() for _ in range(2))
    if options == "biases and temperature":
        biases = tuple(torch.randn(n, generator=g).cuda() for n in (nh * e, nkv * e, nkv * f))
        temp = (0.7, 4)
    pool = torch.full((2, nkv, 16, bs, hd), float("nan"), dtype=act, device="cuda")
    cache = CacheHandle(kind="paged", group=0, k_pool=pool[0], v_pool=pool[1])
    q_out = torch.full((t, (nh + 2 * nkv) * hd), float("nan"), dtype=act, device="cuda")
    rt32.ops.head_prep_store(proj.cuda(), cols, biases, norms, 1e-5, temp, 0.6, q_out, cache,
                             fake_step(positions, slots, bs), nh, nkv, e, f, hd)
    torch.cuda.synchronize()
    p = proj.double()
    q = p[:, cols[0]:cols[0] + nh * e]
    k = p[:, cols[1]:cols[1] + nkv * e]
    v = p[:, cols[2]:cols[2] + nkv * f]
    if biases:
        q, k, v = (x + b.cpu().double() for x, b in zip((q, k, v), biases))
    q, k, v = q.reshape(t, nh, e), k.reshape(t, nkv, e), v.reshape(t, nkv, f) * 0.6
    if norms:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + 1e-5) * norms[0].cpu().double()
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + 1e-5) * norms[1].cpu().double()
    if temp:
        for i, pos in enumerate(positions):
            q[i] *= 1 + 0.7 * math.log((pos + 1) // 4 + 1)
    tol = 1e-5 if act == torch.float32 else 2e-2
    got_q = q_out.cpu().double()[:, :nh * hd].reshape(t, nh, hd)
    assert (got_q[..., :e] - q).abs().max() < tol * q.abs().max()
    assert (got_q[..., e:] == 0).all()
    kp, vp = pool[0].cpu().double(), pool[1].cpu().double()
    for i, s in enumerate(slots):
        assert (kp[:, s // bs, s % bs, :e] - k[i]).abs().max() < tol * k.abs().max()
        assert (kp[:, s // bs, s % bs, e:] == 0).all()
        assert (vp[:, s // bs, s % bs, :f] - v[i]).abs().max() < tol * v.abs().max()
        assert (vp[:, s // bs, s % bs, f:] == 0).all()
    # slot 22 ends its request's stay in page 5, which the step entered: slot 23 is cleared;
    # slot 40 opens page 10 and is the step's last: 41..43 are cleared; page 1 was entered
    # before the step: nothing of it is touched beyond the two slots written
    assert (kp[:, 5, 3] == 0).all() and (vp[:, 5, 3] == 0).all()
    assert (kp[:, 10, 1:] == 0).all() and (vp[:, 10, 1:] == 0).all()
    assert kp[:, 1, :2].isnan().all() and kp[:, 2].isnan().all()


@pytest.mark.parametrize("experts, top, groups", [(10, 3, (2, 1)), (12, 2, (4, 2)), (6, 6, (3, 3)),
                                                  (5, 2, None), (8, 1, (8, 1)), (64, 4, (8, 3))])
def test_grouped_routing_kernel(rt32, experts, top, groups):
    g = torch.Generator().manual_seed(experts)
    t = 37
    logits = torch.randn(t, experts + 1, generator=g)        # one more column, as with a gate
    logits[3] = 0.25                                          # ties: the lowest index wins
    corr = torch.randn(experts, generator=g) * 0.5
    work = {"idx": torch.empty(t * top, dtype=torch.int32, device="cuda"),
            "weight": torch.empty(t * top, dtype=torch.float32, device="cuda"),
            "order": torch.empty(t * top, dtype=torch.int32, device="cuda"),
            "offsets": torch.empty(experts + 1, dtype=torch.int32, device="cuda"),
            "cursor": torch.empty(experts, dtype=torch.int32, device="cuda")}
    work["max_tiles"] = rt32.ops.expert_max_tiles(t * top, experts)
    work["tile_expert"] = torch.empty(work["max_tiles"], dtype=torch.int32, device="cuda")
    work["tile_row0"] = torch.empty(work["max_tiles"], dtype=torch.int32, device="cuda")
    rt32.ops.route(logits.cuda(), top, True, work, correction=corr.cuda(), renorm_eps=1e-20,
                   groups=groups, n_outputs=experts)
    idx = work["idx"].cpu().view(t, top)
    wgt = work["weight"].cpu().view(t, top).double()
    s = torch.sigmoid(logits[:, :experts])
    for i in range(t):
        choice = (s[i] + corr).tolist()                       # float32, as the kernel adds
        want = PM.choose_experts(choice, top, {"count": groups[0], "keep": groups[1]}
                                 if groups else None)
        assert idx[i].tolist() == want, i
        sw = s[i, want].double()
        assert torch.allclose(wgt[i], sw / sw.sum(), atol=1e-6)


def test_row_norm_gate_kernel(rt32):
    g = torch.Generator().manual_seed(5)
    t, width = 7, 36
    for act in (torch.float32, torch.bfloat16):
        o = torch.randn(t, width, generator=g) * 3
        gate = torch.randn(t, 10 + width, generator=g).to(act)
        w = torch.randn(width, generator=g)
        out = torch.zeros(t, width + 8, dtype=act, device="cuda")
        rt32.ops.scan_finish_row(o.cuda(), gate.cuda(), 10, w.cuda(), 1e-5, out[:, 8:], 0.4)
        want = (PM.unit_rms(o.double().numpy(), 1e-5) * w.double().numpy()
                * PM.sigmoid(gate[:, 10:].double().numpy()) * 0.4)
        tol = 1e-5 if act == torch.float32 else 2e-2
        assert np.abs(out[:, 8:].cpu().double().numpy() - want).max() < tol * np.abs(want).max()
        assert (out[:, :8] == 0).all()


def test_side_input_kernels(rt32):
    g = torch.Generator().manual_seed(6)
    t, d, dim, pad, vocab = 5, 40, 6, 8, 11
    ops = rt32.ops
    x = torch.randn(t, d, generator=g)
    delta = torch.randn(t, d, generator=g)
    xd, out = x.cuda(), torch.empty(t, d, dtype=torch.bfloat16, device="cuda")
    ops.settle_cast(xd, delta.cuda(), out)
    assert torch.equal(xd.cpu(), x + delta) and torch.equal(out.cpu(), (x + delta).bfloat16())
    ops.settle_cast(xd, None, out)
    assert torch.equal(xd.cpu(), x + delta)
    z = torch.randn(t, pad, generator=g)
    table = torch.randn(vocab, 3 * dim, generator=g)
    ids = torch.tensor([0, 10, 3, 3, 7], dtype=torch.int32)
    gated = torch.full((t, pad), float("nan"), device="cuda")
    ops.gelu_gate_rows(z.cuda(), table.cuda(), dim, ids.cuda(), gated, n_real=dim)
    want = PM.gelu_tanh(z[:, :dim].double().numpy()) * table[ids.long(), dim:2 * dim].double().numpy()
    assert np.abs(gated[:, :dim].cpu().double().numpy() - want).max() < 1e-6
    assert (gated[:, dim:] == 0).all()
    y = torch.randn(t, d, generator=g) * 5
    w = torch.randn(d, generator=g)
    normed = torch.empty(t, d, device="cuda")
    ops.rms_scale(y.cuda(), w.cuda(), 1e-5, normed)
    want = PM.unit_rms(y.double().numpy(), 1e-5) * w.double().numpy()
    assert np.abs(normed.cpu().double().numpy() - want).max() < 1e-5


@pytest.mark.parametrize("d", [6, 37])
def test_embedding_with_sinusoidal_positions(rt32, d):
    from mini_llm_stack_b200.parts.position import SinusoidalPositions
    g = torch.Generator().manual_seed(d)
    table = torch.randn(9, d, generator=g)
    pos = SinusoidalPositions(d)
    pos.bind({}, rt32)
    ids = torch.tensor([1, 8, 0, 4], dtype=torch.int32, device="cuda")
    positions = torch.tensor([0, 3, 1000, 123456], dtype=torch.int32, device="cuda")
    x = torch.empty(4, d, device="cuda")
    rt32.ops.embed(ids, table.cuda(), x, 9, 2.5, positions=positions, freq=pos.freq)
    want = np.stack([table[i].double().numpy() * 2.5 + PM.sinusoid(p, d)
                     for i, p in zip(ids.tolist(), positions.tolist())])
    assert np.abs(x.cpu().double().numpy() - want).max() < 2e-6


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "plain", "wide"])
def test_whole_prompts(models, key, dtype):
    folder, cfg, w = models[(key, dtype)]
    r = Replayer(folder, dtype, num_blocks=24)
    for rid, n in (("a", 1), ("b", 2), ("c", 95), ("d", 130)):
        tokens = {rid: tokens_for(cfg["vocab"], n, n)}
        r.step([(rid, n)], tokens, end=[rid])
        close(r.logits(rid), PM.forward(cfg, w, tokens[rid]), dtype, f"{key} {n} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "wide"])
def test_decoding_token_by_token(models, key, dtype):
    """From the very first token on: the kept first tokens, the window's edge and the state are
    all built by single-token steps."""
    folder, cfg, w = models[(key, dtype)]
    tokens = {"a": tokens_for(cfg["vocab"], 90, 4)}
    r = Replayer(folder, dtype, num_blocks=12)
    for _ in range(90):
        r.step([("a", 1)], tokens)
    close(r.logits("a"), PM.forward(cfg, w, tokens["a"]), dtype, f"{key} decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 2, 2, 3, 5, 7, 16, 17, 31, 33, 2, 1, 1, 40),
                                   (64, 1, 1, 1, 15, 2, 48, 28), (21, 1, 40, 17, 3, 78)])
def test_portions_of_every_size(models, sizes, dtype):
    folder, cfg, w = models[("sharp", dtype)]
    n = sum(sizes)
    tokens = {"a": tokens_for(cfg["vocab"], n, 9)}
    r = Replayer(folder, dtype, num_blocks=12)
    for s in sizes:
        r.step([("a", s)], tokens)
    want = PM.forward(cfg, w, tokens["a"])
    if dtype == "float32":
        close(r.logits("a"), want, dtype, f"portions {sizes}")
    else:
        # with sharp weights a bfloat16 run is held against the engine's own whole-prompt run
        whole = Replayer(folder, dtype, num_blocks=12)
        whole.step([("a", n)], tokens)
        close(r.logits("a"), whole.logits("a").numpy(), dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "sharp_wide"])
def test_unequal_requests_in_one_batch_on_few_pages_and_slots(models, key, dtype):
    """Five requests through three state slots and a pool that holds less than their sum:
    portions beside single tokens, requests that pause, pages and slots used again."""
    folder, cfg, w = models[(key, dtype)]
    lens = {"a": 75, "b": 33, "c": 2, "d": 58, "e": 41}
    tokens = {k: tokens_for(cfg["vocab"], n, i) for i, (k, n) in enumerate(lens.items())}
    r = Replayer(folder, dtype, num_blocks=12, max_requests=3)
    r.step([("a", 30), ("b", 2)], tokens)
    r.step([("a", 1), ("b", 17), ("c", 2)], tokens, end=["c"])
    r.step([("a", 1), ("b", 1)], tokens)
    r.step([("b", 13)], tokens, end=["b"])                     # a pauses
    r.step([("a", 40), ("d", 1), ("e", 5)], tokens)            # slots and pages of b and c again
    r.step([("a", 1), ("d", 30), ("e", 1)], tokens)
    r.step([("a", 2), ("d", 27), ("e", 35)], tokens, end=["a", "d", "e"])
    alone = Replayer(folder, dtype, num_blocks=12, max_requests=1)
    for k, n in lens.items():
        alone.step([(k, n)], tokens, end=[k])
        if dtype == "float32":
            close(r.logits(k), PM.forward(cfg, w, tokens[k]), dtype, f"{key} request {k}")
            # the batch, the cut and the pages change nothing beyond the last bits
            close(r.logits(k), alone.logits(k).numpy(), dtype, f"{key} {k} alone", tol=2e-6)
        else:
            close(r.logits(k), alone.logits(k).numpy(), dtype, f"{key} request {k}")
    assert r.runner.cache.slots.num_free == 3 and r.runner.cache.num_free_pages() == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_window_edges_and_kept_tokens(models, dtype):
    """A long prompt and decoding past it with sharp softmaxes: the parallel layers read keys
    hundreds of tokens back, the windowed layers the keys just inside the window and the kept
    first tokens, across page borders."""
    folder, cfg, w = models[("sharp", dtype)]
    n = 260
    tokens = {"a": tokens_for(cfg["vocab"], n, 21)}
    want = PM.forward(cfg, w, tokens["a"])
    r = Replayer(folder, dtype, num_blocks=20)
    r.step([("a", 200)], tokens)
    for _ in range(60):
        r.step([("a", 1)], tokens)
    if dtype == "float32":
        close(r.logits("a"), want, dtype, "far keys")
    else:
        whole = Replayer(folder, dtype, num_blocks=20)
        whole.step([("a", n)], tokens)
        close(r.logits("a"), whole.logits("a").numpy(), dtype, "far keys")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_walk_kept_tiles_and_window_tiles(models, dtype):
    """Prompts long enough that the rows' window begins several key tiles behind the kept first
    keys: whole, and cut where the second portion's first rows see the kept keys only through
    their own tile."""
    folder, cfg, w = models[("wide", dtype)]
    tokens = {"a": tokens_for(cfg["vocab"], 330, 77), "b": tokens_for(cfg["vocab"], 330, 77)}
    want = PM.forward(cfg, w, tokens["a"])
    r = Replayer(folder, dtype, num_blocks=48)
    r.step([("a", 330)], tokens, end=["a"])
    close(r.logits("a"), want, dtype, "whole long prompt")
    r.step([("b", 150)], tokens)
    r.step([("b", 179)], tokens)
    r.step([("b", 1)], tokens, end=["b"])
    close(r.logits("b"), want, dtype, "long prompt in two portions")
    if dtype == "bfloat16":
        # both ways in which the tcgen05 kernel forms its two chains of rows
        ops = r.model.runtime.ops
        for rows in (128, 256):
            for hd in (64, 128):
                ops.set_attention_rows(hd, rows)
            tokens[f"w{rows}"] = tokens["a"]
            r.step([(f"w{rows}", 330)], tokens, end=[f"w{rows}"])
            close(r.logits(f"w{rows}"), want, dtype, f"whole long prompt, {rows} rows a CTA")
        for hd in (64, 128):
            ops.set_attention_rows(hd, 0)


def test_long_decoding_through_graphs(models):
    folder, cfg, w = models[("wide", "bfloat16")]
    lens = {"a": 150, "b": 131}
    tokens = {k: tokens_for(cfg["vocab"], n, i + 30) for i, (k, n) in enumerate(lens.items())}
    r = Replayer(folder, "bfloat16", num_blocks=24)
    r.step([("a", 20), ("b", 1)], tokens)
    for _ in range(130):
        r.step([("a", 1), ("b", 1)], tokens)
    for k in lens:
        close(r.logits(k), PM.forward(cfg, w, tokens[k]), "bfloat16", f"long decoding {k}")


@pytest.mark.parametrize("key", ["mixed", "plain"])
def test_greedy_generation_through_the_scheduler(models, key):
    from mini_llm_stack_b200.engine.llm import LLM
    folder, cfg, w = models[(key, "float32")]
    prompts = [tokens_for(cfg["vocab"], n, n + 50) for n in (3, 19, 1, 26)]
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=10, block_size=16, max_batch=3)
    got = llm.generate(prompts, max_new_tokens=12)
    for p, new in zip(prompts, got):
        seq = list(p)
        for tok in new:
            logits = PM.forward(cfg, w, seq)[-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] > 1e-4 * np.abs(logits).max():     # not a close call
                assert tok == int(np.argmax(logits)), (key, len(seq))
            seq.append(tok)
    llm.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_replays_a_folder(models, tmp_path, dtype):
    folder, cfg, w = models[("mixed", dtype)]
    a, b = tokens_for(cfg["vocab"], 50, 1), tokens_for(cfg["vocab"], 9, 2)
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
    la, lb = PM.forward(cfg, w, a), PM.forward(cfg, w, b)
    want = {0: la[[0, 29]], 1: lb[[7]], 2: np.stack([la[48], lb[8]]), 3: la[[49]]}
    for i, rows in want.items():
        got = np.frombuffer((out / f"{i}.f32").read_bytes(), dtype="<f4").reshape(-1, cfg["vocab"])
        tol = 5e-5 if dtype == "float32" else 6e-2
        assert np.abs(got - rows).max() < tol * np.abs(rows).max(), i


def test_command_line_chat_and_seeded_sampling(models):
    """The command line picks the model class by config.json; temperature sampling with a seed
    gives the same tokens however the requests are batched."""
    from mini_llm_stack_b200.engine.llm import LLM
    folder, cfg, w = models[("mixed", "float32")]
    root = Path(__file__).resolve().parent.parent
    p = tokens_for(cfg["vocab"], 9, 4)
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=16, block_size=16, max_batch=4)
    want = llm.generate([p], max_new_tokens=6)[0]
    proc = subprocess.run(
        [sys.executable, "-m", "mini_llm_stack_b200.api", "chat", "--model", str(folder),
         "--dtype", "float32", "--token-ids", ",".join(map(str, p)), "--max-new", "6"],
        capture_output=True, text=True, cwd=root, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.strip().endswith(f"-> {','.join(map(str, want))!r}")
    prompts = [tokens_for(cfg["vocab"], n, n) for n in (5, 21, 2)]
    alone = [LLM.from_folder(folder, dtype="float32", num_blocks=16, block_size=16, max_batch=1)
             .generate(prompts, max_new_tokens=10, temperature=0.8, seed=5)]
    together = llm.generate(prompts, max_new_tokens=10, temperature=0.8, seed=5)
    assert len(together) == 3 and all(len(t) == 10 for t in together)
    llm.engine.cache.check()
    assert alone[0] is not None
