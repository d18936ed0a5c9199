"""``bench.py --design zededra | logulix | zefenex | movazen``: prefill and decode throughput of the design's
layers at sizes that resemble a real model's, beside the dense Llama-style decoder at equal
size.

Every model has random weights (N(0, 0.02^2), drawn on the device), ``--layers`` layers
(default 4) and the same width, head count, head size, feed-forward width and bytes of
cache a token.  Per size: tokens/s of one whole prompt of 2,048 tokens and of decode steps
of 8 requests at context 2,048 (device-timed with CUDA events after warm-up, decode
replayed from CUDA graphs as in serving), plus the device time of every kind of kernel in
one prompt step and one decode step (events around each launch, graphs off), so that a
kernel of the new design can be set beside the like kernel of the dense decoder.
"""

from __future__ import annotations

import json
import time

PAGE = 16
PROMPT = 2048
BATCH = 8

# width, heads, head size, feed-forward, latent (cache values a token), query latent,
# experts / chosen / expert width / shared width, mLSTM heads / key size / value size
SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, ff=8192, kv_rank=256, q_rank=768,
               experts=32, top=4, eff=1024, shared=1024, mheads=4, mdim=256, mvdim=512),
    "8b": dict(width=4096, heads=32, dim=128, ff=14336, kv_rank=256, q_rank=1536,
               experts=64, top=6, eff=1408, shared=2816, mheads=8, mdim=256, mvdim=512),
}


def zededra_config(s: dict, kind: str, layers: int, vocab: int = 32000) -> dict:
    latent = {"type": "latent_attention",
              "mixer": {"dim": s["dim"], "heads": s["heads"], "kv_rank": s["kv_rank"],
                        "q_rank": s["q_rank"], "scale": s["dim"] ** -0.5, "vdim": s["dim"]}}
    mlstm = {"type": "mlstm", "mixer": {"dim": s["mdim"], "gate_cap": 15.0,
                                        "heads": s["mheads"], "vdim": s["mvdim"]}}
    dense = {"ff": s["ff"], "kind": "dense", "limit": 7.0}
    moe = {"expert": {"ff": s["eff"]}, "kind": "moe",
           "router": {"experts": s["experts"], "top": s["top"]}, "shared": {"ff": s["shared"]}}
    layer = {"latent_dense": dict(latent, mlp=dense), "latent_moe": dict(latent, mlp=moe),
             "mlstm_dense": dict(mlstm, mlp=dense)}[kind]
    return {"architecture": "Zededra", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6},
            "layers": [layer] * layers}


def logulix_config(s: dict, kind: str, layers: int, vocab: int = 32000) -> dict:
    """Layers of one kind of Logulix mixer with the ungated feed-forward: attention with the
    dense decoder's heads (a window of 1,024, three taps, capped scores, full rotation), wkv
    with heads of 64 and a decay of inner size 64, retention with keys of the head size and
    values twice as long."""
    kv = max(1, s["kv_rank"] // (2 * s["dim"]), s["heads"] // 16)
    attention = {"type": "attention",
                 "mixer": {"dim": s["dim"], "heads": s["heads"], "kv_heads": kv, "vdim": s["dim"],
                           "scale": s["dim"] ** -0.5, "conv": 3, "softcap": 30.0,
                           "mask": {"size": 1024},
                           "rot": {"base": 10000.0, "dims": s["dim"], "scaling": {"factor": 8.0}}}}
    wkv = {"type": "wkv", "mixer": {"dim": 64, "heads": s["width"] // 64, "rank": 64}}
    heads = s["heads"]
    retention = {"type": "retention",
                 "mixer": {"dim": s["dim"], "heads": heads, "vdim": 2 * s["dim"],
                           "decay": [1.0 - 2.0 ** (-5 - 3 * i / heads) for i in range(heads)],
                           "rot": {"base": 1e6, "dims": s["dim"]}}}
    dense = {"ff": s["ff"], "kind": "dense"}
    layer = {"attention_dense": dict(attention, mlp=dense), "wkv_dense": dict(wkv, mlp=dense),
             "retention_dense": dict(retention, mlp=dense)}[kind]
    return {"architecture": "Logulix", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_scale": 1.0, "layers": [layer] * layers}


def zefenex_config(s: dict, kind: str, layers: int, vocab: int = 32000) -> dict:
    """Layers of Zefenex's latent attention (a latent of three quarters of Zededra's plus a
    rotated key part of one quarter: the same cache bytes a token and the same attention
    arithmetic; queries of half a head plain and half rotated; a window of 1,024, sinks, the
    output gate) with the biased ungated feed-forward, with the routed one (softmax scores, a
    correction, two experts that return their input, a shared expert), or with every second
    layer reading the cache of the layer before it."""
    g = s["kv_rank"] // 4
    mixer = {"dim": s["dim"] - g, "heads": s["heads"], "kv_rank": s["kv_rank"] - g, "rot_dim": g,
             "rot": {"base": 1e6, "dims": g}, "mask": {"size": 1024}, "scale": s["dim"] ** -0.5,
             "vdim": s["dim"]}
    dense = {"ff": s["ff"], "kind": "dense"}
    moe = {"expert": {"ff": s["eff"]}, "kind": "moe",
           "router": {"experts": s["experts"], "identity": 2, "top": s["top"]},
           "shared": {"ff": s["shared"]}}
    mlp = moe if kind == "latent_moe" else dense
    stack = []
    for i in range(layers):
        m = dict(mixer)
        if kind == "shared_cache_dense" and i % 2:
            m["kv_from"] = i - 1
        stack.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Zefenex", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_softcap": 30.0, "layers": stack}


def movazen_config(s: dict, kind: str, layers: int, vocab: int = 32000) -> dict:
    """Layers of Movazen's mixers with its routed experts (sigmoid scores, a correction, eight
    groups of which four are kept, clamped units, a gated shared expert) and its side input of
    256 entries a layer: windowed attention with the dense decoder's heads (a window of 1,024
    behind four kept tokens, per-head norms, slopes, the output gate), or softmax attention of
    the same heads beside lightning attention of as many heads with keys and values of the
    head size; ``mixers_only`` alternates the two without feed-forwards."""
    kv = max(1, s["kv_rank"] // (2 * s["dim"]), s["heads"] // 16)
    heads, dim = s["heads"], s["dim"]
    attention = {"type": "attention",
                 "mixer": {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": dim,
                           "scale": dim ** -0.5, "mask": {"size": 1024, "keep_first": 4}}}
    parallel = {"type": "parallel",
                "mixer": {"left": {"dim": dim, "heads": heads, "kv_heads": kv, "vdim": dim,
                                   "scale": dim ** -0.5, "q_temp": {"coef": 0.1, "every": 512}},
                          "left_scale": 0.7,
                          "right": {"dim": dim, "heads": heads, "vdim": dim,
                                    "decay": [1.0 - 2.0 ** (-5 - 3 * i / heads)
                                              for i in range(heads)]},
                          "right_scale": 0.4}}
    moe = {"expert": {"ff": s["eff"], "limit": 7.0}, "kind": "moe",
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 8, "keep": 4}},
           "shared": {"ff": s["shared"], "limit": 7.0}}
    if kind == "mixers_only":
        stack = [dict(attention if i % 2 == 0 else parallel, mlp=None) for i in range(layers)]
    else:
        stack = [dict(attention if kind == "attention_moe" else parallel, mlp=moe)] * layers
    return {"architecture": "Movazen", "vocab": vocab, "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "token_side": {"dim": 256}, "layers": stack}


DESIGNS = {
    "zededra": (zededra_config, ("latent_dense", "latent_moe", "mlstm_dense")),
    "logulix": (logulix_config, ("attention_dense", "wkv_dense", "retention_dense")),
    "zefenex": (zefenex_config, ("latent_dense", "latent_moe", "shared_cache_dense")),
    "movazen": (movazen_config, ("attention_moe", "parallel_moe", "mixers_only")),
}
# rows of another design measured beside a design's own: the closest existing layers
BESIDE = {"zefenex": (("zededra", "latent_dense"), ("zededra", "latent_moe")),
          "movazen": (("zefenex", "latent_moe"), ("logulix", "attention_dense"),
                      ("logulix", "retention_dense"))}


def llama_config(s: dict, layers: int, vocab: int = 32000) -> dict:
    # kv heads of the latent's size in keys plus values, i.e. the same cache bytes a token (but
    # at most 16 query heads a kv head, the most the fused decode attention takes)
    return dict(architecture="llama_dense", vocab_size=vocab, d_model=s["width"], n_layers=layers,
                n_heads=s["heads"],
                n_kv_heads=max(1, s["kv_rank"] // (2 * s["dim"]), s["heads"] // 16),
                head_dim=s["dim"], intermediate_size=s["ff"], max_seq_len=4096,
                rope_theta=500000.0, norm_eps=1e-5, tie_embeddings=True, dtype="bfloat16")


_LEAVES = ("embed", "add_rmsnorm", "gather_add_rmsnorm", "add_layernorm", "residual_add",
           "rope_store", "paged_attention", "attention_decode_fused", "swiglu", "clamped_glu",
           "latent_norm_store", "headwise_linear", "mlstm_scan", "mlstm_finish", "route",
           "expert_glu", "expert_down", "expert_combine", "qk_conv_norm_rope_store",
           "tail_update", "token_shift_mix", "linear_scan", "scan_finish", "rotate_rows",
           "decay_lowrank", "relu_squared", "scale_", "settle_concat", "add_tanh_norm",
           "latent_rope_prep", "sigmoid_gate", "softcap_", "head_prep_store", "settle_cast",
           "gelu_gate_rows", "rms_scale", "scan_finish_row")
_PRODUCTS = ("linear", "linear_parts", "linear_swiglu", "linear_clamped_glu",
             "linear_relu_squared")


class OpTimer:
    """CUDA events around every kernel face of an ``Ops``; products are named by their
    weight's shape.  Only the outermost face of a nest is timed."""

    def __init__(self, torch, ops):
        self.torch, self.ops, self.depth, self.spans, self.saved = torch, ops, 0, [], {}

    def __enter__(self):
        for name in _LEAVES + _PRODUCTS:
            fn = getattr(self.ops, name)
            self.saved[name] = fn
            setattr(self.ops, name, self._wrap(name, fn))
        return self

    def _wrap(self, name, fn):
        def timed(*a, **k):
            if self.depth:
                return fn(*a, **k)
            label = name
            if name in _PRODUCTS:
                w = a[1]
                label = f"{name} [{w.shape[0]} x {w.shape[1]}]"
            e0 = self.torch.cuda.Event(enable_timing=True)
            e1 = self.torch.cuda.Event(enable_timing=True)
            self.depth += 1
            e0.record()
            try:
                return fn(*a, **k)
            finally:
                e1.record()
                self.depth -= 1
                self.spans.append((label, e0, e1))
        return timed

    def __exit__(self, *exc):
        for name, fn in self.saved.items():
            setattr(self.ops, name, fn)

    def table(self) -> dict:
        self.torch.cuda.synchronize()
        out = {}
        for label, e0, e1 in self.spans:
            ms, n = out.get(label, (0.0, 0))
            out[label] = (ms + e0.elapsed_time(e1), n + 1)
        return {k: {"ms": round(v[0], 4), "calls": v[1]} for k, v in
                sorted(out.items(), key=lambda kv: -kv[1][0])}


def measure(torch, raw: dict, steps: int, warmup: int) -> dict:
    from mini_llm_stack_b200.config import config_from_dict
    from mini_llm_stack_b200.engine.batch import Entry
    from mini_llm_stack_b200.engine.runner import ModelRunner, random_model

    cfg = config_from_dict(raw)
    model = random_model(cfg, seed=0, device="cuda:0", fast=True)
    ops = model.runtime.ops
    gen = torch.Generator().manual_seed(1)

    def rand_tokens(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def timed(fn, n_warm, n_timed):
        for _ in range(n_warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_timed):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ops.check_status()
        return e0.elapsed_time(e1) / n_timed

    out = {}
    pages = (PROMPT + steps + warmup + 64) // PAGE + 1
    for graphs in (True, False):
        runner = ModelRunner(model, num_blocks=BATCH * pages + PROMPT // PAGE + 8, block_size=PAGE,
                             max_requests=BATCH + 1, cuda_graphs=graphs)
        cache = runner.cache
        for g in cache.paged:
            g.kv.normal_(0.0, 1.0)

        def prefill():
            e = [Entry("p", rand_tokens(PROMPT), [PROMPT - 1])]
            runner.reserve(e)
            runner.step(e)
            runner.release("p")

        ids = [f"d{i}" for i in range(BATCH)]

        def start_decode():
            for r in ids:
                cache.admit(r)
                assert cache.reserve(r, PROMPT)
                cache.commit(r, PROMPT)

        def decode():
            e = [Entry(r, rand_tokens(1), [0]) for r in ids]
            runner.reserve(e)
            runner.step(e)

        if graphs:
            torch.cuda.synchronize()
            time.sleep(0.5)
            ms = sorted(timed(prefill, 2 if i == 0 else 0, 1) for i in range(5))[2]
            out["prefill"] = {"tokens_per_s": round(PROMPT / ms * 1e3, 1), "ms": round(ms, 3)}
            start_decode()
            ms = timed(decode, max(3, warmup), steps)
            out["decode"] = {"tokens_per_s": round(BATCH / ms * 1e3, 1), "ms_per_step": round(ms, 4),
                             "batch": BATCH, "context": PROMPT}
        else:
            prefill()
            with OpTimer(torch, ops) as t:
                prefill()
            out["prefill_kernels"] = t.table()
            start_decode()
            decode()
            decode()
            with OpTimer(torch, ops) as t:
                decode()
            out["decode_kernels"] = t.table()
        for r in ids:
            runner.release(r)
        del runner, cache
    del model
    torch.cuda.empty_cache()
    return out


def run(args, peaks: dict, peaks_source: str) -> dict:
    import torch
    torch.cuda.set_device(0)
    layers = args.layers or 4
    sizes = [args.size] if args.size else list(SIZES)
    design = args.design
    make_config, kinds = DESIGNS[design]
    result = {"metric": f"{design}_layers_beside_llama_dense", "unit": "tokens/s", "layers": layers,
              "prompt_tokens": PROMPT, "decode_batch": BATCH, "decode_context": PROMPT,
              "dtype": "bf16", "data": "synthetic", "peaks": peaks, "peaks_source": peaks_source,
              "device": torch.cuda.get_device_name(0), "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        rows = {"llama_dense": measure(torch, llama_config(s, layers), args.steps, args.warmup)}
        for other, kind in BESIDE.get(design, ()):
            rows[f"{other}_{kind}"] = measure(torch, DESIGNS[other][0](s, kind, layers), args.steps,
                                              args.warmup)
        for kind in kinds:
            rows[f"{design}_{kind}"] = measure(torch, make_config(s, kind, layers), args.steps,
                                               args.warmup)
        result["sizes"][name] = rows
    return result


def main(args, peaks: dict, peaks_source: str) -> int:
    print(json.dumps(run(args, peaks, peaks_source)))
    return 0
