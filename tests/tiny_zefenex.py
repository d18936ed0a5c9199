"""Tiny Zefenex configurations and helpers for the tests.

Sizes are chosen so that nothing the engine could confuse is equal: heads, plain, rotated
and value sizes and latents differ between layers; latents plus rotated parts fall on and
off the attention kernels' head sizes; windows are shorter than a page, between pages,
longer than the prompts, or absent; a layer that reads another layer's cache has a wider or
a narrower window than the layer that fills it; routers choose one, two or three outputs
among experts with and without experts that return their input, with and without a shared
expert; layers have no feed-forward at all; widths are no multiple of eight.
"""

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import random_tensors


def latent(heads, dim, rot_dim, vdim, rank, scale, window=None, base=None, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot_dim": rot_dim, "scale": scale,
         "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
    if base is not None:
        m["rot"] = {"base": base, "dims": rot_dim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, identity=0, shared=None):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if identity:
        out["router"]["identity"] = identity
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp=None):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# two caches, each read by a second layer; the reader of the first sees further back than
# the layer that fills it, the reader of the second less far; every feed-forward kind
Z_MIXED = {
    "architecture": "Zefenex", "vocab": 97, "width": 40, "norm": {"eps": 1e-5},
    "embedding": {"scale": 3.0}, "logit_softcap": 6.0,
    "layers": [
        layer(latent(3, 12, 8, 10, 20, 0.3, window=21, base=500.0), dense(72)),
        layer(latent(2, 6, 8, 14, 20, 0.4, window=33, base=500.0, kv_from=0),
              moe(5, 2, 24, identity=2, shared=16)),
        layer(latent(4, 16, 4, 8, 12, 0.25, base=50.0), None),
        layer(latent(1, 20, 4, 24, 12, 0.35, window=7, base=50.0, kv_from=2), moe(3, 1, 20)),
    ],
}

# no cap on the logits, no scale on the embedding, a width that is no multiple of eight, no
# window anywhere, a router that takes every output it has
Z_PLAIN = {
    "architecture": "Zefenex", "vocab": 53, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        layer(latent(2, 10, 6, 5, 9, 0.3, base=10000.0), moe(2, 3, 12, identity=1)),
        layer(latent(3, 4, 2, 12, 30, 0.5, base=7.0), dense(44)),
        layer(latent(5, 8, 6, 4, 9, 0.2, base=10000.0, kv_from=0), None),
    ],
}

# latent + rotated part = 128 and 64: bfloat16 runs go through the tensor-core attention
# kernels (prompts on tcgen05, decoded tokens on the context-split kernel)
Z_WIDE = {
    "architecture": "Zefenex", "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"scale": 11.3}, "logit_softcap": 20.0,
    "layers": [
        layer(latent(4, 32, 32, 48, 96, 0.125, window=70, base=1e6), dense(192)),
        layer(latent(2, 64, 32, 32, 96, 0.1, window=100, base=1e6, kv_from=0),
              moe(8, 3, 64, identity=2, shared=96)),
        layer(latent(4, 48, 16, 64, 48, 0.12, window=16, base=1e4), moe(4, 2, 32, shared=64)),
    ],
}


def one_layer(mixer, mlp=None, width: int = 40, vocab: int = 61, eps: float = 1e-5, **top) -> dict:
    """A model of the embedding, one layer, the final norm and the head."""
    return dict({"architecture": "Zefenex", "vocab": vocab, "width": width, "norm": {"eps": eps},
                 "layers": [layer(mixer, mlp)]}, **top)


def make_zefenex(folder, raw: dict, seed: int, dtype: str = "bfloat16", std: float = 0.12,
                 norm_std: float = 0.1, patch=None):
    """Write a model folder; returns float64 weights as the file holds them.

    Matrices are drawn with a larger deviation than the engine's default so that every
    mechanism moves the logits; biases, sinks, router corrections, the norms' alphas and the
    layer scales get values of their own kind; ``patch(weights)`` may change tensors before
    they are stored (in the stored dtype's rounding)."""
    cfg = config_from_dict(dict(raw, dtype=dtype))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed + 1000)
    w = {}
    for name, t in random_tensors(cfg, seed, norm_std, dtype="float32"):
        if name.endswith(".alpha"):
            t = torch.rand(t.shape, generator=g) * 0.8 + 0.4
        elif name.endswith(".sink"):
            t = torch.randn(t.shape, generator=g) * 1.5
        elif name.endswith(".correction"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith(".router"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith(".ls1") or name.endswith(".ls2"):
            t = torch.rand(t.shape, generator=g) + 0.5
        elif name.endswith(".uk") or name.endswith(".uv"):
            t = torch.randn(t.shape, generator=g) * 0.4
        elif t.dim() == 2:
            t = torch.randn(t.shape, generator=g) * std
        w[name] = t
    if patch:
        patch(w)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = {n: t.to(store).contiguous() for n, t in w.items()}
    save_file(w, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    return {n: t.double() for n, t in w.items()}
