"""Tiny Movazen configurations and helpers for the tests.

Sizes are chosen so that nothing the engine could confuse is equal: query, key and value
sizes, head counts and group sizes differ between layers and between the halves of a parallel
mixer; head sizes fall on and off the kernels' multiples of 16; windows are shorter than a
page, between pages and longer than the prompts, with kept first tokens inside one page, past
a page's edge, or none; routers choose one, two or three experts with and without groups and
shared expert; layers have no feed-forward; the side input's width is and is not a multiple of
eight, or absent; widths are no multiple of eight.
"""

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import random_tensors


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return {"type": "attention", "mixer": m}


def parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, scale, temp = left
    lm = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if temp is not None:
        lm["q_temp"] = {"coef": temp[0], "every": temp[1]}
    rheads, rdim, rvdim, decay = right
    rm = {"decay": list(decay), "dim": rdim, "heads": rheads, "vdim": rvdim}
    return {"type": "parallel", "mixer": {"left": lm, "left_scale": left_scale, "right": rm,
                                          "right_scale": right_scale}}


def moe(experts, top, ff, limit, groups=None, shared=None):
    out = {"expert": {"ff": ff, "limit": limit}, "kind": "moe",
           "router": {"experts": experts, "top": top}}
    if groups:
        out["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mixer, mlp=None):
    return dict(mixer, mlp=mlp)


# every mechanism, nothing equal to anything else
M_MIXED = {
    "architecture": "Movazen", "vocab": 97, "width": 40, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.5}, "token_side": {"dim": 6},
    "layers": [
        layer(attention(4, 2, 12, 20, 0.3, window=21, keep_first=3),
              moe(6, 2, 24, 1.2, groups=(3, 2), shared=(16, 0.8))),
        layer(parallel((2, 1, 16, 8, 0.25, (0.4, 16)), (3, 8, 12, (0.6, 0.9, 0.99)), 0.7, 0.4)),
        layer(attention(3, 3, 16, 16, 0.2, window=40, keep_first=17), moe(4, 1, 20, 2.0)),
        layer(parallel((4, 4, 8, 24, 0.35, None), (1, 20, 4, (0.95,)), 0.5, 1.2),
              moe(8, 3, 16, 0.9, groups=(4, 2), shared=(24, 1.5))),
    ],
}

# no side input, no embedding scale, a width that is no multiple of eight, attention without a
# window, a window without kept tokens, a router that takes every expert of its kept group
M_PLAIN = {
    "architecture": "Movazen", "vocab": 53, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        layer(attention(2, 1, 10, 6, 0.4), moe(4, 2, 12, 1.0, groups=(2, 1))),
        layer(parallel((3, 1, 4, 12, 0.5, (0.2, 5)), (2, 6, 10, (0.8, 0.97)), 1.0, 1.0),
              moe(2, 2, 8, 3.0, shared=(12, 1.0))),
        layer(attention(6, 2, 8, 8, 0.3, window=5)),
    ],
}

# head sizes of 64 and 128 and a side input of a whole 16-byte row: the sizes at which the
# bfloat16 run takes its tensor-core paths
M_WIDE = {
    "architecture": "Movazen", "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"scale": 4.0}, "token_side": {"dim": 16},
    "layers": [
        layer(attention(4, 2, 64, 48, 0.125, window=70, keep_first=20),
              moe(8, 2, 64, 1.25, groups=(4, 2), shared=(80, 0.9))),
        layer(parallel((4, 2, 64, 64, 0.11, (0.25, 32)), (2, 32, 64, (0.9, 0.995)), 0.7, 0.45),
              moe(4, 2, 32, 2.5)),
        layer(attention(2, 1, 128, 128, 0.09, window=33, keep_first=1)),
    ],
}


def one_layer(mixer_layer, mlp=None, width: int = 40, vocab: int = 61, eps: float = 1e-5,
              **top) -> dict:
    """A model of the embedding, one layer, the final norm and the head."""
    return dict({"architecture": "Movazen", "vocab": vocab, "width": width, "norm": {"eps": eps},
                 "layers": [layer(mixer_layer, mlp)]}, **top)


def decisive_routers(w, raw: dict):
    """Make every router's choice rest on its correction: an uneven ladder of corrections over
    scores that barely move with the token, drawn again until every expert and every group's
    score (the sum of its two largest) stands a fifth of a score or more from the next.  Groups
    and experts are then taken by clear margins (no close call that a 16-bit rounding could
    turn), while the weights of the chosen experts still follow the token's scores."""
    for i, layer in enumerate(raw["layers"]):
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        e = mlp["router"]["experts"]
        count = (mlp["router"].get("groups") or {}).get("count", 1)
        g = torch.Generator().manual_seed(100 + i)
        while True:
            c = 0.3 * torch.randperm(e, generator=g).double() + 0.1 * torch.rand(e, generator=g).double()
            sums = [c[k * (e // count):(k + 1) * (e // count)].sort(descending=True).values[:2].sum()
                    for k in range(count)]
            gaps = [abs(float(a - b)) for k, a in enumerate(sums) for b in sums[k + 1:]]
            if not gaps or min(gaps) >= 0.2:
                break
        w[f"l{i}.mlp.correction"] = c.float()
        w[f"l{i}.mlp.router"] *= 0.08


def make_movazen(folder, raw: dict, seed: int, dtype: str = "bfloat16", std: float = 0.15,
                 norm_std: float = 0.1, patch=None):
    """Write a model folder; returns the config as stored and float64 numpy weights as the
    file holds them.

    Matrices are drawn with a larger deviation than the engine's default so that every
    mechanism moves the logits; biases, router corrections and routers get values of their
    own kind; ``patch(weights)`` may change tensors before they are stored (in the stored
    dtype's rounding)."""
    cfg = config_from_dict(dict(raw, dtype=dtype))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed + 1000)
    w = {}
    for name, t in random_tensors(cfg, seed, norm_std, dtype="float32"):
        if name.endswith(".correction"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith(".router") or name.endswith(".sg"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif name.endswith("norm1") or name.endswith("norm2") or name == "final.norm":
            t = torch.randn(t.shape, generator=g) * norm_std       # stored around zero
        elif name == "side.embed":
            t = torch.randn(t.shape, generator=g)
        elif t.dim() == 2:
            t = torch.randn(t.shape, generator=g) * std
        w[name] = t
    if patch:
        patch(w)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = {n: t.to(store).contiguous() for n, t in w.items()}
    save_file(w, str(folder / "model.safetensors"))
    stored = cfg.to_dict()
    (folder / "config.json").write_text(json.dumps(stored, indent=1))
    return stored, {n: t.double().numpy() for n, t in w.items()}
