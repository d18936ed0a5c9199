"""A plain, slow Movazen in float64 numpy: one function per mechanism, whole sequences only,
loops over tokens, heads and keys.  It shares no code with the engine; the tests hold the
engine against it.

A model is ``(config dict, {tensor name: float64 array})``; ``forward`` returns the logits of
every position and, on request, the residual stream after every layer.
"""

from __future__ import annotations

import math

import numpy as np

RENORM_EPS = 1e-20
GATE_ALPHA = 1.702


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def model_norm(x, w, eps):
    """The model's norm: its weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def sinusoid(position: int, width: int):
    """Entry c of the position vector: sine (c even) or cosine (c odd) of
    position * 10000^(-2 (c // 2) / width)."""
    out = np.zeros(width)
    for c in range(width):
        angle = position * 10000.0 ** (-2.0 * (c // 2) / width)
        out[c] = math.sin(angle) if c % 2 == 0 else math.cos(angle)
    return out


def embed(tokens, table, scale, width):
    return np.stack([table[t] * scale + sinusoid(p, width) for p, t in enumerate(tokens)])


def distance_slopes(n_heads: int):
    return [2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)]


def visible(i: int, j: int, window, keep_first) -> bool:
    """Whether the query at i sees the key at j: causal, inside the window or among the
    sequence's first tokens (no window: every earlier key)."""
    if j > i:
        return False
    if window is None:
        return True
    return i - j < window or j < (keep_first or 0)


def softmax_attention(q, k, v, scale, slopes=None, window=None, keep_first=0, sink=False):
    """q [T, H, e], k [T, G, e], v [T, G, f] -> [T, H, f].  ``slopes``: the score loses
    slope_h * (i - j).  ``sink``: one more term exp(0) in the denominator, without a value."""
    t, n_heads, _ = q.shape
    group = n_heads // k.shape[1]
    out = np.zeros((t, n_heads, v.shape[2]))
    for h in range(n_heads):
        g = h // group
        for i in range(t):
            js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
            s = np.array([float(q[i, h] @ k[j, g]) * scale
                          - (slopes[h] * (i - j) if slopes is not None else 0.0) for j in js])
            m = max(s.max(), 0.0) if sink else s.max()
            w = np.exp(s - m)
            den = w.sum() + (math.exp(-m) if sink else 0.0)
            out[i, h] = (w[:, None] * np.stack([v[j, g] for j in js])).sum(0) / den
    return out


def attention_mixer(h, w, m, eps):
    """The mixer 'attention': per-head norms of q and k, distance bias, window with kept
    first tokens, sigmoid gate on the heads' outputs."""
    t = h.shape[0]
    nh, g, e, f = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(t, nh, e)
    k = (h @ w["k"].T).reshape(t, g, e)
    v = (h @ w["v"].T).reshape(t, g, f)
    q = unit_rms(q, eps) * w["q.norm"]
    k = unit_rms(k, eps) * w["k.norm"]
    mask = m.get("mask") or {}
    o = softmax_attention(q, k, v, m["scale"], slopes=distance_slopes(nh),
                          window=mask.get("size"), keep_first=mask.get("keep_first", 0))
    o = o.reshape(t, nh * f) * sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def query_temperature(position: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((position + 1) // every + 1)


def biased_sink_attention(h, w, m):
    """The left half of 'parallel': biased projections, query temperature, causal softmax
    with one added to its denominator."""
    t = h.shape[0]
    nh, g, e, f = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(t, nh, e)
    k = (h @ w["k"].T + w["k.b"]).reshape(t, g, e)
    v = (h @ w["v"].T + w["v.b"]).reshape(t, g, f)
    temp = m.get("q_temp")
    if temp is not None:
        for p in range(t):
            q[p] *= query_temperature(p, temp["coef"], temp["every"])
    o = softmax_attention(q, k, v, m["scale"], sink=True)
    return o.reshape(t, nh * f) @ w["o"].T


def lightning_attention(h, w, m, eps):
    """The right half of 'parallel': a matrix state a head with a constant decay."""
    t = h.shape[0]
    nh, e, f = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(t, nh, e)
    k = silu(h @ w["k"].T).reshape(t, nh, e)
    v = silu(h @ w["v"].T).reshape(t, nh, f)
    o = np.zeros((t, nh, f))
    for head in range(nh):
        state = np.zeros((e, f))
        for i in range(t):
            state = m["decay"][head] * state + np.outer(k[i, head], v[i, head])
            o[i, head] = state.T @ q[i, head]
    y = unit_rms(o.reshape(t, nh * f), eps) * w["norm"]
    return (y * sigmoid(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = biased_sink_attention(h, sub(w, "left"), m["left"])
    right = lightning_attention(h, sub(w, "right"), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def clamped_unit(h, w, limit):
    g = np.minimum(h @ w["gate"].T, limit)
    u = np.clip(h @ w["up"].T, -limit, limit)
    return (g * sigmoid(GATE_ALPHA * g) * (u + 1.0)) @ w["down"].T


def choose_experts(choice, top: int, groups=None, margins=None):
    """Indices of the ``top`` largest choice scores (lowest index on a tie) among the
    experts of the best groups: a group's score is the sum of its two largest choice scores.
    ``margins`` (a list) receives the gap between the last kept and the first refused group's
    score and the gap between the last chosen and the first refused expert's choice score."""
    choice = np.array(choice, dtype=np.float64)
    n = len(choice)
    allowed = np.ones(n, dtype=bool)
    if groups is not None:
        size = n // groups["count"]
        score = []
        for gi in range(groups["count"]):
            part = sorted(choice[gi * size:(gi + 1) * size], reverse=True)
            score.append(sum(part[:2]))
        ranked = sorted(range(groups["count"]), key=lambda gi: (-score[gi], gi))
        best = ranked[:groups["keep"]]
        if margins is not None and len(ranked) > groups["keep"]:
            margins.append(score[best[-1]] - score[ranked[groups["keep"]]])
        allowed[:] = False
        for gi in best:
            allowed[gi * size:(gi + 1) * size] = True
    order = sorted((i for i in range(n) if allowed[i]), key=lambda i: (-choice[i], i))
    if margins is not None and len(order) > top:
        margins.append(choice[order[top - 1]] - choice[order[top]])
    return order[:top]


def routed_experts(h, w, mlp, margins=None):
    """Mixture of clamped units behind a sigmoid router with a correction for the choice,
    groups, renormalised weights and a gated shared expert.  ``margins`` (a list) collects,
    per token, the smallest gap by which a group or an expert was taken over the next one."""
    router = mlp["router"]
    n, top = router["experts"], router["top"]
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        s = sigmoid(w["router"] @ h[i])
        choice = s + w["correction"]
        gaps = []
        chosen = choose_experts(choice, top, router.get("groups"), gaps)
        if margins is not None:
            margins.append(min(gaps) if gaps else np.inf)
        total = sum(s[j] for j in chosen) + RENORM_EPS
        for j in chosen:
            out[i] += (s[j] / total) * clamped_unit(h[i], sub(w, f"e{j}"), mlp["expert"]["limit"])
        if mlp.get("shared") is not None:
            sw = sub(w, "shared")
            out[i] += sigmoid(float(sw["sg"][0] @ h[i])) * clamped_unit(h[i], sw,
                                                                        mlp["shared"]["limit"])
    return out


def token_side_input(x, tokens, w, table, layer: int, dim: int, eps):
    """What a layer adds at its end from the token's own side vector."""
    e = np.stack([table[t, layer * dim:(layer + 1) * dim] for t in tokens])
    g = gelu_tanh(x @ w["gate"].T) * e
    y = g @ w["proj"].T
    return unit_rms(y, eps) * w["norm"]


def sub(tensors: dict, prefix: str) -> dict:
    return {n[len(prefix) + 1:]: t for n, t in tensors.items() if n.startswith(prefix + ".")}


def forward(config: dict, tensors: dict, tokens, want_layers: bool = False, margins=None):
    eps = config["norm"]["eps"]
    width = config["width"]
    scale = (config.get("embedding") or {}).get("scale", 1.0)
    x = embed(tokens, tensors["embed"], scale, width)
    side = config.get("token_side")
    after = []
    for i, layer in enumerate(config["layers"]):
        w = sub(tensors, f"l{i}")
        h = model_norm(x, w["norm1"], eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, sub(w, "mix"), layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, sub(w, "mix"), layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h = model_norm(x, w["norm2"], eps)
            x = x + routed_experts(h, sub(w, "mlp"), layer["mlp"], margins)
        if side is not None:
            x = x + token_side_input(x, tokens, sub(w, "side"), tensors["side.embed"], i,
                                     side["dim"], eps)
        after.append(x.copy())
    logits = model_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    return (logits, np.stack(after)) if want_layers else logits
