"""A plain, slow Zefenex on whole sequences: one function per mechanism.

Written from the design's equations with torch tensor algebra only; it shares no
code with the engine.  Everything runs in the dtype of the weights it is given
(float64 for an oracle); ``tokens`` is one sequence.  ``rnd`` (identity by default)
is applied to every activation a 16-bit engine would store: with ``to_bf16`` the
functions show how far rounding alone moves a result.

Notation: d = model width, H = heads, e = unrotated and g = rotated query/key size
of a head, f = value size of a head, r = latent size, eps = the model's epsilon.
"""

import math

import torch


def ident(t):
    return t


def to_bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


# --------------------------------------------------------------------------- norms
def plain_tanh_norm(x, w, name):
    """tanh(alpha x) * weight + bias: no mean, no variance."""
    return torch.tanh(w[f"{name}.alpha"] * x) * w[name] + w[f"{name}.b"]


def plain_unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------ rotation
def plain_rotate_half(x, positions, dims, base):
    """The first ``dims`` entries of the last axis turn: entry i with entry i + dims/2
    by the angle position * base^(-2i/dims); the rest stay.  x: [S, ..., n]."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = ang.cos().to(x.dtype).view(shape), ang.sin().to(x.dtype).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------ attention
def plain_latent_kv(h, w, p, m, eps, positions, rnd=ident):
    """What a layer with a down projection of its own caches for every token: the
    normalised latent c [S, r] and the rotated key part shared by all heads [S, g]."""
    r, g = m["kv_rank"], m["rot_dim"]
    down = h @ w[f"{p}.dkv"].T
    c = rnd(plain_unit_rms(down[:, :r], eps) * w[f"{p}.dkv.norm"])
    rot = m.get("rot") or {}
    kr = rnd(plain_rotate_half(down[:, r:r + g], positions, rot.get("dims", 0),
                               rot.get("base", 1.0)))
    return c, kr


def plain_sink_softmax(s, hidden, sink):
    """Softmax over the visible keys of s [H, S, S] whose denominator also holds
    exp(sink_h): a term without key or value."""
    s = s.masked_fill(hidden, float("-inf"))
    top = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    ex = torch.exp(s - top)
    return ex / (ex.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def plain_latent_attention(h, w, p, m, c, kr, positions, rnd=ident):
    """Heads of [e unrotated | g rotated] queries against keys [W_uk c | shared rotated
    part], values W_uv c, a window, a sink in the softmax and a sigmoid gate on the
    heads' outputs before W_o.  ``c``, ``kr``: the cached latent and rotated key part
    (this layer's own or another layer's)."""
    S = h.shape[0]
    H, e, g, f = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    rot = m.get("rot") or {}
    q = rnd(h @ w[f"{p}.q"].T).view(S, H, e + g)
    q_plain = q[..., :e]
    q_rot = rnd(plain_rotate_half(q[..., e:], positions, rot.get("dims", 0), rot.get("base", 1.0)))
    k = rnd(c @ w[f"{p}.uk"].T).view(S, H, e)
    v = rnd(c @ w[f"{p}.uv"].T).view(S, H, f)
    s = (torch.einsum("ihe,jhe->hij", q_plain, k) + torch.einsum("ihg,jg->hij", q_rot, kr)) * m["scale"]
    i = torch.arange(S)
    dist = i[:, None] - i[None, :]
    hidden = dist < 0
    if m.get("mask"):
        hidden = hidden | (dist >= m["mask"]["size"])
    a = plain_sink_softmax(s, hidden, w[f"{p}.sink"].to(h.dtype))
    o = rnd(torch.einsum("hij,jhf->ihf", a, v).reshape(S, H * f))
    o = rnd(o * torch.sigmoid(rnd(h @ w[f"{p}.g"].T)))
    return rnd(o @ w[f"{p}.o"].T)


# --------------------------------------------------------------------- feed-forwards
def plain_relu2_unit(h, w, p, rnd=ident):
    """W_down relu(W_up h + b_up)^2 + b_down."""
    z = torch.relu(h @ w[f"{p}.up"].T + w[f"{p}.up.b"])
    return rnd(rnd(z * z) @ w[f"{p}.down"].T + w[f"{p}.down.b"])


def plain_silu_unit(h, w, p, rnd=ident):
    """W_down (silu(W_gate h) * (W_up h)), no biases."""
    g = h @ w[f"{p}.gate"].T
    return rnd(g * torch.sigmoid(g) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def plain_route(h, w, p, router, flip_below=0.0):
    """Softmax scores over all router outputs; the ``top`` with the largest score +
    correction (lowest index on ties); weights = the chosen scores (without the
    correction) over their sum.  ``flip_below``: where the last chosen output leads the
    first one left out by less than this, the other one is taken (what an engine may do
    whose activations are rounded: the choice is a close call)."""
    s = torch.softmax(h @ w[f"{p}.router"].to(h.dtype).T, dim=-1)
    choice = s + w[f"{p}.correction"].to(h.dtype)
    order = torch.sort(choice, dim=-1, descending=True, stable=True)
    top = router["top"]
    idx = order.indices[:, :top].clone()
    if flip_below and top < choice.shape[1]:
        close = (order.values[:, top - 1] - order.values[:, top]) < flip_below
        idx[close, top - 1] = order.indices[close, top]
    val = torch.gather(s, 1, idx)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20)


def plain_routed_experts(h, w, p, mlp, rnd=ident, flip_below=0.0):
    """Weighted sum of the chosen experts' outputs; the last ``identity`` router outputs
    stand for experts that return their input; a shared expert is added for every token."""
    router = mlp["router"]
    n_real = router["experts"]
    idx, val = plain_route(h, w, p, router, flip_below)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(router["top"]):
            ex = int(idx[t, j])
            y = h[t] if ex >= n_real else plain_silu_unit(h[t][None], w, f"{p}.e{ex}", rnd)[0]
            out[t] += val[t, j] * y
    if mlp.get("shared"):
        out = out + plain_silu_unit(h, w, f"{p}.shared", rnd)
    return rnd(out)


def plain_feedforward(h, w, p, mlp, rnd=ident, flip_below=0.0):
    if mlp["kind"] == "dense":
        return plain_relu2_unit(h, w, p, rnd)
    return plain_routed_experts(h, w, p, mlp, rnd, flip_below)


# ----------------------------------------------------------------------------- model
def plain_zefenex(w, cfg, tokens, trace=None, rnd=ident, first_position=0, flip_below=0.0):
    """Logits [S, vocab] of one whole sequence; ``trace`` (a list) receives the residual
    stream after every layer; ``flip_below``: see ``plain_route``."""
    eps = cfg["norm"]["eps"]
    positions = list(range(first_position, first_position + len(tokens)))
    x = w["embed"][torch.as_tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    cached = {}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}.mix"
        h = rnd(plain_tanh_norm(x, w, f"l{i}.norm1"))
        if m.get("kv_from") is None:
            cached[i] = plain_latent_kv(h, w, p, m, eps, positions, rnd)
        c, kr = cached[i if m.get("kv_from") is None else m["kv_from"]]
        y = plain_latent_attention(h, w, p, m, c, kr, positions, rnd)
        x = x + plain_tanh_norm(y, w, f"l{i}.norm1b") * w[f"l{i}.ls1"]
        if L.get("mlp"):
            h = rnd(plain_tanh_norm(x, w, f"l{i}.norm2"))
            y = plain_feedforward(h, w, f"l{i}.mlp", L["mlp"], rnd, flip_below)
            x = x + plain_tanh_norm(y, w, f"l{i}.norm2b") * w[f"l{i}.ls2"]
        if trace is not None:
            trace.append(x)
    logits = rnd(plain_tanh_norm(x, w, "final.norm")) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
