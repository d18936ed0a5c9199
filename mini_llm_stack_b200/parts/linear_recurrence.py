"""Mixers that carry a matrix state per head from token to token: wkv and retention.

Both keep ``S [e, f]`` per head (key size e, value size f) in the request's state slot
(``FixedState``, float32, zero when the slot is claimed) and walk a step's tokens through
it with the same scan kernel; a portion of a prompt continues from the slot's state, so
cutting a prompt changes no bit.

wkv (e = f), with h' the previous token's h (zeros before the first; kept in the slot):
    mix_s = h + (h' - h) * mu_s          for s in r, k, v, g, w
    r, k, v = W_r mix_r, W_k mix_k, W_v mix_v;   gate = silu(W_g mix_g)
    w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))            float32, per head and key channel
    o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(w_t) S + k_t v_t^T
    out = W_o (o / rms_per_head(o) * g_norm * gate)

retention:
    q, k = rot(W_q h), rot(W_k h) * e^-1/2   (``PartialRotary``, "half" pairing; float32)
    S <- decay_head S + k_t v_t^T;   o_t = S^T q_t
    out = W_o (o / rms_per_head(o) * silu(W_g h))

The decay's products, the mixes that feed them, decays, states, rotations and the head
norms are float32 in both run types; the other projections run in the activation type.
"""

from __future__ import annotations

import torch

from .base import CacheHandle, FixedState, Mixer, StepContext, TensorSpec


class WkvMixer(Mixer):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream
    MIXES = ("r", "k", "v", "g", "w")
    STACK_ROWS = 64       # up to so many rows (four a token) the four projections run as one product

    def __init__(self, d_model: int, n_heads: int, head_dim: int, decay_rank: int, eps: float):
        self.d_model, self.n_heads, self.head_dim = int(d_model), int(n_heads), int(head_dim)
        self.decay_rank, self.eps = int(decay_rank), float(eps)
        self.inner = self.n_heads * self.head_dim

    def tensor_specs(self) -> dict:
        d, c = self.d_model, self.inner
        out = {f"mu.{s}": TensorSpec((d,), kind="vector", init="zeros") for s in self.MIXES}
        out.update({
            "r": TensorSpec((c, d)), "k": TensorSpec((c, d)), "v": TensorSpec((c, d)),
            "g": TensorSpec((c, d)),
            "w1": TensorSpec((self.decay_rank, d)), "w2": TensorSpec((c, self.decay_rank)),
            "w0": TensorSpec((c,), kind="vector", init="zeros"),
            "u": TensorSpec((self.n_heads, self.head_dim)),
            "norm": TensorSpec((c,), kind="vector", init="ones"),
            "o": TensorSpec((d, c)),
        })
        return out

    def state_floats(self) -> int:
        """S of every head, then the previous token's h."""
        return self.inner * self.head_dim + self.d_model

    def cache_spec(self):
        return FixedState((self.state_floats(),), torch.float32)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        ops.require_part("shortconv")
        ops.require_part("scan")
        ops.require_scan(self.head_dim)
        self.mu = torch.stack([tensors[f"mu.{s}"] for s in self.MIXES]).contiguous()
        # the four projections stacked: each alone is a run of its rows
        c = self.inner
        self.w_all = ops.prepare_weight(torch.cat([tensors[s] for s in ("r", "k", "v", "g")], dim=0))
        self.w_rkvg = [self.w_all[i * c:(i + 1) * c] for i in range(4)]
        # the decay is float32 from its mix to its exponentials
        self.w1 = tensors["w1"].float().contiguous()
        self.w2t = tensors["w2"].float().t().contiguous()       # [rank, channels]
        self.w0 = tensors["w0"].contiguous()
        self.u = tensors["u"].contiguous()
        self.g_norm = tensors["norm"].contiguous()
        self.w_o = ops.prepare_weight(tensors["o"])

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t, d, c, nh, e = step.n_tokens, self.d_model, self.inner, self.n_heads, self.head_dim
        s_floats = c * e
        prev = cache.state[:, s_floats:s_floats + d]
        mixes = rt.buffer("wkv_mix", (4, t, d), rt.act_dtype)
        mix_w = rt.buffer("wkv_mix_w", (t, d), torch.float32)
        single = step.max_q_len == 1          # then the kernel moves the previous rows on itself
        ops.token_shift_mix(h, self.mu, prev, mixes, mix_w, step, move_tail=single)
        if not single:
            ops.tail_update(h, 0, d, None, prev, 1, step)
        if 4 * t <= self.STACK_ROWS and self.w_all.dtype == torch.bfloat16:
            # few tokens: the step streams weights, so one product of all four mixes with
            # all four matrices (of whose sixteen blocks four are wanted) beats four products
            both = rt.buffer("wkv_rkvg_all", (4 * t, 4 * c), rt.act_dtype)
            ops.linear(mixes.view(4 * t, d), self.w_all, both)
            r, k, v, gate = ((both[i * t:(i + 1) * t], i * c) for i in range(4))
        else:
            rkvg = rt.buffer("wkv_rkvg", (4, t, c), rt.act_dtype)
            for i, w in enumerate(self.w_rkvg):
                ops.linear(mixes[i], w, rkvg[i])
            r, k, v, gate = ((rkvg[i], 0) for i in range(4))
        lo = rt.buffer("wkv_lo", (t, self.decay_rank), torch.float32)
        ops.linear(mix_w, self.w1, lo)
        decay = rt.buffer("wkv_decay", (t, c), torch.float32)
        ops.decay_lowrank(lo, self.w2t, self.w0, decay)
        o = rt.buffer("scan_out", (t, c), torch.float32)
        ops.linear_scan(r, k, v, cache.state, step, nh, e, e, o, decay_tok=decay, bonus=self.u,
                        read_first=True)
        y = rt.buffer("attn_out", (t, c), rt.act_dtype)
        ops.scan_finish(o, gate[0], gate[1], self.g_norm, self.eps, y, nh, e)
        delta = rt.buffer("delta", (t, d), rt.act_dtype)
        return ops.linear_parts(y, self.w_o, delta)


class RetentionMixer(Mixer):
    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, v_dim: int, decay, eps: float,
                 position=None):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.v_dim, self.eps = int(qk_dim), int(v_dim), float(eps)
        self.decay_values = [float(x) for x in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError("retention needs one decay a head")
        if position is not None and position.pairing != "half":
            raise ValueError("this mixer's kernel rotates entry i with i + dims/2")
        self.position = position

    def tensor_specs(self) -> dict:
        d, h, e, f = self.d_model, self.n_heads, self.qk_dim, self.v_dim
        return {"q": TensorSpec((h * e, d)), "k": TensorSpec((h * e, d)),
                "v": TensorSpec((h * f, d)), "g": TensorSpec((h * f, d)),
                "o": TensorSpec((d, h * f))}

    def cache_spec(self):
        return FixedState((self.n_heads * self.qk_dim * self.v_dim,), torch.float32)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        ops.require_part("scan")
        ops.require_scan(self.qk_dim)
        self.w_qkvg = ops.prepare_weight(torch.cat(
            [tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0))
        self.w_o = ops.prepare_weight(tensors["o"])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)
        if self.position is not None:
            self.position.bind({}, runtime)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t, nh, e, f = step.n_tokens, self.n_heads, self.qk_dim, self.v_dim
        qkvg = rt.buffer("ret_qkvg", (t, 2 * nh * e + 2 * nh * f), rt.act_dtype)
        ops.linear(h, self.w_qkvg, qkvg)
        qk = rt.buffer("ret_qk", (t, 2 * nh * e), torch.float32)
        pos = self.position
        ops.rotate_rows(qkvg, 0, nh * e, step.positions, pos.freq if pos else None,
                        pos.dims if pos else 0, float(e) ** -0.5, qk, nh, e)
        o = rt.buffer("scan_out", (t, nh * f), torch.float32)
        ops.linear_scan((qk, 0), (qk, nh * e), (qkvg, 2 * nh * e), cache.state, step, nh, e, f, o,
                        decay_head=self.decay)
        y = rt.buffer("attn_out", (t, nh * f), rt.act_dtype)
        ops.scan_finish(o, qkvg, 2 * nh * e + nh * f, None, self.eps, y, nh, f)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return ops.linear_parts(y, self.w_o, delta)


class LightningAttention(Mixer):
    """Linear attention with one constant decay a head and a matrix state per head:

        q, k, v = silu(W_q h), silu(W_k h), silu(W_v h)       (heads of e, e and f entries)
        S <- decay_head S + k_t v_t^T;   o_t = S^T q_t          (no other scale)
        out = W_o (rms_norm(o over all heads together) * w * sigmoid(W_g h)) * out_scale

    The state lives in the request's state slot (float32, zero when claimed) and is carried
    from token to token, so cutting a prompt changes no bit.  Activations enter the scan in
    float32; decays, state, sums and the norm are float32 in both run types.  With
    ``project=False`` the mixer has no output projection: ``heads(h, step, cache, out)``
    leaves the normed, gated and scaled heads in ``out`` (which may be a block of columns of
    a wider buffer) for a mixer that owns this one."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, v_dim: int, decay, eps: float,
                 out_scale: float = 1.0, project: bool = True):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.v_dim, self.eps = int(qk_dim), int(v_dim), float(eps)
        self.decay_values = [float(x) for x in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError("lightning attention needs one decay a head")
        self.out_scale, self.project = float(out_scale), bool(project)
        self.out_width = self.n_heads * self.v_dim

    def tensor_specs(self) -> dict:
        d, h, e, f = self.d_model, self.n_heads, self.qk_dim, self.v_dim
        out = {"q": TensorSpec((h * e, d)), "k": TensorSpec((h * e, d)),
               "v": TensorSpec((h * f, d)), "g": TensorSpec((h * f, d)),
               "norm": TensorSpec((h * f,), kind="vector", init="ones")}
        if self.project:
            out["o"] = TensorSpec((d, h * f))
        return out

    def cache_spec(self):
        return FixedState((self.n_heads * self.qk_dim * self.v_dim,), torch.float32)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        ops.require_part("scan")
        ops.require_scan(self.qk_dim)
        self.w_qkvg = ops.prepare_weight(torch.cat(
            [tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0))
        self.g_norm = tensors["norm"].float().contiguous()
        if self.project:
            self.w_o = ops.prepare_weight(tensors["o"])
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def heads(self, h, step: StepContext, cache: CacheHandle, out) -> None:
        rt, ops = self.runtime, self.runtime.ops
        t, nh, e, f = step.n_tokens, self.n_heads, self.qk_dim, self.v_dim
        qkvg = rt.buffer("ret_qkvg", (t, 2 * nh * e + 2 * nh * f), rt.act_dtype)
        ops.linear(h, self.w_qkvg, qkvg)
        o = rt.buffer("scan_out", (t, nh * f), torch.float32)
        ops.linear_scan((qkvg, 0), (qkvg, nh * e), (qkvg, 2 * nh * e), cache.state, step, nh, e, f,
                        o, decay_head=self.decay, silu=True)
        ops.scan_finish_row(o, qkvg, 2 * nh * e + nh * f, self.g_norm, self.eps, out,
                            out_scale=self.out_scale)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        if not self.project:
            raise RuntimeError("this mixer has no output projection: its owner calls heads()")
        rt = self.runtime
        y = rt.buffer("attn_out", (step.n_tokens, self.out_width), rt.act_dtype)
        self.heads(h, step, cache, y)
        delta = rt.buffer("delta", (step.n_tokens, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(y, self.w_o, delta)
