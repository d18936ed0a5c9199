"""Causal attention whose keys and values are read off one cached latent a token.

With d = model width, H heads of query/key size e and value size f, a latent of
size r and a query latent of size rq (all float32 norms, eps inside the root):

    cq = unit_rms(W_dq h) * g_q            q_h = W_uq[h] cq
    c  = unit_rms(W_dkv h) * g_kv          k_h = W_uk[h] c,  v_h = W_uv[h] c
    score_ij = (q_hi . k_hj) * scale,  j <= i;  softmax;  out = W_o concat_h(sum_j p_ij v_hj)

No position enters.  Only c is cached, and neither keys nor values are ever rebuilt:
``q . (W_uk c) = (W_uk^T q) . c`` and ``sum_j p_j W_uv c_j = W_uv sum_j p_j c_j``, so the
query is taken into the latent space, the framework's paged attention kernels run
as multi-query attention with the latent pool as the one key and value head
(``PagedKV(1, r', shared_kv=True)``, r' = r rounded up to the kernels' head sizes,
the padding zero), and the result is taken out of the latent space again.
"""

from __future__ import annotations

import torch

from .attention import plan_paged_attention
from .base import CacheHandle, Mixer, PagedKV, StepContext, TensorSpec


class LatentAttention(Mixer):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    PAD = 16          # the attention kernels take head sizes in steps of 16

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, v_dim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        self.kv_rank, self.q_rank = int(kv_rank), int(q_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.pool_rank = max(self.PAD, -(-self.kv_rank // self.PAD) * self.PAD)

    def tensor_specs(self) -> dict:
        d, h = self.d_model, self.n_heads
        return {
            "dq": TensorSpec((self.q_rank, d)),
            "dq.norm": TensorSpec((self.q_rank,), kind="vector", init="ones"),
            "uq": TensorSpec((h * self.qk_dim, self.q_rank)),
            "dkv": TensorSpec((self.kv_rank, d)),
            "dkv.norm": TensorSpec((self.kv_rank,), kind="vector", init="ones"),
            "uk": TensorSpec((h * self.qk_dim, self.kv_rank)),
            "uv": TensorSpec((h * self.v_dim, self.kv_rank)),
            "o": TensorSpec((d, h * self.v_dim)),
        }

    def cache_spec(self):
        return PagedKV(1, self.pool_rank, None, shared_kv=True)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        h, e, f, r, rp = self.n_heads, self.qk_dim, self.v_dim, self.kv_rank, self.pool_rank
        self.w_down = ops.prepare_weight(torch.cat([tensors["dq"], tensors["dkv"]], dim=0))
        self.g_q = tensors["dq.norm"].contiguous()
        self.g_kv = tensors["dkv.norm"].contiguous()
        self.w_uq = ops.prepare_weight(tensors["uq"])
        uk = tensors["uk"].view(h, e, r)
        uv = tensors["uv"].view(h, f, r)
        # W_uk[h]^T as [H, r', e] and W_uv[h] as [H, f, r'], zero where the latent is padded
        self.w_into = torch.zeros((h, rp, e), dtype=uk.dtype, device=uk.device)
        self.w_into[:, :r] = uk.transpose(1, 2)
        self.w_out_of = torch.zeros((h, f, rp), dtype=uv.dtype, device=uv.device)
        self.w_out_of[:, :, :r] = uv
        self.w_o = ops.prepare_weight(tensors["o"])
        ops.require_part("latent")
        ops.require_attention(rp, h, 1)
        self._facts = ops.attention_facts(rp)

    def plan(self, step: StepContext):
        return plan_paged_attention(step, self._facts, self.n_heads, 1, self.pool_rank)

    def decode_graph_key(self, step: StepContext) -> tuple:
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("latent", self.n_heads, self.pool_rank, plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t = step.n_tokens
        nh, e, f, rp = self.n_heads, self.qk_dim, self.v_dim, self.pool_rank
        down = rt.buffer("latent_down", (t, self.q_rank + self.kv_rank), torch.float32)
        ops.linear(h, self.w_down, down)
        cq = rt.buffer("latent_cq", (t, self.q_rank), rt.act_dtype)
        ops.latent_norm_store(down, self.q_rank, self.kv_rank, self.g_q, self.g_kv, self.eps,
                              cq, cache, step)
        q = rt.buffer("latent_q", (t, nh * e), rt.act_dtype)
        ops.linear(cq, self.w_uq, q)
        # the kernels read a row of [q heads | k heads | v heads]; only the q heads are there
        q_in = rt.buffer("latent_q_in", (t, (nh + 2) * rp), rt.act_dtype)
        ops.headwise_linear(q, e, self.w_into, q_in, rp, t)
        o_in = rt.buffer("latent_o_in", (t, nh * rp), rt.act_dtype)
        ops.paged_attention(q_in, o_in, cache, step, nh, 1, rp, self.scale, 0,
                            plan=self.plan(step))
        o = rt.buffer("attn_out", (t, nh * f), rt.act_dtype)
        ops.headwise_linear(o_in, rp, self.w_out_of, o, f, t)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return ops.linear_parts(o, self.w_o, delta)


class RotaryLatentAttention(Mixer):
    """Latent attention whose heads also carry a rotated part, with an optional window, a
    sink in the softmax and a sigmoid gate on the heads' outputs.

    With e plain and g rotated query/key entries a head, value size f, latent size r:

        q_h = [a_h | b_h] = W_q[h] x             b_h rotated by the token's position
        [c' | k'] = W_dkv x                      c = unit_rms(c') * w (r entries);  k' (g
                                                 entries) rotated: one key part for all heads
        score_h(i, j) = (a_hi . W_uk[h] c_j + b_hi . k_j) * scale,   0 <= i - j < window
        p = exp(score) / (sum_j exp(score) + exp(sink_h));   o_h = sum_j p_j W_uv[h] c_j
        out = W_o (concat_h o_h * sigmoid(W_g x))

    Only ``[c | k]`` is cached (``PagedKV(1, r + g rounded up, shared_kv=True)``), and keys
    and values are never rebuilt: the query's plain part is taken into the latent space
    (``W_uk[h]^T a_h``), the paged attention kernels run as multi-query attention over the
    cached rows, whose first r entries are also the values, and ``W_uv[h]`` is applied to the
    weighted latent.  A mixer with ``own_cache=False`` has no ``W_dkv``: its call reads the
    slot another layer's call fills (``LayerCall.writes`` False).  ``cache_window``: how many
    of the latest tokens the cache keeps (at least ``window``; larger when a reader of this
    cache sees further back; None: all).  ``position``: a ``PartialRotary`` with the "half"
    pairing over the first ``position.dims`` of the g entries, or None."""

    decode_capturable = prompt_capturable = True
    PAD = 16

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, rot_dim: int, v_dim: int,
                 kv_rank: int, scale: float, eps: float, position=None, window=None,
                 sink: bool = True, gate: bool = True, own_cache: bool = True,
                 cache_window=None):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.rot_dim, self.v_dim = int(qk_dim), int(rot_dim), int(v_dim)
        self.kv_rank, self.scale, self.eps = int(kv_rank), float(scale), float(eps)
        self.position, self.window = position, window
        self.has_sink, self.has_gate, self.own_cache = bool(sink), bool(gate), bool(own_cache)
        self.cache_window = cache_window if own_cache else None
        if position is not None and (position.pairing != "half" or position.dims > self.rot_dim):
            raise ValueError("the rotated part turns entry i with entry i + dims/2, dims <= rot_dim")
        if own_cache and window is not None and cache_window is not None and cache_window < window:
            raise ValueError("the cache keeps fewer tokens than the window sees")
        width = self.kv_rank + self.rot_dim
        self.pool_width = max(self.PAD, -(-width // self.PAD) * self.PAD)

    def tensor_specs(self) -> dict:
        d, h = self.d_model, self.n_heads
        out = {"q": TensorSpec((h * (self.qk_dim + self.rot_dim), d))}
        if self.own_cache:
            out["dkv"] = TensorSpec((self.kv_rank + self.rot_dim, d))
            out["dkv.norm"] = TensorSpec((self.kv_rank,), kind="vector", init="ones")
        out["uk"] = TensorSpec((h * self.qk_dim, self.kv_rank))
        out["uv"] = TensorSpec((h * self.v_dim, self.kv_rank))
        if self.has_sink:
            out["sink"] = TensorSpec((h,), kind="vector", init="zeros")
        if self.has_gate:
            out["g"] = TensorSpec((h * self.v_dim, d))
        out["o"] = TensorSpec((d, h * self.v_dim))
        return out

    def cache_spec(self):
        if not self.own_cache:
            return None
        return PagedKV(1, self.pool_width, self.cache_window, shared_kv=True)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        h, e, f, r = self.n_heads, self.qk_dim, self.v_dim, self.kv_rank
        # one product for everything that reads the mixer's input: [q | gate | down]
        rows = [tensors["q"]]
        self.gate_col = self.kv_col = -1
        at = rows[0].shape[0]
        if self.has_gate:
            rows.append(tensors["g"])
            self.gate_col, at = at, at + rows[-1].shape[0]
        if self.own_cache:
            rows.append(tensors["dkv"])
            self.kv_col, at = at, at + rows[-1].shape[0]
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.w_in = ops.prepare_weight(torch.cat(rows, dim=0))
        self.in_width = at
        self.w_norm = tensors["dkv.norm"].contiguous() if self.own_cache else None
        # W_uk[h]^T as [H, r, e] and W_uv[h] as [H, f, r]
        self.w_into = tensors["uk"].view(h, e, r).transpose(1, 2).contiguous()
        self.w_out_of = tensors["uv"].view(h, f, r).contiguous()
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        self.w_o = ops.prepare_weight(tensors["o"])
        if self.position is not None:
            self.position.bind({}, runtime)
        ops.require_part("latent")
        ops.require_attention(self.pool_width, h, 1)
        self._facts = ops.attention_facts(self.pool_width)

    def plan(self, step: StepContext):
        return plan_paged_attention(step, self._facts, self.n_heads, 1, self.pool_width)

    def decode_graph_key(self, step: StepContext) -> tuple:
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("latent", self.n_heads, self.pool_width, plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t = step.n_tokens
        nh, e, g, f = self.n_heads, self.qk_dim, self.rot_dim, self.v_dim
        r, rp = self.kv_rank, self.pool_width
        if cache.kind != "paged" or bool(cache.writes) != self.own_cache:
            raise RuntimeError("a latent mixer with a down projection fills its cache slot; one "
                               "without reads another call's")
        # float32 rows: the norm of the latent, the rotation and the gate see no 16-bit rounding
        proj = rt.buffer("latent_in", (t, self.in_width), torch.float32)
        proj = ops.linear_parts(h, self.w_in, proj)
        q_plain = rt.buffer("latent_q_plain", (t, nh * e), rt.act_dtype)
        # the kernels read a row of [q heads | k heads | v heads]; only the q heads are there
        q_in = rt.buffer("latent_q_in", (t, (nh + 2) * rp), rt.act_dtype)
        pos = self.position
        ops.latent_rope_prep(proj, 0, self.kv_col, nh, e, g, r, rp, pos.dims if pos else 0,
                             pos.freq if pos else None, self.w_norm, self.eps, q_plain, q_in,
                             cache, step)
        ops.headwise_linear(q_plain, e, self.w_into, q_in, rp, t)
        o_in = rt.buffer("latent_o_in", (t, nh * rp), rt.act_dtype)
        ops.paged_attention(q_in, o_in, cache, step, nh, 1, rp, self.scale, self.window or 0,
                            plan=self.plan(step), sink=self.sink)
        o = rt.buffer("attn_out", (t, nh * f), rt.act_dtype)
        ops.headwise_linear(o_in, rp, self.w_out_of, o, f, t)
        if self.has_gate:
            ops.sigmoid_gate(o, proj, self.gate_col)
        if hasattr(proj, "release"):
            proj.release()
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return ops.linear_parts(o, self.w_o, delta)
