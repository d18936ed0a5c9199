"""Grouped-query causal attention over the paged cache.

Reference (train/model.py:73-124, MHA only): q/k/v/o projections without bias,
``nn.Linear`` layout [out, in], output feature j belongs to head ``j // head_dim``;
RoPE on q and k; scores ``(q . k) * scale`` with ``scale = head_dim ** -0.5``
(train/model.py:62); causal mask bottom-right aligned: key j is hidden from
query i iff ``j > i + (Sk - Sq)`` (train/model.py:64-68); softmax and P.V in
float32; output heads concatenated head-major (train/model.py:122) and
projected by ``wo``.  Grouped queries: q head h reads kv head ``h // G``.  A
window w additionally hides keys ``j <= p - w`` from the query at position p.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .base import CacheHandle, Mixer, PagedKV, StepContext, TensorSpec


@dataclass(frozen=True)
class AttentionPlan:
    """How one step's attention is launched (for one shape of heads)."""
    n_tiles: int          # tiles of the mma.sync tile kernel over the requests that are not small
    n_tiles_tc: int       # tiles of the tcgen05 kernel over the same requests
    n_tiles_tc_wide: int  # tiles of twice as many rows: the kernel takes these when they fill the SMs
    any_small: bool       # some request has so few rows that the context-split kernel takes it
    n_split: int          # parts the context of the small requests is cut into


def context_splits(tiles: list, n_kv: int, slots: int = 296, cluster_splits: int = 0,
                   longest: int = 0, cluster_slots: int = 0) -> int:
    """Context splits for decoding requests of ``tiles[i]`` key tiles (64 keys) each.

    The kernel cuts every request at the same multiples of tiles, the tiles of the step's
    longest context (``longest``, if a request that is not among these has more) shared
    out over the splits: a shorter request fills only its first splits, and the CTAs of
    the others leave at once.  ``slots`` CTAs of the split kernel run at a
    time (two an SM: 296 on a B200); the cost of a choice is its number of such waves of
    CTAs that have tiles times the tiles a CTA walks (plus six tiles' worth of start-up),
    plus what placing the empty CTAs costs, plus the merge's time, which grows with the
    number of parts (measured at batch 1: 16 parts beat 32).  Up to ``cluster_splits``
    parts are merged inside the split kernel while ``cluster_slots`` CTAs hold them all;
    beyond that a merge kernel follows, which costs about what two tiles take.  The
    cheapest choice wins; a split is never shorter than 256 keys.
    """
    longest = max(longest, max(tiles))
    forced = os.environ.get("MLS_B200_SPLITS")
    if forced:
        return max(1, min(int(forced), longest))
    best, best_cost = 1, None
    for s in range(1, max(1, min(64, longest // 4)) + 1):
        per = -(-longest // s)
        busy = sum(-(-t // per) for t in tiles) * n_kv
        grid = len(tiles) * n_kv * s
        cost = -(-busy // slots) * (per + 6) + 2.0 * (grid - busy) / slots
        if s > 1:
            cost += 0.3 * s
            if not (cluster_splits and s <= cluster_splits and grid <= (cluster_slots or slots)):
                cost += 2.0
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def plan_paged_attention(step: StepContext, facts: dict, n_heads: int, n_kv_heads: int,
                         head_dim: int):
    """A step's ``AttentionPlan`` for heads of this shape (None where the kernel in use
    needs none), shared through ``step.attn_tiles`` by the mixers of the same shape.

    Requests whose (token, head) rows of one kv head fit ``small_rows`` go to the
    context-split kernel, their context cut so that all SMs have work; the others
    are cut into tiles of rows."""
    f = facts
    if not f["tensor_cores"]:
        return None
    group = n_heads // n_kv_heads
    key = ("gqa", group, n_kv_heads, head_dim)
    plan = step.attn_tiles.get(key)
    if plan is None:
        small = [q * group <= f["small_rows"] for q in step.q_lens]
        big = [q * group for q, s in zip(step.q_lens, small) if not s]
        n_small = sum(small)
        n_split = 1
        if n_small:
            keys = f.get("split_keys", 64)
            tiles = [-(-c // keys) for c, s in zip(step.ctx_lens, small) if s]
            n_split = context_splits(tiles, n_kv_heads, f["split_slots"],
                                     f.get("cluster_splits", 0),
                                     longest=-(-step.max_ctx_len // keys),
                                     cluster_slots=f.get("cluster_slots", 0))
        plan = AttentionPlan(
            n_tiles=sum(-(-r // f["tile_rows"]) for r in big),
            n_tiles_tc=sum(-(-r // f["tc_rows"]) for r in big),
            n_tiles_tc_wide=sum(-(-r // (2 * f["tc_rows"])) for r in big),
            any_small=n_small > 0, n_split=n_split)
        step.attn_tiles[key] = plan
    return plan


class GroupedQueryAttention(Mixer):
    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position, window=None):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.d_model, self.n_heads, self.n_kv_heads = d_model, n_heads, n_kv_heads
        self.head_dim, self.scale, self.window = head_dim, float(scale), window
        self.position = position
        self.wqkv = self.wo = None

    def tensor_specs(self) -> dict:
        d, hd = self.d_model, self.head_dim
        return {
            "wq.weight": TensorSpec((self.n_heads * hd, d)),
            "wk.weight": TensorSpec((self.n_kv_heads * hd, d)),
            "wv.weight": TensorSpec((self.n_kv_heads * hd, d)),
            "wo.weight": TensorSpec((d, self.n_heads * hd)),
        }

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        parts = [tensors["wq.weight"], tensors["wk.weight"], tensors["wv.weight"]]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        # one projection for q, k and v: rows [q heads | k heads | v heads]
        self.wqkv = runtime.ops.prepare_weight(torch.cat(parts, dim=0))
        self.wo = runtime.ops.prepare_weight(tensors["wo.weight"])
        self.position.bind({}, runtime)
        runtime.ops.require_attention(self.head_dim, self.n_heads, self.n_kv_heads)
        self._facts = runtime.ops.attention_facts(self.head_dim)

    # ---------------------------------------------------------- launch planning
    @property
    def decode_capturable(self) -> bool:
        """Forward only launches kernels; the position part has to agree."""
        return bool(getattr(self.position, "decode_capturable", False))

    @property
    def prompt_capturable(self) -> bool:
        return bool(getattr(self.position, "prompt_capturable", False))

    def plan(self, step: StepContext):
        """This step's ``AttentionPlan`` (None where the kernel in use needs none).

        Requests whose (token, head) rows of one kv head fit ``small_rows`` go to the
        context-split kernel, their context cut so that all SMs have work; the others
        are cut into tiles of rows.  Mixers with the same shape of heads share the
        plan of a step."""
        return plan_paged_attention(step, self._facts, self.n_heads, self.n_kv_heads,
                                    self.head_dim)

    def decode_graph_key(self, step: StepContext) -> tuple:
        """What, besides the number of requests, fixes this mixer's launches in a step
        of single tokens: the number of context splits."""
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("gqa", self.n_kv_heads, self.n_heads // self.n_kv_heads, self.head_dim,
                plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt = self.runtime
        t = step.n_tokens
        hd = self.head_dim
        width = (self.n_heads + 2 * self.n_kv_heads) * hd
        qkv = rt.buffer("qkv", (t, width), rt.act_dtype)
        o = rt.buffer("attn_out", (t, self.n_heads * hd), rt.act_dtype)
        if getattr(self.position, "takes_parts", False):
            # the projection may stay in the parts it was cut into along K: the
            # rotation adds them up as it reads them
            src = rt.ops.linear_parts(h, self.wqkv, qkv)
            tables = (self.position.fused_tables()
                      if src is not qkv and step.max_q_len == 1 and cache.kind == "paged"
                      and hasattr(self.position, "fused_tables") else None)
            if tables is not None and rt.ops.can_fuse_rope_attention(
                    hd, step.groups[cache.group].block_size):
                # single decoded tokens: the attention kernel rotates and stores as well
                cos, sin, max_pos = tables
                rt.ops.attention_decode_fused(src, o, cache, step, cos, sin, max_pos,
                                              self.n_heads, self.n_kv_heads, hd, self.scale,
                                              self.window or 0, self.plan(step))
                delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
                return rt.ops.linear_parts(o, self.wo, delta)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads, self.n_kv_heads,
                                           parts=None if src is qkv else src)
        else:
            rt.ops.linear(h, self.wqkv, qkv)
            self.position.rotate_and_store(qkv, step, cache, self.n_heads,
                                           self.n_kv_heads)
        rt.ops.paged_attention(qkv, o, cache, step, self.n_heads, self.n_kv_heads,
                               hd, self.scale, self.window or 0, plan=self.plan(step))
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(o, self.wo, delta)


def distance_slopes(n_heads: int) -> list:
    """One slope a head for a bias on the distance to the key: ``2^(-8 (h + 1) / n_heads)``."""
    return [2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)]


class UnrotatedAttention(Mixer):
    """Grouped-query attention in which nothing is rotated; positions enter through options.

    With H query heads and G key/value heads, queries and keys of size e and values of size f
    (query head h reads head ``h // (H/G)``), per token:

        q, k, v = W_q h, W_k h, W_v h             (+ b_q, b_k, b_v with ``qkv_bias``)
        q_h, k_g <- rms_norm(.) * w_q, w_k        per head, weights [e] for all heads (``head_norm``)
        q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))   ``q_temp = (coef, every)``
        score_ij = (q_i . k_j) * scale - slope_h * (i - j)     ``slopes`` (one a head)
        j visible to i iff j <= i and (i - j < window or j < keep_first)
        softmax over the visible keys, with ``zero_sink`` plus one term exp(0) without a value
        o <- o * sigmoid(W_g h)                   element by element (``gate``)
        out = W_o concat_h(o)

    Keys and values live in the paged cache, every head padded with zeros to the kernels'
    head size (the next multiple of 16 of the larger of e and f), as are the queries, the
    gate's rows and the output projection's columns.  ``v_scale`` multiplies the values
    (a weight on this mixer's output that costs nothing).  With ``project=False`` the mixer
    has no output projection: ``heads(h, step, cache, out)`` leaves the heads' outputs in
    ``out`` (which may be a block of columns of a wider buffer) for a mixer that owns this
    one, and ``padded_columns`` says how that mixer's projection has to be laid out."""

    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, head_dim: int, v_dim: int,
                 scale: float, eps: float = 1e-6, window=None, keep_first: int = 0,
                 qkv_bias: bool = False, head_norm: bool = False, slopes=None,
                 zero_sink: bool = False, q_temp=None, gate: bool = False, v_scale: float = 1.0,
                 project: bool = True):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if slopes is not None and len(slopes) != n_heads:
            raise ValueError("a bias on the distance needs one slope a head")
        self.d_model, self.n_heads, self.n_kv_heads = int(d_model), int(n_heads), int(n_kv_heads)
        self.head_dim, self.v_dim = int(head_dim), int(v_dim)
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.qkv_bias, self.head_norm = bool(qkv_bias), bool(head_norm)
        self.slope_values = [float(x) for x in slopes] if slopes is not None else None
        self.zero_sink, self.gate = bool(zero_sink), bool(gate)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        self.v_scale, self.project = float(v_scale), bool(project)
        self.pad_dim = -(-max(self.head_dim, self.v_dim) // 16) * 16     # the kernels' head size
        self.out_width = self.n_heads * self.pad_dim

    def tensor_specs(self) -> dict:
        d, e, f = self.d_model, self.head_dim, self.v_dim
        cq, ck, cv = self.n_heads * e, self.n_kv_heads * e, self.n_kv_heads * f
        out = {"q": TensorSpec((cq, d)), "k": TensorSpec((ck, d)), "v": TensorSpec((cv, d))}
        if self.qkv_bias:
            out.update({"q.b": TensorSpec((cq,), kind="vector", init="zeros"),
                        "k.b": TensorSpec((ck,), kind="vector", init="zeros"),
                        "v.b": TensorSpec((cv,), kind="vector", init="zeros")})
        if self.head_norm:
            out.update({"q.norm": TensorSpec((e,), kind="vector", init="ones"),
                        "k.norm": TensorSpec((e,), kind="vector", init="ones")})
        if self.gate:
            out["g"] = TensorSpec((self.n_heads * f, d))
        if self.project:
            out["o"] = TensorSpec((d, self.n_heads * f))
        return out

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.pad_dim, self.window, keep_first=self.keep_first)

    def pad_rows(self, w):
        """``w [H * f, d]`` with every head's rows padded with zero rows to the kernels' size."""
        if self.pad_dim == self.v_dim:
            return w
        out = w.new_zeros((self.n_heads, self.pad_dim, w.shape[1]))
        out[:, :self.v_dim] = w.view(self.n_heads, self.v_dim, w.shape[1])
        return out.view(self.n_heads * self.pad_dim, w.shape[1])

    def padded_columns(self, w_o):
        """``w_o [d, H * f]`` with zero columns where the heads' outputs are padded."""
        return self.pad_rows(w_o.t().contiguous()).t().contiguous()

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        parts = [tensors["q"], tensors["k"], tensors["v"]]
        if self.gate:
            parts.append(self.pad_rows(tensors["g"]))
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        # one projection for everything that reads the mixer's input: [q | k | v | gate]
        self.w_in = ops.prepare_weight(torch.cat(parts, dim=0))
        cq, ck = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.cols = (0, cq, cq + ck)
        self.gate_col = cq + ck + self.n_kv_heads * self.v_dim
        f32 = torch.float32
        self.biases = (tuple(tensors[n].to(f32).contiguous() for n in ("q.b", "k.b", "v.b"))
                       if self.qkv_bias else None)
        self.norms = (tuple(tensors[n].to(f32).contiguous() for n in ("q.norm", "k.norm"))
                      if self.head_norm else None)
        self.slopes = (torch.tensor(self.slope_values, dtype=f32, device=runtime.device)
                       if self.slope_values is not None else None)
        self.sink = (torch.zeros(self.n_heads, dtype=f32, device=runtime.device)
                     if self.zero_sink else None)
        if self.project:
            self.w_o = ops.prepare_weight(self.padded_columns(tensors["o"]))
        ops.require_part("headprep")
        if self.gate:
            ops.require_part("latent")               # the gate's kernel lives there
        self._tensor_cores = ops.attention_tensor_cores(self.pad_dim)
        if self._tensor_cores:
            ops.require_attention(self.pad_dim, self.n_heads, self.n_kv_heads)
        self._facts = ops.attention_facts(self.pad_dim)

    def plan(self, step: StepContext):
        if not self._tensor_cores:
            return None
        return plan_paged_attention(step, self._facts, self.n_heads, self.n_kv_heads, self.pad_dim)

    def decode_graph_key(self, step: StepContext) -> tuple:
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("gqa", self.n_kv_heads, self.n_heads // self.n_kv_heads, self.pad_dim,
                plan.n_split)

    def heads(self, h, step: StepContext, cache: CacheHandle, out) -> None:
        """The heads' outputs (gated, if the mixer has a gate) into ``out [T, H * pad_dim]``."""
        rt, ops = self.runtime, self.runtime.ops
        t, hd = step.n_tokens, self.pad_dim
        proj = rt.buffer("attn_proj", (t, self.w_in.shape[0]), torch.float32)
        ops.linear(h, self.w_in, proj)
        q_row = rt.buffer("qkv", (t, (self.n_heads + 2 * self.n_kv_heads) * hd), rt.act_dtype)
        ops.head_prep_store(proj, self.cols, self.biases, self.norms, self.eps, self.q_temp,
                            self.v_scale, q_row, cache, step, self.n_heads, self.n_kv_heads,
                            self.head_dim, self.v_dim, hd)
        ops.paged_attention(q_row, out, cache, step, self.n_heads, self.n_kv_heads, hd, self.scale,
                            self.window or 0, plan=self.plan(step), sink=self.sink,
                            slopes=self.slopes, keep_first=self.keep_first,
                            simt=not self._tensor_cores)
        if self.gate:
            ops.sigmoid_gate(out, proj, self.gate_col)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        if not self.project:
            raise RuntimeError("this mixer has no output projection: its owner calls heads()")
        rt = self.runtime
        o = rt.buffer("attn_out", (step.n_tokens, self.out_width), rt.act_dtype)
        self.heads(h, step, cache, o)
        delta = rt.buffer("delta", (step.n_tokens, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(o, self.w_o, delta)
