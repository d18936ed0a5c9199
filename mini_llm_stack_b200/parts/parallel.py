"""Two mixers side by side that read the same input: ``out = W_o [left heads | right heads]``.

Each half is a mixer built without an output projection (``project=False``) that leaves its
heads' outputs, already multiplied by its weight in the sum, in its block of columns of one
buffer (``heads(h, step, cache, out)``, ``out_width`` columns); the two output projections
``left.o [d, .]`` and ``right.o [d, .]`` run as ONE product over that buffer, which is the
weighted sum of the two halves' outputs.  A half that pads its heads says how its projection's
columns are laid out (``padded_columns``).  The left half keeps pages, the right half a state
of fixed size: the mixer's cache is a ``PagedWithState`` and both halves get its handle.
"""

from __future__ import annotations

import torch

from .base import CacheHandle, FixedState, Mixer, PagedKV, PagedWithState, StepContext, TensorSpec
from .block import join_name, under_prefix


class ParallelMixer(Mixer):
    def __init__(self, d_model: int, left, right, names=("left", "right")):
        self.d_model, self.left, self.right = int(d_model), left, right
        self.names = tuple(names)
        for half in (left, right):
            if getattr(half, "project", True):
                raise ValueError("the halves of a parallel mixer are built with project=False")

    def _halves(self):
        return list(zip(self.names, (self.left, self.right)))

    def tensor_specs(self) -> dict:
        out = {}
        for prefix, half in self._halves():
            for n, s in half.tensor_specs().items():
                out[join_name(prefix, n)] = s
            inner = half.n_heads * half.v_dim
            out[join_name(prefix, "o")] = TensorSpec((self.d_model, inner))
        return out

    def cache_spec(self):
        specs = [half.cache_spec() for _, half in self._halves()]
        paged = [s for s in specs if isinstance(s, PagedKV)]
        fixed = [s for s in specs if isinstance(s, FixedState)]
        if len(paged) == 1 and len(fixed) == 1:
            return PagedWithState(paged[0], fixed[0])
        if len(specs) == 2 and specs[0] is None:
            return specs[1]
        if len(specs) == 2 and specs[1] is None:
            return specs[0]
        raise ValueError("a parallel mixer takes one half with pages and one with a state")

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        outs = []
        for prefix, half in self._halves():
            mine = under_prefix(tensors, prefix)
            w_o = mine.pop("o")
            half.bind(mine, runtime)
            outs.append(half.padded_columns(w_o) if hasattr(half, "padded_columns") else w_o)
        if outs[0].dtype != outs[1].dtype:
            outs = [w.float() for w in outs]
        self.w_o = runtime.ops.prepare_weight(torch.cat(outs, dim=1))

    @property
    def decode_capturable(self) -> bool:
        return all(getattr(h, "decode_capturable", False) for _, h in self._halves())

    @property
    def prompt_capturable(self) -> bool:
        return all(getattr(h, "prompt_capturable", False) for _, h in self._halves())

    def decode_graph_key(self, step: StepContext) -> tuple:
        return tuple(k for _, h in self._halves() if (k := h.decode_graph_key(step)))

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt = self.runtime
        t, wl = step.n_tokens, self.left.out_width
        both = rt.buffer("parallel_heads", (t, wl + self.right.out_width), rt.act_dtype)
        self.left.heads(h, step, cache, both[:, :wl])
        self.right.heads(h, step, cache, both[:, wl:])
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(both, self.w_o, delta)
