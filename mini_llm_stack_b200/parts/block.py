"""The arrangement of a layer's parts: the pre-norm residual block, and the block with a norm
before and behind every sublayer.

Reference (train/model.py:200-217): ``x = x + mixer(norm_a(x))``;
``x = x + feed_forward(norm_b(x))``.  The block owns the order and the names
its parts' tensors carry in a weight file; the parts own the math.
"""

from __future__ import annotations

from .base import CacheHandle, Part, ResidualStream, StepContext


def join_name(prefix: str, name: str) -> str:
    """``prefix.name``; an empty ``name`` is the prefix itself (a part whose one tensor
    carries the part's own name)."""
    if not name:
        return prefix
    return f"{prefix}.{name}" if prefix else name


def under_prefix(tensors: dict, prefix: str) -> dict:
    """The tensors of ``prefix`` under their local names (``prefix`` itself becomes "")."""
    out = {}
    for n, t in tensors.items():
        if n == prefix:
            out[""] = t
        elif n.startswith(prefix + "."):
            out[n[len(prefix) + 1:]] = t
    return out


class PreNormBlock(Part):
    tail = None

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn,
                 names=("attn_norm", "attn", "mlp_norm", "mlp"), tail=None):
        """``tail``: a part that runs last, on the stream itself (``forward(stream, step)``:
        it settles what is pending and pushes its own delta); its prefix is a fifth name."""
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ffn_norm, self.ffn = ffn_norm, ffn
        self.tail = tail
        self.names = tuple(names)
        if tail is not None and len(self.names) < 5:
            raise ValueError("a block with a tail needs a fifth name, the tail's prefix")

    def _named_parts(self):
        """(prefix, part) of the parts there are; a block without a feed-forward
        (``ffn`` None) has no second norm either."""
        return [(n, p) for n, p in zip(self.names, (self.mixer_norm, self.mixer,
                                                    self.ffn_norm, self.ffn, self.tail))
                if p is not None]

    def tensor_specs(self) -> dict:
        out = {}
        for prefix, part in self._named_parts():
            for n, s in part.tensor_specs().items():
                out[join_name(prefix, n)] = s
        return out

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        for prefix, part in self._named_parts():
            part.bind(under_prefix(tensors, prefix), runtime)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def decode_capturable(self) -> bool:
        return all(getattr(p, "decode_capturable", False) for _, p in self._named_parts())

    @property
    def prompt_capturable(self) -> bool:
        return all(getattr(p, "prompt_capturable", False) for _, p in self._named_parts())

    def decode_graph_key(self, step: StepContext) -> tuple:
        return tuple(k for _, p in self._named_parts() if (k := p.decode_graph_key(step)))

    def forward(self, stream: ResidualStream, step: StepContext,
                cache: CacheHandle) -> None:
        h = self.mixer_norm.forward(stream)
        delta = self.mixer.forward(h, step, cache)
        if isinstance(delta, tuple):
            # (delta, a vector for every row): a mixer whose output projection has a bias
            delta, vec = delta
            stream.push_more(vec=vec)
        stream.push(delta)
        if self.ffn is not None:
            h = self.ffn_norm.forward(stream)
            stream.push(self.ffn.forward(h, step))
        if self.tail is not None:
            self.tail.forward(stream, step)


class SandwichBlock(PreNormBlock):
    """A norm before and behind each sublayer, and an optional per-channel scale on what
    joins the stream: ``x <- x + s1 * post1(mixer(pre1(x)))``; ``x <- x + s2 *
    post2(ffn(pre2(x)))``.  The norms behind the sublayers are of a kind that can ride on the
    pending delta (``norm.mapped(delta, scale, bias)``, e.g. ``DynamicTanhNorm``): they cost
    no pass of their own.  A sublayer may return ``(delta, vector)``: the vector (an output
    bias) is added to every row before the norm behind it.

    ``names``: prefixes of (pre1, mixer, post1, pre2, ffn, post2); ``scale_names``: the two
    scale vectors' tensor names, or None for a block without them."""

    def __init__(self, mixer_norm, mixer, mixer_post, ffn_norm, ffn, ffn_post, d_model: int,
                 names=("norm1", "mix", "norm1b", "norm2", "mlp", "norm2b"),
                 scale_names=("ls1", "ls2")):
        self.mixer_norm, self.mixer, self.mixer_post = mixer_norm, mixer, mixer_post
        self.ffn_norm, self.ffn, self.ffn_post = ffn_norm, ffn, ffn_post
        self.d_model = int(d_model)
        self.names, self.scale_names = tuple(names), scale_names
        self.scales = [None, None]

    def _named_parts(self):
        parts = (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn,
                 self.ffn_post)
        return [(n, p) for n, p in zip(self.names, parts) if p is not None]

    def tensor_specs(self) -> dict:
        from .base import TensorSpec
        out = super().tensor_specs()
        if self.scale_names is not None:
            out[self.scale_names[0]] = TensorSpec((self.d_model,), kind="vector", init="ones")
            if self.ffn is not None:
                out[self.scale_names[1]] = TensorSpec((self.d_model,), kind="vector", init="ones")
        return out

    def bind(self, tensors: dict, runtime) -> None:
        super().bind(tensors, runtime)
        if self.scale_names is not None:
            self.scales = [tensors[n].contiguous() if n in tensors else None
                           for n in self.scale_names]

    @staticmethod
    def _push(stream: ResidualStream, post, out, scale) -> None:
        bias = None
        if isinstance(out, tuple):
            out, bias = out
        stream.push(post.mapped(out, scale, bias))

    def forward(self, stream: ResidualStream, step: StepContext, cache: CacheHandle) -> None:
        h = self.mixer_norm.forward(stream)
        self._push(stream, self.mixer_post, self.mixer.forward(h, step, cache), self.scales[0])
        if self.ffn is None:
            return
        h = self.ffn_norm.forward(stream)
        self._push(stream, self.ffn_post, self.ffn.forward(h, step), self.scales[1])
