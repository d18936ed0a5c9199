"""Norms: RMS norm with a learned weight, layer norm with a weight and no bias, and the norm
without statistics (a scaled tanh with a weight and a bias).

Reference formula (train/model.py:29-33): ``xf = x.float()``;
``y = xf * rsqrt(mean(xf**2, -1) + eps)``; ``out = (y * w.float()).to(x.dtype)``.
eps sits inside the square root, added to the mean; the weight multiplies after
the normalisation; no bias.  All of it runs in float32 with one rounding at the
end.  The residual stream's pending addend is added in the same pass.
"""

from __future__ import annotations

import torch

from .base import Norm, ResidualStream, TensorSpec


class RMSNorm(Norm):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, dim: int, eps: float, tensor_name: str = "weight", one_plus: bool = False):
        """``tensor_name``: the local name of the weight ("" = the part's own prefix).
        ``one_plus``: the weight is stored around zero and multiplies as ``1 + w`` (the sum is
        taken once, in float32, when the weight is bound)."""
        self.dim = int(dim)
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.one_plus = bool(one_plus)
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.dim,), kind="vector",
                                             init="zeros" if self.one_plus else "ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        w = tensors[self.tensor_name]
        self.weight = (w.float() + 1.0).contiguous() if self.one_plus else w.contiguous()

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        """Add the pending delta into the stream, return the normalised rows.

        With ``rows`` (int32 row indices) only those rows are read, summed and
        normalised: the output is [n_rows, dim] and the stream itself is left
        as it was.
        """
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        if more_rows is not None or more_vec is not None:
            # (also before picked rows: the addends go into every row of the stream)
            rt.ops.residual_add(stream.x, more_rows, more_vec)
        delta = stream.take_pending()
        if rows is None:
            t = stream.x.shape[0]
            h = rt.buffer("normed", (t, self.dim), rt.act_dtype)
            rt.ops.add_rmsnorm(stream.x, delta, self.weight, self.eps, h)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
            rt.ops.gather_add_rmsnorm(stream.x, delta, rows, n_rows, self.weight,
                                      self.eps, h)
        return h


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w`` with the biased variance and no bias, in
    float32 with one rounding.  Adds the stream's pending delta and its other waiting
    addends (``ResidualStream.push_more``) in the same pass.  ``tensor_name`` is the
    local name of the weight ("" = the part's own prefix)."""

    decode_capturable = prompt_capturable = True

    def __init__(self, dim: int, eps: float, tensor_name: str = "weight"):
        self.dim, self.eps, self.tensor_name = int(dim), float(eps), tensor_name
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.dim,), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.tensor_name].contiguous()
        runtime.ops.require_part("layernorm")

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        delta = stream.take_pending()
        if rows is None:
            h = rt.buffer("normed", (stream.x.shape[0], self.dim), rt.act_dtype)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
        rt.ops.add_layernorm(stream.x, delta, self.weight, self.eps, h, rows=rows, n_rows=n_rows,
                             more_rows=more_rows, more_vec=more_vec)
        return h


class MappedDelta:
    """A sublayer's output that still has to pass an element-wise norm (and a per-channel
    scale) before it joins the residual stream: ``(n(delta + bias)) * scale``.  A consumer
    that knows the kind (``DynamicTanhNorm.forward``) applies the map in the pass in which it
    adds the delta; any other consumer gets the mapped values through ``resolve()`` (one
    kernel of its own, float32)."""

    def __init__(self, delta, norm: "DynamicTanhNorm", scale=None, bias=None):
        self.delta, self.norm, self.scale, self.bias = delta, norm, scale, bias

    @property
    def shape(self):
        return self.delta.shape

    def post(self) -> tuple:
        return (self.norm.alpha, self.norm.weight, self.norm.bias, self.scale)

    def release(self) -> None:
        if hasattr(self.delta, "release"):
            self.delta.release()

    def resolve(self):
        rt = self.norm.runtime
        t, d = self.delta.shape
        out = rt.buffer("mapped_delta", (t, d), torch.float32)
        rt.ops.add_tanh_norm(None, self.delta, None, None, post=self.post(), bias=self.bias,
                             y_out=out)
        return out

    def float(self):
        return self.resolve()


class DynamicTanhNorm(Norm):
    """``tanh(alpha * x) * w + b`` with a learned scalar ``alpha`` and vectors ``w``, ``b``: no
    mean, no variance, nothing reduced over the row; float32 inside, one rounding.

    Tensors: the weight under ``tensor_name`` ("" = the part's own prefix), ``alpha`` and
    ``b`` beside it.  As a block's first norm of a sublayer it adds the stream's pending
    delta in the same pass (``forward``); behind a sublayer it does not run by itself:
    ``mapped(delta, scale)`` wraps the sublayer's output, and whoever adds that to the
    stream applies the map while it reads the rows anyway."""

    decode_capturable = prompt_capturable = True

    def __init__(self, dim: int, tensor_name: str = "weight"):
        self.dim, self.tensor_name = int(dim), tensor_name
        self.weight = self.bias = None
        self.alpha = 1.0

    def _name(self, suffix: str) -> str:
        return f"{self.tensor_name}.{suffix}" if self.tensor_name else suffix

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.dim,), kind="vector", init="ones"),
                self._name("b"): TensorSpec((self.dim,), kind="vector", init="zeros"),
                self._name("alpha"): TensorSpec((), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.tensor_name].contiguous()
        self.bias = tensors[self._name("b")].to(self.weight.dtype).contiguous()
        self.alpha = float(tensors[self._name("alpha")])     # read once, at load time
        runtime.ops.require_part("tanhnorm")

    def mapped(self, delta, scale=None, bias=None) -> MappedDelta:
        """``delta`` (a tensor or ``SplitParts``; ``bias`` a vector added to every row first)
        as what this norm, then ``scale``, make of it, for ``ResidualStream.push``."""
        return MappedDelta(delta, self, scale, bias)

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        if more_rows is not None or more_vec is not None:
            rt.ops.require_part("layernorm")
            rt.ops.residual_add(stream.x, more_rows, more_vec)
        delta = stream.take_pending()
        post = bias = None
        if isinstance(delta, MappedDelta):
            post, bias, delta = delta.post(), delta.bias, delta.delta
        if rows is None:
            h = rt.buffer("normed", (stream.x.shape[0], self.dim), rt.act_dtype)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
        rt.ops.add_tanh_norm(stream.x, delta, (self.alpha, self.weight, self.bias), h, post=post,
                             bias=bias, rows=rows, n_rows=n_rows)
        return h
