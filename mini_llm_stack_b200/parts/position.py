"""Rotary position encoding: rotate-half pairing over the whole head by table
(``RotaryPosition``), and a rotation of a head's first entries with either pairing and
scaled frequencies (``PartialRotary``); a sinusoidal vector added to the embedding
(``SinusoidalPositions``).

Reference (train/model.py:36-52): ``inv_freq[i] = theta ** -(2i / head_dim)``
for i in [0, head_dim/2); ``angle[p, i] = p * inv_freq[i]``; cos and sin tables
[max_seq_len, head_dim/2] are built in float32.  Applied to q and k only:
``x1, x2 = halves of x``; ``out = cat(x1*cos - x2*sin, x2*cos + x1*sin)`` with
the row of the tables picked by the token's absolute position
(serve/engine.py:53-58 for single decoded tokens).  The tables are built on
the host with the reference's own expression so that every machine holds the
same float32 values; the rotation itself runs in float32 and rounds once.
"""

from __future__ import annotations

import torch

from .base import CacheHandle, PositionEncoding, StepContext


def rotary_tables(head_dim: int, max_positions: int, theta: float):
    """cos, sin [max_positions, head_dim/2] in float32 (train/model.py:41-45)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    t = torch.arange(max_positions).float()
    freqs = torch.outer(t, inv_freq)
    return freqs.cos(), freqs.sin()


class RotaryPosition(PositionEncoding):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream
    applies_to = "qk"

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.cos = self.sin = None

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        cos, sin = rotary_tables(self.head_dim, self.max_positions, self.theta)
        self.cos = cos.contiguous().to(runtime.device)
        self.sin = sin.contiguous().to(runtime.device)

    @property
    def takes_parts(self) -> bool:
        """Whether ``rotate_and_store`` accepts ``parts`` (the projection left as the
        parts of a cut along K) in place of filled ``qkv`` rows."""
        return self.runtime.ops.rope_takes_parts(self.head_dim)

    def fused_tables(self):
        """(cos, sin, max_positions) for a mixer whose kernel rotates by table row itself
        (rotate-half of q and k, k and v stored at the step's slots), or None if this
        encoding cannot be applied that way."""
        return self.cos, self.sin, self.max_positions

    def rotate_and_store(self, qkv, step: StepContext, cache: CacheHandle,
                         n_heads: int, n_kv_heads: int, parts=None) -> None:
        """Rotate q and k of ``qkv`` in place; store rotated k and raw v.

        The keys and values of this step's tokens go into the pages before
        attention runs (write-then-attend, serve/engine.py:99-100,137-139).
        A call that reads another call's cache (``cache.writes`` False) rotates
        only its queries.
        """
        g = step.groups[cache.group]
        self.runtime.ops.rope_store(
            qkv, step.positions, self.cos, self.sin, g.slot_map,
            cache.k_pool, cache.v_pool, step.n_tokens, n_heads, n_kv_heads,
            self.head_dim, self.max_positions, cache.writes, parts=parts)


class PartialRotary(PositionEncoding):
    """Rotation of the first ``dims`` entries of every head; the rest pass unchanged.

    The pair number i (0 <= i < dims/2) at position p turns by the angle
    ``p * base^(-2i/dims) / factor`` (``factor``: linear scaling of the frequencies):
    ``(u, v) -> (u cos - v sin, v cos + u sin)``.  ``pairing`` says which entries form
    pair i: "interleaved" (2i, 2i + 1) or "half" (i, i + dims/2).  There is no table
    and so no bound on the positions: the kernels that rotate form the angle in float64
    from the position and this part's float64 frequencies, and round its cosine and
    sine once to float32."""

    decode_capturable = prompt_capturable = True

    def __init__(self, dims: int, base: float, factor: float = 1.0, pairing: str = "half"):
        if pairing not in ("interleaved", "half"):
            raise ValueError(f"pairing must be 'interleaved' or 'half', not {pairing!r}")
        if dims < 0 or dims % 2:
            raise ValueError("the rotated entries of a head come in pairs")
        self.dims, self.base, self.factor = int(dims), float(base), float(factor)
        self.pairing = pairing
        self.freq = None

    def frequencies(self):
        """``base^(-2i/dims) / factor`` for i < dims/2, float64 on the host."""
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.base, dtype=torch.float64),
                         -2.0 * i / max(self.dims, 1)) / self.factor

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.freq = self.frequencies().to(runtime.device).contiguous()


class SinusoidalPositions(PositionEncoding):
    """A vector added to a token's embedding: entry 2i is ``sin(p * base^(-2i/width))`` and
    entry 2i + 1 the cosine of the same angle, p the token's position.  There is no table and
    so no bound on the positions: the embedding kernel forms the angle in float64 from the
    position and this part's float64 frequencies."""

    decode_capturable = prompt_capturable = True

    def __init__(self, width: int, base: float = 10000.0):
        self.width, self.base = int(width), float(base)
        self.freq = None

    def frequencies(self):
        """``base^(-2i/width)`` for every pair of entries, float64 on the host."""
        i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.width)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.freq = self.frequencies().to(runtime.device).contiguous()
