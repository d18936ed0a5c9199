"""A model put together from parts: embedding, blocks in a given order, head.

Reference (train/model.py:220-244): ``embed -> blocks -> final_norm -> lm_head``
with ``lm_head.weight`` being ``embed.weight`` when tied (train/model.py:228-229).
Here the order in which blocks run is a list of calls: a call names a block
(the same block may be called twice) and the cache slot it uses; a call may
read the slot an earlier call filled instead of owning one.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import CacheHandle, Part, ResidualStream, StepContext, TensorSpec
from .block import join_name, under_prefix


@dataclass(frozen=True)
class LayerCall:
    layer: int                    # index into ComposedModel.blocks
    cache_slot: Optional[int]     # index into ComposedModel.cache_specs()
    writes: bool = True           # False: reads a slot an earlier call filled
    entry: Optional[tuple] = None  # (index into ComposedModel.entries, number of the pass):
    #                                what is added to the stream right before this call


class PassEntry(Part):
    """What enters the residual stream at the start of a pass over a run of layers that
    is repeated: before every pass but the first the embedding's output (the stream as
    it was before the first layer), and before every pass the pass's own row of a
    learned table ``[passes, d_model]``.  Both are handed to the stream as waiting
    addends, so the first norm of the pass adds them while it reads the rows anyway."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, passes: int, tensor_name: str = "step",
                 add_embedding: bool = True):
        self.d_model, self.passes = int(d_model), int(passes)
        self.tensor_name, self.add_embedding = tensor_name, add_embedding
        self.table = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.passes, self.d_model), kind="matrix")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.table = tensors[self.tensor_name].contiguous()

    def needs_embedding(self, number: int) -> bool:
        return self.add_embedding and number > 0

    def forward(self, stream: ResidualStream, number: int, embedded) -> None:
        stream.push_more(rows=embedded if (self.add_embedding and number > 0) else None,
                         vec=self.table[number])


class PassProjection(Part):
    """What happens to the residual stream at the start of every pass over a run of layers
    that is repeated (the first pass too): ``x <- W [x; x0]`` with x0 the embedding's
    output and ``W [d_model, 2 d_model]`` (x's columns first).  The stream's waiting
    addends are settled first; the product is written over the stream in float32."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, tensor_name: str = "in"):
        self.d_model, self.tensor_name = int(d_model), tensor_name
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.d_model, 2 * self.d_model))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = runtime.ops.prepare_weight(tensors[self.tensor_name])
        runtime.ops.require_part("layernorm")        # the stream's helpers live there

    def needs_embedding(self, number: int) -> bool:
        return True

    def forward(self, stream: ResidualStream, number: int, embedded) -> None:
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        if more_rows is not None or more_vec is not None:
            rt.ops.residual_add(stream.x, more_rows, more_vec)
        t = stream.x.shape[0]
        both = rt.buffer("pass_in", (t, 2 * self.d_model), rt.act_dtype)
        rt.ops.settle_concat(stream.x, stream.take_pending(), embedded, both)
        rt.ops.linear(both, self.weight, stream.x)


class TokenEmbedding(Part):
    """``x[t] = E[token[t]] * scale``, plus the vector of an additive position part
    (``position``, e.g. ``SinusoidalPositions``) if there is one.  (The reference has neither
    scaling nor a position term: ``scale`` 1, train/model.py:239.)"""

    decode_capturable = prompt_capturable = True

    def __init__(self, vocab_size: int, d_model: int, tensor_name: str = "weight",
                 scale: float = 1.0, position=None):
        self.vocab_size, self.d_model = int(vocab_size), int(d_model)
        self.tensor_name, self.scale = tensor_name, float(scale)
        self.position = position
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.vocab_size, self.d_model))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.tensor_name].contiguous()
        if self.position is not None:
            self.position.bind({}, runtime)

    def forward(self, step: StepContext, buffer: str = "residual"):
        rt = self.runtime
        x = rt.buffer(buffer, (step.n_tokens, self.d_model), rt.residual_dtype)
        if self.position is not None:
            rt.ops.embed(step.token_ids, self.weight, x, self.vocab_size, self.scale,
                         positions=step.positions, freq=self.position.freq)
        else:
            rt.ops.embed(step.token_ids, self.weight, x, self.vocab_size, self.scale)
        return x


class OutputHead(Part):
    """``logits = (h @ W^T) * scale`` in float32; W is the embedding table when tied.  With
    ``softcap`` c > 0 the logits then become ``c * tanh(logits / c)``."""

    decode_capturable = prompt_capturable = True

    def __init__(self, vocab_size: int, d_model: int, tied_to: Optional[TokenEmbedding],
                 tensor_name: str = "weight", scale: float = 1.0, softcap: float = 0.0):
        self.vocab_size, self.d_model = int(vocab_size), int(d_model)
        self.tied_to = tied_to
        self.tensor_name, self.scale, self.softcap = tensor_name, float(scale), float(softcap)
        self.weight = None

    def tensor_specs(self) -> dict:
        if self.tied_to is not None:
            return {}
        return {self.tensor_name: TensorSpec((self.vocab_size, self.d_model))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        w = self.tied_to.weight if self.tied_to is not None else tensors[self.tensor_name]
        self.weight = runtime.ops.prepare_weight(w)

    def forward(self, h, n_rows: int):
        rt = self.runtime
        logits = rt.buffer("logits", (n_rows, self.vocab_size), rt.logits_dtype)
        rt.ops.linear(h, self.weight, logits)
        if self.scale != 1.0:
            rt.ops.scale_(logits, self.scale)
        if self.softcap > 0.0:
            rt.ops.softcap_(logits, self.softcap)
        return logits


class ComposedModel:
    """Embedding, blocks, the list of calls, final norm and output head."""

    def __init__(self, config, embedding: TokenEmbedding, blocks: list,
                 calls: list, final_norm, head: OutputHead,
                 names=("embed", "blocks", "final_norm", "lm_head"), aliases=None,
                 block_prefix=None, entries=()):
        """``names``: prefixes of the embedding's, the blocks', the final norm's and the
        head's tensors; ``block_prefix(i)`` overrides ``"<blocks>.<i>"``.  ``entries``:
        ``[(prefix, PassEntry)]`` that calls refer to by ``LayerCall.entry``."""
        self.config = config
        self._block_prefix = block_prefix or (lambda i: f"{names[1]}.{i}")
        self.entries = list(entries)
        self._aliases = aliases          # callable: tensor name -> other names a file may use
        self.embedding, self.blocks, self.calls = embedding, list(blocks), list(calls)
        self.final_norm, self.head = final_norm, head
        self.names = tuple(names)
        self.runtime = None
        # one cache spec per slot, taken from the block of the call that owns it
        self._slot_specs = []
        for call in self.calls:
            if call.cache_slot is None:
                continue
            if call.writes:
                if call.cache_slot != len(self._slot_specs):
                    raise ValueError("cache slots must be numbered in call order")
                self._slot_specs.append(self.blocks[call.layer].cache_spec())
            elif not (0 <= call.cache_slot < len(self._slot_specs)):
                raise ValueError("a call reads a cache slot no earlier call owns")

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> dict:
        e, b, f, h = self.names
        out = {join_name(e, n): s for n, s in self.embedding.tensor_specs().items()}
        for prefix, part in self.entries:
            out.update({join_name(prefix, n): s for n, s in part.tensor_specs().items()})
        for i, blk in enumerate(self.blocks):
            for n, s in blk.tensor_specs().items():
                out[join_name(self._block_prefix(i), n)] = s
        out.update({join_name(f, n): s for n, s in self.final_norm.tensor_specs().items()})
        out.update({join_name(h, n): s for n, s in self.head.tensor_specs().items()})
        return out

    def name_aliases(self) -> dict:
        """For the names of ``tensor_specs`` and ``tied_names``: other spellings a
        weight file may use for the same tensor (the architecture's builder says which)."""
        if self._aliases is None:
            return {}
        names = list(self.tensor_specs()) + list(self.tied_names())
        return {n: a for n in names if (a := list(self._aliases(n)))}

    def tied_names(self) -> dict:
        """Names a file may hold although the model takes them from another."""
        e, _, _, h = self.names
        if self.head.tied_to is not None and h:
            return {f"{h}.weight": join_name(e, self.embedding.tensor_name)}
        return {}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        e, b, f, h = self.names

        def sub(prefix):
            return under_prefix(tensors, prefix) if prefix else {}

        self.embedding.bind(sub(e), runtime)
        for prefix, part in self.entries:
            part.bind(sub(prefix), runtime)
        for i, blk in enumerate(self.blocks):
            blk.bind(sub(self._block_prefix(i)), runtime)
        self.final_norm.bind(sub(f), runtime)
        self.head.bind(sub(h), runtime)

    # -------------------------------------------------------------------- cache
    def cache_specs(self) -> list:
        return list(self._slot_specs)

    # ------------------------------------------------------------------- graphs
    def _all_parts(self) -> list:
        return [self.embedding, *(p for _, p in self.entries), *self.blocks, self.final_norm,
                self.head]

    @property
    def decode_capturable(self) -> bool:
        """Whether a step of single decoded tokens may be replayed from a CUDA graph:
        only if every part says so (``Part.decode_capturable``)."""
        return all(getattr(p, "decode_capturable", False) for p in self._all_parts())

    @property
    def prompt_capturable(self) -> bool:
        """The same for a step of any shape (``Part.prompt_capturable``)."""
        return all(getattr(p, "prompt_capturable", False) for p in self._all_parts())

    def decode_graph_key(self, step: StepContext) -> tuple:
        """What the parts add to the key of a decode step's graph, without repeats."""
        seen = []
        for p in self._all_parts():
            k = p.decode_graph_key(step)
            if k and k not in seen:
                seen.append(k)
        return tuple(seen)

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepContext, handles: list):
        """Run the step's tokens; float32 logits [n_out, vocab] at ``out_rows``."""
        self.runtime.ops.begin_step(step.n_tokens)
        stream = ResidualStream(self.embedding.forward(step))
        embedded = None
        if any(c.entry is not None and self.entries[c.entry[0]][1].needs_embedding(c.entry[1])
               for c in self.calls):
            # the stream moves on in place: a pass that starts over from the embedding's
            # output reads a second copy of it
            embedded = self.embedding.forward(step, buffer="embedded")
        none = CacheHandle()
        for call in self.calls:
            if call.entry is not None:
                self.entries[call.entry[0]][1].forward(stream, call.entry[1], embedded)
            handle = none
            if call.cache_slot is not None:
                handle = handles[call.cache_slot]
                if not call.writes:
                    handle = handle.reader()
            self.blocks[call.layer].forward(stream, step, handle)
        if step.n_out == 0:
            stream.drop_pending()
            return None
        h = self.final_norm.forward(stream, rows=step.out_rows, n_rows=step.n_out)
        return self.head.forward(h, step.n_out)
