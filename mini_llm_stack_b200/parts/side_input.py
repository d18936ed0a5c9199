"""A layer's input from a per-token side table.

The model holds one table ``[vocab, layers * dim]`` (``SideTable``); layer i owns the columns
``[i * dim, (i + 1) * dim)``.  At the end of a layer, on the residual stream x as the layer's
other parts leave it (not normalised), ``TokenSideInput`` adds

    e = table[token][i * dim : (i + 1) * dim]
    g = gelu_tanh(W_gate x) * e
    y = W_proj g
    x <- x + y / sqrt(mean(y^2) + eps) * w_norm          (a plain weight)

The stream's pending delta is settled first (one kernel that also leaves x in the activation
type for the gate's product); the normalised y is pushed as the stream's next pending delta,
so the next norm adds it while it reads the rows anyway.  The gate's outputs are padded with
zeros to whole 16-byte rows for the products.
"""

from __future__ import annotations

import torch

from .base import Part, ResidualStream, StepContext, TensorSpec


class SideTable(Part):
    """The table itself, a tensor of the model (``embed`` under the part's prefix)."""

    decode_capturable = prompt_capturable = True

    def __init__(self, vocab_size: int, width: int, tensor_name: str = "embed"):
        self.vocab_size, self.width, self.tensor_name = int(vocab_size), int(width), tensor_name
        self.table = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.vocab_size, self.width))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.table = tensors[self.tensor_name].contiguous()


class TokenSideInput(Part):
    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, dim: int, column: int, table: SideTable, eps: float):
        self.d_model, self.dim, self.column = int(d_model), int(dim), int(column)
        self.table, self.eps = table, float(eps)
        self.pad = -(-self.dim // 8) * 8

    def tensor_specs(self) -> dict:
        return {"gate": TensorSpec((self.dim, self.d_model)),
                "proj": TensorSpec((self.d_model, self.dim)),
                "norm": TensorSpec((self.d_model,), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        gate, proj = tensors["gate"], tensors["proj"]
        if self.pad != self.dim:
            g = gate.new_zeros((self.pad, self.d_model))
            g[:self.dim] = gate
            p = proj.new_zeros((self.d_model, self.pad))
            p[:, :self.dim] = proj
            gate, proj = g, p
        self.w_gate = runtime.ops.prepare_weight(gate)
        self.w_proj = runtime.ops.prepare_weight(proj)
        self.w_norm = tensors["norm"].float().contiguous()
        runtime.ops.require_part("side")

    def forward(self, stream: ResidualStream, step: StepContext) -> None:
        rt, ops = self.runtime, self.runtime.ops
        t = step.n_tokens
        more_rows, more_vec = stream.take_more()
        if more_rows is not None or more_vec is not None:
            ops.require_part("layernorm")
            ops.residual_add(stream.x, more_rows, more_vec)
        x_act = rt.buffer("side_x", (t, self.d_model), rt.act_dtype)
        ops.settle_cast(stream.x, stream.take_pending(), x_act)
        z = rt.buffer("side_z", (t, self.pad), torch.float32)
        ops.linear(x_act, self.w_gate, z)
        g = rt.buffer("side_g", (t, self.pad), rt.act_dtype)
        ops.gelu_gate_rows(z, self.table.table, self.column, step.token_ids, g, n_real=self.dim)
        y = rt.buffer("side_y", (t, self.d_model), torch.float32)
        y = ops.linear_parts(g, self.w_proj, y)
        delta = rt.buffer("side_delta", (t, self.d_model), torch.float32)
        ops.rms_scale(y, self.w_norm, self.eps, delta)
        stream.push(delta)
