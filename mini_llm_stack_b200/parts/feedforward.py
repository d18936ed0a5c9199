"""Feed-forwards: dense SwiGLU, a clamped gated unit, an ungated unit with the square of
relu, and routed experts.

Reference (train/model.py:127-135): ``w_down(silu(w_gate x) * (w_up x))`` with
``silu(z) = z * sigmoid(z)``, no biases.  Gate and up share one projection
here; ``silu(gate) * up`` is computed in float32, in the projection's own
epilogue where the tcgen05 kernel takes the sizes.
"""

from __future__ import annotations

import torch

from .base import FeedForward, StepContext, TensorSpec


class SwiGLUFeedForward(FeedForward):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, d_model: int, intermediate_size: int,
                 names=("w_gate.weight", "w_up.weight", "w_down.weight")):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.names = tuple(names)             # local names of the gate, up and down matrices
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        g, u, dn = self.names
        return {g: TensorSpec((i, d)), u: TensorSpec((i, d)), dn: TensorSpec((d, i))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        tensors = {"w_gate.weight": tensors[self.names[0]], "w_up.weight": tensors[self.names[1]],
                   "w_down.weight": tensors[self.names[2]]}
        parts = [tensors["w_gate.weight"], tensors["w_up.weight"]]
        if parts[0].dtype != parts[1].dtype:
            parts = [p.float() for p in parts]
        ops = runtime.ops
        # one kernel for projection and activation where the tensor-core kernel takes
        # the sizes: its weight holds gate and up rows interleaved in blocks of 16
        self.fused = (parts[0].dtype == torch.bfloat16
                      and ops.can_fuse_swiglu(self.d_model, self.intermediate_size))
        if self.fused:
            self.w_gate_up = ops.prepare_weight(ops.interleave_gate_up(parts[0], parts[1]))
        else:
            self.w_gate_up = ops.prepare_weight(torch.cat(parts, dim=0))
        self.w_down = ops.prepare_weight(tensors["w_down.weight"])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        i = self.intermediate_size
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        if self.fused:
            rt.ops.linear_swiglu(h, self.w_gate_up, act)
        else:
            gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
            rt.ops.linear(h, self.w_gate_up, gu)
            rt.ops.swiglu(gu, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)


class ClampedGLUFeedForward(FeedForward):
    """``W_down (g' * sigmoid(alpha * g') * (u' + 1))`` with ``g' = min(W_gate h, limit)``
    and ``u' = clamp(W_up h, -limit, limit)``; no biases.  The activation runs in
    float32, in the projection's own epilogue where the tcgen05 kernel takes the sizes
    (as ``SwiGLUFeedForward`` does), else on the projection's output."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 names=("gate", "up", "down")):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.names = tuple(names)

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        g, u, dn = self.names
        return {g: TensorSpec((i, d)), u: TensorSpec((i, d)), dn: TensorSpec((d, i))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        g, u, dn = self.names
        ops = runtime.ops
        self.fused = (tensors[g].dtype == torch.bfloat16 and tensors[u].dtype == torch.bfloat16
                      and ops.can_fuse_swiglu(self.d_model, self.intermediate_size))
        if self.fused:
            self.w_gate_up = ops.prepare_weight(ops.interleave_gate_up(tensors[g], tensors[u]))
        else:
            self.w_gate_up = ops.prepare_weight(torch.cat([tensors[g], tensors[u]], dim=0))
        self.w_down = ops.prepare_weight(tensors[dn])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t, i = h.shape[0], self.intermediate_size
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        if self.fused:
            rt.ops.linear_clamped_glu(h, self.w_gate_up, act, self.alpha, self.limit)
        else:
            gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
            rt.ops.linear(h, self.w_gate_up, gu)
            rt.ops.clamped_glu(gu, act, self.alpha, self.limit)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)


class SquaredReluFeedForward(FeedForward):
    """``W_down relu(W_up h + b_up)^2 + b_down``: no gate; the biases (tensors ``<up>.b``,
    ``<down>.b``) only with ``biases``.  The activation runs in float32, in the projection's
    own epilogue where the tcgen05 kernel takes the sizes (as ``SwiGLUFeedForward`` does), else
    on the projection's output (left in float32 where a bias is still to be added).  With
    biases ``forward`` returns ``(delta, b_down)``: the block adds the vector to every row."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, intermediate_size: int, names=("up", "down"),
                 biases: bool = False):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.names, self.biases = tuple(names), bool(biases)
        self.b_up = self.b_down = None

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        up, down = self.names
        out = {up: TensorSpec((i, d))}
        if self.biases:
            out[f"{up}.b"] = TensorSpec((i,), kind="vector", init="zeros")
        out[down] = TensorSpec((d, i))
        if self.biases:
            out[f"{down}.b"] = TensorSpec((d,), kind="vector", init="zeros")
        return out

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.w_up = runtime.ops.prepare_weight(tensors[self.names[0]])
        self.w_down = runtime.ops.prepare_weight(tensors[self.names[1]])
        if self.biases:
            self.b_up = tensors[f"{self.names[0]}.b"].contiguous()
            self.b_down = tensors[f"{self.names[1]}.b"].contiguous()
        self.fused = (self.w_up.dtype == torch.bfloat16
                      and runtime.ops.can_fuse_activation(self.d_model))

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        act = rt.buffer("ffn_act", (t, self.intermediate_size), rt.act_dtype)
        if self.fused:
            rt.ops.linear_relu_squared(h, self.w_up, act, bias=self.b_up)
        elif self.b_up is not None:
            z = rt.buffer("ffn_up", (t, self.intermediate_size), torch.float32)
            rt.ops.linear(h, self.w_up, z)
            rt.ops.relu_squared(z, act, bias=self.b_up)
        else:
            rt.ops.linear(h, self.w_up, act)
            rt.ops.relu_squared(act, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        delta = rt.ops.linear_parts(act, self.w_down, delta)
        return (delta, self.b_down) if self.b_down is not None else delta


class RoutedExperts(FeedForward):
    """A mixture of small SwiGLU experts behind a float32 router.

    Router logits ``z = W_r h`` and scores ``s = sigmoid(z)`` or, with ``score="softmax"``,
    ``softmax(z)`` over all router outputs, in float32; a token takes its ``top`` outputs
    with the largest scores (lowest index on a tie; with ``correction`` the vector
    ``correction`` [outputs] is added for the choice only) and weighs them by the scores
    themselves (``renormalise``: divided by their sum + ``renorm_eps``).  ``weigh`` says
    where a weight multiplies: "input" (the expert sees ``w * h``) or "output".  The last
    ``identity`` router outputs stand for experts without tensors that return their input
    (times the weight).  A ``shared`` feed-forward, if any, runs for every token and is
    added; with ``shared_gate`` it is first multiplied by ``sigmoid(w_sg . h)``, one number a
    token (tensor ``shared.sg`` [1, d]).  ``groups = (count, keep)``: the router's outputs form
    ``count`` equal groups of neighbours, a group's score is the sum of its two largest choice
    scores, and only outputs of the ``keep`` best groups can be chosen.  ``limit`` > 0: the
    experts are clamped units, ``g' * sigmoid(alpha g') * (u' + 1)`` with ``g' = min(g, limit)``
    and ``u' = clamp(u, -limit, limit)``, instead of ``silu(g) * u``.  Tensors: ``router``
    [E + identity, d] and ``e<i>.gate / up / down`` for each of the E experts; the shared
    part's under ``shared``."""

    decode_capturable = prompt_capturable = True   # routing, sorting and the products stay on the device

    def __init__(self, d_model: int, n_experts: int, top: int, expert_size: int, shared=None,
                 weigh: str = "input", renormalise: bool = False, score: str = "sigmoid",
                 correction: bool = False, identity: int = 0, renorm_eps: float = 0.0,
                 groups=None, limit: float = 0.0, alpha: float = 1.0, shared_gate: bool = False):
        if weigh not in ("input", "output"):
            raise ValueError(f"weigh must be 'input' or 'output', not {weigh!r}")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"score must be 'sigmoid' or 'softmax', not {score!r}")
        if not 0 < int(top) <= int(n_experts) + int(identity):
            raise ValueError("top must lie in 1..n_experts + identity")
        if identity and weigh != "output":
            raise ValueError("experts that return their input are weighed on their output")
        self.d_model, self.n_experts, self.top = int(d_model), int(n_experts), int(top)
        self.expert_size, self.shared = int(expert_size), shared
        self.weigh, self.renormalise = weigh, bool(renormalise)
        self.score, self.has_correction = score, bool(correction)
        self.identity, self.renorm_eps = int(identity), float(renorm_eps)
        self.n_outputs = self.n_experts + self.identity
        self.correction = None
        self.groups = (int(groups[0]), int(groups[1])) if groups else None
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or self.n_outputs % count or not 1 <= keep <= count:
                raise ValueError("the router's outputs must form equal groups, of which some are kept")
            if self.top > keep * (self.n_outputs // count):
                raise ValueError("the kept groups hold fewer outputs than a token takes")
        self.limit, self.alpha = float(limit), float(alpha)
        self.shared_gate = bool(shared_gate)
        if self.shared_gate and shared is None:
            raise ValueError("a gate on the shared expert needs a shared expert")

    def tensor_specs(self) -> dict:
        d, f = self.d_model, self.expert_size
        out = {"router": TensorSpec((self.n_outputs, d))}
        if self.has_correction:
            out["correction"] = TensorSpec((self.n_outputs,), kind="vector", init="zeros")
        for i in range(self.n_experts):
            out[f"e{i}.gate"] = TensorSpec((f, d))
            out[f"e{i}.up"] = TensorSpec((f, d))
            out[f"e{i}.down"] = TensorSpec((d, f))
        if self.shared is not None:
            out.update({f"shared.{n}": s for n, s in self.shared.tensor_specs().items()})
        if self.shared_gate:
            out["shared.sg"] = TensorSpec((1, d))
        return out

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        n = self.n_experts
        self.w_router = tensors["router"].float().contiguous()       # scores are float32
        if self.shared_gate:
            # the gate's row rides behind the router's: one float32 product gives both
            self.w_router = torch.cat([self.w_router, tensors["shared.sg"].float()], 0).contiguous()
        if self.has_correction:
            self.correction = tensors["correction"].float().contiguous()
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{i}.gate"], tensors[f"e{i}.up"]], 0)
                                      for i in range(n)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{i}.down"] for i in range(n)]).contiguous()
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items()
                              if k.startswith("shared.") and k != "shared.sg"}, runtime)
        runtime.ops.require_part("experts")

    def _work(self, t: int) -> dict:
        rt, n_slots = self.runtime, t * self.top
        tiles = rt.ops.expert_max_tiles(n_slots, self.n_experts)   # outputs without weights get none
        i32 = torch.int32
        return {"idx": rt.buffer("route_idx", (n_slots,), i32),
                "weight": rt.buffer("route_weight", (n_slots,), torch.float32),
                "order": rt.buffer("route_order", (n_slots,), i32),
                "offsets": rt.buffer("route_offsets", (self.n_outputs + 1,), i32),
                "cursor": rt.buffer("route_cursor", (self.n_outputs,), i32),
                "tile_expert": rt.buffer("route_tile_expert", (tiles,), i32),
                "tile_row0": rt.buffer("route_tile_row0", (tiles,), i32),
                "max_tiles": tiles}

    def forward(self, h, step: StepContext):
        rt, ops = self.runtime, self.runtime.ops
        t = h.shape[0]
        logits = rt.buffer("route_logits", (t, self.w_router.shape[0]), torch.float32)
        ops.linear(h, self.w_router, logits)
        work = self._work(t)
        ops.route(logits, self.top, self.renormalise, work, softmax=self.score == "softmax",
                  correction=self.correction, renorm_eps=self.renorm_eps, n_real=self.n_experts,
                  groups=self.groups, n_outputs=self.n_outputs)
        n_slots = t * self.top
        y = rt.buffer("expert_act", (n_slots, self.expert_size), rt.act_dtype)
        per_slot = rt.buffer("expert_out", (n_slots, self.d_model), torch.float32)
        ops.expert_glu(h, self.w_gate_up, y, work, self.top, self.weigh == "input",
                       alpha=self.alpha, limit=self.limit)
        ops.expert_down(y, self.w_down, per_slot, work, self.top, self.weigh == "output")
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(h, step)
            if not isinstance(shared, torch.Tensor):
                shared = shared.float()              # a product left as its K-parts
        delta = rt.buffer("routed_delta", (t, self.d_model), rt.act_dtype)
        gate = logits[:, self.n_outputs] if self.shared_gate else None
        if self.identity:
            ops.expert_combine(per_slot, self.top, shared, delta, work=work,
                               n_real=self.n_experts, h=h, shared_gate=gate)
        else:
            ops.expert_combine(per_slot, self.top, shared, delta, shared_gate=gate)
        return delta
