"""Movazen: layers of windowed attention with a bias on the distance, or of softmax attention
beside lightning attention, each followed by routed experts or nothing and by an input from a
per-token side table; RMS norms whose weights are stored around zero, a scaled embedding with a
sinusoidal position vector, an untied output head.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1 / norm2``, ``l<i>.mix.*`` (``left.*`` and
``right.*`` inside a parallel mixer), ``l<i>.mlp.*``, ``l<i>.side.gate / proj / norm``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.movazen_config import MovazenConfig
from ..config.registry import register_architecture
from .attention import UnrotatedAttention, distance_slopes
from .block import PreNormBlock
from .feedforward import ClampedGLUFeedForward, RoutedExperts
from .linear_recurrence import LightningAttention
from .model import ComposedModel, LayerCall, OutputHead, TokenEmbedding
from .norm import RMSNorm
from .parallel import ParallelMixer
from .position import SinusoidalPositions
from .side_input import SideTable, TokenSideInput

RENORM_EPS = 1e-20       # added to the sum of the chosen experts' scores before the division
GATE_ALPHA = 1.702       # the experts' gate: g * sigmoid(GATE_ALPHA * g)
POSITION_BASE = 10000.0


def _mixer(cfg: MovazenConfig, layer: dict):
    m = layer["mixer"]
    if layer["type"] == "attention":
        mask = m.get("mask") or {}
        return UnrotatedAttention(cfg.width, m["heads"], m["kv_heads"], m["dim"], m["vdim"],
                                  m["scale"], cfg.norm_eps, window=mask.get("size"),
                                  keep_first=mask.get("keep_first", 0), head_norm=True,
                                  slopes=distance_slopes(m["heads"]), gate=True)
    left, right = m["left"], m["right"]
    temp = left.get("q_temp")
    return ParallelMixer(
        cfg.width,
        UnrotatedAttention(cfg.width, left["heads"], left["kv_heads"], left["dim"], left["vdim"],
                           left["scale"], cfg.norm_eps, qkv_bias=True, zero_sink=True,
                           q_temp=(temp["coef"], temp["every"]) if temp else None,
                           v_scale=m["left_scale"], project=False),
        LightningAttention(cfg.width, right["heads"], right["dim"], right["vdim"], right["decay"],
                           cfg.norm_eps, out_scale=m["right_scale"], project=False))


def _feedforward(cfg: MovazenConfig, mlp):
    if mlp is None:
        return None
    shared = None
    if mlp.get("shared") is not None:
        shared = ClampedGLUFeedForward(cfg.width, mlp["shared"]["ff"], mlp["shared"]["limit"],
                                       alpha=GATE_ALPHA, names=("gate", "up", "down"))
    router = mlp["router"]
    groups = router.get("groups")
    return RoutedExperts(cfg.width, router["experts"], router["top"], mlp["expert"]["ff"],
                         shared=shared, weigh="output", renormalise=True, score="sigmoid",
                         correction=True, renorm_eps=RENORM_EPS,
                         groups=(groups["count"], groups["keep"]) if groups else None,
                         limit=mlp["expert"]["limit"], alpha=GATE_ALPHA,
                         shared_gate=shared is not None)


def build_movazen(cfg: MovazenConfig) -> ComposedModel:
    embedding = TokenEmbedding(cfg.vocab, cfg.width, tensor_name="", scale=cfg.embedding_scale,
                               position=SinusoidalPositions(cfg.width, POSITION_BASE))

    def norm():
        return RMSNorm(cfg.width, cfg.norm_eps, tensor_name="", one_plus=True)

    entries, table = [], None
    if cfg.side_dim:
        table = SideTable(cfg.vocab, len(cfg.layers) * cfg.side_dim, tensor_name="embed")
        entries.append(("side", table))
    blocks, calls = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = _feedforward(cfg, layer.get("mlp"))
        tail = (TokenSideInput(cfg.width, cfg.side_dim, i * cfg.side_dim, table, cfg.norm_eps)
                if table is not None else None)
        blocks.append(PreNormBlock(norm(), _mixer(cfg, layer), norm() if ffn is not None else None,
                                   ffn, names=("norm1", "mix", "norm2", "mlp", "side"), tail=tail))
        calls.append(LayerCall(i, i, writes=True))
    return ComposedModel(cfg, embedding, blocks, calls, norm(),
                         OutputHead(cfg.vocab, cfg.width, tied_to=None, tensor_name=""),
                         names=("embed", None, "final.norm", "head"),
                         block_prefix=lambda i: f"l{i}", entries=entries)


register_architecture("Movazen", MovazenConfig, build_movazen, aliases=("movazen",))
