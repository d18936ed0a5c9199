"""Zefenex: layers of latent attention with a rotated key part, a window, a sink and an output
gate, each followed by a dense or a routed feed-forward; the norm without statistics before
and behind every sublayer, a per-channel scale on what joins the stream, a scaled embedding
and capped logits.  A layer may read the cache of an earlier layer instead of filling one.

Tensor names: ``embed``, ``l<i>.norm1 / norm1b / norm2 / norm2b`` (with ``.b`` and ``.alpha``
beside each), ``l<i>.ls1 / ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zefenex_config import ZefenexConfig
from .block import SandwichBlock
from .feedforward import RoutedExperts, SquaredReluFeedForward, SwiGLUFeedForward
from .latent_attention import RotaryLatentAttention
from .model import ComposedModel, LayerCall, OutputHead, TokenEmbedding
from .norm import DynamicTanhNorm
from .position import PartialRotary

RENORM_EPS = 1e-20       # added to the sum of the chosen experts' scores before the division


def _mixer(cfg: ZefenexConfig, index: int):
    m = cfg.layers[index]["mixer"]
    rot = m.get("rot")
    position = PartialRotary(rot["dims"], rot["base"], 1.0, "half") if rot and rot["dims"] else None
    own = m.get("kv_from") is None
    return RotaryLatentAttention(
        cfg.width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"],
        cfg.norm_eps, position=position, window=(m.get("mask") or {}).get("size"),
        sink=True, gate=True, own_cache=own,
        cache_window=cfg.kept_window(index) if own else None)


def _feedforward(cfg: ZefenexConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return SquaredReluFeedForward(cfg.width, mlp["ff"], names=("up", "down"), biases=True)
    shared = None
    if mlp.get("shared") is not None:
        shared = SwiGLUFeedForward(cfg.width, mlp["shared"]["ff"], names=("gate", "up", "down"))
    router = mlp["router"]
    return RoutedExperts(cfg.width, router["experts"], router["top"], mlp["expert"]["ff"],
                         shared=shared, weigh="output", renormalise=True, score="softmax",
                         correction=True, identity=router.get("identity") or 0,
                         renorm_eps=RENORM_EPS)


def build_zefenex(cfg: ZefenexConfig) -> ComposedModel:
    embedding = TokenEmbedding(cfg.vocab, cfg.width, tensor_name="", scale=cfg.embedding_scale)

    def norm():
        return DynamicTanhNorm(cfg.width, tensor_name="")

    blocks, calls, slot_of_layer = [], [], {}
    for i, layer in enumerate(cfg.layers):
        ffn = _feedforward(cfg, layer.get("mlp"))
        blocks.append(SandwichBlock(norm(), _mixer(cfg, i), norm(),
                                    norm() if ffn is not None else None, ffn,
                                    norm() if ffn is not None else None, cfg.width))
        src = layer["mixer"].get("kv_from")
        if src is None:
            slot_of_layer[i] = len(slot_of_layer)
            calls.append(LayerCall(i, slot_of_layer[i], writes=True))
        else:
            calls.append(LayerCall(i, slot_of_layer[src], writes=False))
    return ComposedModel(cfg, embedding, blocks, calls, norm(),
                         OutputHead(cfg.vocab, cfg.width, tied_to=None, tensor_name="",
                                    softcap=cfg.logit_softcap),
                         names=("embed", None, "final.norm", "head"),
                         block_prefix=lambda i: f"l{i}")


register_architecture("Zefenex", ZefenexConfig, build_zefenex, aliases=("zefenex",))
