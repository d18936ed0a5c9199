"""Typed configuration of the Movazen decoder, read from its config.json.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``token_side.dim`` (the width of a layer's share of the per-token side table; absent: no side
input) and ``layers``, a list in which every entry names its mixer (``type``: ``attention`` or
``parallel``), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: a
mixture of experts, or null for none).

* ``attention``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values),
  ``scale`` and an optional ``mask`` with ``size`` (the window) and ``keep_first`` (the
  sequence's first tokens the window does not hide).
* ``parallel``: ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and an optional
  ``q_temp`` with ``coef`` and ``every``), ``right`` (``heads``, ``dim``, ``vdim`` and ``decay``,
  one number a head) and the weights ``left_scale`` and ``right_scale`` of the two halves.
* ``mlp``: ``kind`` ``moe``; ``expert`` (``ff``, ``limit``); ``router`` (``experts``, ``top`` and
  optional ``groups`` with ``count`` and ``keep``); an optional ``shared`` expert (``ff``,
  ``limit``).

Every size and constant of a model comes from there.  Positions are not bounded by a table, so
a sequence is as long as the engine lets it be (``max_seq_len``, an engine-side bound that
config.json may carry).
"""

from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError, canonical_dtype_name

DEFAULT_MAX_SEQ_LEN = 1 << 20


def _need(cond, msg):
    if not cond:
        raise ConfigError(msg)


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _positive_int(v, what):
    _need(_is_int(v) and v > 0, f"{what} must be a positive integer, got {v!r}")
    return v


def _number(v, what, positive=True):
    _need(isinstance(v, (int, float)) and not isinstance(v, bool) and (v > 0 or not positive),
          f"{what} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


def _keys(d, want: set, what: str, optional: set = frozenset()):
    _need(isinstance(d, dict), f"{what} must be an object, got {d!r}")
    missing, unknown = want - set(d), set(d) - want - optional
    _need(not missing, f"{what} lacks {sorted(missing)}")
    _need(not unknown, f"{what} has keys this architecture does not know: {sorted(unknown)}")


def _check_softmax_heads(m, what: str, optional: set) -> None:
    _keys(m, {"dim", "heads", "kv_heads", "scale", "vdim"}, what, optional=optional)
    for k in ("dim", "heads", "kv_heads", "vdim"):
        _positive_int(m[k], f"{what}.{k}")
    _need(m["heads"] % m["kv_heads"] == 0,
          f"{what}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    _number(m["scale"], f"{what}.scale")


def _check_attention(m, what: str) -> None:
    _check_softmax_heads(m, what, {"mask"})
    if m.get("mask") is not None:
        _keys(m["mask"], {"size"}, f"{what}.mask", optional={"keep_first"})
        _positive_int(m["mask"]["size"], f"{what}.mask.size")
        keep = m["mask"].get("keep_first", 0)
        _need(_is_int(keep) and keep >= 0,
              f"{what}.mask.keep_first must be a count, got {keep!r}")


def _check_parallel(m, what: str) -> None:
    _keys(m, {"left", "right", "left_scale", "right_scale"}, what)
    _number(m["left_scale"], f"{what}.left_scale", positive=False)
    _number(m["right_scale"], f"{what}.right_scale", positive=False)
    left, right = m["left"], m["right"]
    _check_softmax_heads(left, f"{what}.left", {"q_temp"})
    if left.get("q_temp") is not None:
        _keys(left["q_temp"], {"coef", "every"}, f"{what}.left.q_temp")
        _number(left["q_temp"]["coef"], f"{what}.left.q_temp.coef", positive=False)
        _positive_int(left["q_temp"]["every"], f"{what}.left.q_temp.every")
    _keys(right, {"decay", "dim", "heads", "vdim"}, f"{what}.right")
    for k in ("dim", "heads", "vdim"):
        _positive_int(right[k], f"{what}.right.{k}")
    _need(isinstance(right["decay"], list) and len(right["decay"]) == right["heads"],
          f"{what}.right.decay must hold one number a head")
    for x in right["decay"]:
        _number(x, f"{what}.right.decay", positive=False)


def _check_unit(u, what: str) -> None:
    _keys(u, {"ff", "limit"}, what)
    _positive_int(u["ff"], f"{what}.ff")
    _number(u["limit"], f"{what}.limit")


def _check_mlp(mlp, what: str) -> None:
    if mlp is None:
        return
    _need(isinstance(mlp, dict) and mlp.get("kind") == "moe",
          f"{what}.kind must be 'moe' (or the feed-forward null), got {mlp!r}")
    _keys(mlp, {"kind", "expert", "router"}, what, optional={"shared"})
    _check_unit(mlp["expert"], f"{what}.expert")
    router = mlp["router"]
    _keys(router, {"experts", "top"}, f"{what}.router", optional={"groups"})
    n = _positive_int(router["experts"], f"{what}.router.experts")
    top = _positive_int(router["top"], f"{what}.router.top")
    _need(top <= n, f"{what}.router.top ({top}) exceeds the {n} experts")
    if router.get("groups") is not None:
        _keys(router["groups"], {"count", "keep"}, f"{what}.router.groups")
        count = _positive_int(router["groups"]["count"], f"{what}.router.groups.count")
        keep = _positive_int(router["groups"]["keep"], f"{what}.router.groups.keep")
        _need(n % count == 0, f"{what}.router: {n} experts do not form {count} equal groups")
        _need(keep <= count, f"{what}.router.groups.keep ({keep}) exceeds the {count} groups")
        _need(top <= keep * (n // count),
              f"{what}.router.top ({top}) exceeds the experts of {keep} groups")
    if mlp.get("shared") is not None:
        _check_unit(mlp["shared"], f"{what}.shared")


@dataclass(frozen=True)
class MovazenConfig:
    architecture: str = "Movazen"
    vocab: int = 256
    width: int = 64
    layers: tuple = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    side_dim: int = 0              # 0: no per-token side input
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    dtype: str = "bfloat16"

    # what the framework reads
    @property
    def vocab_size(self) -> int:
        return self.vocab

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_seq_len, "max_seq_len")
        _need(self.norm_eps > 0, "norm.eps must be positive")
        _need(_is_int(self.side_dim) and self.side_dim >= 0, "token_side.dim must be a count")
        canonical_dtype_name(self.dtype)
        _need(len(self.layers) > 0, "layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            _keys(layer, {"type", "mixer"}, what, optional={"mlp"})
            if layer["type"] == "attention":
                _check_attention(layer["mixer"], f"{what}.mixer")
            elif layer["type"] == "parallel":
                _check_parallel(layer["mixer"], f"{what}.mixer")
            else:
                raise ConfigError(f"{what}.type {layer['type']!r} is not known "
                                  f"(attention, parallel)")
            _check_mlp(layer.get("mlp"), f"{what}.mlp")

    @classmethod
    def from_dict(cls, raw: dict) -> "MovazenConfig":
        known = {"architecture", "vocab", "width", "layers", "norm", "embedding", "token_side",
                 "max_seq_len", "dtype"}
        unknown = sorted(set(raw) - known)
        _need(not unknown, f"config.json has keys this architecture does not know: {unknown}")
        for req in ("vocab", "width", "layers", "norm"):
            _need(req in raw, f"config.json lacks the required key {req!r}")
        _keys(raw["norm"], {"eps"}, "norm")
        scale = 1.0
        if raw.get("embedding") is not None:
            _keys(raw["embedding"], {"scale"}, "embedding")
            scale = _number(raw["embedding"]["scale"], "embedding.scale")
        side = 0
        if raw.get("token_side") is not None:
            _keys(raw["token_side"], {"dim"}, "token_side")
            side = _positive_int(raw["token_side"]["dim"], "token_side.dim")
        _need(isinstance(raw["layers"], list), "layers must be a list")
        return cls(architecture=raw.get("architecture", "Movazen"), vocab=raw["vocab"],
                   width=raw["width"], layers=tuple(raw["layers"]),
                   norm_eps=float(raw["norm"]["eps"]), embedding_scale=scale, side_dim=side,
                   max_seq_len=raw.get("max_seq_len", DEFAULT_MAX_SEQ_LEN),
                   dtype=canonical_dtype_name(raw.get("dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": list(self.layers), "norm": {"eps": self.norm_eps}}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        out.update({"vocab": self.vocab, "width": self.width})
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            out["max_seq_len"] = self.max_seq_len
        if self.dtype != "bfloat16":
            out["dtype"] = self.dtype
        return out
