"""Typed configuration of the Zefenex decoder, read from its config.json.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
an optional ``logit_softcap`` and ``layers``, a list in which every entry names its mixer
(``type``: ``latent_attention``), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).  A mixer may read
the cache of an earlier layer (``kv_from``) instead of filling one; its window
(``mask.size``) and rotation (``rot.base``, ``rot.dims``) may be absent.  Every size and
constant of a model comes from there.  Positions are not bounded by a table, so a sequence
is as long as the engine lets it be (``max_seq_len``, an engine-side bound that config.json
may carry).
"""

from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError, canonical_dtype_name

DEFAULT_MAX_SEQ_LEN = 1 << 20

_MIXER_REQUIRED = {"dim", "heads", "kv_rank", "rot_dim", "scale", "vdim"}
_MIXER_OPTIONAL = {"kv_from", "mask", "rot"}


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


def _check_mixer(m, what: str, index: int, layers) -> None:
    _keys(m, _MIXER_REQUIRED, what, optional=_MIXER_OPTIONAL)
    for k in ("dim", "heads", "kv_rank", "vdim"):
        _positive_int(m[k], f"{what}.{k}")
    _need(_is_int(m["rot_dim"]) and m["rot_dim"] >= 0,
          f"{what}.rot_dim must be a non-negative integer, got {m['rot_dim']!r}")
    _number(m["scale"], f"{what}.scale")
    if m.get("mask") is not None:
        _keys(m["mask"], {"size"}, f"{what}.mask")
        _positive_int(m["mask"]["size"], f"{what}.mask.size")
    if m.get("rot") is not None:
        _keys(m["rot"], {"base", "dims"}, f"{what}.rot")
        _number(m["rot"]["base"], f"{what}.rot.base")
        dims = m["rot"]["dims"]
        _need(_is_int(dims) and 0 <= dims <= m["rot_dim"] and dims % 2 == 0,
              f"{what}.rot.dims must be an even number of the {m['rot_dim']} rotated "
              f"entries, got {dims!r}")
    src = m.get("kv_from")
    if src is not None:
        _need(_is_int(src) and 0 <= src < index,
              f"{what}.kv_from must name an earlier layer, got {src!r}")
        other = layers[src]["mixer"]
        _need(other.get("kv_from") is None,
              f"{what}.kv_from names layer {src}, which has no cache of its own")
        for k in ("kv_rank", "rot_dim"):
            _need(other.get(k) == m[k], f"{what}.{k} differs from layer {src}'s, whose cache it reads")
        _need((other.get("rot") or None) == (m.get("rot") or None),
              f"{what}.rot differs from layer {src}'s, whose cache it reads")


def _check_mlp(mlp, what):
    if mlp is None:
        return
    _need(isinstance(mlp, dict) and "kind" in mlp, f"{what} needs a 'kind'")
    if mlp["kind"] == "dense":
        _keys(mlp, {"kind", "ff"}, what)
        _positive_int(mlp["ff"], f"{what}.ff")
    elif mlp["kind"] == "moe":
        _keys(mlp, {"kind", "expert", "router"}, what, optional={"shared"})
        _keys(mlp["expert"], {"ff"}, f"{what}.expert")
        _positive_int(mlp["expert"]["ff"], f"{what}.expert.ff")
        _keys(mlp["router"], {"experts", "top"}, f"{what}.router", optional={"identity"})
        n = _positive_int(mlp["router"]["experts"], f"{what}.router.experts")
        ident = mlp["router"].get("identity") or 0
        _need(_is_int(ident) and ident >= 0, f"{what}.router.identity must be a count")
        top = _positive_int(mlp["router"]["top"], f"{what}.router.top")
        _need(top <= n + ident, f"{what}.router.top ({top}) exceeds the {n + ident} router outputs")
        if mlp.get("shared") is not None:
            _keys(mlp["shared"], {"ff"}, f"{what}.shared")
            _positive_int(mlp["shared"]["ff"], f"{what}.shared.ff")
    else:
        raise ConfigError(f"{what}.kind {mlp['kind']!r} is not known (dense, moe)")


@dataclass(frozen=True)
class ZefenexConfig:
    architecture: str = "Zefenex"
    vocab: int = 256
    width: int = 64
    layers: tuple = ()
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0     # 0: the logits are not capped
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
        _need(self.logit_softcap >= 0, "logit_softcap must not be negative")
        canonical_dtype_name(self.dtype)
        _need(len(self.layers) > 0, "layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            _keys(layer, {"type", "mixer"}, what, optional={"mlp"})
            _need(layer["type"] == "latent_attention",
                  f"{what}.type {layer['type']!r} is not known (latent_attention)")
            _check_mixer(layer["mixer"], f"{what}.mixer", i, self.layers)
            _check_mlp(layer.get("mlp"), f"{what}.mlp")

    def cache_readers(self, index: int) -> list:
        """The layers that read layer ``index``'s cache (itself first)."""
        return [index] + [i for i, layer in enumerate(self.layers)
                          if layer["mixer"].get("kv_from") == index]

    def kept_window(self, index: int):
        """How many of the latest tokens layer ``index``'s cache has to keep: the widest
        window among the layers that read it, None if one of them sees everything."""
        sizes = [(self.layers[i]["mixer"].get("mask") or {}).get("size")
                 for i in self.cache_readers(index)]
        return None if any(s is None for s in sizes) else max(sizes)

    @classmethod
    def from_dict(cls, raw: dict) -> "ZefenexConfig":
        known = {"architecture", "vocab", "width", "layers", "norm", "embedding",
                 "logit_softcap", "max_seq_len", "dtype"}
        unknown = sorted(set(raw) - known)
        _need(not unknown, f"config.json has keys this architecture does not know: {unknown}")
        for req in ("vocab", "width", "layers", "norm"):
            _need(req in raw, f"config.json lacks the required key {req!r}")
        _keys(raw["norm"], {"eps"}, "norm")
        scale = 1.0
        if raw.get("embedding") is not None:
            _keys(raw["embedding"], {"scale"}, "embedding")
            scale = _number(raw["embedding"]["scale"], "embedding.scale")
        _need(isinstance(raw["layers"], list), "layers must be a list")
        cap = raw.get("logit_softcap") or 0.0
        return cls(architecture=raw.get("architecture", "Zefenex"), vocab=raw["vocab"],
                   width=raw["width"], layers=tuple(raw["layers"]),
                   norm_eps=float(raw["norm"]["eps"]), embedding_scale=scale,
                   logit_softcap=_number(cap, "logit_softcap", positive=False),
                   max_seq_len=raw.get("max_seq_len", DEFAULT_MAX_SEQ_LEN),
                   dtype=canonical_dtype_name(raw.get("dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": list(self.layers)}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        out.update({"norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width})
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            out["max_seq_len"] = self.max_seq_len
        if self.dtype != "bfloat16":
            out["dtype"] = self.dtype
        return out
