"""Python faces of the CUDA kernels, and the runtime the parts run on.

Each method checks shapes and types on the host, then calls one exported C
launcher with raw device pointers on torch's current stream.  Nothing here
computes on the CPU and nothing falls back to a library implementation of a
part of the model; the only library call is the plain bfloat16 matrix product
where the own kernel does not apply (the reference multiplies with
``nn.Linear``, i.e. a library GEMM: train/model.py:79-82,130-132,227).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import library

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_LL = ctypes.c_longlong

_ERRORS = {100001: "a size this kernel does not support",
           100002: "the driver refused to encode a tensor map"}


# torch's own fast path to the current stream's handle (a C call without the argument
# handling of torch.cuda.current_stream, which costs several microseconds a launch)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        why = _ERRORS.get(rc)
        if why is None:
            why = f"CUDA error {rc}"
        raise KernelError(f"{what}: {why}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _decl(lib, name, argtypes, restype=ctypes.c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


class SplitParts:
    """A matrix product left as the parts of a cut along K: float32 [parts, M, N].

    Their sum, taken in the order of the slices, is the product.  ``add_rmsnorm``
    adds them up while it reads the residual row anyway, which saves the kernel
    that would do nothing else.  The parts live in one scratch buffer of the
    kernels' owner: they are read (or given up) before the next product that
    wants the buffer, which otherwise takes the ordinary way.
    """

    __slots__ = ("parts", "_ops")

    def __init__(self, parts, ops):
        self.parts = parts
        self._ops = ops

    @property
    def shape(self):
        return self.parts.shape[1:]

    def release(self) -> None:
        if self._ops is not None:
            self._ops._parts_busy = False
            self._ops = None

    def float(self):
        """The product as a float32 tensor of its own."""
        out = self.parts[0].clone()
        for k in range(1, self.parts.shape[0]):
            out += self.parts[k]
        self.release()
        return out

    def clone(self):
        return self.float()

    def to(self, dtype):
        return self.float().to(dtype)


class Ops:
    """The kernels, bound to one device.  Fails at construction without a GPU."""

    def __init__(self, device, act_dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError(
                "this engine runs on a CUDA device only (sm_100a kernels); "
                f"device {device!r} is not one and there is no CPU path")
        self.act_dtype = act_dtype
        self._device_index = (self.device.index if self.device.index is not None
                              else torch.cuda.current_device())
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._libs: list = []                    # every kernel library in use
        self._chained = True                     # what the libraries were last told
        core = self._load("core")
        self._embed = _decl(core, "mls_embed", [_P, _P, _I, _P, _I, _I, _I, _F, _P, _P, _P, _P])
        self._add_rmsnorm = _decl(core, "mls_add_rmsnorm",
                                  [_P, _P, _I, _P, _I, _F, _P, _I, _I, _I, _P, _I, _LL, _P, _P])
        self._gemm_f32 = _decl(core, "mls_gemm_f32", [_P, _I, _P, _P, _I, _I, _I, _P])
        self._rope_store = _decl(core, "mls_rope_store",
                                 [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                  _LL, _I, _P, _I, _LL, _P, _P])
        self._attention_simt = _decl(core, "mls_attention_simt",
                                     [_P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _I, _F, _LL, _P, _P, _I, _LL, _P])
        self._swiglu = _decl(core, "mls_swiglu", [_P, _P, _I, _I, _I, _P])
        self._clamped_glu = _decl(core, "mls_clamped_glu", [_P, _P, _I, _I, _I, _F, _F, _P])
        self._unary_act = _decl(core, "mls_unary_act", [_P, _I, _P, _I, _LL, _I, _P, _I, _I, _P])
        self._softcap_f32 = _decl(core, "mls_softcap_f32", [_P, _LL, _F, _P])
        self._scale_f32 = _decl(core, "mls_scale_f32", [_P, _LL, _F, _P])
        self._part_libs: dict = {}               # kernels of parts only some models have
        self._sample = _decl(core, "mls_sample", [_P, _P, _P, _P, _I, _I, _P, _P])
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._attention_libs: dict = {}
        self._attention_lib_handles: dict = {}
        self._split_ctas_per_sm: dict = {}       # head size -> CTAs of the split kernel an SM holds
        self._attention_fused: dict = {}         # head size -> decode attention that also rotates
        self._tc_rows: dict = {}                 # head size -> rows of a tile of the tcgen05 kernel
        self._scratch: dict = {}
        self._transposed: dict = {}              # id(weight) -> (weight, its transposed view)
        self._gemm = None
        self._tiles_set = False
        self._parts_busy = False
        self.attention_impl = os.environ.get("MLS_B200_ATTENTION", "auto")
        self.gemm_impl = os.environ.get("MLS_B200_GEMM", "auto")
        self.generation = 0          # grows whenever a buffer kernels were given moves
        self.launches = 0            # launches of this package's own kernels
        self.library_launches = 0    # plain matrix products handed to the library

    # ------------------------------------------------------------------ helpers
    def _load(self, name: str, defines: dict | None = None):
        lib = library.load(name, defines)
        lib.mls_set_chained.argtypes = [_I]
        lib.mls_set_chained.restype = None
        lib.mls_set_chained(1 if self._chained else 0)
        self._libs.append(lib)
        return lib

    CHAINED_UP_TO = 256      # tokens of a step whose kernels start under their predecessors

    def begin_step(self, n_tokens: int) -> None:
        """Tell the kernel libraries how to launch this step's kernels: chained
        (each may start, and fetch what no kernel writes, while the one before it
        still runs) pays when kernels are short, plain when they are long."""
        on = n_tokens <= self.CHAINED_UP_TO
        if on != self._chained:
            self._chained = on
            for lib in self._libs:
                lib.mls_set_chained(1 if on else 0)

    def scratch(self, tag: str, n_floats: int):
        """Float32 scratch memory that lives as long as the kernels' owner."""
        buf = self._scratch.get(tag)
        if buf is None or buf.numel() < n_floats:
            buf = torch.empty(max(n_floats, 1 << 16), dtype=torch.float32, device=self.device)
            self._scratch[tag] = buf
            self.generation += 1
        return buf

    def _stream(self):
        """The raw handle of torch's current stream on this device (asked for at every
        launch: a captured step runs on the capture's stream)."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def check_status(self) -> None:
        """Raise if a kernel met a token, position or slot outside its table (waits
        for the device)."""
        self.raise_for_status(int(self.status.item()))

    def raise_for_status(self, code: int) -> None:
        """Raise for a status word already read (``code`` != 0), and clear it on the
        device so that the next step starts clean."""
        if code:
            self.status.zero_()
            what = [n for b, n in ((1, "a token id outside the vocabulary"),
                                   (2, "a position outside the rotary table"),
                                   (4, "a cache slot outside the pool"),
                                   (8, "a bounded wait inside a kernel ran out"),
                                   (16, "shared memory of a kernel was not aligned"))
                    if code & b]
            raise KernelError("a kernel refused its input: " + ("; ".join(what) or
                                                                f"status {code}"))

    # ------------------------------------------------------------------ kernels
    def embed(self, token_ids, table, x, vocab: int, scale: float = 1.0, positions=None,
              freq=None) -> None:
        """``x[t] = table[token[t]] * scale``; with ``freq`` (float64, one a pair of entries)
        plus the sinusoidal vector of ``positions[t]``: sine at 2i, cosine at 2i + 1 of
        ``position * freq[i]``."""
        t, d = x.shape
        _need(freq is None or (freq.dtype == torch.float64 and freq.numel() >= (d + 1) // 2
                               and freq.is_contiguous() and positions is not None
                               and positions.dtype == torch.int32 and positions.numel() >= t),
              "embed: positions and one float64 frequency a pair of entries")
        _need(x.dtype == torch.float32 and x.is_contiguous(), "embed: x must be float32")
        _need(table.shape == (vocab, d) and table.is_contiguous(), "embed: bad table")
        _need(token_ids.dtype == torch.int32 and token_ids.numel() >= t, "embed: bad ids")
        self.launches += 1
        _check(self._embed(_ptr(token_ids), _ptr(table), _code(table.dtype), _ptr(x), t, d,
                           vocab, float(scale), _ptr(self.status),
                           _ptr(positions) if freq is not None else None, _ptr(freq),
                           self._stream()), "embed")

    def _delta_args(self, delta, t: int, d: int, what: str):
        """(pointer, type code, parts, part stride) of a pending residual delta."""
        if delta is None:
            return None, 0, 1, 0
        if hasattr(delta, "resolve"):
            # a delta that still has a map to go through, met by a consumer that does not
            # apply it itself: the map runs as a kernel of its own
            delta = delta.resolve()
        if isinstance(delta, SplitParts):
            parts = delta.parts
            _need(parts.shape[1:] == (t, d) and parts.is_contiguous()
                  and parts.dtype == torch.float32, f"{what}: bad delta parts")
            return parts.data_ptr(), 0, parts.shape[0], t * d
        _need(delta.shape == (t, d) and delta.is_contiguous(), f"{what}: bad delta")
        return delta.data_ptr(), _code(delta.dtype), 1, 0

    def add_rmsnorm(self, x, delta, weight, eps: float, h) -> None:
        """``x += delta`` (a tensor, ``SplitParts`` or None), ``h = rmsnorm(x) * weight``."""
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be float32")
        _need(h.shape == (t, d) and h.is_contiguous(), "add_rmsnorm: bad output")
        _need(weight.shape == (d,), "add_rmsnorm: bad weight")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "add_rmsnorm")
        self.launches += 1
        _check(self._add_rmsnorm(_ptr(x), dp, dcode, _ptr(weight), _code(weight.dtype),
                                 float(eps), _ptr(h), _code(h.dtype), t, d, None, parts, stride,
                                 _ptr(self.status), self._stream()), "add_rmsnorm")
        if isinstance(delta, SplitParts):
            delta.release()

    def gather_add_rmsnorm(self, x, delta, rows, n_rows: int, weight, eps: float, h) -> None:
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "gather_add_rmsnorm: bad x")
        _need(h.shape == (n_rows, d) and h.is_contiguous(), "gather_add_rmsnorm: bad output")
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "gather_add_rmsnorm: rows")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "gather_add_rmsnorm")
        self.launches += 1
        _check(self._add_rmsnorm(_ptr(x), dp, dcode, _ptr(weight), _code(weight.dtype),
                                 float(eps), _ptr(h), _code(h.dtype), n_rows, d, _ptr(rows),
                                 parts, stride, _ptr(self.status), self._stream()),
               "gather_add_rmsnorm")
        if isinstance(delta, SplitParts):
            delta.release()

    def prepare_weight(self, w):
        """A matrix [out, in] made ready for ``linear`` (contiguous, on device)."""
        return w.contiguous()

    def linear(self, a, w, out) -> None:
        """``out[M, N] = a[M, K] @ w[N, K]^T`` with float32 accumulation."""
        m, k = a.shape
        n = w.shape[0]
        _need(w.shape == (n, k) and out.shape == (m, n), "linear: shapes do not fit")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(),
              "linear: operands must be contiguous")
        if m == 0:
            return
        if w.dtype == torch.float32:
            # a matrix held in 32 bits is multiplied in true 32-bit arithmetic (16-bit rows
            # of ``a`` are widened as the kernel loads them)
            _need(a.dtype in (torch.float32, torch.bfloat16), f"linear: input dtype {a.dtype}")
            o32 = out if out.dtype == torch.float32 else torch.empty(
                (m, n), dtype=torch.float32, device=out.device)
            self.launches += 1
            _check(self._gemm_f32(_ptr(a), _code(a.dtype), _ptr(w), _ptr(o32), m, n, k,
                                  self._stream()), "gemm_f32")
            if o32 is not out:
                out.copy_(o32)
            return
        _need(w.dtype == torch.bfloat16, f"linear: weight dtype {w.dtype}")
        a16 = a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)
        if self._use_own_gemm(m, n, k):
            self._gemm_bf16(a16, w, out, m, n, k)
            return
        self.library_launches += 1
        held = self._transposed.get(id(w))           # the view costs a microsecond a call
        if held is None or held[0] is not w:
            held = self._transposed[id(w)] = (w, w.t())
        if out.dtype == torch.float32:
            torch.mm(a16, held[1], out_dtype=torch.float32, out=out)
        else:
            torch.mm(a16, held[1], out=out)

    def _use_own_gemm(self, m: int, n: int, k: int) -> bool:
        """The tcgen05 kernel takes rows that are whole 16-byte chunks; the choice
        between it and the library is ``MLS_B200_GEMM`` (tcgen05 | tcgen05-tiles | cublas |
        auto; prompts of more than 128 rows run on pairs of CTAs, with ``tcgen05-tiles``
        on one CTA a tile)."""
        if self.gemm_impl == "cublas" or k % 8 != 0:
            return False
        if self.gemm_impl in ("tcgen05", "tcgen05-tiles"):
            return True
        # auto: a few rows (decoding) go to the tcgen05 kernel, which asks for its
        # first weights while the kernel before it still runs; more rows go to the
        # library (as the reference's nn.Linear does) unless the kernel fuses work
        # (``linear_swiglu``)
        return m <= 64

    def _gemm_splits(self, m: int, n: int, k: int) -> int:
        """Parts along K for the weight-major orientation (M <= 64): the weights are
        read once; every tile x part is a CTA, and two CTAs fit an SM: as many CTAs
        as fit at the same time, at least 256 of K each."""
        tiles = (n + 127) // 128
        kblocks = (k + 63) // 64
        splits = max(1, min(kblocks // 4, (2 * self.sm_count) // tiles))
        per = -(-kblocks // splits)
        return -(-kblocks // per)

    def _gemm_library(self):
        if self._gemm is None:
            lib = self._load("gemm")
            self._gemm = _decl(lib, "mls_gemm_bf16",
                               [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P])
            self._gemm_gated = _decl(lib, "mls_gemm_bf16_gated",
                                     [_P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P, _P, _P])
            self._gemm_prompt_scratch = _decl(lib, "mls_gemm_prompt_scratch_floats", [_I, _I, _I],
                                              restype=ctypes.c_longlong)
            self._gemm_lib = lib
        return self._gemm_lib

    def set_gemm_tail_cut(self, mode: str) -> None:
        """Whether a prompt's product cuts the tiles of its last round along K: "never",
        "auto" (where it measured faster; the default) or "always" (wherever every piece
        gets four k-blocks)."""
        _need(mode in ("never", "auto", "always"), f"set_gemm_tail_cut: unknown mode {mode!r}")
        fn = _decl(self._gemm_library(), "mls_gemm_set_tail_cut", [_I], restype=None)
        fn(("never", "auto", "always").index(mode))

    def _gemm_bf16(self, a, w, out, m: int, n: int, k: int, epilogue: int = 0,
                   leave_parts: bool = False, gate=None):
        """The tcgen05 product.  ``leave_parts``: the K-parts are not added up but
        returned as ``SplitParts`` (the caller has checked that there are several)."""
        self._gemm_library()
        if self.gemm_impl == "tcgen05-tiles" or self._tiles_set:
            # prompts of more than 128 rows on one CTA a tile instead of pairs of CTAs
            self._gemm_lib.mls_gemm_set_prompt_kernel.argtypes = [_I]
            self._gemm_lib.mls_gemm_set_prompt_kernel.restype = None
            self._tiles_set = self.gemm_impl == "tcgen05-tiles"
            self._gemm_lib.mls_gemm_set_prompt_kernel(0 if self._tiles_set else 1)
        swap = 1 if m <= 64 else 0
        splits, partial, sums = 1, None, 0
        if swap:
            splits = self._gemm_splits(m, n, k)
            if splits > 1:
                tag = "gemm_kept_parts" if leave_parts else "gemm_partials"
                partial = self.scratch(tag, splits * m * n)
                sums = 0 if leave_parts else 1
        else:
            # a prompt's product cuts the tiles of its last round along K when that gives
            # every pair of SMs a piece; a second kernel adds the pieces up
            floats = self._gemm_prompt_scratch(m, n, k)
            if floats:
                partial = self.scratch("gemm_tail_parts", floats)
                sums = 1
        _need(not leave_parts or splits > 1, "gemm_bf16: no parts to leave")
        self.launches += 1 + sums
        out_f32 = 1 if (out is not None and out.dtype == torch.float32) else 0
        if gate is not None:          # epilogue 1 with another gated unit: (alpha, limit, shift)
            _check(self._gemm_gated(_ptr(a), _ptr(w), _ptr(out), out_f32, m, n, k, swap, splits,
                                    float(gate[0]), float(gate[1]), float(gate[2]), _ptr(partial),
                                    _ptr(self.status), self._stream()), "gemm_bf16_gated")
            return None
        _check(self._gemm(_ptr(a), _ptr(w), None if leave_parts else _ptr(out), out_f32,
                          m, n, k, swap, splits, epilogue, _ptr(partial), _ptr(self.status),
                          self._stream()), "gemm_bf16")
        if leave_parts:
            self._parts_busy = True
            return SplitParts(partial[:splits * m * n].view(splits, m, n), self)
        return None

    def linear_parts(self, a, w, out):
        """A product for a consumer that can add up K-parts while it reads its input
        anyway (``add_rmsnorm`` for what goes to the residual stream, ``rope_store``
        for q, k and v): returns ``out``, filled, or the product's parts
        (``SplitParts``) with ``out`` untouched."""
        m, k = a.shape
        n = w.shape[0]
        if (0 < m <= 64 and n % 4 == 0 and w.dtype == torch.bfloat16
                and not self._parts_busy
                and w.shape == (n, k) and a.is_contiguous() and w.is_contiguous()
                and self._use_own_gemm(m, n, k) and self._gemm_splits(m, n, k) > 1):
            a16 = a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)
            return self._gemm_bf16(a16, w, None, m, n, k, leave_parts=True)
        self.linear(a, w, out)
        return out

    def can_fuse_swiglu(self, d_model: int, inter: int) -> bool:
        """Whether gate-up projection and SwiGLU can run as one kernel."""
        return (self.act_dtype == torch.bfloat16 and self.gemm_impl != "cublas"
                and inter % 16 == 0 and d_model % 8 == 0)

    @staticmethod
    def interleave_gate_up(w_gate, w_up):
        """Rows [16 gate | 16 up | 16 gate | ...]: the layout ``linear_swiglu`` reads."""
        i, d = w_gate.shape
        both = torch.stack([w_gate.view(i // 16, 16, d), w_up.view(i // 16, 16, d)], dim=1)
        return both.reshape(2 * i, d).contiguous()

    def linear_swiglu(self, a, w_interleaved, out) -> None:
        """``out[M, I] = silu(a @ Wg^T) * (a @ Wu^T)`` in one kernel; the weight holds
        gate and up rows interleaved in blocks of 16 (``interleave_gate_up``)."""
        m, k = a.shape
        n = w_interleaved.shape[0]
        _need(out.shape == (m, n // 2) and a.dtype == torch.bfloat16 and
              w_interleaved.dtype == torch.bfloat16, "linear_swiglu: shapes or types do not fit")
        _need(a.is_contiguous() and w_interleaved.is_contiguous() and out.is_contiguous(),
              "linear_swiglu: operands must be contiguous")
        if m == 0:
            return
        self._gemm_bf16(a, w_interleaved, out, m, n, k, epilogue=1)

    def linear_clamped_glu(self, a, w_interleaved, out, alpha: float, limit: float) -> None:
        """``out[M, I] = g' * sigmoid(alpha * g') * (u' + 1)`` with ``g' = min(a @ Wg^T, limit)``
        and ``u' = clamp(a @ Wu^T, -limit, limit)`` in one kernel; the weight as for
        ``linear_swiglu`` (``interleave_gate_up``)."""
        m, k = a.shape
        n = w_interleaved.shape[0]
        _need(out.shape == (m, n // 2) and a.dtype == torch.bfloat16 and
              w_interleaved.dtype == torch.bfloat16, "linear_clamped_glu: shapes or types")
        _need(a.is_contiguous() and w_interleaved.is_contiguous() and out.is_contiguous(),
              "linear_clamped_glu: operands must be contiguous")
        if m == 0:
            return
        self._gemm_bf16(a, w_interleaved, out, m, n, k, epilogue=1, gate=(alpha, limit, 1.0))

    def can_fuse_activation(self, k: int) -> bool:
        """Whether a product and an ungated activation of its outputs can run as one kernel."""
        return (self.act_dtype == torch.bfloat16 and self.gemm_impl != "cublas" and k % 8 == 0)

    def linear_relu_squared(self, a, w, out, bias=None) -> None:
        """``out[M, N] = relu(a @ w^T + bias)^2``; without a bias in one kernel (the tcgen05
        product's epilogue), with one as the product in float32 and the activation on it."""
        m, k = a.shape
        n = w.shape[0]
        _need(w.shape == (n, k) and out.shape == (m, n) and a.dtype == torch.bfloat16
              and w.dtype == torch.bfloat16, "linear_relu_squared: shapes or types do not fit")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(),
              "linear_relu_squared: operands must be contiguous")
        if m == 0:
            return
        if bias is not None:
            z = self.scratch("biased_product", m * n)[:m * n].view(m, n)
            self.linear(a, w, z)
            self.relu_squared(z, out, bias=bias)
            return
        self._gemm_bf16(a, w, out, m, n, k, epilogue=2)

    def rope_takes_parts(self, hd: int) -> bool:
        """Whether ``rope_store`` can read its rows from a product's K-parts."""
        return self.act_dtype == torch.bfloat16 and (hd // 2) % 8 == 0

    def rope_store(self, qkv, positions, cos, sin, slot_map, k_pool, v_pool, n_tokens: int,
                   n_heads: int, n_kv: int, hd: int, max_pos: int, writes: bool,
                   parts=None) -> None:
        """Rotate q and k, store rotated k and raw v in the pages, leave rotated q in
        ``qkv``.  With ``parts`` (``SplitParts`` of the projection) the rows are
        read from there instead of from ``qkv``."""
        _need(qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv) * hd,
              "rope_store: bad qkv")
        _need(k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype,
              "rope_store: cache and activations differ in type")
        _need(k_pool.is_contiguous() and v_pool.is_contiguous(), "rope_store: pool layout")
        kvh, pages, block, hd2 = k_pool.shape
        _need(kvh == n_kv and hd2 == hd, "rope_store: pool shape does not fit the heads")
        _need(cos.shape == (max_pos, hd // 2) and cos.dtype == torch.float32,
              "rope_store: bad tables")
        pp, n_parts, stride = None, 0, 0
        if parts is not None:
            _need(self.rope_takes_parts(hd) and qkv.dtype == torch.bfloat16
                  and tuple(parts.shape) == tuple(qkv.shape) and parts.parts.is_contiguous(),
                  "rope_store: these parts cannot be read")
            pp, n_parts = parts.parts.data_ptr(), parts.parts.shape[0]
            stride = qkv.shape[0] * qkv.shape[1]
        self.launches += 1
        _check(self._rope_store(_ptr(qkv), _code(qkv.dtype), _ptr(positions), _ptr(cos),
                                _ptr(sin), _ptr(slot_map), _ptr(k_pool), _ptr(v_pool),
                                n_tokens, n_heads, n_kv, hd, block, max_pos,
                                pages * block, 1 if writes else 0, pp, n_parts, stride,
                                _ptr(self.status), self._stream()), "rope_store")
        if parts is not None:
            parts.release()

    def require_attention(self, hd: int, n_heads: int = 0, n_kv: int = 0) -> None:
        """Make sure attention kernels for this head size exist, or say why not."""
        _need(hd % 16 == 0 and 16 <= hd <= 512,
              f"attention kernels take head sizes 16..512 in steps of 16, not {hd}")
        if hd > 256:
            return          # beyond the tensor-core kernels: the one-warp-per-row kernel, both types
        if self.act_dtype == torch.bfloat16 and hd not in self._attention_libs:
            lib = self._load("attention", {"MLS_HEAD_DIM": int(hd)})
            fn = _decl(lib, "mls_attention_mma",
                       [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _F, _I, _I, _I,
                        _P, _P, _LL, _P, _I, _P, _P, _I, _LL, _P])
            tc = _decl(lib, "mls_attention_tc",
                       [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _F, _I, _I, _I, _LL,
                        _P, _P, _LL, _P, _I, _P])
            fused = _decl(lib, "mls_attention_decode_fused",
                          [_P, _I, _LL, _P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I,
                           _I, _I, _F, _I, _I, _P, _P, _LL, _P, _P])
            self._attention_fused[hd] = fused
            rows_fn = lib.mls_attention_tc_rows
            rows_fn.restype = ctypes.c_int
            self._tc_rows[hd] = int(rows_fn()) or 128
            self._attention_libs[hd] = (fn, tc)
            self._attention_lib_handles[hd] = lib
            per_sm = _decl(lib, "mls_attention_split_ctas_per_sm", [_I])
            tma = self.attention_impl in ("auto", "mma") and hd % 64 == 0
            self._split_ctas_per_sm[hd] = int(per_sm(1 if tma else 0)) or 2

    def set_attention_rows(self, hd: int, rows: int) -> None:
        """Fix the rows a CTA of the tcgen05 attention kernel owns: 256 (two row tiles),
        128 (one, its keys in halves) or 0 (chosen by the step's size; the default)."""
        _need(rows in (0, 128, 256), "set_attention_rows: 0, 128 or 256")
        self.require_attention(hd)
        lib = self._attention_lib_handles[hd]
        fn = _decl(lib, "mls_attention_tc_set_rows", [_I], restype=None)
        fn(rows)

    def attention_tensor_cores(self, hd: int) -> bool:
        """Whether the tensor-core attention kernels take this step's attention (else
        the one-warp-per-row kernel does, which takes every head size up to 512)."""
        return (self.act_dtype == torch.bfloat16 and self.attention_impl != "simt"
                and hd <= 256 and hd % 16 == 0)

    def attention_facts(self, hd: int) -> dict:
        """What a mixer needs to know of the attention kernels to plan a step's
        launches: ``small_rows`` (requests whose (token, head) rows of one kv head are
        at most this many go to the context-split kernel), ``tile_rows`` and
        ``tc_rows`` (rows of a tile of the mma.sync and of the tcgen05 tile kernel),
        ``split_keys`` (keys of a tile of the split kernel), ``split_slots`` (CTAs of the
        split kernel the GPU runs at a time: as many an SM as the kernel's registers and
        shared memory allow),
        ``cluster_splits`` (up to so many context splits are merged inside the kernel),
        ``tensor_cores`` (False: the one-warp-per-row kernel runs, which needs no plan)."""
        tma = self.attention_impl in ("auto", "mma") and hd % 64 == 0
        return {"small_rows": 16, "tile_rows": 64, "tc_rows": self._tc_rows.get(hd, 128),
                "split_keys": 64,
                "split_slots": self._split_ctas_per_sm.get(hd, 2) * self.sm_count,
                "cluster_slots": 2 * self.sm_count,   # CTAs up to which the splits merge in clusters
                # most context splits that merge inside the split kernel (a merge kernel
                # takes over beyond that)
                "cluster_splits": 8 if tma and os.environ.get(
                    "MLS_B200_CLUSTER_MERGE", "1") != "0" else 0,
                "tensor_cores": self.attention_tensor_cores(hd)}

    def paged_attention(self, qkv, out, cache, step, n_heads: int, n_kv: int, hd: int,
                        scale: float, window: int, plan=None, softcap: float = 0.0,
                        sink=None, slopes=None, keep_first: int = 0, simt: bool = False) -> None:
        """Attention of the step's tokens over the pages.  ``slopes`` (float32 [n_heads]): the
        score of head h loses ``slopes[h] * (position - key's position)``.  ``keep_first``: a
        window does not hide the sequence's first so many keys.  ``out`` may be a block of
        columns of a wider buffer.  Of the tensor-core kernels the tcgen05 kernel (prompts) and
        the ``mma.sync`` ones without TMA take the first two, so a bfloat16 call with either runs
        there (rows of a wider buffer are taken by all of them, 16 bytes apart for those with
        TMA); ``simt`` sends the call to the one-warp-per-row kernel.  ``softcap`` c > 0: scores become
        ``c * tanh(score / c)`` before the softmax.  ``sink`` (float32 [n_heads]): the softmax's
        denominator of head h also holds ``exp(sink[h])``, a term without key or value.  ``plan`` (the mixer's, from
        ``attention_facts``): ``n_tiles`` / ``n_tiles_tc`` / ``n_tiles_tc_wide`` tiles of the
        requests that are not small, ``any_small``, ``n_split`` context splits for the small ones."""
        g = step.groups[cache.group]
        t = step.n_tokens
        _need(out.shape == (t, n_heads * hd) and out.stride(1) == 1, "attention: bad out")
        _need(cache.k_pool.dtype == qkv.dtype, "attention: cache and activations differ")
        _need(slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (n_heads,)
                                 and slopes.is_contiguous()), "attention: slopes are float32 [heads]")
        keep_first = int(keep_first or 0) if window else 0
        plain = slopes is None and keep_first == 0 and out.stride(0) % 8 == 0
        _need(plain or not (softcap and slopes is not None),
              "attention: a cap on the scores and slopes together are not supported")
        _need(sink is None or (sink.dtype == torch.float32 and sink.shape == (n_heads,)
                               and sink.is_contiguous()), "attention: sinks are float32 [heads]")
        if (self.attention_tensor_cores(hd) and qkv.dtype == torch.bfloat16 and not simt
                and out.stride(0) % 2 == 0):
            fns = self._attention_libs.get(hd)
            _need(fns is not None, f"attention kernels for head size {hd} were not required")
            fn, tc = fns
            _need(plan is not None, "attention: the tensor-core kernels need the mixer's plan")
            n_tiles, n_small, n_split, n_tiles_tc = (plan.n_tiles, 1 if plan.any_small else 0,
                                                     plan.n_split, plan.n_tiles_tc)
            if (n_tiles and hd in (64, 128) and g.block_size in (8, 16, 32, 64)
                    and self.attention_impl == "auto" and out.stride(0) % 8 == 0):
                # prompts and portions: the tcgen05 kernel; what is left for the call
                # below are the requests of a few rows
                self.launches += 1
                _check(tc(_ptr(qkv), _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool),
                          _ptr(g.block_table), g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len),
                          step.n_requests, n_heads, n_kv, g.block_size, float(scale), int(window),
                          float(softcap), n_tiles_tc, plan.n_tiles_tc_wide, n_small, cache.k_pool.shape[1],
                          _ptr(self.status), _ptr(sink), out.stride(0), _ptr(slopes), keep_first,
                          self._stream()), "attention_tc")
                n_tiles = 0
                if not n_small:
                    return
            part_o = part_lse = None
            if n_split > 1:
                units = t * n_heads
                scratch = self.scratch("attention_partials", n_split * units * (hd + 1))
                part_o = scratch[:n_split * units * hd]
                part_lse = scratch[n_split * units * hd:]
            tma = (self.attention_impl != "no_tma" and plain and hd % 64 == 0
                   and g.block_size in (8, 16, 32, 64))
            self.launches += (1 if n_tiles else 0) + (n_small and self._split_launches(
                n_split, tma, step.n_requests * n_kv * n_split))
            _check(fn(_ptr(qkv), _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool),
                      _ptr(g.block_table), g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len),
                      step.n_requests, t, n_heads, n_kv, g.block_size, float(scale), int(window),
                      float(softcap), n_tiles, n_small, n_split, _ptr(part_o), _ptr(part_lse),
                      cache.k_pool.shape[1], _ptr(self.status),
                      0 if (self.attention_impl == "no_tma" or not plain) else 1, _ptr(sink),
                      _ptr(slopes), keep_first, out.stride(0), self._stream()),
                   "attention_mma")
            return
        self.launches += 1
        _check(self._attention_simt(
            _ptr(qkv), _ptr(out), _code(qkv.dtype), _ptr(cache.k_pool), _ptr(cache.v_pool),
            _ptr(g.block_table), g.max_blocks, _ptr(step.positions), _ptr(step.req_of_token),
            t, n_heads, n_kv, hd, g.block_size, float(scale), int(window), float(softcap),
            cache.k_pool.shape[1], _ptr(sink), _ptr(slopes), keep_first, out.stride(0),
            self._stream()), "attention_simt")

    def _split_launches(self, n_split: int, tma: bool, n_ctas: int) -> int:
        """Kernels the context-split attention launches: two to eight splits merge inside
        clusters of the one kernel if all its CTAs are resident at once, else through a
        merge kernel."""
        if n_split == 1:
            return 1
        in_clusters = (tma and n_split <= 8 and n_ctas <= 2 * self.sm_count
                       and os.environ.get("MLS_B200_CLUSTER_MERGE", "1") != "0")
        return 1 if in_clusters else 2

    def can_fuse_rope_attention(self, hd: int, block_size: int) -> bool:
        """Whether a step of single decoded tokens can leave the rotation and the cache
        write to the attention kernel (``attention_decode_fused``)."""
        return (self.act_dtype == torch.bfloat16 and self.attention_impl == "auto"
                and hd % 64 == 0 and block_size in (8, 16, 32, 64)
                and os.environ.get("MLS_B200_FUSED_ROPE", "1") != "0")

    def attention_decode_fused(self, parts, out, cache, step, cos, sin, max_pos: int,
                               n_heads: int, n_kv: int, hd: int, scale: float, window: int,
                               plan) -> None:
        """A step of one token a request: rotate q and k (read as the K-parts of their
        projection), store k and v, attend.  One kernel (and the merge of the context
        splits) instead of ``rope_store`` + ``paged_attention``; the bits are the same."""
        g = step.groups[cache.group]
        t = step.n_tokens
        width = (n_heads + 2 * n_kv) * hd
        _need(step.max_q_len == 1 and t == step.n_requests, "fused attention: single tokens only")
        _need(isinstance(parts, SplitParts) and tuple(parts.shape) == (t, width)
              and parts.parts.is_contiguous(), "fused attention: bad parts")
        _need(out.shape == (t, n_heads * hd) and out.is_contiguous()
              and out.dtype == torch.bfloat16, "fused attention: bad out")
        _need(cache.k_pool.dtype == torch.bfloat16 and cache.k_pool.is_contiguous()
              and cache.v_pool.is_contiguous(), "fused attention: pool layout")
        _need(cos.shape == (max_pos, hd // 2) and cos.dtype == torch.float32, "fused attention: tables")
        fn = self._attention_fused.get(hd)
        _need(fn is not None and plan is not None, "fused attention: kernels were not required")
        n_split = plan.n_split
        part_o = part_lse = None
        if n_split > 1:
            units = t * n_heads
            scratch = self.scratch("attention_partials", n_split * units * (hd + 1))
            part_o = scratch[:n_split * units * hd]
            part_lse = scratch[n_split * units * hd:]
        self.launches += self._split_launches(n_split, True, step.n_requests * n_kv * n_split)
        _check(fn(parts.parts.data_ptr(), parts.parts.shape[0], t * width, _ptr(step.positions),
                  _ptr(cos), _ptr(sin), max_pos, _ptr(g.slot_map), 1 if cache.writes else 0,
                  _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool), _ptr(g.block_table),
                  g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len), step.n_requests, n_heads,
                  n_kv, g.block_size, float(scale), int(window), n_split, _ptr(part_o),
                  _ptr(part_lse), cache.k_pool.shape[1], _ptr(self.status), self._stream()),
               "attention_decode_fused")
        parts.release()

    def swiglu(self, gu, out) -> None:
        t, inter = out.shape
        _need(gu.shape == (t, 2 * inter) and gu.dtype == out.dtype, "swiglu: shapes")
        _need(gu.is_contiguous() and out.is_contiguous(), "swiglu: layout")
        self.launches += 1
        _check(self._swiglu(_ptr(gu), _ptr(out), _code(out.dtype), t, inter, self._stream()),
               "swiglu")

    def relu_squared(self, z, out, bias=None) -> None:
        """``out = relu(z + bias)^2`` element by element (``out`` may be ``z``; a float32 ``z``
        may go to a bfloat16 ``out``); ``bias`` [columns] is optional."""
        _need(z.shape == out.shape and z.is_contiguous() and out.is_contiguous()
              and (z.dtype == out.dtype or z.dtype == torch.float32), "relu_squared: operands")
        _need(bias is None or (bias.shape == (z.shape[-1],) and bias.is_contiguous()),
              "relu_squared: bad bias")
        self.launches += 1
        _check(self._unary_act(_ptr(z), _code(z.dtype), _ptr(out), _code(out.dtype), z.numel(), 0,
                               _ptr(bias), _code(bias.dtype) if bias is not None else 0,
                               z.shape[-1], self._stream()), "relu_squared")

    def softcap_(self, x, cap: float) -> None:
        """``x = cap * tanh(x / cap)`` on float32 values."""
        _need(x.dtype == torch.float32 and x.is_contiguous() and cap > 0, "softcap_: float32 values")
        self.launches += 1
        _check(self._softcap_f32(_ptr(x), x.numel(), float(cap), self._stream()), "softcap_")

    def scale_(self, x, scale: float) -> None:
        """``x *= scale`` on float32 values."""
        _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_: float32 values")
        self.launches += 1
        _check(self._scale_f32(_ptr(x), x.numel(), float(scale), self._stream()), "scale_")

    # ------------------------------------------- parts only some architectures have
    def _part_lib(self, name: str):
        """The kernels of a kind of part, built and loaded when a model first needs them."""
        fns = self._part_libs.get(name)
        if fns is not None:
            return fns
        lib = self._load(name)
        if name == "layernorm":
            fns = {"add_layernorm": _decl(lib, "mls_add_layernorm",
                                          [_P, _P, _I, _I, _LL, _P, _P, _I, _P, _I, _F, _P, _I,
                                           _I, _I, _P, _P]),
                   "residual_add": _decl(lib, "mls_residual_add", [_P, _P, _P, _I, _I, _I, _P]),
                   "settle_concat": _decl(lib, "mls_settle_concat",
                                          [_P, _P, _I, _I, _LL, _P, _P, _I, _I, _I, _P])}
        elif name == "latent":
            fns = {"norm_store": _decl(lib, "mls_latent_norm_store",
                                       [_P, _I, _I, _I, _I, _P, _P, _I, _F, _P, _I, _P, _P, _I,
                                        _LL, _P, _P]),
                   "headwise": _decl(lib, "mls_headwise_linear",
                                     [_P, _LL, _LL, _P, _P, _LL, _LL, _I, _I, _I, _I, _I, _P]),
                   "rope_prep": _decl(lib, "mls_latent_rope_prep",
                                      [_P, _I, _LL, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P,
                                       _P, _I, _F, _P, _P, _I, _I, _I, _P, _P, _I, _LL, _P, _P]),
                   "gate": _decl(lib, "mls_sigmoid_gate",
                                 [_P, _I, _P, _I, _LL, _I, _I, _I, _I, _P])}
        elif name == "tanhnorm":
            fns = {"add_tanh_norm": _decl(lib, "mls_add_tanh_norm",
                                          [_P, _P, _I, _I, _LL, _P, _F, _P, _P, _P, _F, _P, _P, _I,
                                           _P, _I, _P, _P, _I, _I, _P])}
        elif name == "mlstm":
            fns = {"columns": _decl(lib, "mls_mlstm_columns", [_I, _I]),
                   "scan": _decl(lib, "mls_mlstm_scan",
                                 [_P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _F, _P, _P, _P, _LL,
                                  _I, _I, _I, _I, _P, _P, _P]),
                   "finish": _decl(lib, "mls_mlstm_finish",
                                   [_P, _P, _P, _I, _I, _P, _I, _F, _P, _I, _I, _I, _I, _P])}
        elif name == "experts":
            fns = {"tile_rows": _decl(lib, "mls_expert_tile_rows", []),
                   "topk": _decl(lib, "mls_route_topk",
                                 [_P, _I, _I, _I, _I, _I, _I, _P, _F, _I, _I, _P, _P, _P]),
                   "sort": _decl(lib, "mls_route_sort",
                                 [_P, _I, _I, _I, _P, _P, _P, _P, _I, _P, _P]),
                   "glu": _decl(lib, "mls_expert_glu",
                                [_P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _F,
                                 _P]),
                   "down": _decl(lib, "mls_expert_down",
                                 [_P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _P]),
                   "combine": _decl(lib, "mls_expert_combine",
                                    [_P, _I, _P, _I, _P, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P])}
        elif name == "shortconv":
            fns = {"qk": _decl(lib, "mls_qk_conv_norm_rope_store",
                               [_P, _I, _LL, _P, _P, _I, _P, _P, _I, _F, _P, _LL, _I, _P, _P, _P, _P,
                                _P, _I, _P, _I, _I, _P, _P, _P, _I, _LL, _I, _I, _I, _I, _I, _P, _P]),
                   "shift_mix": _decl(lib, "mls_token_shift_mix",
                                      [_P, _I, _P, _I, _I, _P, _LL, _I, _P, _P, _P, _P, _P, _I, _I,
                                       _P]),
                   "tail": _decl(lib, "mls_tail_update",
                                 [_P, _I, _I, _I, _P, _I, _P, _LL, _I, _I, _P, _P, _I, _P])}
        elif name == "headprep":
            fns = {"prep": _decl(lib, "mls_head_prep_store",
                                 [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _F, _F, _I, _F, _P, _P, _P,
                                  _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P])}
        elif name == "side":
            fns = {"settle_cast": _decl(lib, "mls_settle_cast",
                                        [_P, _P, _I, _I, _LL, _P, _I, _I, _I, _P]),
                   "gelu_gate": _decl(lib, "mls_gelu_gate_rows",
                                      [_P, _P, _I, _I, _I, _P, _I, _P, _I, _I, _I, _I, _P, _P]),
                   "rms_scale": _decl(lib, "mls_rms_scale",
                                      [_P, _I, _I, _LL, _P, _F, _P, _I, _I, _P])}
        elif name == "scan":
            fns = {"scan": _decl(lib, "mls_linear_scan",
                                 [_P, _I, _I, _I, _P, _I, _I, _I, _P, _I, _I, _I, _P, _I, _P, _P,
                                  _I, _I, _P, _P, _P, _LL, _I, _I, _I, _I, _P, _I, _P]),
                   "finish_row": _decl(lib, "mls_scan_finish_row",
                                       [_P, _P, _I, _I, _I, _P, _F, _F, _P, _LL, _I, _I, _P]),
                   "finish": _decl(lib, "mls_scan_finish",
                                   [_P, _P, _I, _I, _I, _P, _I, _F, _P, _I, _I, _I, _P]),
                   "rotate": _decl(lib, "mls_rotate_rows",
                                   [_P, _I, _I, _I, _I, _P, _P, _I, _F, _P, _I, _I, _I, _P]),
                   "decay": _decl(lib, "mls_decay_lowrank",
                                  [_P, _I, _P, _P, _I, _P, _I, _I, _P])}
        else:
            raise KernelError(f"no kernels of a part called {name!r}")
        self._part_libs[name] = fns
        return fns

    def require_part(self, name: str) -> None:
        """Build and load a part's kernels now (at bind time, not in the first step)."""
        self._part_lib(name)

    def add_layernorm(self, x, delta, weight, eps: float, h, rows=None, n_rows: int = 0,
                      more_rows=None, more_vec=None) -> None:
        """``x += delta + more_rows + more_vec`` (each optional; ``delta`` a tensor or
        ``SplitParts``), ``h = layernorm(x) * weight`` (no bias).  With ``rows`` only
        those rows are read and ``x`` stays as it is."""
        t, d = x.shape
        n_out = t if rows is None else n_rows
        _need(x.dtype == torch.float32 and x.is_contiguous(), "add_layernorm: x must be float32")
        _need(h.shape == (n_out, d) and h.is_contiguous(), "add_layernorm: bad output")
        _need(weight.shape == (d,), "add_layernorm: bad weight")
        _need(more_rows is None or (more_rows.shape == (t, d) and more_rows.dtype == torch.float32
                                    and more_rows.is_contiguous()), "add_layernorm: bad rows")
        _need(more_vec is None or (more_vec.shape == (d,) and more_vec.is_contiguous()),
              "add_layernorm: bad vector")
        _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= n_rows),
              "add_layernorm: bad row indices")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "add_layernorm")
        self.launches += 1
        _check(self._part_lib("layernorm")["add_layernorm"](
            _ptr(x), dp, dcode, parts, stride, _ptr(more_rows), _ptr(more_vec),
            _code(more_vec.dtype) if more_vec is not None else 0, _ptr(weight),
            _code(weight.dtype), float(eps), _ptr(h), _code(h.dtype), n_out, d, _ptr(rows),
            self._stream()), "add_layernorm")
        if isinstance(delta, SplitParts):
            delta.release()

    def residual_add(self, x, more_rows=None, more_vec=None) -> None:
        """``x += more_rows + more_vec`` on the float32 residual stream."""
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "residual_add: x must be float32")
        _need(more_rows is None or (more_rows.shape == (t, d) and more_rows.dtype == torch.float32
                                    and more_rows.is_contiguous()), "residual_add: bad rows")
        _need(more_vec is None or (more_vec.shape == (d,) and more_vec.is_contiguous()),
              "residual_add: bad vector")
        self.launches += 1
        _check(self._part_lib("layernorm")["residual_add"](
            _ptr(x), _ptr(more_rows), _ptr(more_vec),
            _code(more_vec.dtype) if more_vec is not None else 0, t, d, self._stream()),
            "residual_add")

    def clamped_glu(self, gu, out, alpha: float, limit: float) -> None:
        """``out = g' * sigmoid(alpha * g') * (u' + 1)`` with ``g' = min(g, limit)`` and
        ``u' = clamp(u, -limit, limit)``; a row of ``gu`` holds [gate | up]."""
        t, inter = out.shape
        _need(gu.shape == (t, 2 * inter) and gu.dtype == out.dtype, "clamped_glu: shapes")
        _need(gu.is_contiguous() and out.is_contiguous(), "clamped_glu: layout")
        self.launches += 1
        _check(self._clamped_glu(_ptr(gu), _ptr(out), _code(out.dtype), t, inter, float(alpha),
                                 float(limit), self._stream()), "clamped_glu")

    def latent_norm_store(self, down, q_rank: int, rank: int, wq, wkv, eps: float, cq, cache,
                          step) -> None:
        """From the down projections ``down [T, q_rank + rank]`` (float32): the normalised
        query latent into ``cq`` and the normalised key/value latent into the pool at the
        step's slots (rows zero-padded to the pool's width)."""
        g = step.groups[cache.group]
        t = step.n_tokens
        pool = cache.k_pool
        _need(down.shape == (t, q_rank + rank) and down.dtype == torch.float32
              and down.is_contiguous(), "latent_norm_store: bad projections")
        _need(pool.is_contiguous() and pool.shape[0] == 1 and pool.shape[3] >= rank,
              "latent_norm_store: bad pool")
        _need(q_rank == 0 or (cq.shape == (t, q_rank) and cq.dtype == pool.dtype
                              and cq.is_contiguous()), "latent_norm_store: bad query latent")
        _need(wkv.shape == (rank,) and (q_rank == 0 or (wq.shape == (q_rank,)
                                                        and wq.dtype == wkv.dtype)),
              "latent_norm_store: bad norm weights")
        self.launches += 1
        _check(self._part_lib("latent")["norm_store"](
            _ptr(down), t, q_rank, rank, pool.shape[3], _ptr(wq), _ptr(wkv), _code(wkv.dtype),
            float(eps), _ptr(cq), _code(pool.dtype), _ptr(g.slot_map), _ptr(pool), g.block_size,
            pool.shape[1] * pool.shape[2], _ptr(self.status), self._stream()),
            "latent_norm_store")

    def headwise_linear(self, src, src_width: int, w, dst, dst_width: int, n_tokens: int) -> None:
        """``dst[t, h, :N] = w[h] @ src[t, h, :K]`` for ``w [H, N, K]``: rows of ``src`` /
        ``dst`` are ``src.shape[1]`` / ``dst.shape[1]`` wide and hold the heads
        ``src_width`` / ``dst_width`` apart."""
        heads, n, k = w.shape
        _need(w.is_contiguous() and src.is_contiguous() and dst.is_contiguous()
              and src.dtype == w.dtype == dst.dtype, "headwise_linear: operands")
        _need(src.shape[0] >= n_tokens and dst.shape[0] >= n_tokens
              and src.shape[1] >= (heads - 1) * src_width + k
              and dst.shape[1] >= (heads - 1) * dst_width + n, "headwise_linear: shapes")
        if (w.dtype == torch.bfloat16 and n_tokens > 64 and self.gemm_impl != "tcgen05"
                and src.shape[1] % 8 == 0 and dst.shape[1] % 8 == 0 and src_width % 8 == 0
                and dst_width % 8 == 0 and k % 8 == 0 and n % 8 == 0):
            # many rows: a plain batched product, handed to the library as the plain
            # products of more than 64 rows are (the heads are the batch)
            held = self._transposed.get(id(w))
            if held is None or held[0] is not w:
                held = self._transposed[id(w)] = (w, w.transpose(1, 2))
            a = src.as_strided((heads, n_tokens, k), (src_width, src.shape[1], 1))
            o = dst.as_strided((heads, n_tokens, n), (dst_width, dst.shape[1], 1))
            self.library_launches += 1
            torch.bmm(a, held[1], out=o)
            return
        self.launches += 1
        _check(self._part_lib("latent")["headwise"](
            _ptr(src), src.shape[1], src_width, _ptr(w), _ptr(dst), dst.shape[1], dst_width,
            _code(w.dtype), n_tokens, heads, n, k, self._stream()), "headwise_linear")

    def mlstm_state_width(self, e: int, f: int) -> int:
        """Floats of one head's state: the memory [e, f], the normaliser [e] and one
        stabiliser per group of columns a CTA owns."""
        fc = int(self._part_lib("mlstm")["columns"](e, f))
        return e * f + e + (f + fc - 1) // fc

    def mlstm_scan(self, qkvg, offsets: tuple, gates, bias_i, bias_f, cap: float, step, state,
                   n_heads: int, e: int, f: int, num, den) -> None:
        """Walk every request's tokens through the matrix memory.  ``qkvg [T, *]`` holds
        q, k and v at the column ``offsets``; ``gates [T, 2H]`` float32 the input and
        forget pre-activations; ``num [T, H*f]``, ``den [T, H]`` float32 come out."""
        t = step.n_tokens
        width = n_heads * self.mlstm_state_width(e, f)
        _need(state.dtype == torch.float32 and state.is_contiguous()
              and state[0].numel() == width, "mlstm_scan: bad state")
        _need(gates.shape == (t, 2 * n_heads) and gates.dtype == torch.float32
              and gates.is_contiguous(), "mlstm_scan: bad gates")
        _need(qkvg.is_contiguous() and num.shape == (t, n_heads * f) and den.shape == (t, n_heads)
              and num.dtype == den.dtype == torch.float32, "mlstm_scan: bad buffers")
        _need(bias_i.shape == (n_heads,) and bias_f.dtype == bias_i.dtype, "mlstm_scan: bad biases")
        q_off, k_off, v_off = offsets
        self.launches += 1
        _check(self._part_lib("mlstm")["scan"](
            _ptr(qkvg), _code(qkvg.dtype), qkvg.shape[1], q_off, k_off, v_off, _ptr(gates),
            _ptr(bias_i), _ptr(bias_f), _code(bias_i.dtype), float(cap), _ptr(step.cu_q),
            _ptr(step.state_slot), _ptr(state), width, step.n_requests, n_heads, e, f, _ptr(num),
            _ptr(den), self._stream()), "mlstm_scan")

    def mlstm_finish(self, num, den, qkvg, g_off: int, weight, eps: float, out, n_heads: int,
                     f: int) -> None:
        """``out = unit_rms_per_head(num / den) * weight * sigmoid(gate)``."""
        t = num.shape[0]
        _need(out.shape == (t, n_heads * f) and out.is_contiguous() and out.dtype == qkvg.dtype,
              "mlstm_finish: bad output")
        _need(weight.shape == (n_heads * f,), "mlstm_finish: bad weight")
        self.launches += 1
        _check(self._part_lib("mlstm")["finish"](
            _ptr(num), _ptr(den), _ptr(qkvg), qkvg.shape[1], g_off, _ptr(weight),
            _code(weight.dtype), float(eps), _ptr(out), _code(out.dtype), t, n_heads, f,
            self._stream()), "mlstm_finish")

    def route(self, logits, top: int, renorm: bool, work: dict, softmax: bool = False,
              correction=None, renorm_eps: float = 0.0, n_real=None, groups=None,
              n_outputs=None) -> None:
        """Choose and sort: from float32 router ``logits [T, E]`` the ``top`` outputs a token
        with the largest score (sigmoid, or ``softmax`` over all outputs) plus ``correction``
        (float32 [E], in the choice only), the scores themselves as weights (``renorm``:
        divided by their sum + ``renorm_eps``), then the (token, choice) slots ordered by
        expert.  Outputs from ``n_real`` on stand for experts without weights and get no
        tiles.  ``groups = (count, keep)``: the outputs form ``count`` equal groups of
        neighbours, and only those of the ``keep`` groups whose two largest choice scores have
        the largest sum can be chosen.  ``n_outputs``: the first so many columns of a wider
        ``logits`` row are the router's.  ``work`` holds the int32 / float32 arrays
        (``expert_work``)."""
        t, row = logits.shape
        n_experts = row if n_outputs is None else int(n_outputs)
        n_groups, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        _need(n_experts <= row and n_groups >= 1 and n_experts % n_groups == 0
              and 1 <= keep <= n_groups and n_groups <= 256
              and top <= keep * (n_experts // n_groups), "route: groups do not fit the outputs")
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "route: logits")
        _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous()
                                     and correction.shape == (n_experts,)), "route: correction")
        fns = self._part_lib("experts")
        self.launches += 2
        _check(fns["topk"](_ptr(logits), row, t, n_experts, top, 1 if renorm else 0,
                           1 if softmax else 0, _ptr(correction), float(renorm_eps), n_groups, keep,
                           _ptr(work["idx"]), _ptr(work["weight"]), self._stream()), "route_topk")
        _check(fns["sort"](_ptr(work["idx"]), t * top, n_experts,
                           n_experts if n_real is None else int(n_real), _ptr(work["order"]),
                           _ptr(work["offsets"]), _ptr(work["tile_expert"]),
                           _ptr(work["tile_row0"]), work["max_tiles"], _ptr(work["cursor"]),
                           self._stream()), "route_sort")

    def expert_max_tiles(self, n_slots: int, n_experts: int) -> int:
        rows = int(self._part_lib("experts")["tile_rows"]())
        return (n_slots + rows - 1) // rows + n_experts

    @staticmethod
    def _many_rows(n_slots: int, n_experts: int) -> int:
        """Whether an expert has, on average, rows for more than two 32-row tiles: a CTA of
        the tensor-core kernel then takes four tiles of an expert against one load of its
        weights (the sums are the same either way)."""
        return 1 if n_slots >= 64 * n_experts else 0

    def expert_glu(self, h, w_gate_up, y, work: dict, top: int, scale_in: bool,
                   alpha: float = 1.0, limit: float = 0.0) -> None:
        """``y[p] = silu(Wg[e] a) * (Wu[e] a)`` for the sorted slots; ``w_gate_up [E, 2F, K]``.
        ``limit`` > 0: the clamped unit ``g' * sigmoid(alpha g') * (u' + 1)`` with
        ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)`` instead."""
        n_experts, f2, k = w_gate_up.shape
        _need(h.dtype == w_gate_up.dtype == y.dtype and h.is_contiguous() and y.is_contiguous()
              and w_gate_up.is_contiguous() and h.shape[1] == k and y.shape[1] == f2 // 2,
              "expert_glu: operands")
        self.launches += 1
        _check(self._part_lib("experts")["glu"](
            _ptr(h), _ptr(w_gate_up), _ptr(y), _code(h.dtype), _ptr(work["order"]),
            _ptr(work["offsets"]), _ptr(work["tile_expert"]), _ptr(work["tile_row0"]),
            work["max_tiles"], _ptr(work["weight"]), top, 1 if scale_in else 0, f2 // 2, k,
            self._many_rows(y.shape[0], n_experts), float(alpha), float(limit), self._stream()),
            "expert_glu")

    def expert_down(self, y, w_down, per_slot, work: dict, top: int, scale_out: bool) -> None:
        """``per_slot[slot] = Wd[e] y[p]`` (float32); ``w_down [E, D, F]``."""
        n_experts, d, f = w_down.shape
        _need(y.dtype == w_down.dtype and y.is_contiguous() and w_down.is_contiguous()
              and y.shape[1] == f and per_slot.dtype == torch.float32 and per_slot.is_contiguous()
              and per_slot.shape[1] == d, "expert_down: operands")
        self.launches += 1
        _check(self._part_lib("experts")["down"](
            _ptr(y), _ptr(w_down), _ptr(per_slot), _code(y.dtype), _ptr(work["order"]),
            _ptr(work["offsets"]), _ptr(work["tile_expert"]), _ptr(work["tile_row0"]),
            work["max_tiles"], _ptr(work["weight"]), top, 1 if scale_out else 0, d, f,
            self._many_rows(y.shape[0], n_experts), self._stream()), "expert_down")

    def expert_combine(self, per_slot, top: int, shared, delta, work=None, n_real=None,
                       h=None, shared_gate=None) -> None:
        """``delta[t] = sum_j per_slot[t * top + j] + shared[t]``; with ``n_real`` a choice of
        an output from ``n_real`` on adds ``weight * h[t]`` instead (an expert that returns
        its input).  ``shared_gate``: a float32 column (one number a token, any row stride);
        the shared addend is multiplied by its sigmoid."""
        t, d = delta.shape
        _need(per_slot.shape == (t * top, d) and delta.is_contiguous(), "expert_combine: shapes")
        _need(shared is None or (shared.shape == (t, d) and shared.is_contiguous()),
              "expert_combine: bad shared addend")
        idx = weight = None
        if n_real is not None:
            _need(work is not None and h is not None and h.shape == (t, d) and h.is_contiguous()
                  and h.dtype == delta.dtype, "expert_combine: identity experts need h and the routing")
            idx, weight = work["idx"], work["weight"]
        _need(shared_gate is None or (shared is not None and shared_gate.dtype == torch.float32
                                      and shared_gate.dim() == 1 and shared_gate.shape[0] == t),
              "expert_combine: the shared addend's gate is one float32 number a token")
        self.launches += 1
        _check(self._part_lib("experts")["combine"](
            _ptr(per_slot), top, _ptr(shared), _code(shared.dtype) if shared is not None else 0,
            _ptr(idx), _ptr(weight), int(n_real or 0), _ptr(h), _ptr(shared_gate),
            shared_gate.stride(0) if shared_gate is not None else 0,
            _ptr(delta), _code(delta.dtype), t, d, self._stream()), "expert_combine")

    def add_tanh_norm(self, x, delta, norm, h, post=None, bias=None, rows=None, n_rows: int = 0,
                      y_out=None) -> None:
        """The norm without statistics, ``n(v) = tanh(alpha v) * w + b``, in the pass that adds a
        sublayer's output to the stream: ``y = delta (+ bias)``; with ``post = (alpha, w, b,
        scale)`` ``y = n_post(y) * scale`` (``scale`` may be None); ``x += y``;
        ``h = n(x)`` with ``norm = (alpha, w, b)``.  ``delta``: a tensor, ``SplitParts`` or None.
        With ``rows`` only those rows are read and ``x`` stays as it is.  ``x`` None and ``h``
        None with ``y_out`` (float32): only the mapped delta is written."""
        src = x if x is not None else y_out
        t, d = src.shape
        n_out = t if rows is None else n_rows
        _need(x is None or (x.dtype == torch.float32 and x.is_contiguous()),
              "add_tanh_norm: x must be float32")
        _need(h is None or (h.shape == (n_out, d) and h.is_contiguous()), "add_tanh_norm: bad output")
        _need(y_out is None or (y_out.shape == (n_out, d) and y_out.dtype == torch.float32
                                and y_out.is_contiguous()), "add_tanh_norm: bad mapped output")
        vecs = [v for v in ((norm or ())[1:] + (tuple(post[1:]) if post else ()) + (bias,))
                if v is not None]
        _need(all(v.shape == (d,) and v.is_contiguous() and v.dtype == vecs[0].dtype for v in vecs),
              "add_tanh_norm: vectors of one type and of the row's width")
        _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= n_rows),
              "add_tanh_norm: bad row indices")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "add_tanh_norm")
        p_alpha, p_w, p_b, p_s = post if post else (0.0, None, None, None)
        alpha, w, b = norm if norm else (0.0, None, None)
        self.launches += 1
        _check(self._part_lib("tanhnorm")["add_tanh_norm"](
            _ptr(x), dp, dcode, parts, stride, _ptr(bias), float(p_alpha), _ptr(p_w), _ptr(p_b),
            _ptr(p_s), float(alpha), _ptr(w), _ptr(b), _code(vecs[0].dtype) if vecs else 0,
            _ptr(h), _code(h.dtype) if h is not None else 0, _ptr(y_out), _ptr(rows), n_out, d,
            self._stream()), "add_tanh_norm")
        if isinstance(delta, SplitParts):
            delta.release()

    def _row_parts(self, proj, t: int, what: str):
        """(pointer, parts, part stride, row width) of a float32 projection given as a tensor
        ``[T, W]`` or as the ``SplitParts`` of its product."""
        if isinstance(proj, SplitParts):
            parts = proj.parts
            _need(parts.dtype == torch.float32 and parts.is_contiguous() and parts.shape[1] == t,
                  f"{what}: bad parts")
            return parts.data_ptr(), parts.shape[0], t * parts.shape[2], parts.shape[2]
        _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[0] == t,
              f"{what}: the projection must be float32 rows")
        return proj.data_ptr(), 1, 0, proj.shape[1]

    def latent_rope_prep(self, proj, q_col: int, kv_col: int, n_heads: int, e: int, g: int,
                         r: int, rp: int, rot_dims: int, freq, w_kv, eps: float, q_plain, q_in,
                         cache, step) -> None:
        """From the float32 projection row ``[... q heads (e plain | g rotated) ... r + g
        down-projected ...]`` (a tensor or ``SplitParts``): the heads' plain parts into
        ``q_plain [T, H * e]``, their rotated parts into ``q_in[t, h * rp + r : + g]`` (zeros up
        to ``rp``), and, if the call writes its cache, ``[unit_rms(down[:r]) * w_kv | rotated
        down[r:] | 0]`` into the pool at the step's slots.  The first ``rot_dims`` of the g
        entries turn, entry i with i + rot_dims/2, by ``position * freq[i]`` (float64)."""
        t = step.n_tokens
        ptr, n_parts, stride, width = self._row_parts(proj, t, "latent_rope_prep")
        writes = bool(cache.writes)
        pool = cache.k_pool
        grp = step.groups[cache.group]
        _need(q_plain.shape == (t, n_heads * e) and q_plain.is_contiguous()
              and q_in.is_contiguous() and q_in.shape[0] == t and q_in.shape[1] >= n_heads * rp
              and q_plain.dtype == q_in.dtype == pool.dtype, "latent_rope_prep: bad query buffers")
        _need(pool.is_contiguous() and pool.shape[0] == 1 and pool.shape[3] == rp,
              "latent_rope_prep: bad pool")
        _need(rot_dims == 0 or (freq is not None and freq.dtype == torch.float64
                                and freq.numel() >= rot_dims // 2), "latent_rope_prep: frequencies")
        _need(not writes or w_kv.shape == (r,), "latent_rope_prep: bad norm weight")
        self.launches += 1
        _check(self._part_lib("latent")["rope_prep"](
            ptr, n_parts, stride, width, q_col, kv_col, t, n_heads, e, g, r, rp, rot_dims,
            _ptr(freq), _ptr(step.positions), _ptr(w_kv) if writes else None,
            _code(w_kv.dtype) if writes else 0, float(eps), _ptr(q_plain), _ptr(q_in),
            q_in.shape[1], _code(pool.dtype), 1 if writes else 0, _ptr(grp.slot_map), _ptr(pool),
            grp.block_size, pool.shape[1] * pool.shape[2], _ptr(self.status), self._stream()),
            "latent_rope_prep")

    def sigmoid_gate(self, o, proj, gate_col: int) -> None:
        """``o[t, c] *= sigmoid(proj[t, gate_col + c])``; ``proj`` a float32 tensor or the
        ``SplitParts`` of its product."""
        t, n = o.shape
        ptr, n_parts, stride, width = self._row_parts(proj, t, "sigmoid_gate")
        _need(o.is_contiguous() and gate_col + n <= width, "sigmoid_gate: operands")
        self.launches += 1
        _check(self._part_lib("latent")["gate"](
            _ptr(o), _code(o.dtype), ptr, n_parts, stride, width, gate_col, t, n,
            self._stream()), "sigmoid_gate")

    def settle_concat(self, x, delta, other, out) -> None:
        """``x += delta`` (a tensor, ``SplitParts`` or None), then ``out[t] = [x[t] | other[t]]``
        in ``out``'s type."""
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and other.shape == (t, d)
              and other.dtype == torch.float32 and other.is_contiguous()
              and out.shape == (t, 2 * d) and out.is_contiguous(), "settle_concat: operands")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "settle_concat")
        self.launches += 1
        _check(self._part_lib("layernorm")["settle_concat"](
            _ptr(x), dp, dcode, parts, stride, _ptr(other), _ptr(out), _code(out.dtype), t, d,
            self._stream()), "settle_concat")
        if isinstance(delta, SplitParts):
            delta.release()

    def qk_conv_norm_rope_store(self, proj, bias, conv_w, taps: int, q_norm, k_norm, eps: float,
                                tail, freq, rot_dims: int, q_out, cache, step, n_heads: int,
                                n_kv: int, hd: int, parts=None, move_tail: bool = False) -> None:
        """From the float32 projection ``proj [T, (H + G) * hd]`` (q heads, then k heads):
        add ``bias``, convolve every channel over time (``conv_w [C, taps]``; the inputs
        before the step come from ``tail [slots, (taps - 1) * C]``), store the convolved k
        as the values, RMS-normalise the whole q row and the whole k row, rotate the first
        ``rot_dims`` entries of every head (2i with 2i + 1, ``freq`` float64), write q into
        ``q_out`` and k into the pages.  ``tail_update`` moves the tail on afterwards, or,
        in a step of one token a request, this kernel itself (``move_tail``).  With ``parts``
        (``SplitParts`` of the projection) the rows are read from there instead of ``proj``."""
        g = step.groups[cache.group]
        t = step.n_tokens
        c = (n_heads + n_kv) * hd
        pool = cache.k_pool
        _need(proj.shape == (t, c) and proj.dtype == torch.float32 and proj.is_contiguous(),
              "qk_conv_norm_rope_store: bad projection")
        _need(pool.is_contiguous() and cache.v_pool.is_contiguous() and pool.shape[0] == n_kv
              and pool.shape[3] == hd and q_out.dtype == pool.dtype and q_out.is_contiguous()
              and q_out.shape[0] >= t and q_out.shape[1] >= n_heads * hd,
              "qk_conv_norm_rope_store: bad pool or output")
        _need(q_norm.shape == (n_heads * hd,) and k_norm.shape == (n_kv * hd,)
              and q_norm.dtype == k_norm.dtype, "qk_conv_norm_rope_store: bad norm weights")
        _need(bias is None or (bias.shape == (c,) and bias.dtype == q_norm.dtype
                               and bias.is_contiguous()), "qk_conv_norm_rope_store: bad bias")
        _need(taps == 0 or (conv_w.shape == (c, taps) and conv_w.dtype == q_norm.dtype
                            and conv_w.is_contiguous()), "qk_conv_norm_rope_store: bad taps")
        _need(taps <= 1 or (tail.dtype == torch.float32 and tail.stride(1) == 1
                            and tail.shape[1] == (taps - 1) * c),
              "qk_conv_norm_rope_store: bad tail")
        _need(rot_dims == 0 or (freq.dtype == torch.float64 and freq.numel() == rot_dims // 2),
              "qk_conv_norm_rope_store: bad frequencies")
        _need(not move_tail or step.max_q_len == 1,
              "qk_conv_norm_rope_store: the tail moves in the kernel only in steps of single tokens")
        src, n_parts, stride = proj.data_ptr(), 1, 0
        if parts is not None:
            _need(tuple(parts.shape) == (t, c) and parts.parts.is_contiguous(),
                  "qk_conv_norm_rope_store: these parts cannot be read")
            src, n_parts, stride = parts.parts.data_ptr(), parts.parts.shape[0], t * c
        self.launches += 1
        _check(self._part_lib("shortconv")["qk"](
            src, n_parts, stride, _ptr(bias), _ptr(conv_w) if taps else None, taps, _ptr(q_norm),
            _ptr(k_norm), _code(q_norm.dtype), float(eps), _ptr(tail) if taps > 1 else None,
            tail.stride(0) if taps > 1 else 0, 1 if (move_tail and taps > 1) else 0,
            _ptr(step.state_slot), _ptr(step.cu_q),
            _ptr(step.req_of_token), _ptr(step.positions), _ptr(freq) if rot_dims else None,
            rot_dims, _ptr(q_out), q_out.shape[1], _code(pool.dtype), _ptr(g.slot_map), _ptr(pool),
            _ptr(cache.v_pool), g.block_size, pool.shape[1] * pool.shape[2], t, n_heads, n_kv, hd,
            1 if cache.writes else 0, _ptr(self.status), self._stream()),
            "qk_conv_norm_rope_store")
        if parts is not None:
            parts.release()

    def tail_update(self, src, col0: int, channels: int, bias, tail, n_tail: int, step) -> None:
        """``tail [slots, n_tail * channels]`` (float32, oldest row first) becomes the last
        ``n_tail`` rows of every request's sequence after this step: rows of ``src[:, col0 :
        col0 + channels]`` (plus ``bias``), or, for a short step, the old tail's."""
        _need(src.is_contiguous() and src.shape[0] >= step.n_tokens
              and src.shape[1] >= col0 + channels, "tail_update: bad rows")
        _need(tail.dtype == torch.float32 and tail.stride(1) == 1
              and tail.shape[1] == n_tail * channels, "tail_update: bad tail")
        _need(bias is None or (bias.shape == (channels,) and bias.is_contiguous()),
              "tail_update: bad bias")
        self.launches += 1
        _check(self._part_lib("shortconv")["tail"](
            _ptr(src), _code(src.dtype), src.shape[1], col0, _ptr(bias),
            _code(bias.dtype) if bias is not None else 0, _ptr(tail), tail.stride(0), n_tail,
            channels, _ptr(step.state_slot), _ptr(step.cu_q), step.n_requests, self._stream()),
            "tail_update")

    def token_shift_mix(self, h, mu, prev, out, out_f32, step, move_tail: bool = False) -> None:
        """``mix_s[t] = h[t] + (h[t - 1] - h[t]) * mu[s]`` for every row s of ``mu [n, d]``,
        with a request's row before its first of the step from ``prev [slots, d]``
        (float32).  ``out [n or n - 1, T, d]``; with ``out_f32 [T, d]`` the last mix goes
        there in float32.  ``move_tail`` (steps of one token a request only): ``prev`` becomes
        this step's rows in the same kernel."""
        t, d = h.shape
        n = mu.shape[0]
        _need(h.is_contiguous() and mu.shape == (n, d) and mu.is_contiguous(),
              "token_shift_mix: operands")
        _need(prev.dtype == torch.float32 and prev.stride(1) == 1 and prev.shape[1] == d,
              "token_shift_mix: bad previous rows")
        _need(out.dtype == h.dtype and out.is_contiguous() and out.shape[1:] == (t, d)
              and out.shape[0] >= (n - 1 if out_f32 is not None else n), "token_shift_mix: out")
        _need(out_f32 is None or (out_f32.shape == (t, d) and out_f32.dtype == torch.float32
                                  and out_f32.is_contiguous()), "token_shift_mix: float32 out")
        _need(not move_tail or step.max_q_len == 1,
              "token_shift_mix: the previous rows move in the kernel only in steps of single tokens")
        self.launches += 1
        _check(self._part_lib("shortconv")["shift_mix"](
            _ptr(h), _code(h.dtype), _ptr(mu), _code(mu.dtype), n, _ptr(prev), prev.stride(0),
            1 if move_tail else 0, _ptr(step.state_slot), _ptr(step.cu_q), _ptr(step.req_of_token), _ptr(out),
            _ptr(out_f32), t, d, self._stream()), "token_shift_mix")

    def require_scan(self, e: int) -> None:
        """Say at bind time whether the scan kernel takes a key size."""
        _need(0 < e <= 256, f"the scan kernel keeps up to 256 rows of a head's state, not {e}")

    def linear_scan(self, a, k, v, state, step, n_heads: int, e: int, f: int, out,
                    decay_tok=None, decay_head=None, bonus=None, read_first: bool = False,
                    silu: bool = False) -> None:
        """Walk every request's tokens through the matrix state ``S [e, f]`` of every head.
        ``a``, ``k``, ``v``: (tensor [T, *], first column) of the read vector, keys and
        values.  ``decay_tok [T, H*e]`` float32 (a decay per token and key channel) or
        ``decay_head [H]`` float32 (one a head).  ``read_first``: the token reads
        ``S + diag(bonus) k v^T`` and the state moves on afterwards; else the state takes
        the token in and is then read.  ``silu``: a, k and v pass through ``z * sigmoid(z)`` as
        they are read.  ``state [slots, >= H*e*f]`` float32, ``out [T, H*f]`` float32."""
        t = step.n_tokens
        for (src, off), width in ((a, e), (k, e), (v, f)):
            _need(src.is_contiguous() and src.shape[0] >= t
                  and src.shape[1] >= off + n_heads * width, "linear_scan: bad operand")
        _need(state.dtype == torch.float32 and state.stride(1) == 1
              and state.shape[1] >= n_heads * e * f, "linear_scan: bad state")
        _need(out.shape == (t, n_heads * f) and out.dtype == torch.float32 and out.is_contiguous(),
              "linear_scan: bad out")
        _need((decay_tok is None) != (decay_head is None), "linear_scan: one kind of decay")
        _need(decay_tok is None or (decay_tok.shape == (t, n_heads * e) and decay_tok.is_contiguous()
                                    and decay_tok.dtype == torch.float32), "linear_scan: decay")
        _need(decay_head is None or (decay_head.shape == (n_heads,)
                                     and decay_head.dtype == torch.float32), "linear_scan: decay")
        _need(bonus is None or (bonus.numel() == n_heads * e and bonus.is_contiguous()),
              "linear_scan: bad bonus")
        self.launches += 1
        _check(self._part_lib("scan")["scan"](
            _ptr(a[0]), _code(a[0].dtype), a[0].shape[1], a[1],
            _ptr(k[0]), _code(k[0].dtype), k[0].shape[1], k[1],
            _ptr(v[0]), _code(v[0].dtype), v[0].shape[1], v[1],
            _ptr(decay_tok), n_heads * e, _ptr(decay_head), _ptr(bonus),
            _code(bonus.dtype) if bonus is not None else 0, 1 if read_first else 0,
            _ptr(step.cu_q), _ptr(step.state_slot), _ptr(state), state.stride(0),
            step.n_requests, n_heads, e, f, _ptr(out), 1 if silu else 0, self._stream()),
            "linear_scan")

    def scan_finish(self, o, gate, gate_off: int, weight, eps: float, out, n_heads: int,
                    f: int) -> None:
        """``out = o / rms_per_head(o) * weight * silu(gate)`` (``weight`` may be None)."""
        t = o.shape[0]
        _need(o.shape == (t, n_heads * f) and o.dtype == torch.float32 and o.is_contiguous()
              and out.shape == (t, n_heads * f) and out.is_contiguous()
              and out.dtype == gate.dtype and gate.is_contiguous()
              and gate.shape[1] >= gate_off + n_heads * f, "scan_finish: operands")
        _need(weight is None or weight.shape == (n_heads * f,), "scan_finish: bad weight")
        self.launches += 1
        _check(self._part_lib("scan")["finish"](
            _ptr(o), _ptr(gate), _code(gate.dtype), gate.shape[1], gate_off, _ptr(weight),
            _code(weight.dtype) if weight is not None else 0, float(eps), _ptr(out), t, n_heads,
            f, self._stream()), "scan_finish")

    def scan_finish_row(self, o, gate, gate_off: int, weight, eps: float, out,
                        out_scale: float = 1.0) -> None:
        """``out = o / rms(o over the whole row) * weight * sigmoid(gate) * out_scale``;
        ``weight`` float32 or None; ``out`` may be a block of columns of a wider buffer."""
        t, width = o.shape
        _need(o.dtype == torch.float32 and o.is_contiguous() and out.shape == (t, width)
              and out.stride(1) == 1 and out.dtype == gate.dtype and gate.is_contiguous()
              and gate.shape[1] >= gate_off + width, "scan_finish_row: operands")
        _need(weight is None or (weight.shape == (width,) and weight.dtype == torch.float32
                                 and weight.is_contiguous()), "scan_finish_row: bad weight")
        self.launches += 1
        _check(self._part_lib("scan")["finish_row"](
            _ptr(o), _ptr(gate), _code(gate.dtype), gate.shape[1], gate_off, _ptr(weight),
            float(eps), float(out_scale), _ptr(out), out.stride(0), t, width, self._stream()),
            "scan_finish_row")

    def head_prep_store(self, proj, cols: tuple, biases, norms, eps: float, q_temp, v_scale: float,
                        q_out, cache, step, n_heads: int, n_kv: int, e: int, f: int,
                        hd: int) -> None:
        """From the float32 projection ``proj [T, W]`` with q, k and v heads (``e``, ``e`` and
        ``f`` entries each) from the columns ``cols = (q, k, v)`` on: add ``biases = (b_q, b_k,
        b_v)`` (float32, or None), RMS-normalise every q and k head with ``norms = (w_q, w_k)``
        (float32 [e], or None), multiply q by ``1 + coef * ln(floor((p + 1) / every) + 1)``
        (``q_temp = (coef, every)`` or None) and v by ``v_scale``; q goes to ``q_out`` (head h
        at column ``h * hd``), k and v into the pages at the step's slots, every head padded
        with zeros to ``hd`` entries; the rest of a page a request enters is cleared."""
        g = step.groups[cache.group]
        t = step.n_tokens
        pool = cache.k_pool
        _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[0] == t
              and proj.shape[1] >= max(cols[0] + n_heads * e, cols[1] + n_kv * e,
                                       cols[2] + n_kv * f), "head_prep_store: bad projection")
        _need(pool.is_contiguous() and cache.v_pool.is_contiguous() and pool.shape[0] == n_kv
              and pool.shape[3] == hd and hd >= max(e, f) and q_out.dtype == pool.dtype
              and q_out.is_contiguous() and q_out.shape[0] >= t and q_out.shape[1] >= n_heads * hd,
              "head_prep_store: bad pool or output")
        vecs = [v for v in (tuple(biases or ()) + tuple(norms or ())) if v is not None]
        _need(all(v.dtype == torch.float32 and v.is_contiguous() for v in vecs),
              "head_prep_store: float32 vectors")
        b_q, b_k, b_v = biases if biases else (None, None, None)
        w_q, w_k = norms if norms else (None, None)
        _need(b_q is None or (b_q.numel() == n_heads * e and b_k.numel() == n_kv * e
                              and b_v.numel() == n_kv * f), "head_prep_store: bad biases")
        _need(w_q is None or (w_q.numel() == e and w_k.numel() == e), "head_prep_store: bad norms")
        coef, every = q_temp if q_temp else (0.0, 0)
        self.launches += 1
        _check(self._part_lib("headprep")["prep"](
            _ptr(proj), proj.shape[1], cols[0], cols[1], cols[2], _ptr(b_q), _ptr(b_k), _ptr(b_v),
            _ptr(w_q), _ptr(w_k), float(eps), float(coef), int(every), float(v_scale),
            _ptr(step.positions), _ptr(g.slot_map), _ptr(q_out), q_out.shape[1], _code(pool.dtype),
            _ptr(pool), _ptr(cache.v_pool), g.block_size, pool.shape[1], t, n_heads, n_kv, e, f,
            hd, 1 if cache.writes else 0, _ptr(self.status), self._stream()), "head_prep_store")

    def settle_cast(self, x, delta, out) -> None:
        """``x += delta`` (a tensor, ``SplitParts`` or None); ``out = x`` in ``out``'s type."""
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and out.shape == (t, d)
              and out.is_contiguous(), "settle_cast: operands")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "settle_cast")
        self.launches += 1
        _check(self._part_lib("side")["settle_cast"](
            _ptr(x), dp, dcode, parts, stride, _ptr(out), _code(out.dtype), t, d, self._stream()),
            "settle_cast")
        if isinstance(delta, SplitParts):
            delta.release()

    def gelu_gate_rows(self, z, table, col0: int, token_ids, out, n_real=None) -> None:
        """``out[t, c] = gelu_tanh(z[t, c]) * table[token[t], col0 + c]`` for the first
        ``n_real`` columns (all, if None), zeros in the others; ``z`` float32."""
        t, dim = z.shape
        n_real = dim if n_real is None else int(n_real)
        _need(z.dtype == torch.float32 and z.is_contiguous() and out.shape == (t, dim)
              and out.is_contiguous() and table.is_contiguous() and table.dim() == 2
              and 0 <= col0 and n_real <= dim and col0 + n_real <= table.shape[1]
              and token_ids.dtype == torch.int32 and token_ids.numel() >= t,
              "gelu_gate_rows: operands")
        self.launches += 1
        _check(self._part_lib("side")["gelu_gate"](
            _ptr(z), _ptr(table), _code(table.dtype), table.shape[1], col0, _ptr(token_ids),
            table.shape[0], _ptr(out), _code(out.dtype), t, dim, n_real, _ptr(self.status),
            self._stream()), "gelu_gate_rows")

    def rms_scale(self, y, weight, eps: float, out) -> None:
        """``out[t] = y[t] / sqrt(mean(y[t]^2) + eps) * weight`` in float32; ``y`` a tensor or
        ``SplitParts``."""
        t, d = out.shape
        _need(out.dtype == torch.float32 and out.is_contiguous() and weight.shape == (d,)
              and weight.dtype == torch.float32 and weight.is_contiguous(), "rms_scale: operands")
        dp, dcode, parts, stride = self._delta_args(y, t, d, "rms_scale")
        self.launches += 1
        _check(self._part_lib("side")["rms_scale"](
            dp, dcode, parts, stride, _ptr(weight), float(eps), _ptr(out), t, d, self._stream()),
            "rms_scale")
        if isinstance(y, SplitParts):
            y.release()

    def rotate_rows(self, src, q_off: int, k_off: int, positions, freq, dims: int,
                    k_scale: float, out, n_heads: int, e: int) -> None:
        """``out[t] = [rot(q) | rot(k) * k_scale]`` in float32: the first ``dims`` entries of
        every head rotated by position * ``freq`` (float64), entry i paired with i + dims/2."""
        t = out.shape[0]
        _need(src.is_contiguous() and src.shape[0] >= t and out.shape == (t, 2 * n_heads * e)
              and out.dtype == torch.float32 and out.is_contiguous(), "rotate_rows: operands")
        _need(dims == 0 or (freq.dtype == torch.float64 and freq.numel() == dims // 2),
              "rotate_rows: bad frequencies")
        self.launches += 1
        _check(self._part_lib("scan")["rotate"](
            _ptr(src), _code(src.dtype), src.shape[1], q_off, k_off, _ptr(positions),
            _ptr(freq) if dims else None, dims, float(k_scale), _ptr(out), t, n_heads, e,
            self._stream()), "rotate_rows")

    def decay_lowrank(self, lo, w2t, w0, out) -> None:
        """``out = exp(-exp(tanh(lo) @ w2t + w0))``, all float32; ``w2t [rank, C]`` is the
        second matrix of the decay transposed."""
        t, rank = lo.shape
        c = w2t.shape[1]
        _need(lo.dtype == torch.float32 and lo.is_contiguous() and w2t.shape == (rank, c)
              and w2t.dtype == torch.float32 and w2t.is_contiguous() and w0.shape == (c,)
              and out.shape == (t, c) and out.dtype == torch.float32 and out.is_contiguous(),
              "decay_lowrank: operands")
        self.launches += 1
        _check(self._part_lib("scan")["decay"](
            _ptr(lo), rank, _ptr(w2t), _ptr(w0), _code(w0.dtype), _ptr(out), t, c, self._stream()),
            "decay_lowrank")

    def sample(self, logits, temperature, uniform, out) -> None:
        """Tokens for float32 ``logits [n, V]``; rows with temperature <= 0 (or
        ``temperature`` None) take the arg max, lowest index on ties."""
        n, v = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits")
        _need(out.dtype == torch.int32 and out.numel() >= n, "sample: out")
        if temperature is not None:
            _need(temperature.dtype == torch.float32 and uniform.dtype == torch.float32,
                  "sample: temperature and uniform must be float32")
        scratch = None
        if v > 4096:             # chunks of the vocabulary on many SMs, then a pick a row
            scratch = self.scratch("argmax_chunks", 3 * n * ((v + 4095) // 4096))
        self.launches += 2 if scratch is not None else 1
        _check(self._sample(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out), n, v,
                            _ptr(scratch), self._stream()), "sample")


class Runtime:
    """Device, element types, kernels and step buffers shared by a model's parts."""

    residual_dtype = torch.float32
    logits_dtype = torch.float32

    def __init__(self, device="cuda:0", dtype: torch.dtype = torch.bfloat16):
        self.device = torch.device(device)
        self.act_dtype = dtype
        self.ops = Ops(self.device, dtype)
        self._buffers: dict = {}
        self._views: dict = {}               # (tag, dtype, shape) -> the view handed out last time

    def buffer(self, tag: str, shape: tuple, dtype: torch.dtype):
        """A step buffer: the same memory for the same tag, grown when needed."""
        shape = tuple(shape)
        view = self._views.get((tag, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        flat = self._buffers.get(key)
        if flat is None or flat.numel() < n:
            flat = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = flat
            self.ops.generation += 1       # captured graphs point at the old memory
            for old in [k for k in self._views if k[0] == tag and k[1] == dtype]:
                del self._views[old]
        view = flat[:n].view(shape)
        if len(self._views) > 4096:          # many shapes have come and gone
            self._views.clear()
        self._views[(tag, dtype, shape)] = view
        return view
