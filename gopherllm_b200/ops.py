"""Python face of the CUDA kernels.

Every function checks sizes, element types and devices on the host, then calls
one launcher on the current CUDA stream.  There is no CPU implementation and no
library fallback: a tensor that is not on a CUDA device, or a library that does
not build, is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_void_p
from typing import Optional

import torch

from .csrc import build, catalog

PAGE = 64                      # tokens per cache page (GL_PAGE)
F32, BF16 = 0, 1
# (an activation with numbers of its own travels as a tuple: ("xielu", up, down))
ACTIVATIONS = {"none": 0, None: 0, "gelu_new": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3,
               "relu2": 4,      # the square of relu
               "silu": 5}
SAMPLE_WINDOW = 64             # tokens the repeat penalty looks back on (runtime.go:27)
SAMPLE_KMAX = 1024

_ERRORS = {
    -1: "this combination of element types is not built",
    -2: "a size the kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel requires",
    -4: "the launch failed (cudaGetLastError)",
    -5: "the kernel needs more shared memory than the device allows",
    -6: "a CUDA driver entry point is missing or failed",
    -7: "the call needs more scratch than the library's built-in array holds",
}


class KernelError(RuntimeError):
    pass


LAUNCHES = 0       # kernels launched through this module since it was last set to 0


def _check(code: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if _TAPE is not None and _TAPE.calls and _TAPE.calls[-1][2] is None:
        _TAPE.calls[-1][2:] = [what, kernels]
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")


# ---------------------------------------------------------------------------
# A tape of launches.  The layers of a model are mostly the same block with other tensors; what the
# host does for one of them (checks, sizes, argument records: some 100 us for a block of five kernels,
# more than the kernels take for a short prompt) is the same for the next but for a handful of
# pointers.  So the launches of one block's run can be recorded and repeated for another block of the
# same shape with that block's tensors in place of the first one's.
class _StreamArg(c_void_p):
    """The stream argument of a launch (a repeated launch takes the stream that is current then)."""


class LaunchTape:
    """The launches between ``start()`` and ``stop()``: [function, arguments, name, kernels] each, and
    the tensors that were allocated for them meanwhile (kept alive: a repeat uses them again)."""

    def __init__(self):
        self.calls: list = []
        self.temps: list = []
        self.slots: list = []
        self.streams: list = []

    def start(self) -> "LaunchTape":
        global _TAPE
        if _TAPE is not None:
            raise KernelError("a tape of launches is already being recorded")
        _TAPE = self
        return self

    def stop(self) -> "LaunchTape":
        global _TAPE
        _TAPE = None
        return self

    def _pointers(self):
        """Every place a pointer stands: (holder, attribute), a c_void_p argument or a record's field."""
        for call in self.calls:
            for a in call[1]:
                if isinstance(a, _StreamArg):
                    continue
                if isinstance(a, c_void_p):
                    yield a, "value"
                else:
                    st = getattr(a, "_obj", None)
                    if isinstance(st, Structure):
                        for name, typ in st._fields_:
                            if typ is c_void_p:
                                yield st, name

    def bind(self, ptrs: dict) -> None:
        """``ptrs``: name -> address of the recorded block's tensors.  Finds the places that hold one."""
        by_ptr: dict = {}
        for k, v in ptrs.items():
            if v:
                by_ptr.setdefault(v, k)
        self.slots = [(h, attr, by_ptr[getattr(h, attr)]) for h, attr in self._pointers()
                      if getattr(h, attr) in by_ptr]
        self.streams = [a for call in self.calls for a in call[1] if isinstance(a, _StreamArg)]

    def same_as(self, other: "LaunchTape", mine: dict, theirs: dict) -> bool:
        """Whether ``other``, the tape of another block's own run, is this tape with that block's tensors
        (``theirs``) in place of this one's (``mine``) and its temporaries in place of this one's, and
        nothing else different: then repeating this tape with a third block's tensors is that block's run."""
        if mine.keys() != theirs.keys() or len(self.calls) != len(other.calls) or len(self.temps) != len(other.temps):
            return False
        to: dict = {}
        for k, v in mine.items():
            if bool(v) != bool(theirs[k]) or (v and to.setdefault(v, theirs[k]) != theirs[k]):
                return False
        for a, b in zip(self.temps, other.temps):
            if a.shape != b.shape or a.dtype != b.dtype:
                return False
            to[a.data_ptr()] = b.data_ptr()

        def same_pointer(u, v):
            return (not u and not v) or (bool(u) and to.get(u, u) == v)

        for (f0, a0, w0, k0), (f1, a1, w1, k1) in zip(self.calls, other.calls):
            if f0 is not f1:
                return False
            if w0 != w1 or k0 != k1 or len(a0) != len(a1):
                return False
            for u, v in zip(a0, a1):
                if type(u) is not type(v):
                    return False
                if isinstance(u, _StreamArg):
                    continue
                if isinstance(u, c_void_p):
                    if not same_pointer(u.value, v.value):
                        return False
                    continue
                su, sv = getattr(u, "_obj", None), getattr(v, "_obj", None)
                if isinstance(su, Structure):
                    if type(su) is not type(sv):
                        return False
                    for name, typ in su._fields_:
                        x, y = getattr(su, name), getattr(sv, name)
                        if typ is c_void_p:
                            if not same_pointer(x, y):
                                return False
                        elif hasattr(x, "__len__"):
                            if list(x) != list(y):
                                return False
                        elif x != y:
                            return False
                elif getattr(u, "value", u) != getattr(v, "value", v):
                    return False
        return True

    def repeat(self, ptrs: dict) -> None:
        """Launch everything again with these tensors in the recorded block's places."""
        global TAPE_REPEATS
        TAPE_REPEATS += 1
        for h, attr, key in self.slots:
            setattr(h, attr, ptrs[key] or None)
        if self.streams:
            cur = _stream().value
            for a in self.streams:
                a.value = cur
        for fn, args, what, kernels in self.calls:
            _check(_launch(fn, *args), what, kernels)


_TAPE: Optional[LaunchTape] = None
TAPE_REPEATS = 0            # tapes repeated since this was last set to 0
REPEAT_LAYERS = True        # whether a model repeats the recorded launches of equal blocks (engine/model.py)


def _launch(fn, *args) -> int:
    """Every kernel launch of this module goes through here."""
    if _TAPE is not None:
        _TAPE.calls.append([fn, args, None, 1])
    return fn(*args)


def empty(shape, dtype, device) -> torch.Tensor:
    """Uninitialised memory for a kernel's output (what the kernels' callers allocate with, so that a
    tape of launches can keep it)."""
    t = torch.empty(shape, dtype=dtype, device=device)
    if _TAPE is not None:
        _TAPE.temps.append(t)
    return t


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t} is not supported by the kernels (float32 and bfloat16 are)")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> "_StreamArg":
    # (the raw handle straight from the runtime: a step launches a few hundred kernels, and building a
    # Stream object for each costs more host time than a short kernel runs)
    if _RAW_STREAM is not None:
        return _StreamArg(_RAW_STREAM(torch.cuda.current_device()))
    return _StreamArg(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _addr(t: Optional[torch.Tensor]):
    """Address for a structure field (None is a null pointer)."""
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the kernels have no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, has {tuple(t.shape)}")


_LIBS: dict = {}
# GOPHERLLM_DEBUG_BOUNDS=1 selects builds of the kernels that check the indices they take from memory
# (token ids, page numbers, positions) and record a bad one instead of using it; see bounds_status().
DEBUG_BOUNDS = os.environ.get("GOPHERLLM_DEBUG_BOUNDS", "") not in ("", "0")


def _lib(source: str, defines=()):
    if DEBUG_BOUNDS:
        defines = tuple(defines) + ("GL_DEBUG_BOUNDS=1",)
    key = (source, tuple(defines))
    lib = _LIBS.get(key)
    if lib is None:
        lib = _LIBS[key] = build.load(source, key[1])
    return lib


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = scale * table[tokens[t]] as float32."""
    _need(table, "table")
    _need(tokens, "tokens", torch.int32)
    V, D = table.shape
    T = tokens.numel()
    if out is None:
        out = empty((T, D), torch.float32, table.device)
    _need(out, "out", torch.float32, (T, D))
    fn = _lib("rowwise.cu").gl_embed
    _check(_launch(fn, _ptr(table), c_int(dtype_code(table.dtype)), _ptr(tokens), _ptr(out),
              c_int(T), c_int(D), c_int(V), c_float(scale), _stream()), "embed")
    return out


def add_rows(table: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] += table[index[t]] (float32 rows; a table of learned positions added to the residual stream)."""
    _need(table, "table")
    _need(index, "index", torch.int32)
    N, D = table.shape
    _need(out, "out", torch.float32, (index.numel(), D))
    fn = _lib("rowwise.cu").gl_add_rows
    _check(_launch(fn, _ptr(table), c_int(dtype_code(table.dtype)), _ptr(index), _ptr(out),
              c_int(index.numel()), c_int(D), c_int(N), _stream()), "add_rows")
    return out


class _EmbedPairArgs(Structure):
    _fields_ = [("table", c_void_p), ("pair_table", c_void_p), ("tokens", c_void_p), ("tok_seq", c_void_p),
                ("tok_pos", c_void_p), ("seq_slot", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p),
                ("last_token", c_void_p), ("out", c_void_p),
                ("T", c_int), ("D", c_int), ("V", c_int), ("buckets", c_int), ("stride", c_int),
                ("mul_prev", ctypes.c_longlong), ("mul_cur", ctypes.c_longlong), ("scale", c_float)]


def embed_pair(table: torch.Tensor, pair_table: torch.Tensor, ctx, last_token: torch.Tensor, mul_prev: int,
               mul_cur: int, scale: float = 1.0) -> torch.Tensor:
    """out[t] = scale * table[token] + pair_table[(token before * mul_prev + token * mul_cur) mod buckets] as
    float32, buckets = rows of pair_table - 1; a sequence's first token takes the last row.  ``last_token``
    [slots, n] int32 holds, in column 0 of a sequence's row, the token before the step's first; it receives the
    step's last."""
    _need(table, "table")
    _need(pair_table, "pair_table", table.dtype)
    _need(last_token, "last_token", torch.int32)
    V, D = table.shape
    if pair_table.shape[1] != D or pair_table.shape[0] < 2 or last_token.dim() != 2:
        raise KernelError(f"embed_pair: tables {tuple(table.shape)} and {tuple(pair_table.shape)} do not fit")
    T = ctx.tokens.numel()
    out = empty((T, D), torch.float32, table.device)
    a = _EmbedPairArgs(table.data_ptr(), pair_table.data_ptr(), ctx.tokens.data_ptr(), ctx.tok_seq.data_ptr(),
                       ctx.tok_pos.data_ptr(), ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(),
                       last_token.data_ptr(), out.data_ptr(), T, D, V, pair_table.shape[0] - 1, last_token.shape[1],
                       int(mul_prev), int(mul_cur), scale)
    fn = _lib("rowwise.cu").gl_embed_pair
    _check(_launch(fn, byref(a), c_int(dtype_code(table.dtype)), _stream()), "embed_pair")
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 logits: x * scale, then cap * tanh(x / cap) when cap > 0."""
    _need(x, "x", torch.float32)
    fn = _lib("rowwise.cu").gl_scale_softcap
    _check(_launch(fn, _ptr(x), ctypes.c_longlong(x.numel()), c_float(scale), c_float(cap), _stream()), "scale_softcap")
    return x


def norm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
         out_dtype: torch.dtype, rms: bool = False, rows: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm (or RMSNorm) of float32 rows; ``rows`` picks rows of x."""
    _need(x, "x", torch.float32)
    D = x.shape[-1]
    _need(gamma, "gamma", torch.float32, (D,))
    if beta is not None:
        _need(beta, "beta", torch.float32, (D,))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        R = rows.numel()
    else:
        R = x.numel() // D
    if out is None:
        out = empty((R, D), out_dtype, x.device)
    _need(out, "out", out_dtype, (R, D))
    fn = _lib("rowwise.cu").gl_norm
    _check(_launch(fn, _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), c_int(dtype_code(out_dtype)),
              c_int(R), c_int(D), c_float(eps), c_int(1 if rms else 0), _stream()), "norm")
    return out


def advance_decode(tokens, tok_pos, seq_ctx, sampled, history, counter) -> None:
    """After a decode step on the device: tokens <- sampled, positions and cached lengths + 1,
    history[counter] <- sampled, counter + 1 (all int32; history is [max_steps, B])."""
    B = tokens.numel()
    for n, t in (("tokens", tokens), ("tok_pos", tok_pos), ("seq_ctx", seq_ctx)):
        _need(t, n, torch.int32, (B,))
    _need(sampled, "sampled", torch.int32)
    _need(history, "history", torch.int32)
    _need(counter, "counter", torch.int32, (1,))
    if sampled.numel() < B or history.shape[-1] != B:
        raise KernelError("advance_decode: sampled or history does not match the batch")
    fn = _lib("rowwise.cu").gl_advance_decode
    _check(_launch(fn, _ptr(tokens), _ptr(tok_pos), _ptr(seq_ctx), _ptr(sampled), _ptr(history), _ptr(counter),
              c_int(B), c_int(history.shape[0]), _stream()), "advance_decode")


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor):
    """cos and sin of float32(pos) * inv_freq, each [T, half] float32.  With float64 frequencies the
    angle is the 64-bit product pos * inv_freq."""
    _need(pos, "pos", torch.int32)
    T, half = pos.numel(), inv_freq.numel()
    cosv = empty((T, half), torch.float32, pos.device)
    sinv = empty(cosv.shape, cosv.dtype, cosv.device)
    if inv_freq.dtype == torch.float64:
        _need(inv_freq, "inv_freq", torch.float64)
        fn = _lib("qkv_cache.cu").gl_rope_table64
        _check(_launch(fn, _ptr(pos), _ptr(inv_freq), _ptr(cosv), _ptr(sinv), c_int(T), c_int(half), _stream()),
               "rope_table")
        return cosv, sinv
    _need(inv_freq, "inv_freq", torch.float32)
    fn = _lib("qkv_cache.cu").gl_rope_table
    _check(_launch(fn, _ptr(pos), _ptr(inv_freq), _ptr(cosv), _ptr(sinv), c_int(T), c_int(half), _stream()),
           "rope_table")
    return cosv, sinv


class _QkvCacheArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p),
                ("q_gamma", c_void_p), ("q_beta", c_void_p), ("k_gamma", c_void_p), ("k_beta", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("pages", c_void_p),
                ("T", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("half", c_int),
                ("max_pages", c_int), ("interleaved", c_int), ("norm_rms", c_int), ("write_kv", c_int),
                ("eps", c_float), ("q_scale", c_float), ("n_pages", c_int)]


def qkv_to_cache(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 tok_seq: torch.Tensor, tok_pos: torch.Tensor, pages: torch.Tensor,
                 num_heads: int, num_kv_heads: int, head_dim: int, q_scale: float,
                 cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                 interleaved: bool = False,
                 q_norm=None, k_norm=None, norm_eps: float = 0.0, norm_rms: bool = False,
                 write_kv: bool = True) -> None:
    """Head norm, rotation and scale of projected rows; q to ``q_out``, k and v into cache pages.

    qkv: [T, (nH + 2 nKV) * hd]; k_cache, v_cache: [pages, nKV, PAGE, hd];
    pages: [B, max_pages] int32; q_norm / k_norm: (gamma, beta or None) or None.
    """
    _need(qkv, "qkv")
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv, "qkv", shape=(T, width))
    _need(q_out, "q_out", qkv.dtype, (T, num_heads * head_dim))
    _need(k_cache, "k_cache")
    _need(v_cache, "v_cache", k_cache.dtype, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(tok_seq, "tok_seq", torch.int32, (T,))
    _need(tok_pos, "tok_pos", torch.int32, (T,))
    _need(pages, "pages", torch.int32)
    half = 0
    if cos is not None:
        half = cos.shape[-1]
        _need(cos, "cos", torch.float32, (T, half))
        _need(sin, "sin", torch.float32, (T, half))
        if 2 * half > head_dim:
            raise KernelError(f"rotary dimension {2 * half} exceeds head size {head_dim}")
    qg = qb = kg = kb = None
    if q_norm is not None:
        qg, qb = q_norm
        kg, kb = k_norm
        for n, t in (("q_norm.gamma", qg), ("k_norm.gamma", kg)):
            _need(t, n, torch.float32, (head_dim,))
        for n, t in (("q_norm.beta", qb), ("k_norm.beta", kb)):
            if t is not None:
                _need(t, n, torch.float32, (head_dim,))
    a = _QkvCacheArgs(qkv.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                      _addr(cos), _addr(sin), _addr(qg), _addr(qb), _addr(kg), _addr(kb),
                      tok_seq.data_ptr(), tok_pos.data_ptr(), pages.data_ptr(),
                      T, num_heads, num_kv_heads, head_dim, half, pages.shape[-1],
                      1 if interleaved else 0, 1 if norm_rms else 0, 1 if write_kv else 0,
                      norm_eps, q_scale, k_cache.shape[0])
    fn = _lib("qkv_cache.cu").gl_qkv_cache
    _check(_launch(fn, byref(a), c_int(dtype_code(qkv.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "qkv_to_cache")


class _AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("seq_qstart", c_void_p), ("seq_qlen", c_void_p), ("seq_ctx", c_void_p), ("pages", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("max_pages", c_int),
                ("window", c_int), ("max_qlen", c_int), ("score_scale", c_float),
                # (appended: the kernels that check indices read it, the others' records end before it)
                ("n_pages", c_int)]


def _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
               num_heads, num_kv_heads, head_dim, window, max_qlen, score_scale) -> _AttnArgs:
    T = q.shape[0]
    _need(q, "q", shape=(T, num_heads * head_dim))
    _need(out, "out", q.dtype, q.shape)
    _need(k_cache, "k_cache")
    _need(v_cache, "v_cache", k_cache.dtype, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    B = seq_qlen.numel()
    for n, t in (("seq_qstart", seq_qstart), ("seq_qlen", seq_qlen), ("seq_ctx", seq_ctx)):
        _need(t, n, torch.int32, (B,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != B:
        raise KernelError(f"pages has {pages.shape[0]} rows for {B} sequences")
    if num_heads % num_kv_heads:
        raise KernelError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
    return _AttnArgs(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                     seq_qstart.data_ptr(), seq_qlen.data_ptr(), seq_ctx.data_ptr(), pages.data_ptr(),
                     B, num_heads, num_kv_heads, head_dim, pages.shape[-1], window, max_qlen, score_scale,
                     k_cache.shape[0])


def attention_generic(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                      num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                      window: int = 0, score_scale: float = 1.0) -> None:
    """Causal attention of this step's queries over the paged cache, 32-bit arithmetic."""
    if head_dim > 256:
        raise KernelError(f"head size {head_dim} exceeds 256")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, score_scale)
    fn = _lib("attention_generic.cu").gl_attention_generic
    _check(_launch(fn, byref(a), c_int(dtype_code(q.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "attention_generic")


def attention_prefill(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                      num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                      window: int = 0) -> None:
    """Causal attention of runs of new tokens over the bfloat16 cache on tensor cores
    (mma.sync, 32-bit softmax); head sizes 16..256 in steps of 16."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"prefill attention takes head sizes 16..256 in steps of 16, not {head_dim}")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("prefill attention takes bfloat16 queries and cache")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, 1.0)
    lib = _lib("attention_prefill.cu", catalog.head_dim_defines(head_dim))
    _check(_launch(lib.gl_attention_prefill, byref(a), _stream()), "attention_prefill")


def attention_prefill_tc(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                         num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                         window: int = 0) -> None:
    """Causal attention of runs of new tokens over the bfloat16 cache on the 5th-generation
    tensor cores (tcgen05.mma for both products, operands by TMA, scores and partial outputs
    in tensor memory); head sizes 16..128 in steps of 16."""
    if head_dim % 16 or not 16 <= head_dim <= 128:
        raise KernelError(f"tcgen05 prefill attention takes head sizes 16..128 in steps of 16, not {head_dim}")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("prefill attention takes bfloat16 queries and cache")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, 1.0)
    lib = _lib("attention_prefill_tc.cu", catalog.head_dim_defines(head_dim))
    _check(_launch(lib.gl_attention_prefill_tc, byref(a), c_int(q.shape[0]), c_int(k_cache.shape[0]), _stream()),
           "attention_prefill_tc")


class _DecodeArgs(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("seq_ctx", c_void_p), ("pages", c_void_p), ("part_o", c_void_p), ("part_ml", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("max_pages", c_int), ("window", c_int),
                ("splits", c_int)]


class _DecodeQkv(Structure):
    _fields_ = [("qkv", c_void_p), ("cosv", c_void_p), ("sinv", c_void_p), ("half", c_int), ("write_kv", c_int),
                ("q_scale", c_float)]


DECODE_MAX_GROUP = 8      # query heads per key/value head the decode kernel takes
_SM_COUNT = {}


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def decode_blocks_per_sm(head_dim: int, group: int = 1) -> int:
    """Blocks of the decode kernel one SM holds at once (bounded by shared memory)."""
    stages = 2
    smem = 2 * stages * PAGE * (2 * head_dim + 16) + 1024 + 4 * (64 + 5 * head_dim * max(1, group) + 16)
    return max(1, min(8, (227 * 1024) // (smem + 1024)))


def decode_splits(batch: int, num_kv_heads: int, max_len: int, device, head_dim: int,
                  group: int = 1) -> int:
    """How many blocks share one (sequence, key/value head).  Never more blocks than are resident
    at once (a grid a little larger than the machine would run a second, nearly empty wave), never
    more than the longest sequence has pages.  Within that: enough blocks to put about 1.7 on every
    SM, and enough that a block has at most 8 pages to walk through; more blocks than that only
    take the SMs' shared memory from the products that run beside a short attention.  Measured on
    Phi-2 shapes (32 heads of 80, 148 SMs; batches of 2 to 8, 512 to 2,048 positions) this is
    within 3 % of the best split everywhere and up to 11 % a step better than filling every slot."""
    pages = max(1, -(-max_len // PAGE))
    sms = sm_count(device)
    per = max(1, batch * num_kv_heads)
    slots = sms * decode_blocks_per_sm(head_dim, group)
    want = max(-(-(17 * sms // 10) // per), -(-pages // 8))
    return max(1, min(want, slots // per, pages, 8))


def decode_takes_qkv(act_dtype, cache_dtype, head_dim: int, rotary_half: int, interleaved: bool,
                     head_norm: bool) -> bool:
    """Whether decode attention can take the projection's output itself (rotating and scaling the
    queries, rotating and storing the new key and value) instead of a pass of qkv_to_cache first."""
    return (act_dtype == torch.bfloat16 and cache_dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and rotary_half % 8 == 0 and not interleaved and not head_norm)


def attention_decode(q, out, k_cache, v_cache, seq_ctx, pages, num_heads: int, num_kv_heads: int,
                     head_dim: int, splits: int, window: int = 0,
                     scratch: Optional[torch.Tensor] = None, qkv: Optional[torch.Tensor] = None,
                     cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                     q_scale: float = 1.0, write_kv: bool = True) -> None:
    """One query per sequence (row b of q is sequence b) over the bfloat16 cache.
    Up to 8 splits merge inside a thread-block cluster and need no scratch.  More splits, or
    ``scratch`` given (float32, at least B*nH*splits*(hd+2) elements), write partial results
    to scratch (allocated here when needed and not given) for a second kernel to merge.
    With ``qkv`` ([B, (heads + 2 kv heads) * head size], the projection's output; q is None then)
    the kernel rotates (cos, sin: [B, half] float32, split-half pairing) and scales the queries itself,
    and stores the new token's rotated key and its value in the cache (write_kv) before it reads them."""
    B = out.shape[0]
    if qkv is not None:
        _need(qkv, "qkv", torch.bfloat16, (B, (num_heads + 2 * num_kv_heads) * head_dim))
        half = 0
        if cos is not None:
            _need(cos, "cos", torch.float32)
            _need(sin, "sin", torch.float32, cos.shape)
            half = cos.shape[1]
            if cos.shape[0] != B or half % 8 or 2 * half > head_dim:
                raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit {B} tokens of head size {head_dim}")
    else:
        _need(q, "q", torch.bfloat16, (B, num_heads * head_dim))
    _need(out, "out", torch.bfloat16, (B, num_heads * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(seq_ctx, "seq_ctx", torch.int32, (B,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != B:
        raise KernelError(f"pages has {pages.shape[0]} rows for {B} sequences")
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"decode attention takes head sizes 16..256 in steps of 16, not {head_dim}")
    if num_heads % num_kv_heads or num_heads // num_kv_heads > DECODE_MAX_GROUP:
        raise KernelError(f"decode attention takes up to {DECODE_MAX_GROUP} query heads per key/value head")
    lib = _lib("attention_decode.cu", catalog.head_dim_defines(head_dim))
    part_o = part_ml = None
    if splits > 8 or (splits > 1 and scratch is not None):
        n_o, n_ml = B * num_heads * splits * head_dim, B * num_heads * splits * 2
        if scratch is None:
            scratch = empty(n_o + n_ml, torch.float32, out.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < n_o + n_ml:
            raise KernelError("decode attention scratch is too small")
        part_o, part_ml = scratch.data_ptr(), scratch.data_ptr() + 4 * n_o
    a = _DecodeArgs(_addr(q), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                    seq_ctx.data_ptr(), pages.data_ptr(), part_o, part_ml,
                    B, num_heads, num_kv_heads, pages.shape[-1], window, splits)
    launches = 2 if part_o is not None else 1
    if qkv is None:
        _check(_launch(lib.gl_attention_decode, byref(a), _stream()), "attention_decode", launches)
    else:
        x = _DecodeQkv(qkv.data_ptr(), _addr(cos), _addr(sin), cos.shape[1] if cos is not None else 0,
                       int(bool(write_kv)), float(q_scale))
        _check(_launch(lib.gl_attention_decode_qkv, byref(a), byref(x), _stream()), "attention_decode", launches)


def attention(q, out, k_cache, v_cache, ctx, pages, num_heads: int, num_kv_heads: int,
              head_dim: int, window: int = 0) -> None:
    """Attention of a step's queries over the cache with the fastest kernel for the step's
    shape and element type.  ``ctx`` is the step's context (per-sequence starts, lengths,
    cached lengths on the device; the longest query run and sequence on the host)."""
    if (ctx.is_decode and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and head_dim % 16 == 0 and num_heads // num_kv_heads <= DECODE_MAX_GROUP):
        splits = decode_splits(ctx.n_seqs, num_kv_heads, ctx.max_len, q.device, head_dim,
                               num_heads // num_kv_heads)
        attention_decode(q, out, k_cache, v_cache, ctx.seq_ctx, pages, num_heads, num_kv_heads,
                         head_dim, splits, window)
        return
    if q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0:
        if USE_TCGEN05 and head_dim <= TC_ATTENTION_MAX_HEAD_DIM:
            attention_prefill_tc(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                                 num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)
            return
        attention_prefill(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                          num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)
        return
    attention_generic(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                      num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)


class _DecodeLayerArgs(Structure):
    _fields_ = [("x", c_void_p), ("norm_g", c_void_p), ("norm_b", c_void_p),
                ("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_up", c_void_p), ("b_up", c_void_p),
                ("w_out", c_void_p), ("b_out", c_void_p), ("w_down", c_void_p), ("b_down", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p), ("pages", c_void_p), ("seq_ctx", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p),
                ("xn", c_void_p), ("qkv", c_void_p), ("o", c_void_p), ("h", c_void_p),
                ("scratch", c_void_p), ("sync", c_void_p),
                ("M", c_int), ("D", c_int), ("I", c_int), ("nH", c_int), ("nKV", c_int), ("half", c_int),
                ("max_pages", c_int), ("n_pages", c_int), ("window", c_int), ("act", c_int), ("rms", c_int),
                ("write_kv", c_int), ("eps", c_float), ("q_scale", c_float)]


DECODE_LAYER_MAX_ROWS = 64
# Fewer tokens than this go through the separate kernels, which are faster there.  Measured on Phi-2's
# sizes, ms a step of 32 layers, separate kernels against the fused layer: 1 token 1.40 / 1.82, 8 tokens
# 1.92 / 2.21, 16 tokens 2.46 / 2.72, 17 tokens 2.83 / 2.79, 32 tokens 3.81 / 3.61 (1,024 positions each);
# 64 tokens of 128 positions 3.54 / 2.69, of 300 4.48 / 3.50, of 2,048 9.60 / 8.46.
DECODE_LAYER_MIN_ROWS = 17
# ... where the first products' 128-row tiles nearly fill the SMs one to a block (Phi-2: 140 tiles on 148
# SMs).  Where they do not (Phi-1.5: 112 tiles), part of the machine idles through that phase and the separate
# kernels stay ahead up to 32 tokens (Phi-1.5's sizes, 1,024 positions, separate / fused: 17 tokens 1.68 / 1.80,
# 24 tokens 1.94 / 2.08, 32 tokens 2.27 / 2.28, 33 tokens 2.68 / 2.39, 48 tokens 3.07 / 2.87, 64 tokens of
# 2,048 positions 5.57 / 5.15).
DECODE_LAYER_MIN_ROWS_CUT_TILES = 33
# ... and steps whose longest sequence is shorter than this (none: the fused layer is ahead at every
# context length from 17 tokens on).
DECODE_LAYER_MIN_CONTEXT = 0
DECODE_LAYER_MAX_HEAD_DIM = catalog.MAX_HEAD_DIM["decode_layer.cu"]
USE_DECODE_LAYER = True
_DECODE_LAYER_KEEP = None          # a dict here receives the work buffers of the last call (for tests)
_DECODE_LAYER_SYNC: dict = {}      # device index -> the int32 words the fused layer's blocks meet through


def decode_layer_takes(x, w_qkv, w_up, w_out, w_down, cache_dtype, head_dim: int, group: int, rotary_half: int,
                       interleaved: bool, head_norm: bool, longest: int = 1 << 30) -> bool:
    """Whether the fused decode layer takes these types and sizes (the caller falls back to the separate
    kernels otherwise): bfloat16 weights and cache, DECODE_LAYER_MIN_ROWS (or, where the first products' tiles do
    not fill the SMs one to a block, DECODE_LAYER_MIN_ROWS_CUT_TILES) to 64 tokens, a longest sequence
    (``longest``, positions after the step) of at least DECODE_LAYER_MIN_CONTEXT, head sizes up to 128 in steps of 16,
    up to 8 query heads per key/value head, split-half rotation over a multiple of 16 dims, no per-head
    norm, widths that are multiples of 8."""
    tiles = -(-w_qkv.shape[0] // 128) + -(-w_up.shape[0] // 128)
    blocks = sm_count(x.device)
    whole_tiles = tiles * 10 >= blocks * -(-tiles // blocks) * 9
    fewest = DECODE_LAYER_MIN_ROWS if whole_tiles else max(DECODE_LAYER_MIN_ROWS, DECODE_LAYER_MIN_ROWS_CUT_TILES)
    return (USE_DECODE_LAYER and fewest <= x.shape[0] <= DECODE_LAYER_MAX_ROWS
            and longest >= DECODE_LAYER_MIN_CONTEXT and cache_dtype == torch.bfloat16
            and all(w.dtype == torch.bfloat16 for w in (w_qkv, w_up, w_out, w_down))
            and head_dim % 16 == 0 and head_dim <= DECODE_LAYER_MAX_HEAD_DIM and group <= DECODE_MAX_GROUP
            # (head sizes 32 and 96: rows of 64 and 192 bytes put four rows of an ldmatrix on the same banks and
            # are not swizzled by the kernel; the separate kernels take those)
            and (head_dim % 32 != 0 or head_dim % 64 == 0)
            and rotary_half % 8 == 0 and not interleaved and not head_norm
            and x.shape[1] % 8 == 0 and w_up.shape[0] % 8 == 0 and w_out.shape[1] % 8 == 0)


def decode_layer(x: torch.Tensor, norm_g: torch.Tensor, norm_b: Optional[torch.Tensor], eps: float, rms: bool,
                 w_qkv: torch.Tensor, b_qkv, w_up: torch.Tensor, b_up, act, w_out: torch.Tensor, b_out,
                 w_down: torch.Tensor, b_down, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 seq_ctx: torch.Tensor, pages: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                 q_scale: float, cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                 window: int = 0, write_kv: bool = True) -> torch.Tensor:
    """One decode step of a parallel block in one kernel, x updated in place:
    n = norm(x); x += attention(n) · w_outᵀ + b_out + act(n · w_upᵀ + b_up) · w_downᵀ + b_down, with one
    token per sequence (row b of x is sequence b's new token at position seq_ctx[b]); the new token's
    rotated key and its value go into the cache (write_kv).  All calls on a device share a few words of
    synchronisation state: they must follow one another on a stream, never overlap."""
    M, D = x.shape
    _need(x, "x", torch.float32)
    _need(norm_g, "norm weight", torch.float32, (D,))
    if norm_b is not None:
        _need(norm_b, "norm bias", torch.float32, (D,))
    Nqkv, No, I = (num_heads + 2 * num_kv_heads) * head_dim, num_heads * head_dim, w_up.shape[0]
    _need(w_qkv, "w_qkv", torch.bfloat16, (Nqkv, D))
    _need(w_up, "w_up", torch.bfloat16, (I, D))
    _need(w_out, "w_out", torch.bfloat16, (D, No))
    _need(w_down, "w_down", torch.bfloat16, (D, I))
    for n, b, k in (("b_qkv", b_qkv, Nqkv), ("b_up", b_up, I), ("b_out", b_out, D), ("b_down", b_down, D)):
        if b is not None:
            _need(b, n, torch.float32, (k,))
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(seq_ctx, "seq_ctx", torch.int32, (M,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != M:
        raise KernelError(f"pages has {pages.shape[0]} rows for {M} sequences")
    half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32, cos.shape)
        half = cos.shape[1]
        if cos.shape[0] != M:
            raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit {M} tokens")
    if act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} unknown")
    if M > DECODE_LAYER_MAX_ROWS or head_dim % 16 or head_dim > DECODE_LAYER_MAX_HEAD_DIM:
        raise KernelError(f"the fused decode layer takes up to {DECODE_LAYER_MAX_ROWS} tokens and head sizes up to "
                          f"{DECODE_LAYER_MAX_HEAD_DIM} in steps of 16")
    dev = x.device
    lib = _lib("decode_layer.cu", catalog.head_dim_defines(head_dim))
    bf = torch.bfloat16
    xn = empty((M, D), bf, dev)
    qkv = empty((M, Nqkv), bf, dev)
    o = empty((M, No), bf, dev)
    h = empty((M, I), bf, dev)
    a = _DecodeLayerArgs(x.data_ptr(), norm_g.data_ptr(), _addr(norm_b), w_qkv.data_ptr(), _addr(b_qkv),
                         w_up.data_ptr(), _addr(b_up), w_out.data_ptr(), _addr(b_out), w_down.data_ptr(), _addr(b_down),
                         k_cache.data_ptr(), v_cache.data_ptr(), pages.data_ptr(), seq_ctx.data_ptr(),
                         _addr(cos), _addr(sin), xn.data_ptr(), qkv.data_ptr(), o.data_ptr(), h.data_ptr(), None, None,
                         M, D, I, num_heads, num_kv_heads, half, pages.shape[-1], k_cache.shape[0], window,
                         ACTIVATIONS[act], 1 if rms else 0, 1 if write_kv else 0, eps, q_scale)
    n_scratch, n_sync = ctypes.c_longlong(0), ctypes.c_longlong(0)
    _check(lib.gl_decode_layer_sizes(byref(a), byref(n_scratch), byref(n_sync)), "decode_layer", 0)
    idx = dev.index or 0
    sync = _DECODE_LAYER_SYNC.get(idx)
    if sync is None or sync.numel() < n_sync.value:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the fused decode layer's synchronisation words must exist before a capture: "
                              "run the step once outside it")
        # zero once; every call leaves the counters zero again (the generation word only ever grows)
        sync = _DECODE_LAYER_SYNC[idx] = torch.zeros(max(int(n_sync.value), 1 << 16), dtype=torch.int32, device=dev)
    scratch = empty(max(1, int(n_scratch.value)), torch.float32, dev)
    a.scratch, a.sync = scratch.data_ptr(), sync.data_ptr()
    _check(_launch(lib.gl_decode_layer, byref(a), _stream()), "decode_layer")
    if _DECODE_LAYER_KEEP is not None:
        _DECODE_LAYER_KEEP.update(xn=xn, qkv=qkv, o=o, h=h)
    return x


def reset_decode_layer_sync() -> None:
    """Zero the fused decode layer's synchronisation words (after a kernel gave up a wait mid-way they
    may be left counting)."""
    for t in _DECODE_LAYER_SYNC.values():
        t.zero_()


class _GemmArgs(Structure):
    _fields_ = [("a", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("add0", c_void_p),
                ("add1", c_void_p), ("out", c_void_p),
                ("M", c_int), ("N", c_int), ("K", c_int), ("act", c_int),
                # a second product summed into the same output (the tcgen05 kernel reads these; the
                # other kernels' argument structs end before them)
                ("a2", c_void_p), ("w2", c_void_p), ("bias2", c_void_p), ("K2", c_int),
                # a second set of columns from the same rows (tcgen05 kernel only)
                ("wB", c_void_p), ("biasB", c_void_p), ("outB", c_void_p), ("NB", c_int), ("actB", c_int),
                # grouped weights (tcgen05 kernel only): the matrix each tile of 128 rows multiplies
                ("group_of_tile", c_void_p), ("groups", c_int),
                # the numbers of an activation that has some (every product kernel reads these two)
                ("act_p0", c_float), ("act_p1", c_float)]


def _act_code(act):
    """(code, p0, p1) of an activation given by name, or as ("xielu", up, down)."""
    if isinstance(act, tuple):
        if len(act) != 3 or act[0] != "xielu":
            raise KernelError(f"activation {act!r} unknown")
        return 6, float(act[1]), float(act[2])
    if act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} unknown")
    return ACTIVATIONS[act], 0.0, 0.0


def _gemm_args(a, w, bias, act, add0, add1, out) -> _GemmArgs:
    _need(a, "a")
    _need(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"a is [{M}, {K}] but w is {tuple(w.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    for n, t in (("add0", add0), ("add1", add1)):
        if t is not None:
            _need(t, n, torch.float32, (M, N))
    _need(out, "out", shape=(M, N))
    code, p0, p1 = _act_code(act)
    return _GemmArgs(a.data_ptr(), w.data_ptr(), _addr(bias), _addr(add0), _addr(add1), out.data_ptr(),
                     M, N, K, code, None, None, None, 0, None, None, None, 0, 0, None, 0, p0, p1)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
              add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(a · wᵀ + bias) + add0 + add1 on CUDA cores in 32-bit (any element type, any size)."""
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    fn = _lib("gemm_simt.cu").gl_gemm_simt
    _check(_launch(fn, byref(g), c_int(dtype_code(a.dtype)), c_int(dtype_code(w.dtype)),
              c_int(dtype_code(out.dtype)), _stream()), "gemm_simt")
    return out


SKINNY_MAX_ROWS = 64
USE_TCGEN05 = True
TC_ATTENTION_MAX_HEAD_DIM = catalog.MAX_HEAD_DIM["attention_prefill_tc.cu"]


def gemm_tcgen05_cut_tiles(mode: int) -> None:
    """How the tcgen05 product shares work when it adds onto its output: 0 whole tiles (default),
    1 equal shares of (tile, k-block) units whenever possible, -1 shares only when whole tiles would
    fill the SMs unevenly."""
    _lib("gemm_tcgen05.cu").gl_gemm_tcgen05_set_split(c_int(mode))


def _second_product(g: _GemmArgs, a, w, second) -> None:
    """Fill in the operands of a second product summed into the same output."""
    a2, w2, bias2 = second
    _need(a2, "a2", torch.bfloat16)
    _need(w2, "w2", torch.bfloat16)
    if a2.shape[0] != a.shape[0] or w2.shape[0] != w.shape[0] or a2.shape[1] != w2.shape[1] or a2.shape[1] % 8:
        raise KernelError(f"second product [{tuple(a2.shape)}] x [{tuple(w2.shape)}] does not fit the first")
    if bias2 is not None:
        _need(bias2, "bias2", torch.float32, (w.shape[0],))
    g.a2, g.w2, g.bias2, g.K2 = a2.data_ptr(), w2.data_ptr(), _addr(bias2), a2.shape[1]


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                split_k: int = 0, second=None) -> torch.Tensor:
    """The weight-streaming product for up to 64 rows of bfloat16 activations (K a multiple of 8).
    ``second`` = (a2, w2, bias2) sums another product into the same output (K a multiple of 64 then)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[0] > SKINNY_MAX_ROWS or a.shape[1] % 8:
        raise KernelError(f"gemm_skinny takes up to {SKINNY_MAX_ROWS} rows and K a multiple of 8")
    if second is not None:
        if a.shape[1] % 64:
            raise KernelError("gemm_skinny takes a second product only behind a K that is a multiple of 64")
        _second_product(g, a, w, second)
    fn = _lib("gemm_skinny.cu").gl_gemm_skinny
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(split_k), _stream()), "gemm_skinny")
    return out


STREAM_MIN_ROWS, STREAM_MAX_ROWS = 17, 64
# Off: as measured with Phi-2's sizes the mma.sync product is as fast or faster at 17 to 64 rows (64 rows:
# 19.5 / 29.8 / 39.9 µs for the qkv, the up and the joined out+down product against 19.8 / 25.7 / 25.7),
# both far from the weights' streaming time; what a block pays once (tensor-memory allocation, two cluster
# barriers, the reduction through the peers' shared memory) stands against ten to twenty stages of work.
USE_GEMM_STREAM = False


def gemm_stream(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                split_k: int = 0, second=None) -> torch.Tensor:
    """The weight-streaming product for up to 64 rows on the 5th-generation tensor cores: the weights
    are the 128-row operand of tcgen05.mma, the tokens its N (K a multiple of 8).  Meant for 17 to 64
    rows, where the tokens' tile is too large to be fetched again for every 64 weight rows.
    ``second`` = (a2, w2, bias2) sums another product into the same output (K a multiple of 64 then)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[0] > STREAM_MAX_ROWS or a.shape[1] % 8:
        raise KernelError(f"gemm_stream takes up to {STREAM_MAX_ROWS} rows and K a multiple of 8")
    if second is not None:
        if a.shape[1] % 64:
            raise KernelError("gemm_stream takes a second product only behind a K that is a multiple of 64")
        _second_product(g, a, w, second)
    fn = _lib("gemm_stream.cu").gl_gemm_stream
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(split_k), _stream()), "gemm_stream")
    return out


def _few_rows(a, w, bias, act, add0, add1, out_dtype, out, second=None):
    """The weight-streaming product for up to 64 rows: mma.sync for up to 16, tcgen05 above."""
    if USE_GEMM_STREAM and a.shape[0] >= STREAM_MIN_ROWS:
        return gemm_stream(a, w, bias, act, add0, add1, out_dtype, out, second=second)
    return gemm_skinny(a, w, bias, act, add0, add1, out_dtype, out, second=second)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                 add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                 tile_n: int = 0, _defines=(), second=None, fork=None):
    """The tensor-core product (tcgen05.mma fed by TMA, accumulators in tensor memory) for
    bfloat16 operands with K a multiple of 8; meant for many rows.  ``second`` = (a2, w2, bias2)
    sums another product over the same rows and columns into the tile before the epilogue:
    out = act(a·wᵀ + a2·w2ᵀ + bias + bias2) + add0 + add1.  ``fork`` = (wB, biasB, actB) computes a
    second output actB(a·wBᵀ + biasB) in the same launch (nothing added, no ``second``; both
    outputs' rows whole 16-byte units) and makes the result the pair (out, outB)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[1] % 8:
        raise KernelError("gemm_tcgen05 takes K a multiple of 8 (TMA needs 16-byte row pitch)")
    if second is not None:
        _second_product(g, a, w, second)
    out_b = None
    if fork is not None:
        w_b, bias_b, act_b = fork
        _need(w_b, "wB", torch.bfloat16)
        if w_b.shape[1] != a.shape[1] or isinstance(act_b, tuple) or act_b not in ACTIVATIONS:
            raise KernelError(f"second set of columns {tuple(w_b.shape)} does not fit a {tuple(a.shape)}")
        if bias_b is not None:
            _need(bias_b, "biasB", torch.float32, (w_b.shape[0],))
        out_b = empty((a.shape[0], w_b.shape[0]), out.dtype, a.device)
        g.wB, g.biasB, g.outB, g.NB, g.actB = w_b.data_ptr(), _addr(bias_b), out_b.data_ptr(), w_b.shape[0], ACTIVATIONS[act_b]
    if tile_n not in (0, 64, 128, 160, 192, 256, 1160, 1192, 1256):
        raise KernelError("tile_n is 0 (choose), 64, 128, 160 (32-bit output only), 192 or 256; "
                          "1000 more for tiles of 256 rows (160, 192, 256)")
    fn = _lib("gemm_tcgen05.cu", _defines).gl_gemm_tcgen05
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(tile_n), _stream()), "gemm_tcgen05")
    return out if fork is None else (out, out_b)


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, group_of_tile: torch.Tensor, out_dtype: torch.dtype,
                         tile_n: int = 0) -> torch.Tensor:
    """out[r] = a[r] . w[g]^T with g = group_of_tile[r // 128]: ``w`` [groups, N, K] holds one matrix per group,
    every tile of 128 rows of ``a`` [M, K] (M a multiple of 128) multiplies the matrix its entry names, and a
    tile with a negative entry is skipped (its rows of the result stay as they are).  The table lives on the
    device: the host need not know it.  bfloat16 operands, K a multiple of 8, N rows of whole 16-byte units."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    _need(group_of_tile, "group_of_tile", torch.int32)
    M, K = a.shape
    E, N, Kw = w.shape
    if Kw != K or K % 8 or M % 128 or group_of_tile.numel() < M // 128 or (N * out_dtype.itemsize) % 16:
        raise KernelError(f"gemm_tcgen05_grouped: a {tuple(a.shape)}, w {tuple(w.shape)} and {group_of_tile.numel()} tiles do not fit")
    out = empty((M, N), out_dtype, a.device)
    g = _GemmArgs(a.data_ptr(), w.data_ptr(), None, None, None, out.data_ptr(), M, N, K, 0,
                  None, None, None, 0, None, None, None, 0, 0, group_of_tile.data_ptr(), E, 0.0, 0.0)
    fn = _lib("gemm_tcgen05.cu").gl_gemm_tcgen05
    _check(_launch(fn, byref(g), c_int(dtype_code(out_dtype)), c_int(tile_n), _stream()), "gemm_tcgen05_grouped")
    return out


# ---------------------------------------------------------------------------
# Mixers with per-sequence state (csrc/recurrent.cu), attention with mixed heads (csrc/attention_mixed.cu)
class _MemoryScanArgs(Structure):
    _fields_ = [("proj", c_void_p), ("out", c_void_p), ("state", c_void_p), ("lower", c_void_p),
                ("seq_slot", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p),
                ("ld", c_int), ("q_off", c_int), ("k_off", c_int), ("v_off", c_int), ("i_off", c_int), ("f_off", c_int),
                ("B", c_int), ("H", c_int), ("D", c_int), ("V", c_int), ("state_stride", c_int), ("kind", c_int),
                ("cap", c_float), ("q_scale", c_float), ("nm_next", c_void_p),
                ("gates", c_void_p), ("a_log", c_void_p), ("dt_bias", c_void_p), ("gates_ld", c_int), ("KVH", c_int),
                ("rows_per_thread", c_int),
                ("cosv", c_void_p), ("sinv", c_void_p), ("rot_half", c_int), ("k_scale", c_float), ("d_skip", c_void_p)]


MEMORY_GATED, MEMORY_BOUNDED_FORGET, MEMORY_DELTA, MEMORY_DECAY = 0, 1, 2, 3
MEMORY_SCAN_ROWS_PER_THREAD = 0     # 0: the kernel chooses by the grid's size; 32, 8, 4, 2 or 1 forces it (measurements)


def memory_state_size(kind: int, H: int, D: int, V: int) -> int:
    """Floats of a sequence's state row: S [H, D, V]; the gated kind adds a normaliser [H, D] and a running
    maximum [H]."""
    if not 0 < D <= 512 or V <= 0 or H <= 0:
        raise KernelError(f"memory_scan takes 1..512 rows a head, got {D}")
    return H * D * V + (H * (D + 1) if kind == MEMORY_GATED else 0)


class _MemoryChunkArgs(Structure):
    _fields_ = [("proj", c_void_p), ("out", c_void_p), ("nq", c_void_p), ("gates", c_void_p), ("state", c_void_p),
                ("lower", c_void_p), ("chunk_state", c_void_p), ("chunk_decay", c_void_p),
                ("tok_seq", c_void_p), ("seq_slot", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p),
                ("T", c_int), ("ld", c_int), ("q_off", c_int), ("k_off", c_int), ("v_off", c_int), ("i_off", c_int),
                ("f_off", c_int), ("B", c_int), ("H", c_int), ("D", c_int), ("V", c_int), ("cols", c_int),
                ("state_stride", c_int), ("kind", c_int), ("chunk_len", c_int), ("n_chunks", c_int),
                ("cap", c_float), ("q_scale", c_float),
                ("gates_in", c_void_p), ("a_log", c_void_p), ("dt_bias", c_void_p), ("cosv", c_void_p),
                ("sinv", c_void_p), ("d_skip", c_void_p), ("gates_ld", c_int), ("KVH", c_int), ("rot_half", c_int),
                ("k_scale", c_float)]


MEMORY_CHUNKS_MAX_ROWS = 128     # rows a head the chunked walk of the matrix memories takes (a column's rows in registers)
USE_MEMORY_CHUNKS = True
# The plain decay's chunked walk pays from shorter runs on and with shorter chunks than the other kinds' (its gates
# cost one pass, its rows are updated in pairs): a prompt of 256 / 512 / 1,024 / 2,048 tokens of ten such layers
# at width 2,048 took 4.7 / 6.7 / 11.0 / 19.5 ms token by token, 3.7 / 4.5 / 6.0 / 9.9 ms in chunks of 32,
# 4.0 / 4.5 / 6.0 / 8.9 ms in chunks of 64 and 4.6 / 5.0 / 6.1 / 9.0 ms in chunks of 128.
MEMORY_CHUNKS_MAX_BYTES = 1 << 30     # of chunk states a launch of the plain decay may hold
DECAY_CHUNKED_FROM = 256
DECAY_LONG_RUN = 512
DECAY_CHUNK_TOKENS = 64          # runs of at least DECAY_LONG_RUN tokens
DECAY_CHUNK_TOKENS_SHORT = 32


def memory_scan(kind: int, proj: torch.Tensor, state: torch.Tensor, ctx, H: int, D: int, V: int,
                q_off: int, k_off: int, v_off: int, i_off: int, f_off: int,
                lower: Optional[torch.Tensor] = None, cap: float = 0.0, q_scale: float = 1.0,
                gates: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None,
                dt_bias: Optional[torch.Tensor] = None, kv_heads: int = 0,
                decay: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                sin: Optional[torch.Tensor] = None, k_scale: float = 1.0,
                skip: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A matrix memory's run over the step's tokens: float32 [T, H*V], each head's S^T q (divided by the
    gated kind's normaliser); ``state`` [slots, size] float32 is read at ctx.seq_slot and written back.
    ``proj`` [T, ld] holds the projections at the given column offsets.  MEMORY_DELTA (the gated delta rule):
    q and k have ``kv_heads`` heads, each read by H / kv_heads heads; ``gates`` [T, ld'] holds the projection
    behind beta at column i_off + h and the one behind the decay at f_off + h; ``a_log`` and ``dt_bias`` [H].
    MEMORY_DECAY: S <- keep S + take k v^T, o = S^T q + skip[h] v, with q and k of ``kv_heads`` heads (0: one per
    head), rotated first where ``cos`` and ``sin`` [T, half] are given (dim i of a head with dim i + half), then
    times q_scale and k_scale.  Either ``decay`` [H] (keep = decay[h], take = 1) or ``gates`` with ``a_log`` and
    ``dt_bias`` [H]: dt = softplus(gates[t, f_off + h] + dt_bias[h]), keep = exp(-exp(a_log[h]) dt), take = dt.
    Long runs of the gated, the bounded-forget and the plain-decay kind (heads of up to MEMORY_CHUNKS_MAX_ROWS rows)
    are walked as chunks side by side; which form runs depends on the step's longest run alone."""
    _need(proj, "proj")
    rot_half = 0
    if kind == MEMORY_DECAY:
        kv_heads = kv_heads or H
        if kv_heads <= 0 or H % kv_heads:
            raise KernelError(f"memory_scan: {H} heads do not share {kv_heads} heads of q and k")
        if (decay is None) == (gates is None):
            raise KernelError("memory_scan: a plain decay is either fixed per head or follows a step size")
        if decay is not None:
            _need(decay, "decay", torch.float32, (H,))
        else:
            _need(gates, "gates", proj.dtype)
            _need(a_log, "a_log", torch.float32, (H,))
            _need(dt_bias, "dt_bias", torch.float32, (H,))
            if gates.shape[0] != proj.shape[0] or f_off + H > gates.shape[1]:
                raise KernelError("memory_scan: the step sizes' columns do not fit")
        if cos is not None:
            rot_half = cos.shape[-1]
            _need(cos, "cos", torch.float32, (proj.shape[0], rot_half))
            _need(sin, "sin", torch.float32, (proj.shape[0], rot_half))
            if 2 * rot_half > D:
                raise KernelError("memory_scan: more rotated dims than a head has")
        if skip is not None:
            _need(skip, "skip", torch.float32, (H,))
        lower = decay
    if kind == MEMORY_DELTA:
        _need(gates, "gates", proj.dtype)
        _need(a_log, "a_log", torch.float32, (H,))
        _need(dt_bias, "dt_bias", torch.float32, (H,))
        if kv_heads <= 0 or H % kv_heads or gates.shape[0] != proj.shape[0]:
            raise KernelError(f"memory_scan: {H} heads do not share {kv_heads} heads of q and k")
    _need(state, "state", torch.float32)
    T, ld = proj.shape
    if state.shape[1] < memory_state_size(kind, H, D, V):
        raise KernelError("memory_scan: the state row is too small for these sizes")
    if kind == MEMORY_BOUNDED_FORGET:
        _need(lower, "lower", torch.float32, (H * D,))
    out = empty((T, H * V), torch.float32, proj.device)
    gated, plain = kind == MEMORY_GATED, kind == MEMORY_DECAY
    chunk_tokens = SCAN_CHUNK_TOKENS
    if plain:
        chunk_tokens = DECAY_CHUNK_TOKENS if ctx.max_qlen >= DECAY_LONG_RUN else DECAY_CHUNK_TOKENS_SHORT
        # every (sequence, chunk) keeps a whole state: many long sequences take longer chunks
        while (ctx.n_seqs * -(-ctx.max_qlen // chunk_tokens) * H * D * V * 4 > MEMORY_CHUNKS_MAX_BYTES
               and chunk_tokens < 1024):
            chunk_tokens *= 2
    chunks = -(-ctx.max_qlen // chunk_tokens)
    if (USE_MEMORY_CHUNKS and kind in (MEMORY_GATED, MEMORY_BOUNDED_FORGET, MEMORY_DECAY) and D <= MEMORY_CHUNKS_MAX_ROWS
            and ctx.max_qlen >= (DECAY_CHUNKED_FROM if plain else SCAN_CHUNKED_FROM)
            and (not plain or ctx.n_seqs * chunks <= 65535)):          # (the grid's third size)
        # a long run: chunks of tokens side by side, a lane a column (two walks and a carry between them)
        cols = V + (1 if gated else 0)
        chunk_state = empty((ctx.n_seqs, chunks, H, D, cols), torch.float32, proj.device)
        chunk_decay = empty((ctx.n_seqs, chunks, H, D), torch.float32, proj.device)
        nq = empty((T, H), torch.float32, proj.device) if gated else None
        scratch = empty((T, H, 4), torch.float32, proj.device) if gated or plain else None
        c = _MemoryChunkArgs(proj.data_ptr(), out.data_ptr(), _addr(nq), _addr(scratch), state.data_ptr(), _addr(lower),
                             chunk_state.data_ptr(), chunk_decay.data_ptr(), ctx.tok_seq.data_ptr(),
                             ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(),
                             T, ld, q_off, k_off, v_off, i_off, f_off, ctx.n_seqs, H, D, V, cols, state.shape[1], kind,
                             chunk_tokens, chunks, cap, q_scale,
                             _addr(gates) if plain else None, _addr(a_log) if plain else None,
                             _addr(dt_bias) if plain else None, _addr(cos) if rot_half else None,
                             _addr(sin) if rot_half else None, _addr(skip) if plain else None,
                             gates.shape[1] if plain and gates is not None else 0, kv_heads if plain else 0, rot_half,
                             k_scale)
        fn = _lib("recurrent.cu").gl_memory_chunks
        _check(_launch(fn, byref(c), c_int(dtype_code(proj.dtype)), _stream()), "memory_chunks",
               7 if gated else 5 if plain else 4)
        return out
    # the gated kind's new normaliser and maximum, moved into the state rows by a second kernel
    nm = empty((ctx.n_seqs, H, D + 1), torch.float32, proj.device) if kind == MEMORY_GATED else None
    a = _MemoryScanArgs(proj.data_ptr(), out.data_ptr(), state.data_ptr(), _addr(lower),
                        ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(),
                        ld, q_off, k_off, v_off, i_off, f_off, ctx.n_seqs, H, D, V, state.shape[1], kind, cap, q_scale,
                        _addr(nm), _addr(gates), _addr(a_log), _addr(dt_bias),
                        gates.shape[1] if gates is not None else 0, kv_heads, MEMORY_SCAN_ROWS_PER_THREAD,
                        _addr(cos) if rot_half else None, _addr(sin) if rot_half else None, rot_half, k_scale, _addr(skip))
    fn = _lib("recurrent.cu").gl_memory_scan
    _check(_launch(fn, byref(a), c_int(dtype_code(proj.dtype)), _stream()), "memory_scan", 2 if kind == MEMORY_GATED else 1)
    return out


def head_norm_gate(o: torch.Tensor, w: Optional[torch.Tensor], H: int, V: int, eps: float, out_dtype: torch.dtype,
                   gate: Optional[torch.Tensor] = None, gate_off: int = 0, gate_act: str = "sigmoid",
                   gate_first: bool = False) -> torch.Tensor:
    """Each head of float32 ``o`` [T, H*V] divided by its root mean square, times ``w`` ([H*V], or [V]
    shared by the heads; None: no weight), times sigmoid (``gate_act`` "silu": silu) of the gate's columns
    gate_off.. of ``gate`` [T, ld] if given.  ``gate_first``: the gate multiplies o before the norm, and the
    root mean square is the gated values'."""
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"head_norm_gate: gate activation {gate_act!r} unknown")
    _need(o, "o", torch.float32)
    T = o.shape[0]
    _need(o, "o", shape=(T, H * V))
    if w is not None:
        _need(w, "w", torch.float32)
        if w.numel() not in (V, H * V):
            raise KernelError(f"head_norm_gate: weight of {w.numel()} elements fits neither {V} nor {H * V}")
    if gate is not None:
        _need(gate, "gate", out_dtype)
        if gate_off + H * V > gate.shape[1]:
            raise KernelError("head_norm_gate: the gate's columns do not fit its rows")
    out = empty((T, H * V), out_dtype, o.device)
    fn = _lib("recurrent.cu").gl_head_norm_gate
    _check(_launch(fn, _ptr(o), _ptr(w), _ptr(gate), _ptr(out), c_int(T), c_int(H), c_int(V),
                   c_int(0 if w is None or w.numel() == V else 1),
                   c_int(0 if gate is None else gate.shape[1]), c_int(gate_off), c_float(eps),
                   c_int(dtype_code(out_dtype)), c_int(1 if gate_act == "silu" else 0), c_int(1 if gate_first else 0),
                   _stream()), "head_norm_gate")
    return out


class _ConvArgs(Structure):
    _fields_ = [("x", c_void_p), ("out", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("state", c_void_p),
                ("tok_seq", c_void_p), ("seq_slot", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p),
                ("T", c_int), ("B", c_int), ("C", c_int), ("taps", c_int), ("ld", c_int), ("x_off", c_int),
                ("state_stride", c_int), ("tail_off", c_int)]


def conv_silu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, tail_off: int, ctx,
              x_off: int = 0) -> torch.Tensor:
    """silu of a causal per-channel convolution over columns x_off.. of ``x`` [T, ld]; ``w`` [C, taps] with the
    current token's tap last.  The inputs before a run come from ``state`` (the last taps-1 inputs of each
    channel from column tail_off of the sequence's row on), which then takes the run's last inputs."""
    _need(x, "x")
    _need(w, "w", torch.float32)
    C, taps = w.shape
    if bias is not None:
        _need(bias, "bias", torch.float32, (C,))
    _need(state, "state", torch.float32)
    T, ld = x.shape
    if x_off + C > ld or tail_off + C * (taps - 1) > state.shape[1]:
        raise KernelError("conv_silu: columns or state row too small")
    out = empty((T, C), x.dtype, x.device)
    a = _ConvArgs(x.data_ptr(), out.data_ptr(), w.data_ptr(), _addr(bias), state.data_ptr(),
                  ctx.tok_seq.data_ptr(), ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(),
                  T, ctx.n_seqs, C, taps, ld, x_off, state.shape[1], tail_off)
    fn = _lib("recurrent.cu").gl_conv_silu
    _check(_launch(fn, byref(a), c_int(dtype_code(x.dtype)), _stream()), "conv_silu",
           2 if taps > 1 and T != ctx.n_seqs else 1)
    return out


class _SelectiveScanArgs(Structure):
    _fields_ = [("x", c_void_p), ("dtp", c_void_p), ("bc", c_void_p), ("z", c_void_p), ("out", c_void_p),
                ("a_log", c_void_p), ("d_skip", c_void_p), ("state", c_void_p),
                ("seq_slot", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p),
                ("B", c_int), ("C", c_int), ("N", c_int), ("z_ld", c_int), ("z_off", c_int), ("state_stride", c_int),
                ("chunk_state", c_void_p), ("chunk_dt", c_void_p), ("chunk_len", c_int), ("n_chunks", c_int)]


SCAN_MAX_STATE = 256
# A run of at least SCAN_CHUNKED_FROM tokens is walked as chunks of SCAN_CHUNK_TOKENS side by side (two walks
# and a carry between them): a token-by-token walk leaves most of the machine idle when the sequences are few.
SCAN_CHUNK_TOKENS = 128     # (a prompt of 2,048 tokens: 11.3 / 11.4 / 13.0 / 15.5 ms with chunks of 64 / 128 / 256 / 512)
SCAN_CHUNKED_FROM = 1024       # (512 tokens in 4 chunks took 8 % longer than walked in one piece)


def selective_scan(x: torch.Tensor, dtp: torch.Tensor, bc: torch.Tensor, z: torch.Tensor, z_off: int,
                   a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, ctx) -> torch.Tensor:
    """The selective state-space scan of the step's tokens: x [T, C], dtp [T, C] float32 (step size before
    softplus), bc [T, 2N] (input then output projection of the state), z the gate in columns z_off.. of its
    tensor; state rows hold S [C, N] first.  Returns [T, C] in x's type."""
    _need(x, "x")
    T, C = x.shape
    N = a_log.shape[1]
    _need(dtp, "dtp", torch.float32, (T, C))
    _need(bc, "bc", x.dtype, (T, 2 * N))
    _need(z, "z", x.dtype)
    _need(a_log, "a_log", torch.float32, (C, N))
    _need(d_skip, "d_skip", torch.float32, (C,))
    _need(state, "state", torch.float32)
    if N > SCAN_MAX_STATE or state.shape[1] < C * N or z_off + C > z.shape[1]:
        raise KernelError("selective_scan: sizes the kernel does not take")
    out = empty((T, C), x.dtype, x.device)
    a = _SelectiveScanArgs(x.data_ptr(), dtp.data_ptr(), bc.data_ptr(), z.data_ptr(), out.data_ptr(),
                           a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(),
                           ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(),
                           ctx.n_seqs, C, N, z.shape[1], z_off, state.shape[1], None, None, 0, 0)
    kernels = 1
    if ctx.max_qlen >= SCAN_CHUNKED_FROM:
        chunks = -(-ctx.max_qlen // SCAN_CHUNK_TOKENS)
        chunk_state = empty((ctx.n_seqs, chunks, C, N), torch.float32, x.device)
        chunk_dt = empty((ctx.n_seqs, chunks, C), torch.float32, x.device)
        a.chunk_state, a.chunk_dt = chunk_state.data_ptr(), chunk_dt.data_ptr()
        a.chunk_len, a.n_chunks, kernels = SCAN_CHUNK_TOKENS, chunks, 3
    fn = _lib("recurrent.cu").gl_selective_scan
    _check(_launch(fn, byref(a), c_int(dtype_code(x.dtype)), _stream()), "selective_scan", kernels)
    return out


class _QkvRowNormArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p), ("q_gamma", c_void_p), ("k_gamma", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("pages", c_void_p),
                ("T", c_int), ("ld", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("vd", c_int),
                ("half", c_int), ("max_pages", c_int), ("interleaved", c_int), ("write_kv", c_int),
                ("eps", c_float), ("q_scale", c_float), ("n_pages", c_int),
                ("temp_coef", c_float), ("temp_every", c_float), ("q_only", c_int), ("head_unit", c_int),
                ("talk", c_void_p), ("k_joined", c_int)]


def qkv_rownorm_to_cache(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, ctx, pages: torch.Tensor,
                         num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, q_scale: float,
                         cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], interleaved: bool,
                         q_gamma: Optional[torch.Tensor], k_gamma: Optional[torch.Tensor], eps: float,
                         write_kv: bool = True, q_temp: Optional[tuple] = None, q_only: bool = False,
                         head_unit: bool = False, talk: Optional[torch.Tensor] = None,
                         k_joined: bool = False) -> torch.Tensor:
    """Queries and keys normalised over the whole projection (root mean square, weights [nH*hd] and
    [nKV*hd]; None: no norm), rotated and scaled; keys and values written to the tokens' cache rows.
    ``head_unit``: after the rotation every head of q and k is divided by its own root mean square (eps
    inside the root, no weight).
    qkv [T, ld]: q, k, v side by side from column 0 (``q_only``: queries alone, nothing is written).
    ``q_temp`` = (coef, every): q also times 1 + coef * ln(floor((position + 1) / every) + 1).
    ``talk`` [nH, nH] float32: a table that mixes the heads' scores before the softmax, s'_h = sum_g talk[h, g] s_g,
    taken on the queries: the result is [T, nH, nKV*hd], head h holding for every key head c the sum of
    talk[h, g] q_g over c's query heads g, so that s'_h is one product with the position's key heads side by side.
    ``k_joined``: the key cache holds them so, [pages, 1, PAGE, nKV*hd].
    Returns q [T, nH*hd] (with ``talk``: [T, nH*nKV*hd])."""
    _need(qkv, "qkv")
    T, ld = qkv.shape
    nq, nk, nv = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
    if q_only:
        nk = nv = 0
        if write_kv:
            raise KernelError("qkv_rownorm_to_cache: rows of queries alone have nothing to write to the cache")
    if q_temp is not None and not q_temp[1] > 0:
        raise KernelError("qkv_rownorm_to_cache: the query temperature's period must be positive")
    if ld < nq + nk + nv:
        raise KernelError("qkv_rownorm_to_cache: the projection's rows are too short")
    k_shape = (1, PAGE, num_kv_heads * head_dim) if k_joined else (num_kv_heads, PAGE, head_dim)
    if talk is not None:
        _need(talk, "talk", torch.float32, (num_heads, num_heads))
    if tuple(k_cache.shape[1:]) != k_shape or tuple(v_cache.shape[1:]) != (num_kv_heads, PAGE, value_dim):
        raise KernelError(f"cache pages do not fit: keys {tuple(k_cache.shape)}, values {tuple(v_cache.shape)}")
    half = 0
    if cos is not None:
        half = cos.shape[-1]
        _need(cos, "cos", torch.float32, (T, half))
        _need(sin, "sin", torch.float32, (T, half))
    if q_gamma is not None:
        _need(q_gamma, "q_gamma", torch.float32, (nq,))
    if k_gamma is not None:
        _need(k_gamma, "k_gamma", torch.float32, (nk,))
    q = empty((T, nq * num_kv_heads if talk is not None else nq), qkv.dtype, qkv.device)
    a = _QkvRowNormArgs(qkv.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _addr(cos), _addr(sin),
                        _addr(q_gamma), _addr(k_gamma), ctx.tok_seq.data_ptr(), ctx.tok_pos.data_ptr(), pages.data_ptr(),
                        T, ld, num_heads, num_kv_heads, head_dim, value_dim, half, pages.shape[-1],
                        1 if interleaved else 0, 1 if write_kv else 0, eps, q_scale, k_cache.shape[0],
                        q_temp[0] if q_temp is not None else 0.0, q_temp[1] if q_temp is not None else 0.0,
                        1 if q_only else 0, 1 if head_unit else 0, _addr(talk), 1 if k_joined else 0)
    fn = _lib("qkv_cache.cu").gl_qkv_rownorm_cache
    _check(_launch(fn, byref(a), c_int(dtype_code(qkv.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "qkv_rownorm_to_cache")
    return q


class _MixedAttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("pairs", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("mix", c_void_p), ("seq_qstart", c_void_p), ("seq_qlen", c_void_p), ("seq_ctx", c_void_p), ("pages", c_void_p),
                ("T", c_int), ("B", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("vd", c_int),
                ("max_pages", c_int), ("window", c_int), ("max_qlen", c_int), ("n_pages", c_int),
                ("parts", c_void_p), ("ml", c_void_p), ("splits", c_int), ("pages_per_split", c_int),
                ("score_scale", c_float), ("softcap", c_float), ("slopes", c_void_p), ("sinks", c_void_p), ("nVH", c_int),
                ("vs", c_int)]


# A block of the one-token kernel walks its pages one after the other and waits for each: what hides the trips to
# memory is the number of blocks an SM holds (eight fit), so the context is cut until the grid fills them, down
# to a page a block (32 sequences of 1,000 positions, 8 key heads: 253 us a launch with two blocks an SM, a step of
# ten layers 2.78 -> 2.06 ms with eight).
MIXED_DECODE_BLOCKS_PER_SM = 8


def mixed_decode_splits(batch: int, num_kv_heads: int, max_len: int, device) -> int:
    """Ranges of pages a sequence's context is cut into for a one-token step: enough blocks (key heads x
    sequences x ranges) for about MIXED_DECODE_BLOCKS_PER_SM an SM, no range shorter than a page."""
    pages = max(1, -(-int(max_len) // PAGE))
    want = max(1, (MIXED_DECODE_BLOCKS_PER_SM * sm_count(device)) // max(1, batch * num_kv_heads))
    return max(1, min(pages, want, 64))


class _PairsArgs(Structure):
    _fields_ = [("q", c_void_p), ("pairs", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("seq_qstart", c_void_p), ("seq_qlen", c_void_p), ("seq_ctx", c_void_p), ("pages", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("nVal", c_int), ("max_pages", c_int), ("window", c_int),
                ("max_qlen", c_int), ("score_scale", c_float), ("softcap", c_float), ("slopes", c_void_p),
                ("out", c_void_p), ("sinks", c_void_p), ("nVH", c_int), ("vs", c_int), ("v_in_k", c_int)]


USE_PAIRS_TC = True
USE_ROWS_DECODE_TC = True      # one token a sequence, eight or more query heads on a key head: the heads as rows of a tensor-core product


class _RowsDecodeArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("seq_qstart", c_void_p), ("seq_ctx", c_void_p),
                ("pages", c_void_p), ("parts", c_void_p), ("ml", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("nVH", c_int), ("max_pages", c_int), ("window", c_int),
                ("splits", c_int), ("pages_per_split", c_int), ("rows", c_int), ("v_in_k", c_int), ("score_scale", c_float)]


def rows_decode_smem(head_dim: int, value_dim: int, values_in_keys: bool) -> int:
    stages = 16 * (2 * head_dim + 16) + 2 * 64 * (2 * head_dim + 16) + (0 if values_in_keys else 2 * 64 * (2 * value_dim + 16))
    return max(stages, 16 * (2 * head_dim + 16) + (4 * 16 * value_dim + 128) * 4)


def rows_decode_splits(batch: int, runs: int, span_pages: int, device, smem: int) -> int:
    """Ranges of pages a sequence's context is cut into for the kernel whose rows are query heads: enough blocks
    (runs of heads x sequences x ranges) to fill the blocks an SM holds of it twice over, no range shorter than a page."""
    pages = max(1, int(span_pages))
    per_sm = max(1, min(4, (227 * 1024) // max(1, smem)))
    want = max(1, (2 * per_sm * sm_count(device)) // max(1, batch * runs))
    return max(1, min(pages, want, 64))


def attention_mixed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, ctx, pages: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                    mix: Optional[torch.Tensor] = None, window: int = 0, score_scale: float = 1.0,
                    softcap: float = 0.0, slopes: Optional[torch.Tensor] = None,
                    sinks: Optional[torch.Tensor] = None, value_heads: int = 0, values_in_keys: bool = False) -> torch.Tensor:
    """Causal softmax attention of scaled queries [T, nH*hd] over the paged cache; with ``mix`` [nH, nH]
    head h applies sum_g mix[h, g] * (head g's softmax weights) to the values of its own key/value
    head.  A score is (q . k) * score_scale, then softcap * tanh(score / softcap) when softcap > 0, then
    minus slopes[h] * (query position - key position) when ``slopes`` [nH] float32 is given.  With ``sinks``
    [nH] float32 the denominator of head h's softmax also holds exp(sinks[h]), once, with no key and no value.
    ``value_heads`` > 0: the value cache has that many heads (a multiple of the key heads), and without a table
    query head h takes the values of head h / (nH / value_heads): many query heads on one wide key head, each
    with one of several value heads.  ``values_in_keys``: a position's values are the first ``value_dim`` numbers of its
    key row (``v_cache`` is the key cache).
    Returns [T, nH*vd] in q's type.  Prompts in bfloat16 with key and value sizes that are
    multiples of 16 compute the (query head, value head) pairs on the tensor cores (a library per pair
    of sizes); everything else runs the 32-bit kernels."""
    _need(q, "q")
    T = q.shape[0]
    _need(q, "q", shape=(T, num_heads * head_dim))
    if mix is not None:
        _need(mix, "mix", torch.float32, (num_heads, num_heads))
    if slopes is not None:
        _need(slopes, "slopes", torch.float32, (num_heads,))
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (num_heads,))
    n_val = num_kv_heads if mix is not None else 1
    nvh = int(value_heads)
    if nvh and (nvh % num_kv_heads or num_heads % nvh or (mix is not None and nvh != num_kv_heads)):
        raise KernelError(f"attention_mixed: {nvh} value heads do not fit {num_heads} query heads on {num_kv_heads} key heads")
    vs = 0
    if values_in_keys:
        if mix is not None or nvh not in (0, num_kv_heads) or value_dim > head_dim:
            raise KernelError("attention_mixed: values inside the key rows come one row of values a key head, no longer than it")
        v_cache, vs = k_cache, head_dim
    if (tuple(v_cache.shape[1:]) != (nvh or num_kv_heads, PAGE, vs or value_dim)
            or tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim)):
        raise KernelError(f"attention_mixed: cache pages do not fit: keys {tuple(k_cache.shape)}, values {tuple(v_cache.shape)}")
    out = empty((T, num_heads * value_dim), q.dtype, q.device)
    pairs_tc = (USE_PAIRS_TC and ctx.max_qlen > 1 and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
                and head_dim % 16 == 0 and value_dim % 16 == 0 and head_dim <= 256 and value_dim <= 256
                and 2 * 64 * (2 * head_dim + 16) + 2 * 64 * (2 * value_dim + 16) <= 227 * 1024 and not DEBUG_BOUNDS)
    if pairs_tc and mix is None:
        # prompts without a mixing table: the tensor-core kernel rounds and writes the result itself
        p = _PairsArgs(q.data_ptr(), None, k_cache.data_ptr(), v_cache.data_ptr(),
                       ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.seq_ctx.data_ptr(), pages.data_ptr(),
                       ctx.n_seqs, num_heads, num_kv_heads, 1, pages.shape[-1], window, ctx.max_qlen,
                       score_scale, softcap, _addr(slopes), out.data_ptr(), _addr(sinks), nvh, vs, 1 if values_in_keys else 0)
        fn = _lib("attention_mixed_tc.cu", catalog.pair_dim_defines(head_dim, value_dim)).gl_attention_pairs_tc
        _check(_launch(fn, byref(p), _stream()), "attention_pairs_tc")
        return out
    pairs = empty((T, num_heads, n_val, value_dim), torch.float32, q.device)
    a = _MixedAttnArgs(q.data_ptr(), pairs.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _addr(mix),
                       ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.seq_ctx.data_ptr(), pages.data_ptr(),
                       T, ctx.n_seqs, num_heads, num_kv_heads, head_dim, value_dim, pages.shape[-1], window,
                       ctx.max_qlen, k_cache.shape[0], None, None, 0, 0, score_scale, softcap, _addr(slopes), _addr(sinks), nvh, vs)
    group, share = num_heads // num_kv_heads, num_heads // (nvh or num_kv_heads)
    rows = min(share, 16)
    if (USE_ROWS_DECODE_TC and ctx.max_qlen == 1 and mix is None and softcap == 0.0 and slopes is None and not DEBUG_BOUNDS
            and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0 and value_dim % 16 == 0
            and head_dim <= 256 and value_dim <= 256 and group >= 8 and rows >= 4 and share % rows == 0
            and rows_decode_smem(head_dim, value_dim, values_in_keys) <= 227 * 1024):
        # one token a sequence and many query heads on a key head: runs of heads that share a value head are the rows
        # of a tensor-core product over the key head's pages; the ranges are put together by the mixing kernel
        smem = rows_decode_smem(head_dim, value_dim, values_in_keys)
        span = max(1, -(-int(ctx.max_len) // PAGE))          # pages a token's keys can lie on
        if window > 0:
            span = min(span, -(-window // PAGE) + 1)
        splits = rows_decode_splits(ctx.n_seqs, num_heads // rows, span, q.device, smem)
        a.splits = splits
        a.pages_per_split = -(-span // splits)
        parts = empty((ctx.n_seqs, num_heads, 1, splits, value_dim), torch.float32, q.device)
        ml = empty((ctx.n_seqs, num_heads, splits, 2), torch.float32, q.device)
        a.parts, a.ml = parts.data_ptr(), ml.data_ptr()
        r = _RowsDecodeArgs(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), ctx.seq_qstart.data_ptr(),
                            ctx.seq_ctx.data_ptr(), pages.data_ptr(), parts.data_ptr(), ml.data_ptr(), ctx.n_seqs, num_heads,
                            num_kv_heads, nvh or num_kv_heads, pages.shape[-1], window, splits, a.pages_per_split, rows,
                            1 if values_in_keys else 0, score_scale)
        fn = _lib("attention_mixed_tc.cu", catalog.pair_dim_defines(head_dim, value_dim)).gl_attention_rows_decode_tc
        _check(_launch(fn, byref(r), _stream()), "attention_rows_decode_tc")
        _check(_launch(_lib("attention_mixed.cu").gl_head_mix_split, byref(a), c_int(dtype_code(q.dtype)), _stream()), "head_mix_split")
        return out
    if mix is not None:
        by_key_head = group <= 8 and num_kv_heads <= 8
    elif group <= 8:
        by_key_head = group % min(share, group) == 0
    else:                           # runs of eight query heads of a key head, whose value heads are whole within a run or span runs
        by_key_head = group % 8 == 0 and (share % 8 == 0 if share >= 8 else 8 % share == 0)
    if ctx.max_qlen == 1 and by_key_head and value_dim <= 128:
        # one token a sequence: the context in ranges of pages, a block each (sized for the step's longest
        # sequence; a captured step is sized for its bucket's longest), put together by the mixing kernel
        splits = mixed_decode_splits(ctx.n_seqs, num_kv_heads * max(1, group // 8), ctx.max_len, q.device)
        a.splits = splits
        a.pages_per_split = -(-max(1, -(-int(ctx.max_len) // PAGE)) // splits)
        parts = empty((ctx.n_seqs, num_heads, n_val, splits, value_dim), torch.float32, q.device)
        ml = empty((ctx.n_seqs, num_heads, splits, 2), torch.float32, q.device)
        a.parts, a.ml = parts.data_ptr(), ml.data_ptr()
    lib = _lib("attention_mixed.cu")
    if pairs_tc:
        p = _PairsArgs(q.data_ptr(), pairs.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                       ctx.seq_qstart.data_ptr(), ctx.seq_qlen.data_ptr(), ctx.seq_ctx.data_ptr(), pages.data_ptr(),
                       ctx.n_seqs, num_heads, num_kv_heads, n_val, pages.shape[-1], window, ctx.max_qlen,
                       score_scale, softcap, _addr(slopes), None, _addr(sinks), nvh, vs, 0)
        fn = _lib("attention_mixed_tc.cu", catalog.pair_dim_defines(head_dim, value_dim)).gl_attention_pairs_tc
        _check(_launch(fn, byref(p), _stream()), "attention_pairs_tc")
        _check(_launch(lib.gl_head_mix, byref(a), c_int(dtype_code(q.dtype)), _stream()), "head_mix")
        return out
    _check(_launch(lib.gl_attention_mixed, byref(a), c_int(dtype_code(q.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "attention_mixed", 2)
    return out


def gated_act(gu: torch.Tensor, act, inner: Optional[int] = None, row_gate: Optional[int] = None) -> torch.Tensor:
    """act(gate) * up for rows that hold the gate's columns and then the up projection's.  ``inner``: the rows
    are longer than that, the gate's ``inner`` columns first, the up projection's behind them; ``row_gate``: the
    column of such a row whose sigmoid multiplies the whole row's result."""
    _need(gu, "gu")
    T, F2 = gu.shape
    if inner is not None:
        if act not in ACTIVATIONS or 2 * inner > F2 or (row_gate is not None and not 0 <= row_gate < F2):
            raise KernelError("gated_act: the rows do not hold the gate's and the up projection's columns")
        out = empty((T, inner), gu.dtype, gu.device)
        fn = _lib("rowwise.cu").gl_gated_act_rows
        _check(_launch(fn, _ptr(gu), _ptr(out), c_int(T), c_int(inner), c_int(F2), c_int(-1 if row_gate is None else row_gate),
                       c_int(ACTIVATIONS[act]), c_int(dtype_code(gu.dtype)), _stream()), "gated_act")
        return out
    if F2 % 2 or act not in ACTIVATIONS:
        raise KernelError("gated_act: rows of gate and up columns and a known activation expected")
    out = empty((T, F2 // 2), gu.dtype, gu.device)
    fn = _lib("rowwise.cu").gl_gated_act
    _check(_launch(fn, _ptr(gu), _ptr(out), c_int(T), c_int(F2 // 2), c_int(ACTIVATIONS[act]),
                   c_int(dtype_code(gu.dtype)), _stream()), "gated_act")
    return out


def xielu(x: torch.Tensor, up: float, down: float) -> torch.Tensor:
    """In place: up * z^2 + z / 2 above zero, down * (e^z - 1 - z) + z / 2 at and below it."""
    _need(x, "x")
    _check(_launch(_lib("rowwise.cu").gl_xielu, _ptr(x), ctypes.c_longlong(x.numel()), c_float(up), c_float(down),
                   c_int(dtype_code(x.dtype)), _stream()), "xielu")
    return x


# ---------------------------------------------------------------------------
# Attention through a latent (csrc/latent.cu)
class _LatentPrepareArgs(Structure):
    _fields_ = [("proj", c_void_p), ("cq_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p), ("q_gamma", c_void_p), ("kv_gamma", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("pages", c_void_p),
                ("T", c_int), ("ld", c_int), ("q_rank", c_int), ("kv_rank", c_int), ("rot", c_int), ("max_pages", c_int),
                ("n_pages", c_int), ("interleaved", c_int), ("write_kv", c_int), ("eps", c_float)]


def latent_prepare(proj: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, ctx, pages: torch.Tensor,
                   q_rank: int, kv_rank: int, rot: int, q_gamma: torch.Tensor, kv_gamma: torch.Tensor, eps: float,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], interleaved: bool,
                   write_kv: bool = True) -> torch.Tensor:
    """A token's down projections proj [T, ld] = [query latent (q_rank) | c (kv_rank) | key part (rot) | ...]: both
    latents RMS-normed with their weights (32-bit), the key part rotated by the token's angles; the row [c | key part]
    goes to the token's place in k_cache [pages, 1, PAGE, kv_rank + rot], c to v_cache [pages, 1, PAGE, kv_rank]
    (``v_cache`` None or the key cache itself: the values are read from the key rows, nothing more is written).
    Returns the normed query latent [T, q_rank]."""
    _need(proj, "proj")
    T, ld = proj.shape
    if ld < q_rank + kv_rank + rot:
        raise KernelError("latent_prepare: the projection's rows are too short")
    if v_cache is not None and v_cache.data_ptr() == k_cache.data_ptr():
        v_cache = None
    if tuple(k_cache.shape[1:]) != (1, PAGE, kv_rank + rot) or (v_cache is not None and tuple(v_cache.shape[1:]) != (1, PAGE, kv_rank)):
        raise KernelError(f"cache pages do not fit: keys {tuple(k_cache.shape)}, values {tuple(v_cache.shape)}")
    _need(q_gamma, "q_gamma", torch.float32, (q_rank,))
    _need(kv_gamma, "kv_gamma", torch.float32, (kv_rank,))
    if cos is not None:
        _need(cos, "cos", torch.float32, (T, rot // 2))
        _need(sin, "sin", torch.float32, (T, rot // 2))
    cq = empty((T, q_rank), proj.dtype, proj.device)
    a = _LatentPrepareArgs(proj.data_ptr(), cq.data_ptr(), k_cache.data_ptr(), _addr(v_cache), _addr(cos), _addr(sin),
                           q_gamma.data_ptr(), kv_gamma.data_ptr(), ctx.tok_seq.data_ptr(), ctx.tok_pos.data_ptr(),
                           pages.data_ptr(), T, ld, q_rank, kv_rank, rot, pages.shape[-1], k_cache.shape[0],
                           1 if interleaved else 0, 1 if write_kv else 0, eps)
    _check(_launch(_lib("latent.cu").gl_latent_prepare, byref(a), c_int(dtype_code(proj.dtype)),
                   c_int(dtype_code(k_cache.dtype)), _stream()), "latent_prepare")
    return cq


class _HeadLinearArgs(Structure):
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("out", c_void_p), ("gate", c_void_p), ("cosv", c_void_p), ("sinv", c_void_p),
                ("T", c_int), ("H", c_int), ("N", c_int), ("K", c_int),
                ("x_row", c_int), ("x_head", c_int), ("x_off", c_int), ("o_row", c_int), ("o_head", c_int), ("o_off", c_int),
                ("g_row", c_int), ("g_off", c_int), ("tail", c_int), ("interleaved", c_int)]


def head_linear(x: torch.Tensor, w: torch.Tensor, x_head: int, tail: int = 0, cos: Optional[torch.Tensor] = None,
                sin: Optional[torch.Tensor] = None, interleaved: bool = False, gate: Optional[torch.Tensor] = None,
                gate_off: int = 0) -> torch.Tensor:
    """A product per head: out[t, h, :N] = w[h] x[t, h, :K] for x [T, H * x_head] (head h's K inputs start at column
    h * x_head) and w [H, N, K].  ``tail`` > 0: the columns x[t, h, K:K + tail] are copied behind the result, turned by
    the token's angles when cos/sin [T, tail / 2] are given; out is [T, H * (N + tail)].  ``gate`` [T, ld]: the result
    of head h is multiplied by sigmoid(gate[t, gate_off + h])."""
    _need(x, "x")
    _need(w, "w")
    T = x.shape[0]
    H, N, K = w.shape
    if x.shape[1] != H * x_head or K + tail > x_head:
        raise KernelError(f"head_linear: x {tuple(x.shape)} does not hold {H} heads of {K} + {tail} columns")
    if cos is not None:
        _need(cos, "cos", torch.float32, (T, tail // 2))
        _need(sin, "sin", torch.float32, (T, tail // 2))
    g_row = 0
    if gate is not None:
        _need(gate, "gate", x.dtype)
        g_row = gate.shape[1]
        if gate.shape[0] != T or gate_off + H > g_row:
            raise KernelError("head_linear: the gate's rows do not hold a column for every head")
    out = empty((T, H * (N + tail)), x.dtype, x.device)
    a = _HeadLinearArgs(x.data_ptr(), w.data_ptr(), out.data_ptr(), _addr(gate), _addr(cos), _addr(sin), T, H, N, K,
                        x.shape[1], x_head, 0, H * (N + tail), N + tail, 0, g_row, gate_off, tail, 1 if interleaved else 0)
    _check(_launch(_lib("latent.cu").gl_head_linear, byref(a), c_int(dtype_code(x.dtype)), c_int(dtype_code(w.dtype)),
                   _stream()), "head_linear")
    return out


# ---------------------------------------------------------------------------
# A mixture of experts (csrc/moe.cu)
MOE_TILE_ROWS = 32


class _RouteArgs(Structure):
    _fields_ = [("logits", c_void_p), ("ids", c_void_p), ("weights", c_void_p),
                ("T", c_int), ("E", c_int), ("top", c_int), ("groups", c_int), ("keep", c_int), ("scale", c_float),
                ("bias", c_void_p), ("softmax_chosen", c_int)]


def _route_mode(E: int, groups: int, bias, softmax_chosen: bool) -> None:
    if bias is not None:
        _need(bias, "bias", torch.float32, (E,))
    if softmax_chosen and groups != 1:
        raise KernelError("moe_route: the softmax over the chosen logits takes one group of experts")


def moe_route(logits: torch.Tensor, top: int, groups: int = 1, keep: int = 1, scale: float = 1.0,
              bias: Optional[torch.Tensor] = None, softmax_chosen: bool = False):
    """Each token's ``top`` experts by sigmoid(logits) and their weights score / (sum of the chosen scores +
    1e-20) * scale: (ids int32 [T, top], weights float32 [T, top]).  With ``groups`` > 1 the experts form that
    many equal groups of neighbours; a group's score is the sum of its two largest scores and only experts of
    the best ``keep`` groups are chosen from.  ``bias`` [E] float32 is added to the logits first.  With
    ``softmax_chosen`` the ``top`` largest logits are chosen instead and weighted by the softmax over those
    alone (times scale)."""
    _need(logits, "logits", torch.float32)
    T, E = logits.shape
    _route_mode(E, groups, bias, softmax_chosen)
    if not (0 < top <= E and groups >= 1 and E % groups == 0 and 1 <= keep <= groups and keep * (E // groups) >= top):
        raise KernelError(f"moe_route: top {top} of {E} experts in {groups} groups of which {keep} stay is not possible")
    ids = empty((T, top), torch.int32, logits.device)
    weights = empty((T, top), torch.float32, logits.device)
    a = _RouteArgs(logits.data_ptr(), ids.data_ptr(), weights.data_ptr(), T, E, top, groups, keep, scale, _addr(bias),
                   1 if softmax_chosen else 0)
    _check(_launch(_lib("moe.cu").gl_moe_route, byref(a), _stream()), "moe_route")
    return ids, weights


class _RouteFromArgs(Structure):
    # (the kernel's record holds the router's record as a member; written out flat here, with the same layout, so
    # that a tape of launches finds every pointer)
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("K", c_int),
                ("logits", c_void_p), ("ids", c_void_p), ("weights", c_void_p),
                ("T", c_int), ("E", c_int), ("top", c_int), ("groups", c_int), ("keep", c_int), ("scale", c_float),
                ("bias", c_void_p), ("softmax_chosen", c_int)]


def moe_route_from(x: torch.Tensor, w_router: torch.Tensor, top: int, groups: int = 1, keep: int = 1, scale: float = 1.0,
                   bias: Optional[torch.Tensor] = None, softmax_chosen: bool = False):
    """``moe_route`` of the logits x . w_router^T ([T, K] in the activation type, [E, K] float32) in one kernel:
    a token's logits are sums over k in an order of their own, whatever else is in the step.  Inputs too wide
    for a block's shared memory take the plain product and ``moe_route``."""
    _need(x, "x")
    _need(w_router, "w_router", torch.float32)
    T, K = x.shape
    E = w_router.shape[0]
    if w_router.shape[1] != K:
        raise KernelError(f"moe_route_from: router {tuple(w_router.shape)} does not fit x {tuple(x.shape)}")
    _route_mode(E, groups, bias, softmax_chosen)
    if (E + groups + K) * 4 > 48 * 1024:
        return moe_route(gemm_simt(x, w_router, out_dtype=torch.float32), top, groups, keep, scale, bias, softmax_chosen)
    if not (0 < top <= E and groups >= 1 and E % groups == 0 and 1 <= keep <= groups and keep * (E // groups) >= top):
        raise KernelError(f"moe_route: top {top} of {E} experts in {groups} groups of which {keep} stay is not possible")
    ids = empty((T, top), torch.int32, x.device)
    weights = empty((T, top), torch.float32, x.device)
    a = _RouteFromArgs(x.data_ptr(), w_router.data_ptr(), K, None, ids.data_ptr(), weights.data_ptr(), T, E, top, groups,
                       keep, scale, _addr(bias), 1 if softmax_chosen else 0)
    _check(_launch(_lib("moe.cu").gl_moe_route_from, byref(a), c_int(dtype_code(x.dtype)), _stream()), "moe_route")
    return ids, weights


class _PlanArgs(Structure):
    _fields_ = [("ids", c_void_p), ("order", c_void_p), ("tile_expert", c_void_p), ("tile_start", c_void_p),
                ("tile_rows", c_void_p), ("n_tiles", c_void_p), ("A", c_int), ("E", c_int), ("max_tiles", c_int)]


class _ExpertArgs(Structure):
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("out", c_void_p), ("order", c_void_p), ("tile_expert", c_void_p),
                ("tile_start", c_void_p), ("tile_rows", c_void_p), ("n_tiles", c_void_p), ("weights", c_void_p),
                ("A", c_int), ("N", c_int), ("K", c_int), ("top", c_int), ("max_tiles", c_int), ("E", c_int)]


class _PadPlanArgs(Structure):
    _fields_ = [("ids", c_void_p), ("order", c_void_p), ("place", c_void_p), ("tile_expert", c_void_p),
                ("A", c_int), ("E", c_int), ("max_tiles", c_int), ("tile_m", c_int)]


MOE_ROWS_KERNEL_PER_EXPERT = 4     # up to this many (token, choice) pairs an expert on average: the few-rows kernel
USE_MOE_GROUPED = True             # many rows an expert in bfloat16: one grouped product on tcgen05 (False: tiles on mma.sync)
USE_MOE_TC = True        # bfloat16 experts on the tensor cores (False: the CUDA-core kernels, for comparison)


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, add: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * down_e(silu(gate_e(x[t])) * up_e(x[t])) + add[t], e = ids[t, k]; float32
    [T, hidden].  w_gate_up [E, 2F, K] holds every expert's gate rows and then its up rows, w_down [E, hidden, F].
    The step's (token, choice) pairs are sorted by expert on the device and cut into tiles of rows; the grids
    cover the most tiles any choice can make, so nothing depends on the host knowing what the router chose.
    Which kernels run depends on the step's size alone: up to MOE_ROWS_KERNEL_PER_EXPERT pairs an expert on
    average (bfloat16) a weight-streaming kernel, a warp an output column; more (bfloat16): every expert's rows on
    tiles of 128 of their own and each product one tcgen05 product with grouped weights; other types: tiles of 32
    rows on the CUDA cores, every sum over k in ascending order.  ``add`` may be a callable that returns the tensor:
    it is called right before the last kernel, the one that adds it (a branch on a second stream joins there)."""
    _need(x, "x")
    T, K = x.shape
    late_add = add if callable(add) else None
    if late_add is not None:
        add = None
    _need(ids, "ids", torch.int32)
    top = ids.shape[1]
    _need(weights, "weights", torch.float32, (T, top))
    _need(w_gate_up, "w_gate_up")
    _need(w_down, "w_down", w_gate_up.dtype)
    E, F2, Kw = w_gate_up.shape
    F = F2 // 2
    hidden = w_down.shape[1]
    if Kw != K or F2 % 2 or tuple(w_down.shape) != (E, hidden, F) or tuple(ids.shape) != (T, top):
        raise KernelError(f"moe_experts: weights {tuple(w_gate_up.shape)} / {tuple(w_down.shape)} do not fit x {tuple(x.shape)}")
    if add is not None:
        _need(add, "add", torch.float32, (T, hidden))
    if out is None:
        out = empty((T, hidden), torch.float32, x.device)
    _need(out, "out", torch.float32, (T, hidden))
    A = T * top
    dev = x.device
    lib = _lib("moe.cu")
    if (USE_MOE_TC and USE_TCGEN05 and USE_MOE_GROUPED and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
            and A > MOE_ROWS_KERNEL_PER_EXPERT * E and K % 8 == 0 and F % 8 == 0 and hidden % 4 == 0):
        # many rows an expert: rows sorted by expert, every expert on tiles of 128 rows of its own, and each of
        # the two products one product with grouped weights
        tiles = -(-A // 128) + min(E, A)
        order = empty((tiles * 128,), torch.int32, dev)
        place = empty((A,), torch.int32, dev)
        tile_expert = empty((tiles,), torch.int32, dev)
        p = _PadPlanArgs(ids.data_ptr(), order.data_ptr(), place.data_ptr(), tile_expert.data_ptr(), A, E, tiles, 128)
        _check(_launch(lib.gl_moe_plan_padded, byref(p), _stream()), "moe_plan")
        xs = empty((tiles * 128, K), torch.bfloat16, dev)
        _check(_launch(lib.gl_moe_gather_rows, _ptr(x), _ptr(order), _ptr(xs), c_int(tiles * 128), c_int(K), c_int(top),
                       _stream()), "moe_gather_rows")
        gu = gemm_tcgen05_grouped(xs, w_gate_up, tile_expert, torch.bfloat16)
        h = gated_act(gu, "silu")
        y = gemm_tcgen05_grouped(h, w_down, tile_expert, torch.float32)
        if late_add is not None:
            add = late_add()
            _need(add, "add", torch.float32, (T, hidden))
        _check(_launch(lib.gl_moe_combine_placed, _ptr(y), _ptr(place), _ptr(weights), _ptr(add), _ptr(out), c_int(T),
                       c_int(hidden), c_int(top), _stream()), "moe_combine")
        return out
    max_tiles = -(-A // MOE_TILE_ROWS) + min(E, A)
    # (each a tensor of its own: a tape of launches knows temporaries by their first address)
    order = empty((A,), torch.int32, dev)
    tile_expert, tile_start, tile_rows = (empty((max_tiles,), torch.int32, dev) for _ in range(3))
    n_tiles = empty((1,), torch.int32, dev)
    p = _PlanArgs(ids.data_ptr(), order.data_ptr(), tile_expert.data_ptr(), tile_start.data_ptr(), tile_rows.data_ptr(),
                  n_tiles.data_ptr(), A, E, max_tiles)
    _check(_launch(lib.gl_moe_plan, byref(p), _stream()), "moe_plan")
    h = empty((A, F), x.dtype, dev)
    y = empty((A, hidden), torch.float32, dev)
    xd, wd = c_int(dtype_code(x.dtype)), c_int(dtype_code(w_gate_up.dtype))
    g = _ExpertArgs(x.data_ptr(), w_gate_up.data_ptr(), h.data_ptr(), order.data_ptr(), tile_expert.data_ptr(),
                    tile_start.data_ptr(), tile_rows.data_ptr(), n_tiles.data_ptr(), None, A, F, K, top, max_tiles, E)
    _check(_launch(lib.gl_moe_gate_up if USE_MOE_TC else lib.gl_moe_gate_up_simt, byref(g), xd, wd, _stream()), "moe_gate_up")
    d = _ExpertArgs(h.data_ptr(), w_down.data_ptr(), y.data_ptr(), order.data_ptr(), tile_expert.data_ptr(),
                    tile_start.data_ptr(), tile_rows.data_ptr(), n_tiles.data_ptr(), weights.data_ptr(), A, hidden, F, top,
                    max_tiles, E)
    _check(_launch(lib.gl_moe_down if USE_MOE_TC else lib.gl_moe_down_simt, byref(d), xd, wd, _stream()), "moe_down")
    if late_add is not None:
        add = late_add()
        _need(add, "add", torch.float32, (T, hidden))
    _check(_launch(lib.gl_moe_combine, _ptr(y), _ptr(add), _ptr(out), c_int(T), c_int(hidden), c_int(top), _stream()),
           "moe_combine")
    return out


def enter_pass(x: torch.Tensor, base: Optional[torch.Tensor], table: Optional[torch.Tensor], row: int) -> torch.Tensor:
    """x += base + table[row] on the float32 residual stream (either may be None)."""
    _need(x, "x", torch.float32)
    T, D = x.shape
    if base is not None:
        _need(base, "base", torch.float32, (T, D))
    if table is not None:
        _need(table, "table", torch.float32)
        if table.shape[1] != D or not 0 <= row < table.shape[0]:
            raise KernelError(f"enter_pass: row {row} of a table {tuple(table.shape)} for width {D}")
    fn = _lib("rowwise.cu").gl_enter_pass
    _check(_launch(fn, _ptr(x), _ptr(base), _ptr(table), c_int(T), c_int(D), c_int(row), _stream()), "enter_pass")
    return x


def rms_norm_pair(x: torch.Tensor, g1: torch.Tensor, g2: torch.Tensor, eps: float, out_dtype: torch.dtype):
    """Two RMS norms of the same float32 rows with weights g1 and g2, the rows read once."""
    _need(x, "x", torch.float32)
    R, D = x.shape
    _need(g1, "g1", torch.float32, (D,))
    _need(g2, "g2", torch.float32, (D,))
    o1 = empty((R, D), out_dtype, x.device)
    o2 = empty((R, D), out_dtype, x.device)
    fn = _lib("rowwise.cu").gl_rms_norm_pair
    _check(_launch(fn, _ptr(x), _ptr(g1), _ptr(g2), _ptr(o1), _ptr(o2), c_int(dtype_code(out_dtype)), c_int(R), c_int(D),
                   c_float(eps), _stream()), "rms_norm_pair")
    return o1, o2


def round_rows(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """The float32 residual stream in the activation type (itself when that is float32): the input of a
    sublayer that reads the stream as it is."""
    _need(x, "x", torch.float32)
    if out_dtype == torch.float32:
        return x
    if out_dtype != torch.bfloat16:
        raise KernelError(f"round_rows: {out_dtype} is not an activation type")
    out = empty(x.shape, torch.bfloat16, x.device)
    _check(_launch(_lib("rowwise.cu").gl_round_rows, _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _stream()), "round_rows")
    return out


def post_norm_add(a: torch.Tensor, w: torch.Tensor, eps: float, add: torch.Tensor, out: Optional[torch.Tensor] = None,
                  scale: float = 1.0, second=None, rounded: Optional[torch.dtype] = None):
    """out = add + y / sqrt(mean(y^2) + eps) * w with y = scale * a (+ scale2 * a2 for ``second`` = (a2, scale2)),
    float32 rows: a sublayer's output, or the weighted sum of its two branches, normed and added onto the
    stream.  ``rounded`` = bfloat16 also returns the result rounded to that type (the next sublayer's input);
    returns (out, rounded copy or None)."""
    _need(a, "a", torch.float32)
    R, D = a.shape
    _need(w, "w", torch.float32, (D,))
    _need(add, "add", torch.float32, (R, D))
    a2, s2 = (None, 0.0)
    if second is not None:
        a2, s2 = second
        _need(a2, "a2", torch.float32, (R, D))
    if out is None:
        out = empty((R, D), torch.float32, a.device)
    _need(out, "out", torch.float32, (R, D))
    copy = empty((R, D), torch.bfloat16, a.device) if rounded == torch.bfloat16 else None
    fn = _lib("rowwise.cu").gl_post_norm_add
    _check(_launch(fn, _ptr(a), _ptr(a2), _ptr(w), _ptr(add), _ptr(out), _ptr(copy), c_int(R), c_int(D), c_float(eps),
                   c_float(scale), c_float(s2), _stream()), "post_norm_add")
    return out, copy


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float, adds=(), out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = sa * a + sb * b + sum(adds), float32 tensors of one shape; up to two adds."""
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32, tuple(a.shape))
    adds = list(adds)
    if len(adds) > 2:
        raise KernelError("scaled_sum adds at most two tensors")
    for t in adds:
        _need(t, "add", torch.float32, tuple(a.shape))
    adds += [None] * (2 - len(adds))
    if out is None:
        out = empty(a.shape, torch.float32, a.device)
    _need(out, "out", torch.float32, tuple(a.shape))
    _check(_launch(_lib("rowwise.cu").gl_scaled_sum, _ptr(a), _ptr(b), _ptr(adds[0]), _ptr(adds[1]), _ptr(out),
                   ctypes.c_longlong(a.numel()), c_float(sa), c_float(sb), _stream()), "scaled_sum")
    return out


def moe_route_table(tokens: torch.Tensor, table: torch.Tensor, experts: int):
    """Routing by token id: (ids int32 [T, top], weights float32 [T, top]) with ids[t] = table[tokens[t]] and
    every weight 1 / top."""
    _need(tokens, "tokens", torch.int32)
    _need(table, "table", torch.int32)
    T = tokens.shape[0]
    vocab, top = table.shape
    ids = empty((T, top), torch.int32, tokens.device)
    weights = empty((T, top), torch.float32, tokens.device)
    _check(_launch(_lib("moe.cu").gl_moe_route_table, _ptr(tokens), _ptr(table), _ptr(ids), _ptr(weights), c_int(T), c_int(top),
                   c_int(vocab), c_int(experts), _stream()), "moe_route_table")
    return ids, weights


def rms_scale_add(a: torch.Tensor, w: torch.Tensor, eps: float, alpha: float, adds=(), out: Optional[torch.Tensor] = None,
                  second=None):
    """out = alpha * a / sqrt(mean(a^2) + eps) * w + sum(adds), float32 rows; up to three adds.  ``second`` =
    (a2, w2): a second branch normalised and scaled the same way and added in the same pass."""
    _need(a, "a", torch.float32)
    R, D = a.shape
    _need(w, "w", torch.float32, (D,))
    a2 = w2 = None
    if second is not None:
        a2, w2 = second
        _need(a2, "a2", torch.float32, (R, D))
        _need(w2, "w2", torch.float32, (D,))
    adds = list(adds)
    if len(adds) > 3:
        raise KernelError("rms_scale_add adds at most three tensors")
    for t in adds:
        _need(t, "add", torch.float32, (R, D))
    adds += [None] * (3 - len(adds))
    if out is None:
        out = empty((R, D), torch.float32, a.device)
    _need(out, "out", torch.float32, (R, D))
    fn = _lib("rowwise.cu").gl_rms_scale_add
    _check(_launch(fn, _ptr(a), _ptr(w), _ptr(a2), _ptr(w2), _ptr(adds[0]), _ptr(adds[1]), _ptr(adds[2]), _ptr(out),
                   c_int(R), c_int(D), c_float(eps), c_float(alpha), _stream()), "rms_scale_add")
    return out


def wait_failures(clear: bool = False) -> dict:
    """Which of the loaded libraries recorded a bounded wait that ran out (what they computed since is
    invalid): library name -> 1, 0, or -1 if the word could not be read.  ``clear`` sets the words back
    to 0.  Reading a word waits for the device."""
    out = {}
    for key, lib in list(build._loaded.items()):
        if hasattr(lib, "gl_wait_status"):
            out[key] = int(lib.gl_wait_status(c_int(1 if clear else 0)))
    return out


_BOUNDS_KINDS = {1: "token id", 2: "page number", 3: "position in a page table", 4: "row of a table"}


def bounds_status(clear: bool = False) -> dict:
    """In a build that checks indices (GOPHERLLM_DEBUG_BOUNDS=1): library name -> (kind, value, limit,
    count) of the bad indices its kernels met since the words were last cleared; libraries without
    violations are left out.  Empty in an ordinary build."""
    out = {}
    for key, lib in list(build._loaded.items()):
        if hasattr(lib, "gl_bounds_status"):
            words = (c_int * 4)()
            if lib.gl_bounds_status(words, c_int(1 if clear else 0)) != 0:
                out[key] = ("unreadable", 0, 0, 0)
            elif words[0] != 0:
                out[key] = (_BOUNDS_KINDS.get(words[0], str(words[0])), words[1], words[2], words[3])
    return out


def check_wait_failures() -> None:
    """Raise KernelError naming every library whose kernels gave up a bounded wait since the last
    check; the words are cleared, so the next check speaks of what ran after this one."""
    oob = bounds_status(clear=True)
    if oob:
        raise KernelError("kernels met indices outside their tables: " + "; ".join(
            f"{lib}: {kind} {value} (limit {limit}, {count} in all)" for lib, (kind, value, limit, count) in sorted(oob.items())))
    bad = sorted(k for k, v in wait_failures(clear=True).items() if v != 0)
    if bad:
        reset_decode_layer_sync()
        raise KernelError("a kernel gave up waiting (for a TMA copy or a tensor-core product) in "
                          + ", ".join(bad) + ": the results since the last check are invalid")


def linear_pair(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                a2: torch.Tensor, w2: torch.Tensor, bias2: Optional[torch.Tensor],
                add0: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = a·wᵀ + bias + a2·w2ᵀ + bias2 + add0: the last products of two branches that are added
    to the same rows.  In bfloat16 both run as one product over the joined K (one kernel, one pass
    over the output); otherwise one after the other, each adding onto out."""
    if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a2.dtype == torch.bfloat16
            and w2.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a2.shape[1] % 8 == 0):
        if a.shape[0] <= SKINNY_MAX_ROWS:
            if a.shape[1] % 64 == 0:
                return _few_rows(a, w, bias, None, add0, None, torch.float32, out, second=(a2, w2, bias2))
            if a2.shape[1] % 64 == 0:                  # the product whose K fills whole stages goes first
                return _few_rows(a2, w2, bias2, None, add0, None, torch.float32, out, second=(a, w, bias))
        elif USE_TCGEN05:
            return gemm_tcgen05(a, w, bias, None, add0, None, torch.float32, out, second=(a2, w2, bias2))
    out = linear(a, w, bias, add0=add0, out_dtype=torch.float32, out=out)
    return linear(a2, w2, bias2, add0=out, out=out)


def linear_fork(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act,
                w_b: torch.Tensor, bias_b: Optional[torch.Tensor], act_b, out_dtype: Optional[torch.dtype] = None):
    """(act(a·wᵀ + bias), act_b(a·w_bᵀ + bias_b)): the first products of two branches that read the
    same rows.  For many rows of bfloat16 both run as one grid of tensor-core tiles; otherwise one
    after the other."""
    dt = out_dtype or a.dtype
    if (USE_TCGEN05 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w_b.dtype == torch.bfloat16
            and a.shape[0] > SKINNY_MAX_ROWS and a.shape[1] % 8 == 0
            and (w.shape[0] * dt.itemsize) % 16 == 0 and (w_b.shape[0] * dt.itemsize) % 16 == 0):
        return gemm_tcgen05(a, w, bias, act, out_dtype=dt, fork=(w_b, bias_b, act_b))
    return linear(a, w, bias, act, out_dtype=dt), linear(a, w_b, bias_b, act_b, out_dtype=dt)


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
           add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(a · wᵀ + bias) + add0 + add1 with the fastest kernel that takes these
    types and sizes.  float32 operands always run the 32-bit CUDA-core product."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        if a.shape[0] <= SKINNY_MAX_ROWS:
            return _few_rows(a, w, bias, act, add0, add1, out_dtype, out)
        if USE_TCGEN05:
            return gemm_tcgen05(a, w, bias, act, add0, add1, out_dtype, out)
    return gemm_simt(a, w, bias, act, add0, add1, out_dtype, out)


class _SampleArgs(Structure):
    _fields_ = [("logits", c_void_p), ("work", c_void_p), ("state_row", c_void_p), ("recent", c_void_p),
                ("recent_n", c_void_p), ("rng", c_void_p), ("out", c_void_p),
                ("sort_key", c_void_p), ("sort_idx", c_void_p),
                ("B", c_int), ("V", c_int), ("vpad", c_int), ("top_k", c_int),
                ("temperature", c_float), ("top_p", c_float), ("min_p", c_float),
                ("repeat_penalty", c_float)]


def check_sampler(temperature: float, top_k: int, top_p: float, min_p: float, vocab: int) -> None:
    """Raise if the kernel does not take this combination of options."""
    greedy = temperature < 1e-6 or top_k == 1
    if greedy:
        return
    whole = not (0 < top_k < vocab)
    if not whole and top_k > SAMPLE_KMAX:
        raise KernelError(f"top_k {top_k} exceeds {SAMPLE_KMAX} (top_k 0 or >= vocabulary samples the whole row)")


def needs_sort_scratch(temperature: float, top_k: int, top_p: float, min_p: float, vocab: int) -> bool:
    """Whether sampling needs sorting scratch: never (a nucleus or min-p cut with top-k off finds its
    boundary by a search over the weights' bits, not by sorting the row)."""
    return False


def sort_scratch_size(vocab: int) -> int:
    n = 1
    while n < vocab:
        n <<= 1
    return n


def sample(logits: torch.Tensor, work: torch.Tensor, recent: torch.Tensor, recent_n: torch.Tensor,
           rng: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float,
           min_p: float, repeat_penalty: float, state_row: Optional[torch.Tensor] = None,
           sort_key: Optional[torch.Tensor] = None, sort_idx: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits [B, V] into ``out`` [B] int32.

    recent [R, 64] int32 / recent_n [R] int32: each state row's window of recent tokens
    (the choice is appended); rng [R] int64: xorshift64 states; state_row [B] int32 says
    which state row a logits row uses (None: row b uses state b)."""
    _need(logits, "logits", torch.float32)
    B, V = logits.shape
    _need(work, "work", torch.float32)
    if work.numel() < B * V:
        raise KernelError("sampling scratch is smaller than the logits")
    R = recent_n.numel()
    _need(recent, "recent", torch.int32, (R, SAMPLE_WINDOW))
    _need(recent_n, "recent_n", torch.int32, (R,))
    _need(rng, "rng", torch.int64, (R,))
    _need(out, "out", torch.int32)
    if out.numel() < B:
        raise KernelError("out is smaller than the batch")
    if state_row is not None:
        _need(state_row, "state_row", torch.int32)
        if state_row.numel() < B:
            raise KernelError("state_row is smaller than the batch")
    elif R < B:
        raise KernelError(f"{R} sampler states for {B} rows")
    check_sampler(temperature, top_k, top_p, min_p, V)
    vpad = 0
    if needs_sort_scratch(temperature, top_k, top_p, min_p, V):
        vpad = sort_scratch_size(V)
        if sort_key is None:
            sort_key = empty((B, vpad), torch.float32, logits.device)
            sort_idx = empty((B, vpad), torch.int32, logits.device)
        _need(sort_key, "sort_key", torch.float32)
        _need(sort_idx, "sort_idx", torch.int32)
        if sort_key.numel() < B * vpad or sort_idx.numel() < B * vpad:
            raise KernelError("sorting scratch is smaller than the batch needs")
    a = _SampleArgs(logits.data_ptr(), work.data_ptr(), _addr(state_row), recent.data_ptr(),
                    recent_n.data_ptr(), rng.data_ptr(), out.data_ptr(), _addr(sort_key), _addr(sort_idx),
                    B, V, vpad, top_k,
                    temperature, top_p, min_p, repeat_penalty)
    _check(_launch(_lib("sampling.cu").gl_sample, byref(a), _stream()), "sample")


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off in every library loaded so far (on by
    default).  With it a kernel's blocks may be scheduled, and a product may start fetching
    its weights, while the kernel before it is still finishing."""
    for lib in list(build._loaded.values()):
        if hasattr(lib, "gl_set_pdl"):
            lib.gl_set_pdl(c_int(1 if on else 0))


def warm_up(head_dims=()) -> None:
    """Compile (if needed) and load every library a model with these head sizes uses."""
    for src, defines in catalog.all_libraries(head_dims):
        _lib(src, defines)
