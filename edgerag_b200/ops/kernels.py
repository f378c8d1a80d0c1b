"""Python entry points of the CUDA kernels: tensors in, one launch on the current stream each.

Every function checks what a wrong call would turn into a wrong result (device, dtype, layout,
sizes), then calls the ``extern "C"`` function of the library built for the tensors' element type.
Nothing here falls back to PyTorch arithmetic: a missing library or a refused shape raises.
"""

from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import native


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_ELEM = {torch.float32: "float32", torch.bfloat16: "bfloat16"}

_SIGNATURES = {
    "erb_embed_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p, c_void_p],
    "erb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                        c_void_p],
    "erb_residual_add": [c_void_p, c_void_p, c_longlong, c_void_p],
    "erb_rope_cache_write": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_swiglu": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_resolve_ids": [c_void_p, c_int, c_void_p, c_int, c_void_p],
    "erb_gather_cast": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_linear": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_void_p, c_longlong, c_void_p],
    "erb_linear_skinny": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_skinny_glu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_skinny_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "erb_linear_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tune": [c_int],
    "erb_linear_trials": [],
    "erb_linear_tc_parts": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tc_parts_count": [c_int, c_int],
    "erb_residual_add_parts": [c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p],
    "erb_add_rmsnorm_parts": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                              c_int, c_int, c_void_p],
    "erb_linear_tc_glu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tc_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "erb_attention_rows": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "erb_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_float, c_void_p],
    "erb_attention_prefill_tc": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                 c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "erb_attention_decode_bulk": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_float, c_void_p, c_void_p, c_int, c_void_p],
    "erb_attention_decode_gqa": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_void_p, c_void_p, c_void_p],
    "erb_sample_rows": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
}

_functions: dict[tuple[str, str | None, str], object] = {}

#: launches issued through this module: this package's own kernels, and library products
launch_counts = {"own": 0, "library": 0}
_LAUNCHES = {"erb_attention_decode": 2, "erb_attention_prefill_tc": 1, "erb_attention_decode_bulk": 1, "erb_attention_decode_gqa": 1, "erb_linear": 0}
SKINNY_MAX_ROWS = 16     # rows up to which the register-fed weight-streaming kernels are used
TC_MAX_ROWS = 64         # rows up to which the TMA + tcgen05 weight-streaming kernel may be used


def launches() -> int:
    """Kernels launched through this module so far (this package's own and the library's)."""
    return launch_counts["own"] + launch_counts["library"]


def _fn(library: str, elem: str | None, name: str):
    key = (library, elem, name)
    fn = _functions.get(key)
    if fn is None:
        lib = native.load(library, elem)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[name]
        fn.restype = c_int
        fn._erb_lib = lib
        fn._erb_own = _LAUNCHES.get(name, 1)
        _functions[key] = fn
    return fn


def _call(fn, *args) -> None:
    rc = fn(*args)
    if fn._erb_own:
        launch_counts["own"] += fn._erb_own
    else:
        launch_counts["library"] += 1
    if rc != 0:
        raise KernelError(fn._erb_lib.erb_last_error().decode())


def _elem(t: torch.Tensor) -> str:
    try:
        return _ELEM[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The raw handle of the current CUDA stream (the capturing stream inside a graph capture)."""
    # (the C calls directly: torch.cuda.current_device() costs a microsecond of Python per launch)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor | None, name: str, dtype=None, contiguous: bool = True) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


# --- rows ------------------------------------------------------------------------------------

def embed_rows(hidden: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
               embeds: torch.Tensor | None = None, embed_row: torch.Tensor | None = None) -> None:
    """hidden[t] = table[ids[t]], or embeds[embed_row[t]] where embed_row[t] >= 0 (float output)."""
    n, h = hidden.shape
    _need(hidden, "hidden", torch.float32); _need(table, "table"); _need(ids, "ids", torch.int32)
    _need(status, "status", torch.int32); _need(embed_row, "embed_row", torch.int32)
    if table.shape[1] != h or ids.numel() < n:
        raise KernelError("embed_rows: shapes disagree")
    if embeds is not None:
        _need(embeds, "embeds", table.dtype)
        if embeds.shape[1] != h or embed_row is None:
            raise KernelError("embed_rows: embeds need embed_row and the hidden width")
    _call(_fn("elementwise", _elem(table), "erb_embed_rows"), hidden.data_ptr(), table.data_ptr(),
          _ptr(embeds), ids.data_ptr(), _ptr(embed_row), n, h, table.shape[0],
          0 if embeds is None else embeds.shape[0], status.data_ptr(), _stream())


def add_rmsnorm(hidden: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                delta: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                write_back: bool = True, settled: bool = False) -> None:
    """out = weight * round(rmsnorm(hidden (+ delta))); hidden += delta in place when write_back.
    ``delta``: rows of the element type, or float32 partial sums ``[parts, rows, width]`` (what
    ``linear_parts`` leaves) that are added in their order and rounded to the element type once, so that
    the update is what a product stored in the element type would have been.
    ``settled``: ``hidden`` was last written two or more launches ago (the launch just before this one
    wrote ``delta`` at most), so the kernel may read it while that launch is still running."""
    _need(hidden, "hidden", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    _need(rows, "rows", torch.int32)
    h = hidden.shape[1]
    n = out.shape[0]
    in_parts = delta is not None and delta.dim() == 3
    _need(delta, "delta", torch.float32 if in_parts else out.dtype)
    if out.shape[1] != h or weight.numel() != h or (delta is not None and delta.shape[-2:] != hidden.shape):
        raise KernelError("add_rmsnorm: shapes disagree")
    if rows is None and n != hidden.shape[0]:
        raise KernelError("add_rmsnorm: out rows differ from hidden rows")
    if rows is not None and rows.numel() < n:
        raise KernelError("add_rmsnorm: fewer row indices than output rows")
    if in_parts:
        _call(_fn("elementwise", _elem(out), "erb_add_rmsnorm_parts"), hidden.data_ptr(), delta.data_ptr(), delta.shape[0],
              delta.stride(0), weight.data_ptr(), out.data_ptr(), _ptr(rows), n, h, float(eps),
              int(write_back and rows is None), int(bool(settled)), _stream())
        return
    _call(_fn("elementwise", _elem(out), "erb_add_rmsnorm"), hidden.data_ptr(), _ptr(delta), weight.data_ptr(),
          out.data_ptr(), _ptr(rows), n, h, float(eps), int(write_back and rows is None), int(bool(settled)), _stream())


def residual_add(hidden: torch.Tensor, delta: torch.Tensor, dtype: torch.dtype | None = None) -> None:
    """hidden += delta: rows of the model's element type, or float32 partial sums ``[parts, rows, width]``,
    which are added up and rounded to ``dtype`` (the model's element type) once, as ``add_rmsnorm`` does."""
    _need(hidden, "hidden", torch.float32); _need(delta, "delta")
    if delta.dim() == 3:
        _need(delta, "delta", torch.float32)
        if delta.shape[1:] != hidden.shape or dtype is None:
            raise KernelError("residual_add: partial sums need [parts, rows, width] and the element type to round to")
        _call(_fn("elementwise", _ELEM[dtype], "erb_residual_add_parts"), hidden.data_ptr(), delta.data_ptr(), delta.shape[0],
              delta.stride(0), hidden.numel(), _stream())
        return
    if hidden.shape != delta.shape:
        raise KernelError("residual_add: shapes disagree")
    _call(_fn("elementwise", _elem(delta), "erb_residual_add"), hidden.data_ptr(), delta.data_ptr(),
          hidden.numel(), _stream())


def resolve_ids(ids: torch.Tensor, fed: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> None:
    """Replace every id t < 0 of ``ids`` (int32, in place) by ``fed[-t - 1]``: tokens of the step
    before that are still on the device.  ``dtype`` only picks the library that holds the kernel
    (the engine's element type, so that nothing else has to be built)."""
    _need(ids, "ids", torch.int32); _need(fed, "fed", torch.int32)
    _call(_fn("elementwise", _ELEM[dtype], "erb_resolve_ids"), ids.data_ptr(), ids.numel(),
          fed.data_ptr(), fed.numel(), _stream())


def gather_cast(src: torch.Tensor, dst: torch.Tensor, rows: torch.Tensor | None) -> None:
    _need(src, "src", torch.float32); _need(dst, "dst"); _need(rows, "rows", torch.int32)
    _call(_fn("elementwise", _elem(dst), "erb_gather_cast"), src.data_ptr(), dst.data_ptr(), _ptr(rows),
          dst.shape[0], dst.shape[1], _stream())


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None,
                     n_q_heads: int, n_kv_heads: int, head_dim: int, rot_dim: int,
                     slots: torch.Tensor | None = None, k_pages: torch.Tensor | None = None,
                     v_pages: torch.Tensor | None = None, page_size: int = 0) -> None:
    """Rotate q (in place) and k by the halves convention; write rotated k and v to cache slots.

    ``k_pages``/``v_pages``: one layer's pages ``[n_pages, n_kv_heads, page_size, head_dim]``.
    ``slots``: int32 per token, ``page * page_size + offset`` or negative to write nothing.
    """
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(slots, "slots", torch.int32); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * head_dim or positions.numel() < n:
        raise KernelError("rope_cache_write: qkv width or positions disagree with the head counts")
    write = k_pages is not None
    if write:
        if v_pages is None or slots is None or slots.numel() < n:
            raise KernelError("rope_cache_write: cache write needs k_pages, v_pages and slots")
        if tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("rope_cache_write: page layout is not [pages, kv heads, page_size, head_dim]")
    if rot_dim and (inv_freq is None or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 values")
    _call(_fn("elementwise", _elem(qkv), "erb_rope_cache_write"), qkv.data_ptr(), positions.data_ptr(),
          _ptr(inv_freq), _ptr(slots), _ptr(k_pages), _ptr(v_pages), n, n_q_heads, n_kv_heads, head_dim,
          rot_dim, page_size, int(write), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter):
        raise KernelError("swiglu: gate_up must be [tokens, 2 * intermediate]")
    _call(_fn("elementwise", _elem(out), "erb_swiglu"), gate_up.data_ptr(), out.data_ptr(), n, inter, _stream())


# --- matrix products -------------------------------------------------------------------------

_workspaces: dict[int, torch.Tensor] = {}
WORKSPACE_BYTES = 64 << 20


def _workspace(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws


_set_status_word = None
_status_word: torch.Tensor | None = None     # where the tensor-core weight-streaming kernel reports
_status_word_told: int | None = None         # ... and what the library was last told


def linear_status_word(status: torch.Tensor | None) -> None:
    """Name the device word (int32) to which the TMA + tcgen05 weight-streaming kernel reports a wait
    that ran out (code 4000000 + block).  Kept until named again.  The library itself is told when it
    is next used (a model that never brings 17 to 64 rows to a large product never builds it)."""
    global _status_word
    if status is not None:
        _need(status, "status", torch.int32)
    _status_word = status


def _fn_tc(name: str):
    """A function of the tensor-core weight-streaming library, which first hears of the status word if it has changed."""
    global _set_status_word, _status_word_told
    fn = _fn("linear_tc", None, name)
    told = None if _status_word is None else _status_word.data_ptr()
    if told != _status_word_told:
        if _set_status_word is None:
            _set_status_word = fn._erb_lib.erb_linear_tc_set_status_word
            _set_status_word.argtypes = [c_void_p]
            _set_status_word.restype = c_int
        _set_status_word(told)
        _status_word_told = told
    return fn


def linear_few_rows_supported(a: torch.Tensor, weight: torch.Tensor, lda: int) -> bool:
    """Whether the weight-streaming kernel takes these operands (bfloat16, at most 64 rows, 16-byte rows)."""
    k = a.shape[1]
    return (a.dtype == torch.bfloat16 and a.shape[0] <= 64 and k % 8 == 0 and lda % 8 == 0
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_few_rows(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` through the weight-streaming kernel, for up to 64 rows."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_few_rows: shapes or strides disagree")
    if out.dtype not in (torch.bfloat16, torch.float32) or not linear_few_rows_supported(a, weight, lda):
        raise KernelError("linear_few_rows: operands not supported")
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, int(out.dtype == torch.float32), _stream())


def linear_tc(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` for up to 64 bfloat16 rows through the TMA + tcgen05 weight-streaming kernel."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_tc: shapes or strides disagree")
    if out.dtype not in (torch.bfloat16, torch.float32) or not linear_few_rows_supported(a, weight, lda):
        raise KernelError("linear_tc: operands not supported")
    _call(_fn_tc("erb_linear_tc"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, lda, k, ldo,
          int(out.dtype == torch.float32), _stream())


#: weights below this size stay with the library at 17 to 64 rows (measured at 64 rows: 960 x 960, 1.8 MB, 4.2 us in
#: parts against 3.4 us; 960 x 2560, 4.9 MB, 4.3 against 5.9 us; 2048 x 2048, 8.4 MB, 4.5 against 5.8 us)
PARTS_MIN_WEIGHT_ELEMENTS = 2 << 20


def linear_parts_count(a: torch.Tensor, weight: torch.Tensor) -> int:
    """How many partial results ``linear_parts`` leaves for ``a @ weight^T``, or 0 where the product is
    not taken in parts: it is for the bfloat16 rows of a decode step beyond the register kernel's
    (``SKINNY_MAX_ROWS`` < rows <= ``TC_MAX_ROWS``) against a weight with so few rows that whole tiles of
    them would leave most SMs without work (the attention output and the down projection)."""
    m, k = a.shape
    n = weight.shape[0]
    if not (SKINNY_MAX_ROWS < m <= TC_MAX_ROWS) or a.dtype != torch.bfloat16 or n % 4 or a.stride(1) != 1:
        return 0
    if not linear_few_rows_supported(a, weight, a.stride(0)) or -(-n // 128) * 2 > _sms(a.device):
        return 0
    if n * k < PARTS_MIN_WEIGHT_ELEMENTS:
        return 0
    return _parts_count(n, k)


def linear_parts_slices(weight: torch.Tensor) -> int:
    """The number of slices of k, and so of partial results, that ``linear_parts`` makes for this weight (a
    function of its shape alone)."""
    return _parts_count(weight.shape[0], weight.shape[1])


@functools.lru_cache(maxsize=256)
def _parts_count(n: int, k: int) -> int:
    return int(_fn_tc("erb_linear_tc_parts_count")(n, k))


def linear_parts(a: torch.Tensor, weight: torch.Tensor, parts: torch.Tensor) -> None:
    """``parts[s] = a[:, slice s of k] @ weight[:, slice s of k]^T`` in float32 for the
    ``linear_parts_slices`` slices of k; their sum in order is the product (``add_rmsnorm`` and
    ``residual_add`` take them as they are).  Up to ``TC_MAX_ROWS`` bfloat16 rows, n a multiple of 4."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(parts, "parts", torch.float32)
    m, k = a.shape
    n = weight.shape[0]
    if (weight.shape[1] != k or a.stride(1) != 1 or m > TC_MAX_ROWS or n % 4 or not linear_few_rows_supported(a, weight, a.stride(0))
            or tuple(parts.shape) != (linear_parts_slices(weight), m, n)):
        raise KernelError("linear_parts: shapes disagree or the operands are not supported")
    _call(_fn_tc("erb_linear_tc_parts"), a.data_ptr(), weight.data_ptr(), parts.data_ptr(), m, n, k, a.stride(0), k, n,
          _stream())


def linear_tc_glu(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear_glu`` through the TMA + tcgen05 kernel."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    m, k = a.shape
    n = weight.shape[0] // 2
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1 or not linear_glu_supported(a, weight, 64):
        raise KernelError("linear_tc_glu: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    _call(_fn_tc("erb_linear_tc_glu"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, lda, k, ldo,
          _stream())


def linear_tc_rope_store(a: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                         inv_freq: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int) -> None:
    """``linear_rope_store`` through the TMA + tcgen05 kernel (head sizes 32, 64, 128)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(slots, "slots", torch.int32)
    _need(k_pages, "k_pages", torch.bfloat16); _need(v_pages, "v_pages", torch.bfloat16)
    m, k = a.shape
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    if (weight.shape != (width, k) or qkv.shape != (m, width) or a.stride(1) != 1 or qkv.stride(1) != 1
            or positions.numel() < m or slots.numel() < m or inv_freq.numel() != head_dim // 2
            or k_pages.shape[1:] != (n_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape
            or head_dim not in (32, 64, 128) or not linear_rope_store_supported(a, weight, head_dim, head_dim, 64)):
        raise KernelError("linear_tc_rope_store: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = qkv.stride(0) if m > 1 else max(width, qkv.stride(0))
    _call(_fn_tc("erb_linear_tc_rope"), a.data_ptr(), weight.data_ptr(), qkv.data_ptr(), m, k, lda, k, ldo,
          n_q_heads, n_kv_heads, head_dim, positions.data_ptr(), inv_freq.data_ptr(), slots.data_ptr(),
          k_pages.data_ptr(), v_pages.data_ptr(), page_size, _stream())


def linear_glu_supported(a: torch.Tensor, weight: torch.Tensor, max_rows: int = SKINNY_MAX_ROWS) -> bool:
    """Whether the gated products take these operands: a handful of bfloat16 rows (``max_rows``: 16 where
    the register-fed kernel is the better choice, up to 64 for the kernels' own limit), 16-byte rows."""
    lda = a.stride(0) if a.shape[0] > 1 else max(a.shape[1], a.stride(0))
    return a.shape[0] <= max_rows and weight.shape[0] % 2 == 0 and linear_few_rows_supported(a, weight, lda)


def linear_glu(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = silu(a @ gate^T) * (a @ up^T) for ``weight = [gate; up]`` of shape [2N, K], in one
    launch; equal to ``linear`` into an [M, 2N] buffer followed by ``swiglu`` (each product is rounded
    to bfloat16 before the gate)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    m, k = a.shape
    n = weight.shape[0] // 2
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1 or not linear_glu_supported(a, weight, 64):
        raise KernelError("linear_glu: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny_glu"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, _stream())


def linear_rope_store_supported(a: torch.Tensor, weight: torch.Tensor, head_dim: int, rot_dim: int,
                                max_rows: int = SKINNY_MAX_ROWS) -> bool:
    """Whether the products with the rotary epilogue take these operands: a handful of bfloat16 rows
    (``max_rows`` as for ``linear_glu_supported``), full rotation, head sizes in steps of 16."""
    lda = a.stride(0) if a.shape[0] > 1 else max(a.shape[1], a.stride(0))
    return (a.shape[0] <= max_rows and rot_dim == head_dim and head_dim % 16 == 0
            and linear_few_rows_supported(a, weight, lda))


def linear_rope_store(a: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                      inv_freq: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: torch.Tensor,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int) -> None:
    """``linear(a, [Wq; Wk; Wv], qkv)`` followed by ``rope_cache_write`` in one launch, for a few rows:
    rotated q lands in ``qkv``'s q columns (its k and v columns are left as they are), rotated k and
    v in the tokens' cache slots.  Same bits as the two kernels."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(slots, "slots", torch.int32)
    _need(k_pages, "k_pages", torch.bfloat16); _need(v_pages, "v_pages", torch.bfloat16)
    m, k = a.shape
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    if (weight.shape != (width, k) or qkv.shape != (m, width) or a.stride(1) != 1 or qkv.stride(1) != 1
            or positions.numel() < m or slots.numel() < m or inv_freq.numel() != head_dim // 2
            or k_pages.shape[1:] != (n_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape
            or not linear_rope_store_supported(a, weight, head_dim, head_dim, 64)):
        raise KernelError("linear_rope_store: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = qkv.stride(0) if m > 1 else max(width, qkv.stride(0))
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny_rope"), a.data_ptr(), weight.data_ptr(), qkv.data_ptr(), m, k,
          lda, k, ldo, n_q_heads, n_kv_heads, head_dim, positions.data_ptr(), inv_freq.data_ptr(), slots.data_ptr(),
          k_pages.data_ptr(), v_pages.data_ptr(), page_size, _stream())


LINEAR_TUNE_FROM_ROWS = 1024     # rows from which the library's proposals for a shape are timed (as in csrc/gemm.cu)


def linear_tune(dtype: torch.dtype, on: bool) -> None:
    """Switch trials of the library's proposals on or off for the library products (of this element type) that
    follow: while on, a shape of ``LINEAR_TUNE_FROM_ROWS`` rows or more that has had no trial yet gets one
    (every proposal timed on the caller's operands with the weights from DRAM; the fastest stays for the
    process).  A trial costs as much as several steps: it is for a run whose shapes will be used many
    times more, such as the run before a step's layout is captured into a CUDA graph."""
    _fn("gemm", _ELEM[dtype], "erb_linear_tune")(int(bool(on)))


def linear_trials(dtype: torch.dtype) -> int:
    """How many product shapes (of this element type) have had a trial in this process."""
    return int(_fn("gemm", _ELEM[dtype], "erb_linear_trials")())


def linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           library: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ weight[N, K]^T (float accumulation, no TF32).  bfloat16 rows of a
    decode step go through this package's weight-streaming kernels: up to ``SKINNY_MAX_ROWS`` rows the
    register-fed one, up to ``TC_MAX_ROWS`` rows the TMA + tcgen05 one where the product has enough
    rows of w to give every SM a block without a split over k (the output head).  Within each of the
    two a row's bits do not depend on how many other rows the step has.  Everything else, or all with
    ``library=True``, is a library product.

    ``a`` and ``out`` may be row-strided views (last dimension contiguous); ``out`` is float or the
    element type of ``a``.
    """
    _need(a, "a", contiguous=False); _need(weight, "weight", a.dtype); _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear: shapes or strides disagree")
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError("linear: out must be float32 or the input type")
    if m == 0:
        return
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if m <= TC_MAX_ROWS and not accumulate and not library and linear_few_rows_supported(a, weight, lda):
        if m <= SKINNY_MAX_ROWS:
            # a handful of rows: this package's weight-streaming kernel instead of the library product
            _call(_fn("gemm", "bfloat16", "erb_linear_skinny"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
                  lda, k, ldo, int(out.dtype == torch.float32), _stream())
            return
        if n >= 128 * 2 * _sms(a.device):
            _call(_fn_tc("erb_linear_tc"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
                  lda, k, ldo, int(out.dtype == torch.float32), _stream())
            return
    ws = _workspace(a.device)
    _call(_fn("gemm", _elem(a), "erb_linear"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, int(out.dtype == torch.float32), int(accumulate), ws.data_ptr(), ws.numel(), _stream())


# --- attention -------------------------------------------------------------------------------

DECODE_SPLIT_KEYS = 512

def attention_rows(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                   seq_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                   scale: float, window: int = 0) -> None:
    """Causal attention of every token over its sequence's pages (general kernel, any portion sizes).

    ``q``: ``[tokens, >= n_q_heads * D]`` view with unit inner stride (the q part of a qkv buffer);
    ``out``: ``[tokens, n_q_heads * D]``; pages ``[n_pages, n_kv_heads, page_size, D]``;
    ``block_tables`` int32 ``[sequences, max_pages]``.
    """
    _need(q, "q", contiguous=False); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(block_tables, "block_tables", torch.int32); _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32); _need(out, "out", q.dtype, contiguous=False)
    n = q.shape[0]
    _, nkv, page_size, d = k_pages.shape
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < n_q_heads * d or out.shape[1] < n_q_heads * d:
        raise KernelError("attention_rows: q/out layout disagrees with the head counts")
    _call(_fn("attention", _elem(q), "erb_attention_rows"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], seq_of_token.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), n, n_q_heads, nkv, d, page_size, int(window),
          float(scale), _stream())


_sm_counts: dict[int, int] = {}


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch._C._cuda_getDevice()
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def choose_decode_split(n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int = 64) -> int:
    """Keys per split for the decode kernels (see ``_choose_decode_split``; answers are remembered)."""
    return _choose_decode_split(torch._C._cuda_getDevice(), n_seqs, n_kv_heads, max_keys, page_size, head_dim)


@functools.lru_cache(maxsize=4096)
def _choose_decode_split(device: int, n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int) -> int:
    """Keys per split for the decode kernels, from 128 to 2048.

    The bulk kernel runs one block per (sequence, group of neighbouring kv heads, split), two blocks per SM.
    Measured on the decode step (24 layers, contexts of 8,192, batches of 1 to 16): best is the
    largest split that still fills most of one wave of blocks; a little more than one wave is worst
    (the few blocks of the second wave stream alone, far below the memory's bandwidth); from about
    two waves on, the largest such split, but no more than 1024 keys once there are many waves.  A function of the batch's size and of a power-of-two
    bound on its longest context only, so an eager step and a captured one make the same choice.
    """
    sms = _sm_counts.get(device)
    if sms is None:
        sms = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    slots = 2 * sms
    if head_dim in (32, 64, 128):    # the sizes of the bulk-copy kernels: blocks per sequence and split as they group heads
        groups = native.load("attention_tc", None).erb_attention_decode_bulk_groups(n_kv_heads, head_dim, page_size, 512)
    else:                            # the general kernel (and no need to build the other library for it)
        groups = n_kv_heads
    fits = [s for s in (2048, 1024, 512, 256, 128) if s % page_size == 0 or page_size % s == 0]
    if not fits:
        return DECODE_SPLIT_KEYS
    blocks = {s: n_seqs * groups * -(-max_keys // s) for s in fits}
    for s in fits:                       # most of one wave
        if 0.6 * slots <= blocks[s] <= slots:
            return s
    for s in fits:                       # well beyond one wave: splits of 2048 only up to two waves (measured)
        if blocks[s] >= 1.7 * slots and (s <= 1024 or blocks[s] <= 2 * slots):
            return s
    return fits[-1] if blocks[fits[-1]] < slots else min(fits, key=lambda s: abs(blocks[s] - slots))


def context_bound(pages: int) -> tuple[int, int]:
    """(bound, granule) in pages for a batch whose longest context has ``pages`` pages: the bound is
    ``pages`` rounded up to a multiple of the granule, a quarter of the power-of-two bucket it lies in
    (at least 4 pages).  Steps that share a bound share launch shapes (and a captured graph); the
    longest context then lies within one granule below the bound."""
    bucket = max(4, 1 << (max(1, pages) - 1).bit_length())
    granule = max(1, bucket // 4)
    return -(-max(1, pages) // granule) * granule, granule


def choose_decode_plan(n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int = 64,
                       grouped: bool = False, granule: int = 0) -> tuple[int, int]:
    """(keys per split, kv heads per block) for a decode step whose longest context lies in
    (``max_keys`` - ``granule``, ``max_keys``]; heads per block 0 means the kernel's own choice.
    ``grouped``: the kernel for several query heads per kv head runs, which groups by itself."""
    if grouped or head_dim not in (32, 64, 128):
        return choose_decode_split(n_seqs, n_kv_heads, max_keys, page_size, head_dim), 0
    return _choose_decode_plan(torch._C._cuda_getDevice(), n_seqs, n_kv_heads, max_keys, page_size, head_dim,
                               granule if granule > 0 else max_keys)


@functools.lru_cache(maxsize=4096)
def _choose_decode_plan(device: int, n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int,
                        granule: int) -> tuple[int, int]:
    """The bulk kernel runs one block per (sequence, group of kv heads, split), two blocks per SM.  By
    default it groups as many neighbouring heads as make a page's copy about 8 KB, which long contexts
    and large batches need for bandwidth; a small batch or a short context then gives far fewer blocks
    than SMs, each walking through many stages one after the other.  Measured with caches read from
    DRAM (batches of 1 to 64, contexts of 640 to 8,192): best is the plan with the fewest heads per
    block (from 2) and then the longest splits whose blocks fill most of one wave, e.g. 16 sequences
    of 640 tokens 15 us with 2 heads per block and no split against 23 us with 8 heads and splits of
    256; where no such plan exists the rule of ``_choose_decode_split`` with the default grouping
    stands (it is as good for 8 sequences of 8,192 tokens and better beyond).  Splits are either at
    most a granule long or hold the whole context: a split between the two leaves the longest
    context with one full split and a short rest, and the step waits for the full one (8 sequences
    of 640 tokens: 1.53 ms a step with splits of 512, 1.46 ms with splits of 256).  A function of the
    batch's size and of the bound on the longest context only."""
    split = _choose_decode_split(device, n_seqs, n_kv_heads, max_keys, page_size, head_dim)
    lib = native.load("attention_tc", None)
    default = lib.erb_attention_decode_bulk_head_group(n_kv_heads, head_dim, page_size, 512, 0)
    slots = 2 * _sm_counts[device]
    sizes = [s for s in (2048, 1024, 512, 256, 128, 64)
             if s % page_size == 0 and -(-max_keys // s) <= 64 and (s <= granule or s >= max_keys)]
    finest = None
    for hg in (2, 4, 8):
        if hg > default:
            break
        for s in sizes:
            if lib.erb_attention_decode_bulk_head_group(n_kv_heads, head_dim, page_size, s, hg) != hg:
                continue
            blocks = n_seqs * -(-n_kv_heads // hg) * -(-max_keys // s)
            if 0.6 * slots <= blocks <= slots:
                return s, hg
            if hg == 2:
                finest = (s, hg, blocks)
    if finest is not None and finest[2] < 0.6 * slots:       # even the finest plan leaves SMs idle: take it
        return finest[0], finest[1]
    return split, 0


def decode_scratch_floats(n_seqs: int, n_q_heads: int, head_dim: int, max_splits: int) -> tuple[int, int]:
    return n_seqs * n_q_heads * max_splits * head_dim, n_seqs * n_q_heads * max_splits * 2


def attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                     token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                     scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                     window: int = 0, split_keys: int = DECODE_SPLIT_KEYS) -> None:
    """Attention of one new token per sequence, keys cut into splits of ``split_keys`` (split-KV).

    ``token_of_seq`` int32 ``[sequences]`` gives each sequence's row in q/out/positions.  Scratch:
    ``part_acc`` float ``[sequences * heads * max_splits * D]``, ``part_ml`` twice
    ``sequences * heads * max_splits``.
    """
    _need(q, "q", contiguous=False); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(block_tables, "block_tables", torch.int32); _need(token_of_seq, "token_of_seq", torch.int32)
    _need(positions, "positions", torch.int32); _need(out, "out", q.dtype, contiguous=False)
    _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
    n_seqs = token_of_seq.numel()
    _, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError("attention_decode: scratch too small")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode: q/out inner stride must be 1")
    _call(_fn("attention", _elem(q), "erb_attention_decode"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(),
          max_splits, n_seqs, n_q_heads, nkv, d, page_size, int(window), int(split_keys), float(scale), _stream())


def decode_bulk_supported(dtype: torch.dtype, head_dim: int, window: int, n_q_heads: int, n_kv_heads: int,
                          max_splits: int = 1) -> bool:
    """Shapes the bulk-copy decode kernel takes; everything else goes to the general decode kernel."""
    return (dtype == torch.bfloat16 and head_dim in (32, 64, 128) and window <= 0
            and n_q_heads // n_kv_heads <= 8 and max_splits <= 64)


_split_counters: dict[torch.device, torch.Tensor] = {}


def split_counters(device: torch.device, n: int) -> torch.Tensor:
    """The counters by which the split decode kernels find the block that finishes last for each
    (sequence, group of kv heads): one zeroed int32 array per device, shared by all calls (calls on
    one stream follow each other; the kernels leave every counter at zero).  It keeps its address, so
    that captured graphs stay valid."""
    buf = _split_counters.get(device)
    if buf is None:
        buf = _split_counters[device] = torch.zeros(1 << 18, dtype=torch.int32, device=device)
    if n > buf.numel():
        raise KernelError(f"decode attention: {n} (sequence, head group) pairs, at most {buf.numel()}")
    return buf


def reset_split_counters() -> None:
    """Zeroes the counters again: needed after a kernel gave up on a wait (a flagged status), since
    its block did not count."""
    for buf in _split_counters.values():
        buf.zero_()


def attention_decode_bulk(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                          token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                          scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                          status: torch.Tensor, split_keys: int = DECODE_SPLIT_KEYS, head_group: int = 0) -> None:
    """``attention_decode`` for bfloat16 with keys and values streamed by bulk asynchronous copies.
    The splits of a sequence are merged by the block that finishes last (``split_counters``), so
    this is one launch.  ``head_group``: kv heads per block (a power of two; 0: as many as make a
    page's copy about 8 KB)."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(token_of_seq, "token_of_seq", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(part_acc, "part_acc", torch.float32)
    _need(part_ml, "part_ml", torch.float32); _need(status, "status", torch.int32)
    n_seqs = token_of_seq.numel()
    _, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError("attention_decode_bulk: scratch too small")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode_bulk: q/out inner stride must be 1")
    _call(_fn("attention_tc", None, "erb_attention_decode_bulk"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(), max_splits,
          n_seqs, n_q_heads, nkv, d, page_size, int(split_keys), float(scale), status.data_ptr(),
          split_counters(q.device, n_seqs * nkv).data_ptr(), int(head_group), _stream())


@functools.lru_cache(maxsize=4096)
def decode_gqa_supported(dtype: torch.dtype, head_dim: int, window: int, n_q_heads: int, n_kv_heads: int,
                         page_size: int, split_keys: int, max_splits: int = 1) -> bool:
    """Shapes the tensor-core decode kernel for grouped query heads takes: bfloat16, head size 64,
    2 to 8 query heads per kv head, pages of a multiple of 8 tokens, no window."""
    if dtype != torch.bfloat16 or window > 0 or max_splits > 64 or head_dim != 64 or n_q_heads == n_kv_heads:
        return False        # (answered here so that other models need not build the tensor-core library)
    return bool(native.load("attention_tc", None).erb_attention_decode_gqa_supported(
        n_q_heads, n_kv_heads, head_dim, page_size, int(split_keys)))


def attention_decode_gqa(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                         token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                         scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                         status: torch.Tensor, split_keys: int = DECODE_SPLIT_KEYS) -> None:
    """``attention_decode`` for several query heads per kv head on tensor cores: the query heads of a
    kv head are the rows of one matrix tile, pages arrive by TMA tensor copies."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(token_of_seq, "token_of_seq", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(part_acc, "part_acc", torch.float32)
    _need(part_ml, "part_ml", torch.float32); _need(status, "status", torch.int32)
    n_seqs = token_of_seq.numel()
    n_pages, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or v_pages.shape != k_pages.shape:
        raise KernelError("attention_decode_gqa: scratch too small or pools disagree")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode_gqa: q/out inner stride must be 1")
    _call(_fn("attention_tc", None, "erb_attention_decode_gqa"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), n_pages, block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(), max_splits,
          n_seqs, n_q_heads, nkv, d, page_size, int(split_keys), float(scale), status.data_ptr(),
          split_counters(q.device, n_seqs * nkv).data_ptr(), _stream())


#: query rows of one (sequence, head) that a block of the tensor-core prefill kernel takes
PREFILL_TC_ROWS = 256


def prefill_tc_supported(dtype: torch.dtype, head_dim: int, window: int, page_size: int = 16) -> bool:
    """Shapes the tensor-core prefill kernel takes (bfloat16, head size 64, no window, pages of 8 to
    128 tokens, a power of two); everything else goes to the general row kernel."""
    return (dtype == torch.bfloat16 and head_dim == 64 and window <= 0
            and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0)


def prefill_tc_blocks(q_lens) -> int:
    """Blocks per head the tensor-core prefill kernel needs for portions of these lengths."""
    return sum(-(-int(n) // PREFILL_TC_ROWS) for n in q_lens)


def prefill_tc_key_splits(n_blocks: int, n_q_heads: int, max_keys: int, device: torch.device) -> int:
    """Ranges to cut every block's keys into: 1 unless the portions give far fewer blocks than the GPU has
    SMs and the walk over the keys is long (512 new tokens after 7,000 cached ones: 30 to 64 blocks of
    59 key tiles each take 131 us whatever their number; cut so that the blocks fill one wave, 4 tiles
    a range at least).  ``max_keys``: a bound on the longest context that steps of one layout share."""
    sms = _sms(device)
    blocks = n_blocks * n_q_heads
    tiles = -(-max_keys // 128)
    if blocks * 2 > sms or tiles < 8:
        return 1
    return max(1, min(sms // blocks, tiles // 4, 16))


def prefill_tc_scratch_floats(n_rows: int, n_q_heads: int, key_splits: int) -> tuple[int, int]:
    """Floats of ``part_o`` and ``part_ml`` for ``attention_prefill_tc`` with key splits over the first ``n_rows`` rows of the batch."""
    return n_rows * n_q_heads * key_splits * 64, n_rows * n_q_heads * key_splits * 2


def attention_prefill_tc(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                         seq_starts: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_blocks: int,
                         n_q_heads: int, scale: float, status: torch.Tensor, key_splits: int = 1, first_row: int = 0,
                         part_o: torch.Tensor | None = None, part_ml: torch.Tensor | None = None) -> None:
    """Causal attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 64, no window).

    ``qkv`` / ``out``: row t is token t of the batch (the q heads lead each qkv row);
    ``seq_starts`` int32 ``[n + 1]``: token offsets of the n sequences to process, whose block tables
    are the n rows of ``block_tables``; ``n_blocks``: ``prefill_tc_blocks`` of their lengths (an upper
    bound is fine).  ``key_splits`` > 1 (``prefill_tc_key_splits``): every block's keys are cut into
    that many ranges, each a block of its own, and a second kernel merges them; the sequences'
    tokens are then rows ``first_row`` to the end of ``qkv``, and ``part_o`` / ``part_ml`` are float
    scratch of ``prefill_tc_scratch_floats(qkv rows, heads, key_splits)``.
    """
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(seq_starts, "seq_starts", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(status, "status", torch.int32)
    n_pages, nkv, page_size, d = k_pages.shape
    n_seqs = seq_starts.numel() - 1
    if qkv.stride(1) != 1 or out.stride(1) != 1 or block_tables.shape[0] < n_seqs or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill_tc: layout disagrees")
    if key_splits > 1:
        _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
        need_o, need_ml = prefill_tc_scratch_floats(qkv.shape[0], n_q_heads, key_splits)
        if part_o is None or part_ml is None or part_o.numel() < need_o or part_ml.numel() < need_ml or not 0 <= first_row < qkv.shape[0]:
            raise KernelError("attention_prefill_tc: scratch for the key ranges is missing or too small")
    _call(_fn("attention_prefill", None, "erb_attention_prefill_tc"), qkv.data_ptr(), qkv.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), n_pages, block_tables.data_ptr(), block_tables.shape[1], seq_starts.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), n_seqs, int(n_blocks), n_q_heads, nkv, d, page_size,
          float(scale), status.data_ptr(), int(key_splits), int(first_row), qkv.shape[0] - int(first_row), _ptr(part_o), _ptr(part_ml),
          _stream())
    if key_splits > 1:
        launch_counts["own"] += 1          # the merge of the ranges


# --- sampling --------------------------------------------------------------------------------

def sample_rows(logits: torch.Tensor, tokens: torch.Tensor, temperature: torch.Tensor | None = None,
                rng_state: torch.Tensor | None = None) -> None:
    """tokens[r] = argmax(logits[r]) where temperature[r] <= 0, else an inverse-CDF draw."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(tokens, "tokens", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(rng_state, "rng_state", torch.int64)
    if logits.stride(1) != 1 or tokens.numel() < logits.shape[0]:
        raise KernelError("sample_rows: layout disagrees")
    _call(_fn("sampling", None, "erb_sample_rows"), logits.data_ptr(), logits.stride(0) if logits.shape[0] > 1 else max(logits.stride(0), logits.shape[1]),
          logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(rng_state), tokens.data_ptr(), _stream())


def uniform_from_state(state: int) -> float:
    """The uniform in [0, 1) that the sampling kernel derives from a 64-bit state (host copy)."""
    z = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z ^= z >> 31
    return (z >> 40) / 16777216.0
