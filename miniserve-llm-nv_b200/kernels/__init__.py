"""ctypes bindings of the CUDA library: one Python function per kernel entry point.

Every function takes CUDA tensors, checks types, shapes and contiguity on the host,
launches on torch's current stream and returns nothing (outputs are arguments).  There
is no CPU path: a call with a CPU tensor, or on a machine where the library cannot be
built or loaded, raises.
"""

from __future__ import annotations

import ctypes
import logging
from typing import Optional

import torch

from . import build

ABI_VERSION = 5
log = logging.getLogger("miniserve_b200")
_library: Optional[ctypes.CDLL] = None

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def library() -> ctypes.CDLL:
    """The loaded CUDA library (built on first use)."""
    global _library
    if _library is None:
        path = build.library_path()
        lib = ctypes.CDLL(str(path))
        lib.ms_last_error.restype = ctypes.c_char_p
        lib.ms_abi_version.restype = ctypes.c_int
        if lib.ms_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} reports ABI {lib.ms_abi_version()}, bindings expect {ABI_VERSION}; rebuild it")
        # argument and result types from the prototypes in the sources: calls then pass plain Python numbers
        kinds = {"pointer": ctypes.c_void_p, "int": ctypes.c_int, "float": ctypes.c_float, "longlong": ctypes.c_longlong,
                 "string": ctypes.c_char_p, "void": None}
        for name, (result, arguments) in build.exported_signatures().items():
            function = getattr(lib, name)
            function.restype = kinds[result]
            function.argtypes = [kinds[a] for a in arguments]
        _library = lib
    return _library


launch_count = 0   # entry points of this library called so far (each launches one kernel, or a fixed few)


def _check(code: int) -> None:
    global launch_count
    if code != 0:
        raise KernelError(library().ms_last_error().decode())
    launch_count += 1


_device_index: Optional[int] = None


def _stream() -> int:
    """torch's current stream on the library's device (the raw handle: this is called for every launch)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(_device_index)


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The tensor's address (None: a null pointer); the entry points' argument types are known to ctypes."""
    return None if tensor is None else tensor.data_ptr()


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)") from None


def _want(tensor: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if (tensor.is_cuda and tensor.is_contiguous() and (dtype is None or tensor.dtype is dtype)
            and (shape is None or tensor.shape == shape)):
        return                      # (one test for the usual case; what follows words the refusal)
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


_i = int        # (arguments are converted by ctypes from the prototypes' types; these only coerce)
_f = float


# --------------------------------------------------------------------------- memory-bound kernels


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out[n] = scale * float32(table[tokens[n]])``; tokens int32 ``[N]``, out float32 ``[N, H]``."""
    n, hidden = tokens.numel(), table.shape[1]
    _want(tokens, "tokens", torch.int32)
    _want(table, "table")
    _want(out, "out", torch.float32, (n, hidden))
    _check(library().ms_embedding(_ptr(tokens), _ptr(table), _i(_code(table.dtype)), _ptr(out), _i(n), _i(hidden),
                                  _f(scale), _stream()))


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: Optional[float] = None) -> None:
    """In place on float32 ``x``: ``x *= scale``, then with ``cap``: ``x = cap * tanh(x / cap)``."""
    _want(x, "x", torch.float32)
    _check(library().ms_scale_softcap(_ptr(x), x.numel(), _f(scale), _f(cap if cap else 0.0), _stream()))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """Adds ``delta`` into the float32 ``residual`` (in place) and writes its RMSNorm to ``out``.

    With ``rows`` (int32 ``[K]``) only those rows are normalised, into ``out [K, H]``, and
    the residual is left untouched.  ``weight`` may be float32 or bfloat16 whatever ``out`` is.
    """
    hidden = residual.shape[1]
    n_out = residual.shape[0] if rows is None else rows.numel()
    _want(residual, "residual", torch.float32)
    _want(out, "out", None, (n_out, hidden))
    _want(weight, "weight", None, (hidden,))
    if delta is not None:
        _want(delta, "delta", out.dtype, residual.shape)
    if rows is not None:
        _want(rows, "rows", torch.int32)
    _check(library().ms_add_rmsnorm(_ptr(residual), _ptr(delta), _i(_code(out.dtype)), _ptr(weight),
                                    _i(_code(weight.dtype)), _ptr(rows), _ptr(out), _i(n_out), _i(hidden), _f(eps),
                                    _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """RMSNorm over the last dim of ``x [rows, size]`` into ``out`` of the same type and shape."""
    _want(x, "x")
    _want(out, "out", x.dtype, x.shape)
    size = x.shape[-1]
    _want(weight, "weight", None, (size,))
    _check(library().ms_rmsnorm(_ptr(x), _i(_code(x.dtype)), _ptr(weight), _i(_code(weight.dtype)), _ptr(out),
                                _i(x.numel() // size), _i(size), _f(eps), _stream()))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos_sin: torch.Tensor) -> None:
    """``cos_sin[n, j] = (cos, sin)(positions[n] * inv_freq[j])`` in float32; cos_sin ``[N, half, 2]``."""
    n, half = positions.numel(), inv_freq.numel()
    _want(positions, "positions", torch.int32)
    _want(inv_freq, "inv_freq", torch.float32)
    _want(cos_sin, "cos_sin", torch.float32, (n, half, 2))
    _check(library().ms_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(cos_sin), _i(n), _i(half), _stream()))


def qk_norm_rope_append(qkv: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                        rotary_dim: int, interleaved: bool, k_pool: torch.Tensor, v_pool: torch.Tensor,
                        n_q: int, n_kv: int, head_dim: int, q_out: torch.Tensor) -> None:
    """Per-head RMSNorm of q and k, rotation, and the append of k and v to one layer's pools.

    qkv ``[N, (n_q + 2 n_kv) * d]``; slots int32 ``[N]`` (page * page_size + offset, negative:
    no write); pools ``[pages, n_kv, page_size, d]``; q_out ``[N, n_q, d]``; cos_sin float32
    ``[N, rotary_dim / 2, 2]`` or None for no rotation; norm weights ``[d]`` or None.
    """
    n = qkv.shape[0]
    _want(qkv, "qkv", None, (n, (n_q + 2 * n_kv) * head_dim))
    _want(slots, "slots", torch.int32, (n,))
    _want(k_pool, "k_pool", qkv.dtype)
    _want(v_pool, "v_pool", qkv.dtype, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {head_dim}]")
    _want(q_out, "q_out", qkv.dtype, (n, n_q, head_dim))
    weight_code = 0
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _want(weight, name, None, (head_dim,))
            weight_code = _code(weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, rotary_dim // 2, 2))
    else:
        rotary_dim = 0
    _check(library().ms_qk_norm_rope_append(
        _ptr(qkv), _i(_code(qkv.dtype)), _ptr(slots), _ptr(q_weight), _ptr(k_weight), _i(weight_code), _f(eps),
        _ptr(cos_sin), _i(rotary_dim), _i(1 if interleaved else 0), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[2]),
        _i(n_q), _i(n_kv), _i(head_dim), _ptr(q_out), _i(n), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False) -> None:
    """``out[n, c] = silu(gate_up[n, c]) * gate_up[n, I + c]`` for gate_up ``[N, 2 I]``.

    ``paired``: the columns come as :func:`interleave_gate_up` orders a weight's rows (eight gate columns, then
    the up columns of the same features, and so on): ``out[n, 8 j + r] = silu(gate_up[n, 16 j + r]) *
    gate_up[n, 16 j + 8 + r]``.
    """
    n, inter = out.shape
    _want(gate_up, "gate_up", None, (n, 2 * inter))
    _want(out, "out", gate_up.dtype)
    _check(library().ms_silu_mul(_ptr(gate_up), _i(_code(gate_up.dtype)), _ptr(out), _i(n), _i(inter),
                                 _i(1 if paired else 0), _stream()))


# --------------------------------------------------------------------------- attention

MAX_HEAD_DIM = 512      # of the general attention kernel (attention_generic.cu: 16 output lanes per thread)


def attention_kernels(dtype: torch.dtype, head_dim: int, n_q: int, n_kv: int, page_size: int,
                      modified_scores: bool = False) -> dict:
    """Which kernel :func:`paged_attention` runs for these sizes: ``{"decode": name, "prompt": name}`` with the
    names ``tcgen05``, ``mma.sync`` and ``general`` (float32 arithmetic, any size; the only one of the float32
    path, and what bfloat16 falls back to for head sizes the tensor-core kernels are not built for and for
    scores with a soft cap or a distance bias)."""
    lib = library()
    if modified_scores or dtype != torch.bfloat16 or not lib.ms_attention_mma_supports(_i(head_dim)):
        return {"decode": "general", "prompt": "general"}
    prompt = "mma.sync"
    if USE_TCGEN05_ATTENTION and lib.ms_attention_tcgen05_supports(_i(head_dim), _i(n_q), _i(n_kv), _i(page_size)):
        prompt = "tcgen05"
    return {"decode": "mma.sync", "prompt": prompt}



def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                    request_of_token: torch.Tensor, positions: torch.Tensor, query_start: torch.Tensor,
                    context_lens: torch.Tensor, max_query_len: int, max_context_len: int, scale: float,
                    window: Optional[int], out: torch.Tensor, host_query_start: Optional[list] = None,
                    softcap: Optional[float] = None, bias_slopes: Optional[torch.Tensor] = None) -> None:
    """Causal grouped-query attention of every token over its request's paged keys and values.

    q, out ``[N, n_q, d]``; pools of one layer ``[pages, n_kv, page_size, d]``; block_tables
    int32 ``[R, width]``; request_of_token, positions int32 ``[N]``; query_start ``[R + 1]`` and
    context_lens ``[R]`` describe the same batch per request (a request's tokens are the last
    ones of its context).  A token at position p sees keys ``max(0, p - window + 1) .. p`` of
    its own request, which must be in the pool already.

    Score modifiers, both off by default: ``softcap`` turns a scaled score ``s`` into ``softcap * tanh(s /
    softcap)``; ``bias_slopes`` (float32 ``[n_q]``) adds ``slope[head] * (key position - query position)``
    after it.  The general kernel implements them; the tensor-core kernels do not, so a call with either
    runs the general kernel whatever the sizes.

    bfloat16 with a head size the tensor-core kernels are built for runs there
    (``max_query_len``/``max_context_len`` are upper bounds used to shape their grids); everything
    else runs the general float32-arithmetic kernel.  With ``host_query_start`` (the same numbers
    as ``query_start``, on the host) a batch that begins with single-token requests and goes on
    with prompt portions is run as two launches, so that the single tokens get their keys split
    over many thread blocks instead of one block walking a whole context.
    """
    n, n_q, head_dim = q.shape
    _want(q, "q")
    _want(out, "out", q.dtype, q.shape)
    _want(k_pool, "k_pool", q.dtype)
    _want(v_pool, "v_pool", q.dtype, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, n_kv, page_size, {head_dim}]")
    _want(block_tables, "block_tables", torch.int32)
    _want(request_of_token, "request_of_token", torch.int32, (n,))
    _want(positions, "positions", torch.int32, (n,))
    n_requests = context_lens.numel()
    _want(query_start, "query_start", torch.int32, (n_requests + 1,))
    _want(context_lens, "context_lens", torch.int32, (n_requests,))
    lib = library()
    n_kv = k_pool.shape[1]
    modified = bool(softcap) or bias_slopes is not None
    if bias_slopes is not None:
        _want(bias_slopes, "bias_slopes", torch.float32, (n_q,))
    if modified or q.dtype != torch.bfloat16 or not lib.ms_attention_mma_supports(_i(head_dim)):
        _check(lib.ms_paged_attention_generic(
            _ptr(q), _i(_code(q.dtype)), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _i(block_tables.shape[1]),
            _ptr(request_of_token), _ptr(positions), _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim),
            _f(scale), _i(window if window else 0), _f(softcap if softcap else 0.0), _ptr(bias_slopes), _ptr(out),
            _i(n), _stream()))
        return

    def run(first: int, last: int, longest: int, rows: int) -> None:
        """Requests first .. last - 1 (their tokens are found through query_start, which holds absolute rows);
        ``rows``: one past the last row of the batch that these requests own, which sizes the scratch of the
        key splits and the merge that follows them."""
        tables, starts, lens = block_tables[first:last], query_start[first:last + 1], context_lens[first:last]
        count = last - first
        group = n_q // n_kv
        if (USE_TCGEN05_ATTENTION and longest * group > 16
                and lib.ms_attention_tcgen05_supports(_i(head_dim), _i(n_q), _i(n_kv), _i(k_pool.shape[2]))):
            # prompt portions: the TMA + tcgen05 + tensor-memory kernel, its softmax groups taking the key tiles in
            # turn or working on each together
            entry = lib.ms_paged_attention_turns if ATTENTION_IN_TURNS else lib.ms_paged_attention_tcgen05
            _check(entry(
                _ptr(q), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[0]), _ptr(tables), _i(block_tables.shape[1]),
                _ptr(starts), _ptr(lens), _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale),
                _i(window if window else 0), _ptr(out), _i(count), _i(longest), _i(n),
                _ptr(device_error_flag(q.device)), _stream()))
            return
        splits = lib.ms_attention_mma_splits(_i(head_dim), _i(count), _i(n_kv), _i(n_q), _i(longest), _i(max_context_len))
        part_o = part_lse = None
        if splits > 1:
            part_o = torch.empty((rows * n_q * splits, head_dim), dtype=torch.float32, device=q.device)
            part_lse = torch.empty((rows * n_q * splits,), dtype=torch.float32, device=q.device)
        _check(lib.ms_paged_attention_mma(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(tables), _i(block_tables.shape[1]), _ptr(starts), _ptr(lens),
            _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale), _i(window if window else 0), _ptr(out),
            _ptr(part_o), _ptr(part_lse), _i(splits), _i(count), _i(longest), _i(rows), _stream()))

    leading_single = 0
    if host_query_start and max_query_len > 1 and len(host_query_start) == n_requests + 1:
        while (leading_single < n_requests
               and host_query_start[leading_single + 1] - host_query_start[leading_single] == 1):
            leading_single += 1
    if 0 < leading_single < n_requests:
        run(0, leading_single, 1, leading_single)      # single tokens are the batch's first rows, one each
        run(leading_single, n_requests, max_query_len, n)
    else:
        run(0, n_requests, max_query_len, n)


FUSED_DECODE_ATTENTION = __import__("os").environ.get("MINISERVE_B200_FUSED_DECODE_ATTENTION", "1") == "1"


# Steps of this many requests run :func:`decode_attention_fused` where it takes the sizes.  Measured at Qwen3-1.7B
# sizes, context 4,096 (ms per step with / without): 1 request 1.341 / 1.330, 2: 1.370 / 1.366, 4: 1.490 / 1.549,
# 8: 1.731 / 1.801, 16: 2.807 / 2.789, 64: 6.441 / 6.371.  With one or two requests there are few blocks and each
# repeats the queries' norm and rotation; with many the kernel's larger register count costs residency.
FUSED_DECODE_ROWS = (3, 8)


def decode_attention_fused_supported(dtype: torch.dtype, head_dim: int, n_q: int, n_kv: int) -> bool:
    """Whether :func:`decode_attention_fused` takes these sizes (bfloat16, head size 64 or 128, at most 16
    query heads per key/value head); MINISERVE_B200_FUSED_DECODE_ATTENTION=0 turns it off."""
    return bool(FUSED_DECODE_ATTENTION and dtype == torch.bfloat16
                and library().ms_attention_decode_fused_supports(_i(head_dim), _i(n_q), _i(n_kv)))


def decode_attention_fused_preferred(rows: int) -> bool:
    """Whether a step of ``rows`` single tokens is faster with :func:`decode_attention_fused` (see FUSED_DECODE_ROWS)."""
    return FUSED_DECODE_ROWS[0] <= rows <= FUSED_DECODE_ROWS[1]


def decode_attention_fused(qkv: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                           k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                           query_start: torch.Tensor, context_lens: torch.Tensor, max_context_len: int, scale: float,
                           window: Optional[int], n_q: int, n_kv: int, head_dim: int, out: torch.Tensor) -> None:
    """A decode step's attention for requests of ONE new token each, from the projection's output: what
    :func:`qk_norm_rope_append` followed by :func:`paged_attention` computes (per-head RMSNorm of q and k,
    half-split rotation over the whole head, the append of k and v at ``slots``, attention over the cache with the
    keys split over many blocks, and the merge of the splits), with the first of the three kernels folded into
    the second.  Arguments as there; ``cos_sin`` float32 ``[N, d / 2, 2]`` or None; ``max_context_len`` an upper
    bound that the split count is derived from."""
    n = qkv.shape[0]
    _want(qkv, "qkv", torch.bfloat16, (n, (n_q + 2 * n_kv) * head_dim))
    _want(slots, "slots", torch.int32, (n,))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != head_dim:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {head_dim}]")
    _want(out, "out", torch.bfloat16, (n, n_q, head_dim))
    _want(block_tables, "block_tables", torch.int32)
    _want(query_start, "query_start", torch.int32, (n + 1,))
    _want(context_lens, "context_lens", torch.int32, (n,))
    weight_code = 0
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _want(weight, name, None, (head_dim,))
            weight_code = _code(weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (n, head_dim // 2, 2))
    lib = library()
    splits = lib.ms_attention_decode_fused_splits(_i(head_dim), _i(n), _i(n_kv), _i(max_context_len))
    part_o = part_lse = None
    if splits > 1:
        part_o = torch.empty((n * n_q * splits, head_dim), dtype=torch.float32, device=qkv.device)
        part_lse = torch.empty((n * n_q * splits,), dtype=torch.float32, device=qkv.device)
    _check(lib.ms_attention_decode_fused(
        _ptr(qkv), _ptr(slots), _ptr(q_weight), _ptr(k_weight), _i(weight_code), _f(eps), _ptr(cos_sin), _ptr(k_pool),
        _ptr(v_pool), _ptr(block_tables), _i(block_tables.shape[1]), _ptr(query_start), _ptr(context_lens),
        _i(k_pool.shape[2]), _i(n_q), _i(n_kv), _i(head_dim), _f(scale), _i(window if window else 0), _ptr(out),
        _ptr(part_o), _ptr(part_lse), _i(splits), _i(n), _stream()))


# --------------------------------------------------------------------------- matrix products


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_stats: Optional["RowStats"] = None) -> None:
    """``out[M, N] = x[M, K] @ weight[N, K]^T``.  (``row_stats``: see :func:`linear_wide`; the caller has asked
    :func:`fold_supported` first.)

    float32 operands run through the library's own FFMA kernel (true 32-bit, no tensor-core
    mode).  bfloat16 operands go to cuBLAS through ``torch.mm`` with float32 accumulation;
    ``out`` may then be bfloat16 or float32.
    """
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or tuple(out.shape) != (m, n):
        raise KernelError(f"linear: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if row_stats is not None:
        if row_stats.per_row:
            linear_pair(x, weight, out, row_stats=row_stats)
        else:
            linear_wide(x, weight, out, row_stats=row_stats)
        return
    if x.dtype == torch.float32:
        _want(x, "x", torch.float32)
        _want(weight, "weight", torch.float32)
        _want(out, "out", torch.float32)
        _check(library().ms_gemm_f32(_ptr(x), _ptr(weight), _ptr(out), _i(m), _i(n), _i(k), _i(k), _i(k), _i(n),
                                     _stream()))
        return
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16)
    _want(out, "out")
    if m <= STREAM_MAX_ROWS and k % 8 == 0:
        # few rows (decode steps): one of the two weight-streaming kernels, or the library, by measurement
        choice = _few_rows_choice(x, weight, m)
        if choice == "stream":
            linear_stream(x, weight, out)
            return
        if choice == "skinny":
            _check(library().ms_gemm_skinny(_ptr(x), _i(0), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m),
                                            _i(n), _i(k), _stream()))
            return
        if choice == "wide":
            linear_wide(x, weight, out)
            return
    if k % 8 == 0 and out.dtype == torch.bfloat16 and pair_preferred(x.device, m, n):
        choice = _pair_or_library("plain", m, weight)
        if choice != "library":
            linear_pair(x, weight, out, wide=choice == "wide")
            return
    if USE_TCGEN05_GEMM and m >= 128 and k % 8 == 0:
        linear_tcgen05(x, weight, out)
        return
    if out.dtype == torch.bfloat16:
        torch.mm(x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)


# Products of many rows (prompt portions).  The kernel in which two thread blocks share a 256 x 256 tile
# (linear_pair) is level with cuBLAS where its tiles fill the pairs of multiprocessors (measured at 2,048 rows:
# 29.3 / 17.7 / 76.5 / 39.3 us against 29.7 / 17.8 / 76.2 / 37.8 us for the four products of a Qwen3-1.7B layer), and
# it can apply the gated activation as it stores, which the library cannot.  With few tiles, or a last round of
# tiles that leaves most pairs idle, cuBLAS' smaller tiles win, so those shapes stay there
# (MINISERVE_B200_PAIR_GEMM=0: all of them do).  The one-block tcgen05 kernel (linear_tcgen05) reaches 77-92 % of
# cuBLAS and runs only on request (MINISERVE_B200_TCGEN05_GEMM=1).
USE_PAIR_GEMM = __import__("os").environ.get("MINISERVE_B200_PAIR_GEMM", "1") == "1"
USE_TCGEN05_GEMM = __import__("os").environ.get("MINISERVE_B200_TCGEN05_GEMM", "0") == "1"
PAIR_MIN_FILL = 0.8            # of the pairs' time in use, by the count of tiles


_many_row_choices: dict = {}         # (device index, kind, row tiles, N, K) -> "pair" | "wide" | "library"
_many_row_times: dict = {}           # the same keys -> {candidate: microseconds} as measured


def many_row_choices() -> dict:
    """What was chosen for the many-row products so far, with the measured times in microseconds."""
    return {key: (choice, _many_row_times.get(key)) for key, choice in _many_row_choices.items()}


def _pair_or_library(kind: str, rows: int, weight: torch.Tensor, n_q: int = 0, n_kv: int = 0) -> str:
    """For a product of ``rows`` rows that :func:`pair_preferred` lets through: the two-block kernel with the
    element-wise work of ``kind`` in its epilogue ("pair"; "wide": with tiles of 256 x 512, which fetch a quarter less
    from the L2 cache but are fewer), or cuBLAS followed by the separate kernel ("library").
    Measured once per kind, count of 256-row tiles and weight shape, on the weight itself, at the first eager call
    that meets it (kept in the choices file like the few-row choices); with MINISERVE_B200_LINEAR_TUNING=0 it is
    the two-block kernel.  Kinds: "plain" (store), "gated" (against the product and the activation kernel), "add"
    (product adding into the residual stream and the norm that reads it, against product, and norm that adds),
    "qkv" (against product and the norm + rotation + append kernel)."""
    n, k = weight.shape
    tiles_m = (rows + 255) // 256
    key = (torch.device(weight.device).index or 0, kind, tiles_m, n, k)
    choice = _many_row_choices.get(key)
    if choice is None:
        if not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return "pair"
        stored_as = f"rows{tiles_m} {kind}"
        choice = _stored_choice(stored_as, n, k)
        if choice is None:
            choice = _measure_many_rows(key, rows, weight, n_q, n_kv)
            _store_choice(stored_as, n, k, choice)
            log.info("%s products of %d rows with a %d x %d weight run %s (measured, us: %s)", kind, rows, n, k,
                     "the two-block kernel" if choice == "pair" else "cuBLAS and the separate kernel", _many_row_times.get(key))
        _many_row_choices[key] = choice
    return choice


def _measure_many_rows(key: tuple, rows: int, weight: torch.Tensor, n_q: int, n_kv: int) -> str:
    kind = key[1]
    n, k = weight.shape
    device = weight.device
    generator = torch.Generator(device=device).manual_seed(0)
    source = torch.randn((rows, k), dtype=torch.float32, device=device, generator=generator).to(torch.bfloat16)
    x = torch.empty_like(source)
    whole = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
    if kind == "plain":
        candidates = {"pair": lambda: linear_pair(x, weight, whole, wide=False),
                      "wide": lambda: linear_pair(x, weight, whole, wide=True),
                      "library": lambda: torch.mm(x, weight.t(), out=whole)}
    elif kind == "gated":
        half = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=device)

        def by_library() -> None:
            torch.mm(x, weight.t(), out=whole)
            silu_mul(whole, half, paired=True)
        candidates = {"pair": lambda: linear_pair(x, weight, half, gated=True, wide=False),
                      "wide": lambda: linear_pair(x, weight, half, gated=True, wide=True), "library": by_library}
    elif kind == "add":
        residual = torch.zeros((rows, n), dtype=torch.float32, device=device)
        norm_weight = torch.ones(n, dtype=torch.bfloat16, device=device)

        def by_pair(wide: bool) -> None:
            linear_pair(x, weight, residual, add=True, wide=wide)
            add_rmsnorm(residual, None, norm_weight, 1e-6, whole)

        def by_library() -> None:
            delta = torch.mm(x, weight.t())
            add_rmsnorm(residual, delta, norm_weight, 1e-6, whole)
        candidates = {"pair": lambda: by_pair(False), "wide": lambda: by_pair(True), "library": by_library}
    elif kind == "qkv":
        d, page = 128, 64
        q = torch.empty((rows, n_q, d), dtype=torch.bfloat16, device=device)
        pools = [torch.empty(((rows + page - 1) // page, n_kv, page, d), dtype=torch.bfloat16, device=device) for _ in range(2)]
        slots = torch.arange(rows, dtype=torch.int32, device=device)
        norm_weight = torch.ones(d, dtype=torch.bfloat16, device=device)
        cos_sin = torch.zeros((rows, d // 2, 2), dtype=torch.float32, device=device)

        def by_library() -> None:
            torch.mm(x, weight.t(), out=whole)
            qk_norm_rope_append(whole, slots, norm_weight, norm_weight, 1e-6, cos_sin, d, False, pools[0], pools[1], n_q, n_kv, d, q)
        candidates = {"pair": lambda: linear_pair_qkv(x, weight, slots, norm_weight, norm_weight, 1e-6, cos_sin, pools[0],
                                                      pools[1], n_q, n_kv, q),
                      "library": by_library}
    else:
        raise KernelError(f"no many-row product of kind {kind!r}")
    times = _sample_times(candidates, x, rounds=4, source=source)
    _many_row_times[key] = {name: round(1e3 * t, 1) for name, t in times.items()}
    return min(times, key=times.get)


def pair_fill(device: torch.device, m: int, n: int) -> float:
    """The share of the pairs' time that the 256 x 256 tiles of an ``m x n`` product keep busy: tiles / (rounds x pairs)."""
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = max(_multiprocessors[key] // 2, 1)
    tiles = ((m + 255) // 256) * ((n + 255) // 256)
    return tiles / (((tiles + pairs - 1) // pairs) * pairs)


def pair_rounds(device: torch.device, m: int, n: int) -> int:
    """Tiles that the busiest pair of multiprocessors works on, one after the other, in an ``m x n`` product."""
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    pairs = max(_multiprocessors[key] // 2, 1)
    return (((m + 255) // 256) * ((n + 255) // 256) + pairs - 1) // pairs


def pair_preferred(device: torch.device, m: int, n: int, gated: bool = False) -> bool:
    """Whether a bfloat16 product of ``m`` rows with an ``n``-row weight goes to :func:`linear_pair`.  The gated form
    also saves the activation kernel and its traffic, so it is taken at a lower fill."""
    return USE_PAIR_GEMM and m >= 256 and pair_fill(device, m, n) >= (0.6 if gated else PAIR_MIN_FILL)

# Prompt portions in bfloat16 run the tcgen05 attention kernel where it takes the sizes (head size 64 or 128,
# group size dividing 128, pages of 8..128 tokens); MINISERVE_B200_TCGEN05_ATTENTION=0 keeps them on the
# mma.sync kernel.
USE_TCGEN05_ATTENTION = __import__("os").environ.get("MINISERVE_B200_TCGEN05_ATTENTION", "1") == "1"
# ... in the form in which two groups of softmax threads take the key tiles in turn, one thread per query row, with
# three score buffers; MINISERVE_B200_ATTENTION_IN_TURNS=0: all softmax threads on every tile, two per row.
ATTENTION_IN_TURNS = __import__("os").environ.get("MINISERVE_B200_ATTENTION_IN_TURNS", "1") == "1"

_error_flags: dict = {}


def device_error_flag(device: torch.device) -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits set when a wait runs out (0: all well)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_device_errors(device: torch.device) -> None:
    """Raises if a kernel gave up waiting since the last check (synchronises the device)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        return                      # no kernel with bounded waits has run on this device
    flag = _error_flags[key]
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(f"a kernel gave up a bounded wait (code {code}: 1 producer, 2 MMA issue, 3 epilogue, "
                          "4 copies in flight at the end)")


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: bool = False) -> None:
    """``out = x @ weight^T`` (``add``: ``out += ...`` on a float32 ``out``) by the library's tcgen05 kernel.

    bfloat16 operands with an inner size that is a multiple of 8; meant for 128 rows and more.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", torch.float32 if add else None, (m, n))
    _check(library().ms_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(1 if add else 0), _i(m),
                                     _i(n), _i(k), _ptr(device_error_flag(x.device)), _stream()))


PAIR_WIDE = __import__("os").environ.get("MINISERVE_B200_PAIR_WIDE", "0") == "1"


def linear_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: bool = False, gated: bool = False,
                row_stats: Optional["RowStats"] = None, wide: Optional[bool] = None) -> None:
    """``out = x @ weight^T`` by the kernel in which two thread blocks share each 256 x 256 tile (tcgen05 with
    ``cta_group::2``).  ``add``: ``out += ...`` on a float32 ``out``.  ``gated``: ``weight`` is
    :func:`interleave_gate_up` of a gate and an up projection and ``out [M, N / 2] = silu(gate) * up``.
    ``row_stats`` (from :func:`linear_pair_residual`): ``x`` still lacks the division by its rows' root mean square,
    and the results are multiplied by it before they are rounded.

    bfloat16 operands with an inner size that is a multiple of 8; meant for 256 rows and more.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    if gated:
        _want(out, "out", torch.bfloat16, (m, n // 2))
    else:
        _want(out, "out", torch.float32 if add else None, (m, n))
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if add or not row_stats.per_row or row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != m \
                or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"linear_pair: row statistics of shape {tuple(row_stats.partials.shape)} for {m} rows, "
                              f"{row_stats.count} tiles")
    _check(library().ms_gemm_pair(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(2 if gated else 1 if add else 0),
                                  _i(1 if (PAIR_WIDE if wide is None else wide) else 0),
                                  _i(m), _i(n), _i(k), _ptr(row_stats.partials if row_stats else None),
                                  _i(row_stats.count if row_stats else 0), _f(row_stats.eps if row_stats else 0.0), None, None,
                                  _i(0), None, _ptr(device_error_flag(x.device)), _stream()))


QKV_IN_PRODUCT = __import__("os").environ.get("MINISERVE_B200_QKV_IN_PRODUCT", "1") == "1"


def qkv_in_product_supported(rows: int, dtype: torch.dtype, weight: torch.Tensor, head_dim: int, n_q: int, n_kv: int,
                             cos_sin, rotary_dim: int, interleaved: bool) -> bool:
    """Whether a q/k/v projection of ``rows`` rows can norm, rotate and append its heads as it stores them
    (:func:`linear_pair_qkv`): bfloat16, so many rows that it goes to :func:`linear_pair`, heads of 128, and no
    rotation or the half-split one over the whole head."""
    if rows < 256 or not QKV_IN_PRODUCT or dtype != torch.bfloat16:
        return False
    n, k = weight.shape
    return (head_dim == 128 and k % 8 == 0
            and (cos_sin is None or (rotary_dim == head_dim and not interleaved))
            and pair_preferred(weight.device, rows, n) and _pair_or_library("qkv", rows, weight, n_q, n_kv) == "pair")


def linear_pair_qkv(x: torch.Tensor, weight: torch.Tensor, slots: torch.Tensor, q_weight: Optional[torch.Tensor],
                    k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor], k_pool: torch.Tensor,
                    v_pool: torch.Tensor, n_q: int, n_kv: int, q_out: torch.Tensor, row_stats: Optional["RowStats"] = None) -> None:
    """The q/k/v projection ``x @ weight^T`` with :func:`qk_norm_rope_append` applied to the tiles as they leave the
    tensor cores (heads of 128; the arguments mean what they mean there): q heads to ``q_out``, k and v heads to the
    pools, and the projection itself is never written out.  ``row_stats`` as in :func:`linear_pair`."""
    m, k = x.shape
    d = 128
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, ((n_q + 2 * n_kv) * d, k))
    _want(slots, "slots", torch.int32, (m,))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[3] != d:
        raise KernelError(f"pool shape {tuple(k_pool.shape)} is not [pages, {n_kv}, page_size, {d}]")
    _want(q_out, "q_out", torch.bfloat16, (m, n_q, d))
    weight_code = 0
    for name, norm_weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if norm_weight is not None:
            _want(norm_weight, name, None, (d,))
            weight_code = _code(norm_weight.dtype)
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share one element type")
    if cos_sin is not None:
        _want(cos_sin, "cos_sin", torch.float32, (m, d // 2, 2))
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if not row_stats.per_row or row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != m \
                or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"linear_pair_qkv: row statistics of shape {tuple(row_stats.partials.shape)} for {m} rows")
    _check(library().ms_gemm_pair_qkv(
        _ptr(x), _ptr(weight), _ptr(q_out), _i(m), _i(k), _ptr(row_stats.partials if row_stats else None),
        _i(row_stats.count if row_stats else 0), _f(row_stats.eps if row_stats else 0.0), _ptr(slots), _ptr(q_weight),
        _ptr(k_weight), _i(weight_code), _f(eps), _ptr(cos_sin), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[2]), _i(n_q),
        _i(n_kv), _ptr(device_error_flag(x.device)), _stream()))


def pair_column_tiles(n: int) -> int:
    """Rows of ``partials`` that :func:`linear_pair_residual` writes for a weight of ``n`` rows."""
    return (n + 255) // 256


def linear_pair_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float, x_next: torch.Tensor, partials: torch.Tensor) -> "RowStats":
    """:func:`linear_wide_residual` for many rows, by the kernel of :func:`linear_pair`: ``residual += x @ weight^T``
    (float32, in place), ``x_next = bfloat16(residual * norm_weight)`` and the rows' sums of squares, one row of
    ``partials [>= pair_column_tiles(N), M]`` per 256 columns.  ``N`` a multiple of 8."""
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(residual, "residual", torch.float32, (m, n))
    _want(norm_weight, "norm_weight", None, (n,))
    _want(x_next, "x_next", torch.bfloat16, (m, n))
    _want(partials, "partials", torch.float32)
    tiles = pair_column_tiles(n)
    if n % 8 or partials.dim() != 2 or partials.shape[1] != m or partials.shape[0] < tiles:
        raise KernelError(f"linear_pair_residual: weight {tuple(weight.shape)}, partials {tuple(partials.shape)} for {tiles} "
                          f"tiles of {m} rows")
    _check(library().ms_gemm_pair(_ptr(x), _ptr(weight), _ptr(x_next), _i(1), _i(3), _i(0), _i(m), _i(n), _i(k), None, _i(0),
                                  _f(0.0), _ptr(residual), _ptr(norm_weight), _i(_code(norm_weight.dtype)), _ptr(partials),
                                  _ptr(device_error_flag(x.device)), _stream()))
    return RowStats(partials, tiles, eps, per_row=True)


_stream_buffers: dict = {}

# Products of few rows (decode steps) read every weight once; which kernel streams a given weight fastest
# depends on its shape.  For up to SKINNY_MAX_ROWS rows the choice between the mma.sync kernel ("skinny":
# many small blocks, K split over a cluster for narrow weights), the tcgen05 kernel ("stream": one block
# per multiprocessor, its start and the sum over blocks sharing a tile cost some microseconds, which only a
# large weight wins back) and the library is measured once per weight shape, on the weight itself, in captured
# graphs as a decode step runs them (_sample_times), at the first eager call that meets the shape;
# MINISERVE_B200_LINEAR_TUNING=0 turns the measurement off, and then (and while a graph is being captured
# before any eager call) the rule below decides.  From SKINNY_MAX_ROWS + 1 to STREAM_MAX_ROWS rows it is the
# rule alone.  The gated product of a feed-forward (gated_up) chooses the same way between the kernel that
# applies the activation as it stores ("wide") and a plain product followed by the activation kernel.
STREAM_MAX_ROWS = int(__import__("os").environ.get("MINISERVE_B200_STREAM_MAX_ROWS", "16"))
STREAM_MIN_UNITS = int(__import__("os").environ.get("MINISERVE_B200_STREAM_MIN_UNITS", "32"))
LINEAR_TUNING = __import__("os").environ.get("MINISERVE_B200_LINEAR_TUNING", "1") == "1"
FEW_ROWS_KERNEL = __import__("os").environ.get("MINISERVE_B200_FEW_ROWS", "")     # "skinny" | "stream" | "wide" | "library"
if FEW_ROWS_KERNEL not in ("", "skinny", "stream", "wide", "library"):
    raise ValueError(f"MINISERVE_B200_FEW_ROWS={FEW_ROWS_KERNEL!r}: expected skinny, stream, wide or library")
_multiprocessors: dict = {}
_linear_choices: dict = {}           # (device index, N, K) -> "skinny" | "stream" | "wide" | "library"
_gated_choices: dict = {}            # (device index, 2 I, K) -> "wide" | "separate"
_choice_times: dict = {}             # the same keys -> {candidate: microseconds} as measured
FLUSH_BYTES = 256 << 20              # larger than the L2 cache
DRAW = 1.03                          # two measured times closer than this count as level


def _stream_units_per_block(device: torch.device, n: int, k: int) -> float:
    key = torch.device(device).index or 0
    if key not in _multiprocessors:
        _multiprocessors[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return ((n + 255) // 256) * ((k + 63) // 64) / _multiprocessors[key]


def _few_rows_rule(device: torch.device, m: int, n: int, k: int) -> str:
    if m <= SKINNY_MAX_ROWS and wide_supports(n, k) == 2:
        return "wide"                # one wave of blocks, each with its whole share of the weight on the way early
    if _stream_units_per_block(device, n, k) >= STREAM_MIN_UNITS:
        return "stream"
    return "skinny" if m <= SKINNY_MAX_ROWS else "library"


def _few_rows_choice(x: torch.Tensor, weight: torch.Tensor, m: int) -> str:
    n, k = weight.shape
    if FEW_ROWS_KERNEL and m <= SKINNY_MAX_ROWS and (FEW_ROWS_KERNEL != "wide" or wide_supports(n, k)):
        return FEW_ROWS_KERNEL      # pinned (to profile one kernel on every product, or to compare)
    if m > SKINNY_MAX_ROWS:
        return _few_rows_rule(x.device, m, n, k)
    key = (torch.device(x.device).index or 0, n, k)
    choice = _linear_choices.get(key)
    if choice is None:
        if not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return _few_rows_rule(x.device, m, n, k)
        choice = _stored_choice("linear", n, k)
        if choice is not None and (choice != "wide" or wide_supports(n, k)):
            _linear_choices[key] = choice
            return choice
        choice = _linear_choices[key] = _measure_few_rows(weight)
        _store_choice("linear", n, k, choice)
        log.info("products of up to %d rows with a %d x %d weight run the %s kernel (measured, us: %s)", SKINNY_MAX_ROWS, n, k,
                 choice, _choice_times.get(key))
    return choice


def linear_choices() -> dict:
    """What was measured so far: (device index, N, K) -> the kernel chosen for products of few rows."""
    return dict(_linear_choices)


# A measured choice can differ between runs where two kernels are level, and with it the order of a product's sums.
# MINISERVE_B200_CHOICES_FILE names a JSON file that keeps the choices: what it holds is used instead of measuring,
# and what is measured is added to it, so that later runs (and other processes) repeat the first one's choices.
CHOICES_FILE = __import__("os").environ.get("MINISERVE_B200_CHOICES_FILE", "")


def _stored_choice(kind: str, n: int, k: int) -> Optional[str]:
    if not CHOICES_FILE:
        return None
    import json
    try:
        with open(CHOICES_FILE, encoding="utf-8") as handle:
            value = json.load(handle).get(f"{kind} {n}x{k}")
    except (OSError, ValueError):
        return None
    allowed = (("skinny", "stream", "wide", "library") if kind == "linear" else ("pair", "wide", "library") if kind.startswith("rows")
               else ("wide", "separate"))
    return value if value in allowed else None


def _store_choice(kind: str, n: int, k: int, choice: str) -> None:
    if not CHOICES_FILE:
        return
    import json
    import os
    try:
        try:
            with open(CHOICES_FILE, encoding="utf-8") as handle:
                stored = json.load(handle)
        except (OSError, ValueError):
            stored = {}
        stored[f"{kind} {n}x{k}"] = choice
        temporary = f"{CHOICES_FILE}.{os.getpid()}"
        with open(temporary, "w", encoding="utf-8") as handle:
            json.dump(stored, handle, indent=1, sort_keys=True)
        os.replace(temporary, CHOICES_FILE)
    except OSError as error:
        log.warning("cannot keep the kernel choices in %s: %s", CHOICES_FILE, error)


TUNING_REPEATS = 8      # a candidate this many times in one captured graph


def _sample_times(candidates: dict, x: torch.Tensor, rounds: int = 7, source: Optional[torch.Tensor] = None) -> dict:
    """Device time in milliseconds of each of ``candidates`` (name -> callable reading ``x``), measured the way
    a decode step runs them: in a captured graph, after a small kernel of this library that writes ``x`` (so
    that a candidate which can start before its predecessor ends does so), with the L2 cache overwritten
    before it.  A graph holds that sequence TUNING_REPEATS times; the same graph without the candidate is
    timed too and subtracted.  The graphs take turns, round after round, so that a clock that is still rising
    meets all of them alike; the figure is the lower quartile of a graph's samples."""
    device = x.device
    flush = torch.empty(FLUSH_BYTES // 4, dtype=torch.float32, device=device)
    # (``source``: what ``x`` is made from before every run; zeros unless the candidates' speed depends on the data,
    # as that of tensor-core products under the power limit does)
    source = torch.zeros_like(x) if source is None else source
    weight = torch.ones(x.shape[-1], dtype=x.dtype, device=device)

    def capture(run) -> torch.cuda.CUDAGraph:
        def sequence() -> None:
            for _ in range(TUNING_REPEATS):
                flush.zero_()
                rmsnorm(source, weight, 1e-6, x)
                if run is not None:
                    run()
        sequence()                                          # lazy set-up outside the capture
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sequence()
        return graph

    graphs = {name: capture(run) for name, run in candidates.items()}
    graphs[None] = capture(None)
    samples = {name: [] for name in graphs}
    for round_index in range(rounds + 2):
        for name, graph in graphs.items():
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            end.synchronize()
            if round_index >= 2:                            # the first rounds bring the clocks up
                samples[name].append(start.elapsed_time(end))
    quartile = {name: sorted(times)[len(times) // 4] for name, times in samples.items()}
    return {name: (quartile[name] - quartile[None]) / TUNING_REPEATS for name in candidates}


def _measure_few_rows(weight: torch.Tensor) -> str:
    """Times the candidates for ``[8, K] @ weight[N, K]^T`` on the device and names the one to use: the fastest
    of this library's kernels or the vendor library's."""
    n, k = weight.shape
    device = weight.device
    x = torch.zeros((SKINNY_MAX_ROWS, k), dtype=torch.bfloat16, device=device)
    out = torch.empty((SKINNY_MAX_ROWS, n), dtype=torch.bfloat16, device=device)
    candidates = {
        "skinny": lambda: _check(library().ms_gemm_skinny(_ptr(x), _i(0), _ptr(weight), _ptr(out), _i(_code(out.dtype)),
                                                          _i(SKINNY_MAX_ROWS), _i(n), _i(k), _stream())),
        "stream": lambda: linear_stream(x, weight, out),
        "library": lambda: torch.mm(x, weight.t(), out=out),
    }
    if wide_supports(n, k) == 2:
        candidates["wide"] = lambda: linear_wide(x, weight, out)
    times = _sample_times(candidates, x)
    _choice_times[(torch.device(device).index or 0, n, k)] = {name: round(1e3 * t, 2) for name, t in times.items()}
    own = min((name for name in candidates if name != "library"), key=lambda name: times[name])
    # Whole steps decide what the measurement leaves open.  The two kernels that stream weights by TMA and ask
    # for the first of them before their predecessor has ended have kept in the step what they showed here (the
    # output matrix, level with the vendor library here, is 4 % of a step faster with the tcgen05 kernel), so
    # they also win a draw; the mma.sync kernel has lost to the library in the step where it was level with it
    # here (the 8B gate/up projection: 12 us a layer), so it has to be clearly faster.
    if own == "skinny":
        return own if DRAW * times[own] < times["library"] else "library"
    return own if times[own] <= DRAW * times["library"] else "library"


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ weight^T`` for up to 64 rows of bfloat16 ``x`` (inner size a multiple of 8) by the
    library's weight-streaming tcgen05 kernel; ``out`` bfloat16 or float32."""
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", None, (m, n))
    key = torch.device(x.device).index or 0
    tiles = (n + 255) // 256
    buffers = _stream_buffers.get(key)
    if buffers is None or buffers[1].numel() < tiles:
        floats, ints = ctypes.c_longlong(0), ctypes.c_longlong(0)
        _check(library().ms_gemm_stream_buffers(_i(max(n, 1 << 20)), ctypes.addressof(floats), ctypes.addressof(ints)))
        buffers = (torch.empty(floats.value, dtype=torch.float32, device=x.device),
                   torch.zeros(ints.value, dtype=torch.int32, device=x.device))
        _stream_buffers[key] = buffers
    _check(library().ms_gemm_stream(_ptr(x), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m), _i(n), _i(k),
                                    _ptr(buffers[0]), _ptr(buffers[1]), _ptr(device_error_flag(x.device)), _stream()))


_wide_supports: dict = {}


def wide_supports(n: int, k: int) -> int:
    """0: :func:`linear_wide` does not take a weight of ``n`` rows and inner size ``k``; 1: it does, in several
    waves of blocks; 2: with at most one block per multiprocessor, which is what it is made for."""
    answer = _wide_supports.get((n, k))
    if answer is None:
        answer = _wide_supports[(n, k)] = int(library().ms_gemm_wide_supports(_i(n), _i(k)))
    return answer


class RowStats:
    """What is still missing from activations whose norm is folded into the products around it: ``x`` holds
    ``residual * norm weight`` and every row has yet to be divided by the root of its mean square.
    ``partials`` (float32) holds sums of squares of the residual's rows, one row of partial sums per block (or
    column tile) of the product that wrote ``x``: ``[count, 8]`` from the few-row product, ``[count, rows]`` from
    the many-row one (``per_row``).  The product that reads ``x`` adds them up in order and applies
    ``1 / sqrt(total / size + eps)`` to its own results."""

    __slots__ = ("partials", "count", "eps", "per_row")

    def __init__(self, partials: torch.Tensor, count: int, eps: float, per_row: bool = False) -> None:
        self.partials, self.count, self.eps, self.per_row = partials, count, eps, per_row


def wide_blocks(n: int, k: int) -> int:
    """Blocks that :func:`linear_wide` runs for a weight ``[n, k]``: the rows of ``partials`` that
    :func:`linear_wide_residual` writes."""
    return int(library().ms_gemm_wide_blocks(_i(n), _i(k)))


def _wide_call(x, weight, out, out_code: int, mode: int, m: int, n: int, k: int, row_stats: Optional[RowStats],
               residual=None, norm_weight=None, x_next=None, out_partials=None) -> None:
    if row_stats is not None:
        _want(row_stats.partials, "row_stats.partials", torch.float32)
        if row_stats.partials.dim() != 2 or row_stats.partials.shape[1] != 8 or row_stats.partials.shape[0] < row_stats.count:
            raise KernelError(f"row statistics of shape {tuple(row_stats.partials.shape)} for {row_stats.count} blocks")
    _check(library().ms_gemm_wide(
        _ptr(x), _ptr(weight), _ptr(out), _i(out_code), _i(mode), _i(m), _i(n), _i(k),
        _ptr(row_stats.partials if row_stats else None), _i(row_stats.count if row_stats else 0),
        _f(row_stats.eps if row_stats else 0.0), _ptr(residual), _ptr(norm_weight),
        _i(_code(norm_weight.dtype) if norm_weight is not None else 0), _ptr(x_next), _ptr(out_partials),
        _ptr(device_error_flag(x.device)), _stream()))


def linear_wide(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
                row_stats: Optional[RowStats] = None) -> None:
    """``out = x @ weight^T`` for up to 8 rows of bfloat16 ``x`` by the library's kernel for weights of many
    rows (no sum across blocks); ``out`` bfloat16 or float32.

    ``gated``: ``weight [2 I, K]`` holds a gated feed-forward's two projections in blocks of sixteen rows,
    eight gate rows followed by the up rows of the same features (:func:`interleave_gate_up`), and
    ``out [M, I]`` bfloat16 receives ``silu(gate) * up``.  ``row_stats``: ``x`` comes from
    :func:`linear_wide_residual`; its rows' norm is completed on the results (before the activation).
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(out, "out", torch.bfloat16 if gated else None, (m, n // 2 if gated else n))
    _wide_call(x, weight, out, _code(out.dtype), 1 if gated else 0, m, n, k, row_stats)


def linear_wide_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float, x_next: torch.Tensor, partials: torch.Tensor) -> RowStats:
    """``residual += x @ weight^T`` (float32, in place) for up to 8 rows of bfloat16 ``x``, and the input of
    whatever follows an RMSNorm of the new residual: ``x_next = bfloat16(residual * norm_weight)`` with the rows'
    sums of squares left in ``partials`` (float32 ``[>= wide_blocks(N, K), 8]``).  The returned statistics go
    with ``x_next`` into :func:`linear_wide` or :func:`gated_up`.  Only for weights with ``wide_supports == 2``.
    """
    m, k = x.shape
    n = weight.shape[0]
    _want(x, "x", torch.bfloat16)
    _want(weight, "weight", torch.bfloat16, (n, k))
    _want(residual, "residual", torch.float32, (m, n))
    _want(norm_weight, "norm_weight", None, (n,))
    _want(x_next, "x_next", torch.bfloat16, (m, n))
    _want(partials, "partials", torch.float32)
    blocks = wide_blocks(n, k)
    if wide_supports(n, k) != 2 or partials.dim() != 2 or partials.shape[1] != 8 or partials.shape[0] < blocks:
        raise KernelError(f"linear_wide_residual: weight {tuple(weight.shape)} (one wave of blocks only), partials "
                          f"{tuple(partials.shape)} for {blocks} blocks")
    _wide_call(x, weight, None, 1, 2, m, n, k, None, residual, norm_weight, x_next, partials)
    return RowStats(partials, blocks, eps)


ADD_IN_PRODUCT = __import__("os").environ.get("MINISERVE_B200_ADD_IN_PRODUCT", "1") == "1"


def add_in_product_supported(rows: int, dtype: torch.dtype, weight: torch.Tensor) -> bool:
    """Whether a product of ``rows`` rows with ``weight`` can add its results into a float32 matrix as it stores
    them (:func:`linear_add`): bfloat16, and so many rows that it goes to :func:`linear_pair`, whose read-out hands
    its tiles to TMA as additions.  The norm that follows then reads the residual stream and writes its output,
    and no longer reads a separate output, adds it and writes the stream back (at Qwen3-1.7B sizes and 2,048 rows:
    25 MB instead of 50 MB a norm)."""
    if rows < 256 or not ADD_IN_PRODUCT or dtype != torch.bfloat16:      # (what decides for steps of few rows, first)
        return False
    n, k = weight.shape
    return (n % 4 == 0 and k % 8 == 0
            and pair_preferred(weight.device, rows, n) and _pair_or_library("add", rows, weight) != "library")


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> None:
    """``residual += x @ weight^T`` (float32, in place), where :func:`add_in_product_supported` said so."""
    linear_pair(x, weight, residual, add=True, wide=_pair_or_library("add", x.shape[0], weight) == "wide")


def residual_partials_shape(rows: int, n: int, k: int) -> tuple:
    """The shape of the float32 ``partials`` that :func:`linear_residual` wants for ``rows`` rows and a weight ``[n, k]``."""
    return (wide_blocks(n, k), 8) if rows <= SKINNY_MAX_ROWS else (pair_column_tiles(n), rows)


def linear_residual(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                    x_next: torch.Tensor, partials: torch.Tensor) -> RowStats:
    """A product whose results join the residual stream, with the norm that follows folded in (where
    :func:`fold_supported` said so): :func:`linear_wide_residual` for up to 8 rows, :func:`linear_pair_residual`
    for many."""
    if x.shape[0] <= SKINNY_MAX_ROWS:
        return linear_wide_residual(x, weight, residual, norm_weight, eps, x_next, partials)
    return linear_pair_residual(x, weight, residual, norm_weight, eps, x_next, partials)


def fold_supported(rows: int, dtype: torch.dtype, producer: torch.Tensor, consumer: torch.Tensor,
                   consumer_gated: bool = False) -> bool:
    """Whether, in a step of ``rows`` rows, an RMSNorm between the product with the weight ``producer`` and the
    one with ``consumer`` can be folded into the two (:func:`linear_residual`, then ``row_stats``): bfloat16, and
    either at most 8 rows and both weights ones that :func:`linear_wide` is (or would be) chosen for, or so many
    rows that both products go to :func:`linear_pair`."""
    if not FOLD_NORMS or dtype != torch.bfloat16 or rows <= 0:
        return False
    if rows > SKINNY_MAX_ROWS:
        if not FOLD_NORMS_MANY_ROWS or producer.shape[0] % 8 or producer.shape[1] % 8 or consumer.shape[1] % 8:
            return False
        # The folded epilogue moves 10 bytes per element against 2; it pays where a pair has a next tile to
        # accumulate meanwhile (measured at Qwen3-1.7B sizes: 4,096 rows 39.3 against 46.1 us for the o projection and
        # the norm kernel, 8,192 rows 71.9 against 89.4 us; 2,048 rows, one tile per pair, 25.8 against 26.1 us)
        return (pair_preferred(producer.device, rows, producer.shape[0])
                and pair_rounds(producer.device, rows, producer.shape[0]) >= 2
                and pair_preferred(consumer.device, rows, consumer.shape[0], gated=consumer_gated)
                and _pair_or_library("add", rows, producer) != "library"
                and _pair_or_library("gated" if consumer_gated else "plain", rows, consumer) != "library")
    for weight, gated in ((producer, False), (consumer, consumer_gated)):
        n, k = weight.shape
        if k % 8 or wide_supports(n, k) != 2:
            return False
        key = (torch.device(weight.device).index or 0, n, k)
        if FEW_ROWS_KERNEL:
            chosen = FEW_ROWS_KERNEL
        else:
            chosen = (_gated_choices if gated else _linear_choices).get(key, "wide")    # not measured yet: the rule says wide
        if chosen != "wide":
            return False
    return True


FOLD_NORMS = __import__("os").environ.get("MINISERVE_B200_FOLD_NORMS", "1") == "1"
FOLD_NORMS_MANY_ROWS = __import__("os").environ.get("MINISERVE_B200_FOLD_NORMS_MANY_ROWS", "1") == "1"


GATE_UP_BLOCK = 8    # rows of the gate projection beside as many of the up projection, for linear_wide(gated=True)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``[2 I, K]``: rows 16 j .. 16 j + 7 are the gate rows 8 j .. 8 j + 7, the next eight the same up rows."""
    inter, k = gate.shape
    if inter % GATE_UP_BLOCK != 0 or up.shape != gate.shape:
        raise KernelError(f"interleave_gate_up: {tuple(gate.shape)} and {tuple(up.shape)}; rows must be a multiple of 8")
    blocks = inter // GATE_UP_BLOCK
    return torch.stack((gate.reshape(blocks, GATE_UP_BLOCK, k), up.reshape(blocks, GATE_UP_BLOCK, k)), dim=1).reshape(2 * inter, k)


WIDE_GATED_MIN_ROWS = 8192     # of the paired weight: the rule when nothing was measured


def gated_up(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_stats: Optional[RowStats] = None) -> None:
    """``out[M, I] = silu(x @ gate^T) * (x @ up^T)`` with ``weight = interleave_gate_up(gate, up)``.
    (``row_stats``: see :func:`linear_wide`; the caller has asked :func:`fold_supported` first.)

    Few rows of bfloat16 go through :func:`linear_wide`, which applies the activation as it stores, where that
    is faster than the product (:func:`linear`) followed by :func:`silu_mul`: measured once per weight shape
    like the choice among the plain products, with the same switch.
    """
    m, k = x.shape
    two_i = weight.shape[0]
    _want(out, "out", x.dtype, (m, two_i // 2))
    if row_stats is not None:
        if row_stats.per_row:
            linear_pair(x, weight, out, gated=True, row_stats=row_stats)
        else:
            linear_wide(x, weight, out, gated=True, row_stats=row_stats)
        return
    if x.dtype == torch.bfloat16 and 0 < m <= SKINNY_MAX_ROWS and _gated_choice(x, weight) == "wide":
        linear_wide(x, weight, out, gated=True)
        return
    if x.dtype == torch.bfloat16 and k % 8 == 0 and pair_preferred(x.device, m, two_i, gated=True):
        choice = _pair_or_library("gated", m, weight)
        if choice != "library":
            linear_pair(x, weight, out, gated=True, wide=choice == "wide")    # many rows: the activation is applied as the tiles are stored
            return
    gate_up = torch.empty((m, two_i), dtype=x.dtype, device=x.device)
    linear(x, weight, gate_up)
    silu_mul(gate_up, out, paired=True)


def _gated_choice(x: torch.Tensor, weight: torch.Tensor) -> str:
    n, k = weight.shape
    key = (torch.device(x.device).index or 0, n, k)
    choice = _gated_choices.get(key)
    if choice is None:
        fits = wide_supports(n, k) if k % 8 == 0 and n % (2 * GATE_UP_BLOCK) == 0 else 0
        if not fits:
            choice = _gated_choices[key] = "separate"
        elif not LINEAR_TUNING or torch.cuda.is_current_stream_capturing():
            return "wide" if fits == 2 and n >= WIDE_GATED_MIN_ROWS else "separate"
        else:
            choice = _stored_choice("gated", n, k)
            if choice is not None:
                _gated_choices[key] = choice
                return choice
            choice = _gated_choices[key] = _measure_gated(weight)
            _store_choice("gated", n, k, choice)
            log.info("gated products of up to %d rows with a %d x %d weight run %s (measured, us: %s)", SKINNY_MAX_ROWS, n, k,
                     "the kernel that applies the activation" if choice == "wide" else "a plain product and the activation kernel",
                     _choice_times.get(key + ("gated",)))
    return choice


def _measure_gated(weight: torch.Tensor) -> str:
    n, k = weight.shape
    device = weight.device
    x = torch.zeros((SKINNY_MAX_ROWS, k), dtype=torch.bfloat16, device=device)
    gate_up = torch.empty((SKINNY_MAX_ROWS, n), dtype=torch.bfloat16, device=device)
    out = torch.empty((SKINNY_MAX_ROWS, n // 2), dtype=torch.bfloat16, device=device)

    def separate() -> None:
        linear(x, weight, gate_up)
        silu_mul(gate_up, out, paired=True)

    separate()                                              # the plain product's own choice is made outside the timing
    times = _sample_times({"wide": lambda: linear_wide(x, weight, out, gated=True), "separate": separate}, x)
    _choice_times[(torch.device(device).index or 0, n, k, "gated")] = {name: round(1e3 * t, 2) for name, t in times.items()}
    return "wide" if times["wide"] <= times["separate"] else "separate"


def choice_times() -> dict:
    """The measurements behind :func:`linear_choices` and :func:`gated_choices`: key -> {candidate: microseconds}
    (gated products have a fourth key element)."""
    return {key: dict(times) for key, times in _choice_times.items()}


def gated_choices() -> dict:
    """What was measured so far: (device index, 2 I, K) -> how the gated product of few rows runs."""
    return dict(_gated_choices)


SKINNY_MAX_ROWS = 8    # above this the weight-streaming kernel re-reads the activations too often


FUSE_GATED_INPUT = False    # applying the activation while streaming recomputes it in every block: slower (measured twice)


def gated_linear(gate_up: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out = (silu(gate_up[:, :I]) * gate_up[:, I:]) @ weight[N, I]^T``.

    With few rows in bfloat16 the activation is applied while the product streams the weights;
    otherwise it is one kernel (:func:`silu_mul`) followed by :func:`linear`.
    """
    m, two_i = gate_up.shape
    inter = two_i // 2
    n = weight.shape[0]
    if two_i != 2 * inter or weight.shape[1] != inter or tuple(out.shape) != (m, n):
        raise KernelError(f"gated_linear: gate_up {tuple(gate_up.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if FUSE_GATED_INPUT and gate_up.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and inter % 8 == 0:
        _want(gate_up, "gate_up", torch.bfloat16)
        _want(weight, "weight", torch.bfloat16)
        _want(out, "out")
        _check(library().ms_gemm_skinny(_ptr(gate_up), _i(1), _ptr(weight), _ptr(out), _i(_code(out.dtype)), _i(m),
                                        _i(n), _i(inter), _stream()))
        return
    hidden = torch.empty((m, inter), dtype=gate_up.dtype, device=gate_up.device)
    silu_mul(gate_up, hidden)
    linear(hidden, weight, out)


# --------------------------------------------------------------------------- sampling

SAMPLING_RECORD_WORDS = 8


def sample(logits: torch.Tensor, records: Optional[torch.Tensor], slot_of_row: Optional[torch.Tensor],
           draw_index: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """Chooses one token per row of float32 ``logits [K, V]`` into int32 ``out [K]``.

    ``records`` int32 ``[slots, 8]`` holds per state slot the bit patterns of (temperature,
    top_p) and the integers (top_k, seed low word, seed high word); ``slot_of_row`` and
    ``draw_index`` are int32 ``[K]``.  ``records=None`` means argmax for every row.
    """
    k, vocab = logits.shape
    _want(logits, "logits", torch.float32)
    _want(out, "out", torch.int32, (k,))
    if records is not None:
        _want(records, "records", torch.int32)
        if records.dim() != 2 or records.shape[1] != SAMPLING_RECORD_WORDS:
            raise KernelError(f"records must be [slots, {SAMPLING_RECORD_WORDS}] int32")
        _want(slot_of_row, "slot_of_row", torch.int32, (k,))
        _want(draw_index, "draw_index", torch.int32, (k,))
    # candidates of the first of the two kernels: (value, index) for every chunk of every row
    scratch = torch.empty((k, library().ms_sample_chunks(_i(vocab)), 2), dtype=torch.int32, device=logits.device)
    _check(library().ms_sample(_ptr(logits), _i(logits.stride(0)), _i(vocab), _ptr(records), _ptr(slot_of_row),
                               _ptr(draw_index), _ptr(out), _i(k), _ptr(scratch), _stream()))
