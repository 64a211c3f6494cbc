"""Python face of the CUDA kernels in ``csrc/``: one function per kernel.

Each function checks its arguments (device, dtype, shape, contiguity) and
launches on the current CUDA stream of torch through the library's C
interface.  There is no other implementation behind these names: tensors that
are not on a CUDA device, a missing compiler or a failed build raise an error.

Conventions: the residual stream ``x32`` is float32; activations, matrices
and the cache are in the run dtype (bfloat16 or float32, never mixed in one
call); norm weights, biases and logits are float32; index tensors are int32.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import torch

from .csrc.build import ensure_built

_lib = None
_lib_lock = threading.Lock()

_F32, _BF16 = 0, 1
launches = 0            # kernels launched through this module since import (bench reads it)


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The kernel library, built on first use."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                path = ensure_built()
                lib = ctypes.CDLL(str(path))
                lib.li_last_error.restype = ctypes.c_char_p
                _lib = lib
    return _lib


def library_file() -> str:
    library()
    return str(ensure_built(verbose=False))


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"run dtype must be float32 or bfloat16, got {t.dtype}")


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(f"{name}: the kernels run on CUDA devices only, tensor is on '{t.device}'")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None and t.shape != tuple(shape):
        raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# the current stream's handle without building a Stream object (a few hundred launches a step ask for it)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor):
    if _raw_stream is not None:
        index = t.device.index
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device() if index is None else index))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check(rc: int, what: str) -> None:
    global launches
    launches += 1
    if rc != 0:
        msg = library().li_last_error()
        raise KernelError(f"{what}: {msg.decode() if msg else 'error ' + str(rc)}")


_i = ctypes.c_int
_f = ctypes.c_float
_l = ctypes.c_longlong


# --------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, out32: torch.Tensor) -> None:
    """out32[t, :] = float(table[ids[t], :])."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table, "embedding table")
    _need(ids, "token ids", torch.int32)
    _need(out32, "embedding output", torch.float32, (T, H))
    _check(library().li_embedding(_p(table), _i(_dt(table)), _p(ids), _p(out32), _i(T), _i(H), _i(V), _stream(out32)), "embedding")


def add_pair_rows(x32: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, q_start: torch.Tensor,
                  seq_of_token: torch.Tensor, slots: torch.Tensor, state: torch.Tensor, mul_prev: int, mul_cur: int) -> None:
    """``x32[t] += pairs[(prev * mul_prev + ids[t] * mul_cur) mod buckets]`` with ``prev`` the token before ``t`` in its
    sequence: the one before it in the step, or, for the first token of a portion, the sequence's last token of the step
    before, kept in ``state[slot, 0]`` (int32); a sequence's first token (position 0) takes row ``buckets``, the table's
    last.  The state moves on to the portion's last token in the same launch."""
    T, H = x32.shape
    _need(x32, "residual stream", torch.float32)
    _need(pairs, "table of pairs", None, (pairs.shape[0], H))
    _need(ids, "token ids", torch.int32)
    _need(positions, "positions", torch.int32, (T,))
    _need(q_start, "q_start", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(slots, "state slots", torch.int32)
    _need(state, "state of previous tokens", torch.int32)
    if state.dim() != 2 or pairs.shape[0] < 2:
        raise KernelError(f"add_pair_rows: state {tuple(state.shape)}, table {tuple(pairs.shape)}")
    _check(library().li_add_pair_rows(_p(x32), _p(pairs), _i(_dt(pairs)), _p(ids), _p(positions), _p(q_start), _p(seq_of_token), _p(slots),
                                      _p(state), _l(state.shape[1]), _i(pairs.shape[0] - 1), _l(int(mul_prev)), _l(int(mul_cur)), _i(T), _i(H),
                                      _stream(x32)), "add_pair_rows")


def rmsnorm(x32: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    T, H = x32.shape
    _need(x32, "rmsnorm input", torch.float32)
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "rmsnorm output", None, (T, H))
    _check(library().li_rmsnorm(_p(x32), _p(weight), _f(eps), _p(out), _i(_dt(out)), _i(T), _i(H), _stream(out)), "rmsnorm")


def add_rmsnorm(x32: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """x32 += delta (float32 sum, kept in x32); out = rmsnorm(x32)."""
    T, H = x32.shape
    _need(x32, "add_rmsnorm residual", torch.float32)
    _need(delta, "add_rmsnorm delta", None, (T, H))
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "add_rmsnorm output", delta.dtype, (T, H))
    _check(library().li_add_rmsnorm(_p(x32), _p(delta), _i(_dt(delta)), _p(weight), _f(eps), _p(out), _i(T), _i(H), _stream(out)),
           "add_rmsnorm")


def gather_rmsnorm(x32: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[r] = rmsnorm(x32[rows[r]])."""
    T, H = x32.shape
    R = rows.shape[0]
    _need(x32, "gather_rmsnorm input", torch.float32)
    _need(rows, "gather_rmsnorm rows", torch.int32)
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "gather_rmsnorm output", None, (R, H))
    _check(library().li_gather_rmsnorm(_p(x32), _p(rows), _p(weight), _f(eps), _p(out), _i(_dt(out)), _i(R), _i(T), _i(H), _stream(out)),
           "gather_rmsnorm")


def residual_add(x32: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x32, "residual", torch.float32)
    _need(delta, "delta", None, x32.shape)
    _check(library().li_residual_add(_p(x32), _p(delta), _i(_dt(delta)), _l(x32.numel()), _stream(x32)), "residual_add")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """``out[i] = mean + std * n(key, i)`` (flat index i) with n standard normal from the library's counter-based
    generator; float32 or bfloat16.  ``litinfer_b200.weights.random_init`` restates the recipe on the host."""
    _need(out, "fill_normal output")
    _check(library().li_fill_normal(_p(out), _i(_dt(out)), _l(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)), _f(mean), _f(std),
                                    _stream(out)), "fill_normal")


def fill_randint(out: torch.Tensor, key: int, high: int) -> None:
    """``out[i]`` = an integer in [0, high) from (key, i); int32."""
    _need(out, "fill_randint output", torch.int32)
    _check(library().li_fill_randint(_p(out), _l(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)), _i(high), _stream(out)),
           "fill_randint")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """``out[r] = src[rows[r]]`` for float32 rows (int32 ``rows`` on the device)."""
    _need(src, "gather source", torch.float32)
    _need(rows, "gather rows", torch.int32, (out.shape[0],))
    _need(out, "gather output", torch.float32, (rows.shape[0], src.shape[1]))
    _check(library().li_gather_rows(_p(src), _p(rows), _p(out), _i(src.shape[0]), _i(rows.shape[0]), _l(src.shape[1]), _stream(out)), "gather_rows")


def table_gather(resident: torch.Tensor, updates: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, trash_page: int) -> None:
    """Bring the resident block tables (int32 ``[slots + 1, cols]``, the last row all sink page) up to date with
    ``updates`` (a count, then triples of slot, logical page, page id) for the step's sequences (``slots`` int32 ``[S]``)
    and copy each sequence's row into the step's table ``out`` (int32 ``[S, max_blocks]``)."""
    _need(resident, "resident block tables", torch.int32)
    _need(updates, "table updates", torch.int32)
    _need(slots, "state slots", torch.int32)
    S = slots.shape[0]
    _need(out, "the step's block table", torch.int32, (S, out.shape[1]))
    if resident.dim() != 2 or updates.numel() < 1 or (updates.numel() - 1) % 3:
        raise KernelError(f"table_gather: resident {tuple(resident.shape)}, {updates.numel()} words of updates")
    _check(library().li_table_gather(_p(resident), _i(resident.shape[0]), _i(resident.shape[1]), _p(updates), _i((updates.numel() - 1) // 3),
                                     _p(slots), _p(out), _i(S), _i(out.shape[1]), _i(int(trash_page)), _stream(out)), "table_gather")


OVERLAP_KINDS = {"gemm": 1, "streaming_products": 2, "attention": 4, "rest": 8}


def allow_overlap(but: tuple = ()) -> None:
    """The launches that follow may begin while the kernel before them still runs (programmatic dependent launch),
    except the kinds of kernel named in ``but`` (keys of OVERLAP_KINDS).  The step function sets this per step."""
    library().li_pdl_allow(ctypes.c_int(sum(OVERLAP_KINDS[k] for k in but)))


def scale_inplace(x32: torch.Tensor, factor: float) -> None:
    """x32 *= factor (float32, in place)."""
    _need(x32, "scale operand", torch.float32)
    _check(library().li_scale_inplace(_p(x32), _l(x32.numel()), _f(factor), _stream(x32)), "scale")


def logit_cap(logits: torch.Tensor, cap: float) -> None:
    """logits = cap * tanh(logits / cap) (float32, in place)."""
    _need(logits, "logits", torch.float32)
    _check(library().li_logit_cap(_p(logits), _l(logits.numel()), _f(cap), _stream(logits)), "logit_cap")


EPILOGUES = {None: 0, "swiglu": 1, "glu_clamped": 2}
GATED = ("swiglu", "glu_clamped")


def _linear_args(a, weight, bias, out, epilogue):
    M, Kd = a.shape
    N = weight.shape[0]
    _need(a, "linear input")
    _need(weight, "linear weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "linear bias", torch.float32, (N,))
    if epilogue not in EPILOGUES:
        raise KernelError(f"linear: unknown epilogue {epilogue!r}")
    _need(out, "linear output", None, (M, N // 2 if epilogue in GATED else N))
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError(f"linear output must be {a.dtype} or float32, got {out.dtype}")
    return M, N, Kd


def _gated_params(epilogue, bias, epilogue_params):
    """What goes in the bias argument of the library's call: a gated product has no bias, and the clamped unit's two
    parameters (float32 ``[limit, alpha]`` on the device) travel in its place."""
    if epilogue == "glu_clamped":
        if bias is not None or epilogue_params is None:
            raise KernelError("linear: the glu_clamped epilogue takes no bias and needs epilogue_params = [limit, alpha]")
        _need(epilogue_params, "epilogue parameters", torch.float32, (2,))
        return epilogue_params
    if epilogue_params is not None:
        raise KernelError(f"linear: epilogue {epilogue!r} takes no parameters")
    return bias


def linear(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
           epilogue: Optional[str] = None, row_scale=None, epilogue_params: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = a[M, K] weight[N, K]^T (+ bias[N]); float32 accumulation;
    out is in the run dtype or float32.

    ``row_scale=(ssq, width, eps)``: every token's row of the product is multiplied by
    ``1 / sqrt(sum_p ssq[t, p] / width + eps)`` before bias and epilogue (see :func:`linear_add_scaled`); an error
    unless :func:`linear_scaled_accepts`.

    ``epilogue="swiglu"`` (bfloat16 only): ``weight`` holds gate and up rows interleaved in
    groups of 8 (see :func:`interleave_gate_up`) and out[M, N / 2] = up * gate / (1 + exp(-gate)).
    ``epilogue="glu_clamped"`` with ``epilogue_params`` = float32 ``[limit, alpha]`` on the device: the same layout, and
    out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    M, N, Kd = _linear_args(a, weight, bias, out, epilogue)
    bias = _gated_params(epilogue, bias, epilogue_params)
    if M == 0:
        return
    if row_scale is not None:
        _check(library().li_linear_scaled(_p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)), _i(_dt(out)), _i(M), _i(N), _i(Kd),
                                          _i(EPILOGUES[epilogue]), *_row_scale_args(row_scale, M), _stream(out)), "linear (scaled)")
        return
    _check(library().li_linear(_p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)), _i(_dt(out)), _i(M), _i(N), _i(Kd),
                               _i(EPILOGUES[epilogue]), _stream(out)), "linear")


def _row_scale_args(row_scale, M: int):
    ssq, width, eps = row_scale
    _need(ssq, "partial sums of squares", torch.float32)
    if ssq.dim() != 2 or ssq.shape[0] != M:
        raise KernelError(f"partial sums of squares of shape {tuple(ssq.shape)} for {M} tokens")
    return _p(ssq), _i(ssq.shape[1]), _i(int(width)), _f(float(eps))


def linear_scaled_accepts(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether :func:`linear` takes ``row_scale`` for these operands (bfloat16, at most 64 tokens)."""
    M, Kd = a.shape
    return bool(library().li_linear_scaled_accepts(_p(a), _p(weight), _p(out), _i(_dt(a)), _i(M), _i(weight.shape[0]), _i(Kd)))


def linear_add_scaled_parts(a: torch.Tensor, weight: torch.Tensor, x32: torch.Tensor, hprime: torch.Tensor) -> int:
    """How many partial sums per token :func:`linear_add_scaled` writes for these operands; 0 if no kernel takes them."""
    M, Kd = a.shape
    return int(library().li_linear_add_scaled_parts(_p(a), _p(weight), _p(x32), _p(hprime), _i(_dt(a)), _i(M), _i(weight.shape[0]), _i(Kd)))


def linear_add_scaled(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], x32: torch.Tensor,
                      norm_weight: torch.Tensor, hprime: torch.Tensor, ssq: torch.Tensor) -> None:
    """The product into the residual stream with the next RMSNorm half done, as one kernel (few bfloat16 tokens):
    ``x32 += a weight^T (+ bias)``; ``hprime = bfloat16(norm_weight * x32)``; ``ssq[t, p]`` = the sum of the new
    ``x32[t]^2`` over the columns of the product's tile p.  The normalised activation is
    ``hprime[t] / sqrt(sum_p ssq[t, p] / N + eps)``; :func:`linear` applies that factor to its own result
    (``row_scale``), :func:`apply_row_scale` to hprime itself."""
    M, Kd = a.shape
    N = weight.shape[0]
    _need(a, "linear input", torch.bfloat16)
    _need(weight, "linear weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "linear bias", torch.float32, (N,))
    _need(x32, "residual stream", torch.float32, (M, N))
    _need(norm_weight, "rmsnorm weight", torch.float32, (N,))
    _need(hprime, "weighted sum", a.dtype, (M, N))
    parts = linear_add_scaled_parts(a, weight, x32, hprime)
    if parts == 0:
        raise KernelError(f"linear_add_scaled: no kernel for {M} tokens, N={N}, K={Kd}")
    _need(ssq, "partial sums of squares", torch.float32, (M, parts))
    _check(library().li_linear_add_scaled(_p(a), _p(weight), _p(bias), _p(x32), _p(norm_weight), _p(hprime), _p(ssq), _i(_dt(a)),
                                          _i(M), _i(N), _i(Kd), _stream(hprime)), "linear_add_scaled")


def apply_row_scale(hprime: torch.Tensor, ssq: torch.Tensor, width: int, eps: float, out: torch.Tensor) -> None:
    """``out[t] = hprime[t] / sqrt(sum_p ssq[t, p] / width + eps)`` (bfloat16)."""
    M, H = hprime.shape
    _need(hprime, "weighted sum", torch.bfloat16)
    _need(out, "normalised output", torch.bfloat16, (M, H))
    p_ssq, nparts, w, e = _row_scale_args((ssq, width, eps), M)
    _check(library().li_apply_row_scale(_p(hprime), p_ssq, nparts, w, e, _p(out), _i(M), _i(H), _stream(out)), "apply_row_scale")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up rows as one [2 I, K] matrix in the order the swiglu epilogue reads:
    8 gate rows, the 8 up rows of the same outputs, the next 8 gate rows, ... (I a multiple of 8)."""
    I, Kd = gate.shape
    if I % 8 or up.shape != gate.shape:
        raise KernelError(f"interleave_gate_up: shapes {tuple(gate.shape)} / {tuple(up.shape)}, rows must be a multiple of 8")
    return torch.stack((gate.view(I // 8, 8, Kd), up.view(I // 8, 8, Kd)), dim=1).reshape(2 * I, Kd).contiguous()


LINEAR_IMPLEMENTATIONS = {"simt": 0, "gemv": 1, "tcgen05": 2, "gemv_tcgen05": 3}


def linear_with(which: str, a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                epilogue: Optional[str] = None, epilogue_params: Optional[torch.Tensor] = None) -> None:
    """:func:`linear` through one named kernel (``simt``, ``gemv``, ``tcgen05``, ``gemv_tcgen05``); an error
    if that kernel refuses the sizes.  For tests and measurements of a kernel alone."""
    M, N, Kd = _linear_args(a, weight, bias, out, epilogue)
    bias = _gated_params(epilogue, bias, epilogue_params)
    _check(library().li_linear_with(_i(LINEAR_IMPLEMENTATIONS[which]), _p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)),
                                    _i(_dt(out)), _i(M), _i(N), _i(Kd), _i(EPILOGUES[epilogue]), _stream(out)), f"linear[{which}]")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, denominators: torch.Tensor, rotary_dim: int,
                  slot_mapping: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  num_heads: int, num_kv_heads: int, head_dim: int, write: bool = True) -> None:
    """Rotate q (in place in ``qkv``) and k; store rotated k and plain v at each
    token's slot of the caches: keys ``[pages, kv_heads, page_size, head_dim]``, values
    transposed ``[pages, kv_heads, head_dim, page_size]``.
    With ``write`` false only q is rotated.  ``rotary_dim`` 0 (``denominators`` may be None): nothing is
    rotated, keys and values are stored as they are."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (num_heads + 2 * num_kv_heads) * head_dim))
    _need(positions, "positions", torch.int32, (T,))
    if rotary_dim:
        _need(denominators, "rope denominators", torch.float32, (rotary_dim // 2,))
    _need(slot_mapping, "slot mapping", torch.int32, (T,))
    _need(k_cache, "key cache", qkv.dtype)
    pages, nkv, page_size, dh = k_cache.shape
    _need(v_cache, "value cache", qkv.dtype, (pages, nkv, dh, page_size))
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    _check(library().li_rope_kv_write(
        _p(qkv), _i(_dt(qkv)), _p(positions), _p(denominators if rotary_dim else None), _i(rotary_dim), _p(slot_mapping), _p(k_cache), _p(v_cache),
        _i(T), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages), _i(1 if write else 0), _stream(qkv)),
        "rope_kv_write")


def linear_rope_kv(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], qkv: torch.Tensor,
                   positions: torch.Tensor, denominators: torch.Tensor, rotary_dim: int, slot_mapping: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                   write: bool = True, fused: bool = True, row_scale=None, cos_sin: Optional[torch.Tensor] = None) -> None:
    """The fused q|k|v projection followed by :func:`rope_kv_write`: ``qkv = a weight^T + bias``, q rotated in
    place, k rotated and v stored into the caches.  Keys and values are only guaranteed to be in the caches
    afterwards, not in ``qkv``.  For a few bfloat16 tokens both steps run as one kernel (the rotation is the
    product's epilogue); ``fused=False`` forces two kernels, for tests.  ``row_scale`` as in :func:`linear`.
    ``cos_sin``: the step's table from :func:`rope_table`; with it a long bfloat16 step (head_dim 128) rotates and
    writes the cache in the epilogue of the tensor-memory product too.  ``rotary_dim`` 0 (``denominators`` may be
    None): no rotation, as in :func:`rope_kv_write`."""
    T, Kd = a.shape
    N = (num_heads + 2 * num_kv_heads) * head_dim
    _need(a, "linear input")
    _need(weight, "qkv weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "qkv bias", torch.float32, (N,))
    _need(qkv, "qkv", a.dtype, (T, N))
    _need(positions, "positions", torch.int32, (T,))
    if rotary_dim:
        _need(denominators, "rope denominators", torch.float32, (rotary_dim // 2,))
    _need(slot_mapping, "slot mapping", torch.int32, (T,))
    if cos_sin is not None:
        _need(cos_sin, "rope table", torch.float32, (T, rotary_dim // 2, 2))
    _need(k_cache, "key cache", a.dtype)
    pages, nkv, page_size, dh = k_cache.shape
    _need(v_cache, "value cache", a.dtype, (pages, nkv, dh, page_size))
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    _check(library().li_linear_rope_kv(
        _p(a), _p(weight), _p(bias), _p(qkv), _i(_dt(a)), _p(positions), _p(denominators if rotary_dim else None), _i(rotary_dim), _p(slot_mapping),
        _p(k_cache), _p(v_cache), _i(T), _i(Kd), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages),
        _i(1 if write else 0), _i(1 if fused else 0),
        *(_row_scale_args(row_scale, T) if row_scale is not None else (_p(None), _i(0), _i(0), _f(0.0))), _p(cos_sin), _stream(qkv)),
        "linear_rope_kv")


def rope_table(positions: torch.Tensor, denominators: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, j] = (cos, sin)(float(positions[t]) / denominators[j])``: the angles of a step, for products that rotate in
    their epilogue (:func:`linear_rope_kv`)."""
    T = positions.shape[0]
    half = denominators.shape[0]
    _need(positions, "positions", torch.int32, (T,))
    _need(denominators, "rope denominators", torch.float32, (half,))
    _need(out, "rope table", torch.float32, (T, half, 2))
    _check(library().li_rope_table(_p(positions), _p(denominators), _i(half), _p(out), _i(T), _stream(out)), "rope_table")


ATTENTION_IMPLEMENTATIONS = {"general": 0, "decode": 1, "prefill": 2, "prefill_tcgen05": 3}


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, q_start: torch.Tensor, ctx_lens: torch.Tensor,
                    seq_of_token: torch.Tensor, positions: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                    max_q_len: int, max_ctx_len: int, implementation: Optional[str] = None,
                    old_lens: Optional[torch.Tensor] = None, singles: int = 0,
                    units: Optional[torch.Tensor] = None, unit_slots: Tuple[int, int] = (0, 0),
                    softcap: float = 0.0, slopes: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                    keep_first: int = 0, sinks: Optional[torch.Tensor] = None) -> None:
    """Causal grouped-query attention of the step's tokens over the paged cache.

    Queries are the first ``num_heads * head_dim`` columns of ``qkv`` (already
    rotated).  The token at position p of sequence s sees the cached keys
    ``max(0, p - window + 1) .. p`` of s, found through ``block_table[s]``.
    ``implementation`` (``general``, ``decode``, ``prefill``, ``prefill_tcgen05``) forces one kernel, for
    tests and measurements; it is an error if that kernel refuses the sizes.
    ``old_lens`` (int32 ``[S]``): how many keys of each sequence were in the cache before this step; needed when
    several sequences of the step are tokens of one request (None: all but each sequence's last key).
    ``singles``: how many sequences of a step with longer portions have one token (negative: not known).  They then
    go to the decode kernel, the rest to the kernel for portions (bfloat16).
    ``units`` (int32, from ``engine.batch.attention_units``): the work list of the kernel for long portions, with
    ``unit_slots`` = how many entries to launch when the single tokens are the decode kernel's, and when not.
    ``softcap`` > 0: a score s becomes ``softcap * tanh(s / softcap)`` (after the scale).  ``slopes`` (float32
    ``[num_heads]``): ``slopes[h] * (p - key)`` is taken off the scores of head h, a penalty linear in the distance.
    ``gate`` (run dtype ``[T, num_heads]``): head h's output is multiplied by ``sigmoid(gate[t, h])``.
    ``keep_first`` (with a window): the keys ``0 .. keep_first - 1`` stay visible behind the window, at their own positions.
    ``sinks`` (float32 ``[num_heads]``): ``exp(sinks[h])`` joins the denominator of head h's softmax once; it has no key
    and no value and is not scaled."""
    T = qkv.shape[0]
    S = ctx_lens.shape[0]
    _need(qkv, "qkv", None, (T, (num_heads + 2 * num_kv_heads) * head_dim))
    _need(out, "attention output", qkv.dtype, (T, num_heads * head_dim))
    _need(k_cache, "key cache", qkv.dtype)
    _need(v_cache, "value cache", qkv.dtype, (k_cache.shape[0], k_cache.shape[1], k_cache.shape[3], k_cache.shape[2]))
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (S + 1,))
    _need(ctx_lens, "ctx_lens", torch.int32, (S,))
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    pages, nkv, page_size, dh = k_cache.shape
    if block_table.dim() != 2 or block_table.shape[0] != S:
        raise KernelError(f"block table must be [{S}, max_blocks], got {tuple(block_table.shape)}")
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    if block_table.shape[1] * page_size < max_ctx_len:
        raise KernelError(f"block table of {block_table.shape[1]} pages cannot cover a context of {max_ctx_len}")
    if old_lens is not None:
        _need(old_lens, "old_lens", torch.int32, (S,))
    if units is not None:
        _need(units, "attention work list", torch.int32)
        if units.numel() < 4 + 4 * max(unit_slots) or units.data_ptr() % 16:
            raise KernelError(f"attention work list of {units.numel()} words cannot hold {max(unit_slots)} entries (or is not 16-byte aligned)")
    args = (_p(qkv), _p(out), _p(k_cache), _p(v_cache), _i(_dt(qkv)), _p(block_table), _i(block_table.shape[1]),
            _p(q_start), _p(ctx_lens), _p(seq_of_token), _p(positions), _i(T), _i(S),
            _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages), _f(scale),
            _i(0 if window is None else int(window)), _i(max_q_len), _i(max_ctx_len), _p(old_lens), _i(int(singles)),
            _p(units), _i(int(unit_slots[0])), _i(int(unit_slots[1])), _f(float(softcap or 0.0)), _p(slopes), _p(gate), _i(int(keep_first or 0)), _p(sinks), _stream(out))
    if sinks is not None:
        _need(sinks, "softmax sinks", torch.float32, (num_heads,))
    if slopes is not None:
        _need(slopes, "distance slopes", torch.float32, (num_heads,))
    if gate is not None:
        _need(gate, "head gate", qkv.dtype, (T, num_heads))
    if implementation is None:
        _check(library().li_paged_attention(*args), "paged_attention")
    else:
        _check(library().li_paged_attention_with(_i(ATTENTION_IMPLEMENTATIONS[implementation]), *args),
               f"paged_attention[{implementation}]")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = up * gate / (1 + exp(-gate)) with gate_up = [gate | up] along the last axis."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    _need(out, "swiglu output", gate_up.dtype, (T, I2 // 2))
    _check(library().li_swiglu(_p(gate_up), _p(out), _i(_dt(out)), _i(T), _i(I2 // 2), _stream(out)), "swiglu")


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
    gate_up = [gate | up] along the last axis."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    _need(out, "glu output", gate_up.dtype, (T, I2 // 2))
    _check(library().li_glu_clamped(_p(gate_up), _p(out), _i(_dt(out)), _i(T), _i(I2 // 2), _f(limit), _f(alpha), _stream(out)), "glu_clamped")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = a N(z) + b N(z^2) + c N(z^3) + e`` per row of ``z`` [T, n], powers element by element, ``N(v) = v / sqrt(mean(v^2)
    + eps)``; ``coef`` = (a, b, c, e), float32 on the device.  Means and the result in float32, one rounding."""
    T, n = z.shape
    _need(z, "polynorm input")
    _need(coef, "polynorm coefficients", torch.float32, (4,))
    _need(out, "polynorm output", z.dtype, (T, n))
    _check(library().li_polynorm(_p(z), _i(_dt(z)), _p(coef), _f(eps), _p(out), _i(T), _i(n), _stream(out)), "polynorm")


def mul_sigmoid(x: torch.Tensor, gate: torch.Tensor, gate_col: int = 0, group: int = 1) -> None:
    """``x[t, i] *= sigmoid(gate[t, gate_col + i // group])`` in place (float32 arithmetic, one rounding): an output gate per
    element, or with ``group`` a head's width one per head."""
    T, n = x.shape
    _need(x, "gated activation")
    _need(gate, "gate", x.dtype)
    if gate.dim() != 2 or gate.shape[0] != T or group < 1 or n % group or gate_col + n // group > gate.shape[1]:
        raise KernelError(f"mul_sigmoid: a gate of shape {tuple(gate.shape)} from column {gate_col} for {T} rows of {n} in groups of {group}")
    _check(library().li_mul_sigmoid(_p(x), _p(gate), _i(_dt(x)), _i(gate.shape[1]), _i(int(gate_col)), _i(int(group)), _i(T), _i(n), _stream(x)),
           "mul_sigmoid")


class WeightedPair:
    """Two activations that stand for ``sa * a + sb * b`` (two mixers side by side) until a kernel that consumes the sum
    takes it in (:func:`hc_update`); :meth:`materialize` adds them up with a kernel of its own."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, sa: float, sb: float) -> None:
        self.a, self.b, self.sa, self.sb = a, b, float(sa), float(sb)

    def materialize(self) -> torch.Tensor:
        out = torch.empty_like(self.a)
        weighted_sum2(self.a, self.b, self.sa, self.sb, out)
        return out


def weighted_sum2(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float, out: torch.Tensor) -> None:
    """out = sa * a + sb * b (run dtype in and out, the sum in float32)."""
    _need(a, "first operand")
    _need(b, "second operand", a.dtype, a.shape)
    _need(out, "weighted sum", a.dtype, a.shape)
    _check(library().li_weighted_sum2(_p(a), _p(b), _f(sa), _f(sb), _p(out), _i(_dt(a)), _l(a.numel()), _stream(out)), "weighted_sum2")


# --------------------------------------------------------------------------
# several residual streams (hyper-connections) and learned positions
# --------------------------------------------------------------------------

def add_position_rows(x32: torch.Tensor, table: torch.Tensor, positions: torch.Tensor) -> None:
    """x32[t] += table[positions[t]] (learned absolute positions; the table in the run dtype)."""
    T, H = x32.shape
    _need(x32, "residual stream", torch.float32)
    _need(table, "position table", None, (table.shape[0], H))
    _need(positions, "positions", torch.int32, (T,))
    _check(library().li_add_position_rows(_p(x32), _p(table), _i(_dt(table)), _p(positions), _i(T), _i(H), _i(table.shape[0]), _stream(x32)),
           "add_position_rows")


def hc_expand(x32: torch.Tensor, xs: torch.Tensor) -> None:
    """xs[t, a] = x32[t] for every stream a; xs float32 ``[T, streams, H]``."""
    T, H = x32.shape
    _need(x32, "residual stream", torch.float32)
    _need(xs, "streams", torch.float32, (T, xs.shape[1], H))
    _check(library().li_hc_expand(_p(x32), _p(xs), _i(T), _i(xs.shape[1]), _i(H), _stream(xs)), "hc_expand")


def hc_read_norm(xs: torch.Tensor, in_w: Optional[torch.Tensor], rows: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out: torch.Tensor) -> None:
    """out[r] = rmsnorm(sum_s in_w[s] xs[rows[r], s]) * weight.  ``in_w`` None: the plain sum of the streams;
    ``rows`` None: every token in order."""
    T, s, H = xs.shape
    _need(xs, "streams", torch.float32)
    if in_w is not None:
        _need(in_w, "read weights", torch.float32, (s,))
    R = T if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "normalised output", None, (R, H))
    _check(library().li_hc_read_norm(_p(xs), _p(in_w), _p(rows), _p(weight), _f(eps), _p(out), _i(_dt(out)), _i(R), _i(T), _i(s), _i(H),
                                     _stream(out)), "hc_read_norm")


def hc_update(xs: torch.Tensor, y, mix: torch.Tensor, out_w: torch.Tensor, next_in: Optional[torch.Tensor] = None,
              next_weight: Optional[torch.Tensor] = None, eps: float = 0.0, next_out: Optional[torch.Tensor] = None) -> None:
    """xs[t, r] = sum_s mix[s, r] xs[t, s] + out_w[r] y[t], every stream from the old ones, in place; with ``next_out``
    also the next sublayer's input: next_out[t] = rmsnorm(sum_r next_in[r] xs[t, r]) * next_weight.
    ``y`` may be a :class:`WeightedPair` (a, b, sa, sb): the sublayer's output is then sa * a + sb * b, summed in float32."""
    T, s, H = xs.shape
    y2, s1, s2 = None, 1.0, 0.0
    if isinstance(y, WeightedPair):
        y, y2, s1, s2 = y.a, y.b, float(y.sa), float(y.sb)
        _need(y2, "sublayer output (second)", y.dtype, (T, H))
    _need(xs, "streams", torch.float32)
    _need(y, "sublayer output", None, (T, H))
    _need(mix, "stream mix", torch.float32, (s, s))
    _need(out_w, "write weights", torch.float32, (s,))
    if next_out is not None:
        _need(next_in, "read weights", torch.float32, (s,))
        _need(next_weight, "rmsnorm weight", torch.float32, (H,))
        _need(next_out, "normalised output", y.dtype, (T, H))
    _check(library().li_hc_update(_p(xs), _p(y), _p(y2), _f(s1), _f(s2), _i(_dt(y)), _p(mix), _p(out_w), _p(next_in if next_out is not None else None),
                                  _p(next_weight if next_out is not None else None), _f(eps), _p(next_out), _i(T), _i(s), _i(H), _stream(xs)),
           "hc_update")


# --------------------------------------------------------------------------
# mixers with a state of fixed size per request
# --------------------------------------------------------------------------

def _state_args(state: torch.Tensor, offset: int):
    _need(state, "state", torch.float32)
    if state.dim() != 2:
        raise KernelError(f"state must be [slots, elements], got {tuple(state.shape)}")
    return _p(state), _l(state.shape[1]), _l(int(offset))


def causal_conv_silu(x: torch.Tensor, col: int, weight: torch.Tensor, bias: torch.Tensor, state: torch.Tensor, state_off: int,
                     q_start: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, shift: bool = False) -> None:
    """Depthwise causal convolution and silu over the C channels at column ``col`` of ``x`` [T, *]:
    ``out[t, c] = silu(bias[c] + sum_k weight[c, k] * input_(t - taps + 1 + k)[c])``; inputs before a sequence's portion
    come from ``state[slot, state_off:]`` ([taps - 1, C], oldest first).  The state is not changed
    (:func:`conv_state_shift` does that afterwards), unless ``shift``: the caller promises that every sequence of the
    step has one token, and the state moves on in the same launch."""
    T = x.shape[0]
    C, taps = weight.shape
    _need(x, "convolution input")
    _need(weight, "convolution weight", torch.float32)
    _need(bias, "convolution bias", torch.float32, (C,))
    _need(out, "convolution output", x.dtype, (T, C))
    _need(q_start, "q_start", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(slots, "state slots", torch.int32)
    st, stride, off = _state_args(state, state_off)
    if state_off + (taps - 1) * C > state.shape[1]:
        raise KernelError("causal_conv_silu: the state is too small for the convolution's inputs")
    _check(library().li_causal_conv_silu(_p(x), _i(_dt(x)), _i(x.shape[1]), _i(col), _p(weight), _p(bias), st, stride, off, _p(q_start),
                                         _p(seq_of_token), _p(slots), _p(out), _i(T), _i(C), _i(taps), _i(1 if shift else 0), _stream(out)), "causal_conv_silu")


def conv_state_shift(x: torch.Tensor, col: int, channels: int, taps: int, state: torch.Tensor, state_off: int, q_start: torch.Tensor,
                     slots: torch.Tensor) -> None:
    """After a step's convolution: each sequence's state keeps the last ``taps - 1`` inputs it has now seen."""
    _need(x, "convolution input")
    _need(q_start, "q_start", torch.int32)
    S = q_start.shape[0] - 1
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, off = _state_args(state, state_off)
    _check(library().li_conv_state_shift(_p(x), _i(_dt(x)), _i(x.shape[1]), _i(col), st, stride, off, _p(q_start), _p(slots), _i(S),
                                         _i(channels), _i(taps), _stream(x)), "conv_state_shift")


class ScanChunks:
    """The long portions of a step cut into chunks that the scans run side by side (see :func:`ssm_scan`):
    ``seg`` int32 ``[chunks, 4]`` (first token, end, chunk, state slot) and ``runs`` int32 ``[sequences, 3]`` (first chunk,
    chunks, state slot) on the device.  Made from the step's host-side metadata, once per step."""

    LENGTH = 64              # tokens a chunk
    FROM = 128               # the longest portion of a step from which its scans run in chunks

    def __init__(self, q_start, slots, device, length: int = LENGTH) -> None:
        seg, runs = [], []
        for s, slot in enumerate(slots):
            lo, hi = int(q_start[s]), int(q_start[s + 1])
            if hi <= lo:
                continue
            first = len(seg)
            for b in range(lo, hi, length):
                seg.append((b, min(hi, b + length), len(seg), int(slot)))
            runs.append((first, len(seg) - first, int(slot)))
        self.count, self.nruns = len(seg), len(runs)
        self.seg = torch.tensor(seg, dtype=torch.int32).to(device)
        self.runs = torch.tensor(runs, dtype=torch.int32).to(device)


def _scan_passes(chunks: Optional["ScanChunks"], elements: int, heads: int, device):
    """(seg pointer, S, mode, chunk states, chunk decays) of every pass a scan makes: one over whole sequences, or two over chunks."""
    if chunks is None:
        return None
    return (torch.empty((chunks.count, elements), dtype=torch.float32, device=device),
            torch.empty((chunks.count, heads), dtype=torch.float32, device=device))


def ssm_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, y32: torch.Tensor, heads: int, head_dim: int,
             state_size: int, groups: int, chunks: Optional[ScanChunks] = None) -> None:
    """The selective state-space recurrence per head, state ``S [state_size, head_dim]`` at the start of ``state[slot]``:
    ``dt = softplus(proj[t, dt_col + h] + dt_bias[h])``; ``S = exp(-exp(A_log[h]) dt) S + dt B_t x_t^T``;
    ``y_t = S^T C_t + D[h] x_t``.  ``xbc`` [T, heads * head_dim + 2 * groups * state_size] holds x | B | C.  The state
    is kept column by column, ``[heads, head_dim, state_size]``.

    ``chunks``: the step's sequences cut into chunks (a step with long portions).  Every chunk then runs twice, side by side
    with the others: from a state of zeros to find what it adds, and, after the states have been carried from chunk to
    chunk in order (:func:`ScanChunks`, ``li_scan_carry``), from the state it really starts with, for its outputs."""
    T, C = xbc.shape
    _need(xbc, "x|B|C")
    _need(proj, "projection", xbc.dtype)
    for t, n in ((dt_bias, "dt_bias"), (A_log, "A_log"), (D, "D")):
        _need(t, n, torch.float32, (heads,))
    _need(y32, "scan output", torch.float32, (T, heads * head_dim))
    S = q_start.shape[0] - 1
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, _ = _state_args(state, 0)
    if heads * head_dim * state_size > state.shape[1] or dt_col + heads > proj.shape[1]:
        raise KernelError("ssm_scan: the state or the projection is too small")
    dt_ptr = ctypes.c_void_p(proj.data_ptr() + dt_col * proj.element_size())

    def run(seg, n, mode, cstate, cdecay):
        _check(library().li_ssm_scan(_p(xbc), _i(_dt(xbc)), _i(C), dt_ptr, _i(proj.shape[1]), _p(dt_bias), _p(A_log), _p(D), st, stride,
                                     _p(q_start), _p(slots), _p(y32), _i(n), _i(heads), _i(head_dim), _i(state_size), _i(groups),
                                     _p(seg), _i(mode), _p(cstate), _p(cdecay), _stream(y32)), "ssm_scan")

    if chunks is None or chunks.count == 0:
        return run(None, S, 0, None, None)
    cstate, cdecay = _scan_passes(chunks, heads * head_dim * state_size, heads, xbc.device)
    run(chunks.seg, chunks.count, 1, cstate, cdecay)
    _check(library().li_scan_carry(st, stride, _p(cstate), _p(cdecay), _p(None), _p(chunks.seg), _p(chunks.runs), _i(chunks.nruns), _i(heads),
                                   _i(head_dim * state_size), _i(0), _stream(y32)), "scan_carry")
    run(chunks.seg, chunks.count, 2, cstate, cdecay)


def decay_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
               slots: torch.Tensor, out32: torch.Tensor, heads: int, dim: int, vdim: int, chunks: Optional[ScanChunks] = None) -> None:
    """Linear attention with a constant decay per head, state ``S [dim, vdim]`` per head at the start of
    ``state[slot]``: ``S = decay[h] S + k_t v_t^T``; ``out_t = S^T q_t``; q, k, v are silu of the columns of ``qkv``
    at ``q_col``, ``k_col``, ``v_col`` (heads side by side).  The state is kept column by column, ``[heads, vdim, dim]``.
    ``chunks``: as in :func:`ssm_scan`."""
    T = qkv.shape[0]
    _need(qkv, "q|k|v")
    _need(decay, "decay", torch.float32, (heads,))
    _need(out32, "scan output", torch.float32, (T, heads * vdim))
    S = q_start.shape[0] - 1
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, _ = _state_args(state, 0)
    if heads * dim * vdim > state.shape[1]:
        raise KernelError("decay_scan: the state is too small")

    def run(seg, n, mode, cstate):
        _check(library().li_decay_scan(_p(qkv), _i(_dt(qkv)), _i(qkv.shape[1]), _i(q_col), _i(k_col), _i(v_col), _p(decay), st, stride, _p(q_start),
                                       _p(slots), _p(out32), _i(n), _i(heads), _i(dim), _i(vdim), _p(seg), _i(mode), _p(cstate), _stream(out32)),
               "decay_scan")

    if chunks is None or chunks.count == 0:
        return run(None, S, 0, None)
    cstate = torch.empty((chunks.count, heads * dim * vdim), dtype=torch.float32, device=qkv.device)
    run(chunks.seg, chunks.count, 1, cstate)
    _check(library().li_scan_carry(st, stride, _p(cstate), _p(None), _p(decay), _p(chunks.seg), _p(chunks.runs), _i(chunks.nruns), _i(heads),
                                   _i(dim * vdim), _i(0), _stream(out32)), "scan_carry")
    run(chunks.seg, chunks.count, 2, cstate)


def gla_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, za: torch.Tensor, za_col: int, tau: float, state: torch.Tensor,
             q_start: torch.Tensor, slots: torch.Tensor, out32: torch.Tensor, heads: int, dim: int, vdim: int,
             chunks: Optional[ScanChunks] = None) -> None:
    """Linear attention with a decay per token and key channel, state ``S [dim, vdim]`` per head at the start of
    ``state[slot]``: ``S = diag(a_t) S + k_t v_t^T``; ``out_t = S^T q_t / sqrt(dim)``; ``a_t = sigmoid(z_t)^(1 / tau)`` with
    the float32 logits z in the ``heads * dim`` columns of ``za`` from ``za_col``; q, k, v are the columns of ``qkv`` at
    ``q_col``, ``k_col``, ``v_col`` as they are.  The state is kept column by column, ``[heads, vdim, dim]``.
    ``chunks``: as in :func:`ssm_scan`; a chunk's decay is a number per head and key channel."""
    T = qkv.shape[0]
    _need(qkv, "q|k|v")
    _need(za, "decay logits", torch.float32)
    _need(out32, "scan output", torch.float32, (T, heads * vdim))
    S = q_start.shape[0] - 1
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, _ = _state_args(state, 0)
    if heads * dim * vdim > state.shape[1] or za.shape[0] != T:
        raise KernelError("gla_scan: the state or the decays are too small")

    def run(seg, n, mode, cstate, cdecay):
        _check(library().li_gla_scan(_p(qkv), _i(_dt(qkv)), _i(qkv.shape[1]), _i(q_col), _i(k_col), _i(v_col), _p(za), _i(za.shape[1]), _i(za_col),
                                     _f(1.0 / float(tau)), _f(float(dim) ** -0.5), st, stride, _p(q_start), _p(slots), _p(out32), _i(n), _i(heads),
                                     _i(dim), _i(vdim), _p(seg), _i(mode), _p(cstate), _p(cdecay), _stream(out32)), "gla_scan")

    if chunks is None or chunks.count == 0:
        return run(None, S, 0, None, None)
    cstate = torch.empty((chunks.count, heads * dim * vdim), dtype=torch.float32, device=qkv.device)
    cdecay = torch.empty((chunks.count, heads * dim), dtype=torch.float32, device=qkv.device)
    run(chunks.seg, chunks.count, 1, cstate, cdecay)
    _check(library().li_scan_carry(st, stride, _p(cstate), _p(cdecay), _p(None), _p(chunks.seg), _p(chunks.runs), _i(chunks.nruns), _i(heads),
                                   _i(dim * vdim), _i(dim), _stream(out32)), "scan_carry")
    run(chunks.seg, chunks.count, 2, cstate, cdecay)


def delta_row_elements(dim: int) -> int:
    """How many floats a prepared vector of ``dim`` key channels takes (32, 64, 128 or 256: zeros behind ``dim``)."""
    if dim > 256:
        raise KernelError(f"the delta rule takes keys of at most 256 elements, got {dim}")
    return 32 if dim <= 32 else 64 if dim <= 64 else 128 if dim <= 128 else 256


def delta_prepare(proj: torch.Tensor, col: int, b_col: int, conv_w: torch.Tensor, state: torch.Tensor, state_off: int, q_start: torch.Tensor,
                  seq_of_token: torch.Tensor, slots: torch.Tensor, za: torch.Tensor, za_col: int, A_log: torch.Tensor, prep_qk: torch.Tensor,
                  prep_g: torch.Tensor, v32: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float = 1e-6,
                  shift: bool = False) -> None:
    """What the gated delta rule needs of every token and does not depend on the state.  ``proj`` [T, *] holds the channels
    q | k | v (``kv_heads * dim``, ``kv_heads * dim``, ``heads * vdim``) from column ``col`` and beta's input at ``b_col + h``.
    Each channel passes a causal convolution (``conv_w`` float32 [channels, taps], the last column the token's own; inputs
    before a portion from ``state[slot, state_off:]`` as [taps - 1, channels], oldest first) and silu.  q and k become unit
    vectors per key head (``x / sqrt(sum x^2 + unit_eps)``, q also times ``dim^-1/2``).  Written, all float32, with ``DP`` =
    :func:`delta_row_elements`: ``prep_qk`` [T, kv_heads, 2 DP + 4] = (q | k | k . q), ``prep_g`` [T, heads, DP + 4] = (g | beta)
    with ``g = exp(-exp(A_log[h]) softplus(za[:, za_col + h dim + i]))`` (``za`` float32) and ``beta = sigmoid(.)``, ``v32``
    [T, heads * vdim].  The state is not changed (:func:`conv_state_shift` does that afterwards), unless ``shift``: the caller
    promises that every sequence of the step has one token."""
    T = proj.shape[0]
    C = 2 * kv_heads * dim + heads * vdim
    DP = delta_row_elements(dim)
    _need(proj, "projections")
    _need(conv_w, "convolution weight", torch.float32)
    if conv_w.dim() != 2 or conv_w.shape[0] != C:
        raise KernelError(f"delta_prepare: convolution weight of shape {tuple(conv_w.shape)} for {C} channels")
    taps = conv_w.shape[1]
    _need(za, "decay inputs", torch.float32)
    _need(A_log, "A_log", torch.float32, (heads,))
    _need(prep_qk, "prepared q and k", torch.float32, (T, kv_heads, 2 * DP + 4))
    _need(prep_g, "prepared decays", torch.float32, (T, heads, DP + 4))
    _need(v32, "prepared values", torch.float32, (T, heads * vdim))
    _need(q_start, "q_start", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(slots, "state slots", torch.int32)
    st, stride, off = _state_args(state, state_off)
    if state_off + (taps - 1) * C > state.shape[1] or za.shape[0] != T:
        raise KernelError("delta_prepare: the state or the decays are too small")
    _check(library().li_delta_prepare(_p(proj), _i(_dt(proj)), _i(proj.shape[1]), _i(int(col)), _i(int(b_col)), _p(conv_w), _i(taps), st, stride, off,
                                      _p(q_start), _p(seq_of_token), _p(slots), _p(za), _i(za.shape[1]), _i(int(za_col)), _p(A_log),
                                      _f(float(dim) ** -0.5), _f(float(unit_eps)), _p(prep_qk), _p(prep_g), _p(v32), _i(T), _i(heads), _i(kv_heads),
                                      _i(dim), _i(vdim), _i(1 if shift else 0), _stream(v32)), "delta_prepare")


def delta_scan(prep_qk: torch.Tensor, prep_g: torch.Tensor, v32: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
               out32: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int) -> None:
    """The gated delta rule with a decay per token, head and key channel over what :func:`delta_prepare` made, state
    ``S [dim, vdim]`` per head at the start of ``state[slot]`` (kept column by column, ``[heads, vdim, dim]``):
    ``S = diag(g_t) S``; ``u = beta_t (v_t - S^T k_t)``; ``S = S + k_t u^T``; ``out_t = S^T q_t``; head h uses the q and k of key
    head ``h // (heads / kv_heads)``.  A sequence's tokens run in order, in one piece."""
    T = v32.shape[0]
    DP = delta_row_elements(dim)
    _need(prep_qk, "prepared q and k", torch.float32, (T, kv_heads, 2 * DP + 4))
    _need(prep_g, "prepared decays", torch.float32, (T, heads, DP + 4))
    _need(v32, "prepared values", torch.float32, (T, heads * vdim))
    _need(out32, "scan output", torch.float32, (T, heads * vdim))
    S = q_start.shape[0] - 1
    _need(q_start, "q_start", torch.int32)
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, _ = _state_args(state, 0)
    if heads * dim * vdim > state.shape[1]:
        raise KernelError("delta_scan: the state is too small")
    _check(library().li_delta_scan(_p(prep_qk), _p(prep_g), _p(v32), st, stride, _p(q_start), _p(slots), _p(out32), _i(S), _i(heads), _i(kv_heads),
                                   _i(dim), _i(vdim), _stream(out32)), "delta_scan")


def channel_scan(x: torch.Tensor, x_col: int, bc: torch.Tensor, b_col: int, c_col: int, dt32: torch.Tensor, z: torch.Tensor, z_col: int,
                 A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, y: torch.Tensor,
                 chunks: Optional[ScanChunks] = None) -> None:
    """The selective scan with a state row per channel, ``S [inner, N]`` at the start of ``state[slot]``:
    ``dt = softplus(dt32[t])`` (float32, one per channel); ``S[c] = exp(-exp(A_log[c]) dt_c) S[c] + dt_c x_c B_t``;
    ``y[t, c] = (S[c] . C_t + D[c] x_c) silu(z_c)``.  x: the ``inner`` columns of ``x`` from ``x_col``; B and C: N columns of
    ``bc`` from ``b_col`` and ``c_col``; z: the columns of ``z`` from ``z_col``; y in the run dtype.  ``chunks``: as in
    :func:`ssm_scan`; a chunk's decay is a number per element of the state."""
    T = x.shape[0]
    inner, N = A_log.shape
    _need(x, "scan input")
    _need(bc, "B|C", x.dtype)
    _need(z, "gate", x.dtype)
    _need(dt32, "step sizes", torch.float32, (T, inner))
    _need(A_log, "A_log", torch.float32)
    _need(D, "D", torch.float32, (inner,))
    _need(y, "scan output", x.dtype, (T, inner))
    S = q_start.shape[0] - 1
    _need(slots, "state slots", torch.int32, (S,))
    st, stride, _ = _state_args(state, 0)
    if inner * N > state.shape[1] or bc.shape[0] != T or z.shape[0] != T:
        raise KernelError("channel_scan: the state or an input is too small")

    def run(seg, n, mode, cstate, cdecay):
        _check(library().li_channel_scan(_p(x), _i(_dt(x)), _i(x.shape[1]), _i(x_col), _p(bc), _i(bc.shape[1]), _i(b_col), _i(c_col), _p(dt32),
                                         _i(dt32.shape[1]), _p(z), _i(z.shape[1]), _i(z_col), _p(A_log), _p(D), st, stride, _p(q_start), _p(slots),
                                         _p(y), _i(n), _i(inner), _i(N), _p(seg), _i(mode), _p(cstate), _p(cdecay), _stream(y)), "channel_scan")

    if chunks is None or chunks.count == 0:
        return run(None, S, 0, None, None)
    cstate = torch.empty((chunks.count, inner * N), dtype=torch.float32, device=x.device)
    cdecay = torch.empty((chunks.count, inner * N), dtype=torch.float32, device=x.device)
    run(chunks.seg, chunks.count, 1, cstate, cdecay)
    _check(library().li_scan_carry(st, stride, _p(cstate), _p(cdecay), _p(None), _p(chunks.seg), _p(chunks.runs), _i(chunks.nruns), _i(1),
                                   _i(inner * N), _i(inner * N), _stream(y)), "scan_carry")
    run(chunks.seg, chunks.count, 2, cstate, cdecay)


def gated_rmsnorm(y32: torch.Tensor, gate: torch.Tensor, gate_col: int, weight: torch.Tensor, eps: float, groups: int, gate_first: bool,
                  out: torch.Tensor, gate_act: str = "sigmoid") -> None:
    """RMSNorm of ``y32`` [T, n] in ``groups`` equal parts, times ``weight``.  ``gate_first``: y is multiplied by
    silu(gate) before the norm; otherwise the normalised result is multiplied by sigmoid(gate) (``gate_act`` "silu": by
    silu(gate)).  The gate is the n columns of ``gate`` from ``gate_col``."""
    T, n = y32.shape
    _need(y32, "norm input", torch.float32)
    _need(gate, "gate")
    _need(weight, "rmsnorm weight", torch.float32, (n,))
    _need(out, "norm output", gate.dtype, (T, n))
    _check(library().li_gated_rmsnorm(_p(y32), _p(gate), _i(_dt(gate)), _i(gate.shape[1]), _i(gate_col), _p(weight), _f(eps),
                                      _i(0 if gate_first else (2 if gate_act == "silu" else 1)), _p(out), _i(T), _i(n), _i(groups), _stream(out)),
           "gated_rmsnorm")


# --------------------------------------------------------------------------
# norms on both sides of a sublayer, a vector per pass, norms of column ranges
# --------------------------------------------------------------------------

class RowSum:
    """An activation [T, H] that stands for ``sum_k rows[place_of[t * top + k]]`` (times ``weights[t, k]`` if given): what a
    mixture of experts leaves, until a kernel that consumes the sum takes it in (:func:`norm_add_norm`);
    :meth:`materialize` adds the rows up with a kernel of its own (:func:`moe_combine`)."""

    def __init__(self, rows: torch.Tensor, place_of: torch.Tensor, top: int, weights: Optional[torch.Tensor] = None) -> None:
        self.rows, self.place_of, self.top, self.weights = rows, place_of, int(top), weights
        self.shape = (place_of.numel() // self.top, rows.shape[1])
        self.dtype = rows.dtype

    def materialize(self) -> torch.Tensor:
        y = torch.empty(self.shape, dtype=self.rows.dtype, device=self.rows.device)
        moe_combine(self.rows, self.place_of, self.weights, self.top, y)
        return y


SCALE_ONLY = 2          # the `centered` of a "norm" that is a factor per channel and nothing else


def norm_add_norm(x32: torch.Tensor, y, post: Optional[tuple], nxt: Optional[tuple], out: Optional[torch.Tensor],
                  rows: Optional[torch.Tensor] = None) -> None:
    """Per token: ``x32 += post(y)``, then ``out = nxt(x32)``.  A norm is a tuple ``(weight, centered, eps)``: centered takes
    the mean off and divides by the root of the variance (mean of squared deviations) + eps, not centered divides by the
    root of the mean of squares + eps; both multiply by the weight.  ``centered`` 2 (:data:`SCALE_ONLY`): no statistic at
    all, the row times the weight (a learned factor per channel).  ``post`` None: ``x32 += y``; ``y`` None: nothing is
    added; ``nxt`` None: no output; ``nxt`` with a weight of None: ``out`` is ``x32`` as it is, in the run dtype.  ``rows`` (int32, only without ``y``): ``out[r] = nxt(x32[rows[r]])``.  ``y`` may be a
    :class:`RowSum`: the sum is then taken inside this kernel, in float32."""
    n_src, H = x32.shape
    _need(x32, "residual stream", torch.float32)
    R = n_src if rows is None else rows.shape[0]
    places, top, y_weights = None, 0, None
    if isinstance(y, RowSum):
        if H > 8192:
            y = y.materialize()
        else:
            places, top, y_weights, y = y.place_of, y.top, y.weights, y.rows
            _need(y, "rows of the sublayer's output", None, (y.shape[0], H))
            _need(places, "places of a token's rows", torch.int32, (n_src * top,))
            if y_weights is not None:
                _need(y_weights, "weights of a token's rows", torch.float32, (n_src, top))
    if y is not None and places is None:
        _need(y, "sublayer output", None, (n_src, H))
    if y is not None:
        if rows is not None:
            raise KernelError("norm_add_norm: gathered rows cannot take a sublayer's output")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    wp, cp, ep = post if post is not None else (None, False, 0.0)
    wn, cn, en = nxt if nxt is not None else (None, False, 0.0)
    if wp is not None:
        _need(wp, "norm weight (after the sublayer)", torch.float32, (H,))
    if wn is not None:
        _need(wn, "norm weight (before the next sublayer)", torch.float32, (H,))
    if nxt is not None:
        _need(out, "normalised output", y.dtype if y is not None else None, (R, H))
    dt = _dt(y) if y is not None else _dt(out)
    _check(library().li_norm_add_norm(_p(x32), _p(y), _i(dt), _p(wp), _i(int(cp)), _f(ep), _p(wn), _i(int(cn)), _f(en),
                                      _p(out if nxt is not None else None), _p(rows), _i(R), _i(n_src), _i(H), _p(places), _i(top), _p(y_weights),
                                      _stream(x32)), "norm_add_norm")


def add_row(x32: torch.Tensor, row: torch.Tensor) -> None:
    """x32[t] += row for every token (float32)."""
    T, H = x32.shape
    _need(x32, "residual stream", torch.float32)
    _need(row, "row", torch.float32, (H,))
    _check(library().li_add_row(_p(x32), _p(row), _i(T), _i(H), _stream(x32)), "add_row")


def rmsnorm_cols(x: torch.Tensor, col: int, n: int, width: int, weight: torch.Tensor, eps: float, out: torch.Tensor, col_a: int,
                 col_b: int = -1) -> None:
    """RMS norm of the columns ``col .. col + n - 1`` of ``x`` (the mean of squares over ``width`` elements: fewer than n when
    the last columns are zero padding), times ``weight`` [n]; written to ``out`` at column ``col_a`` and, if given, ``col_b``."""
    T = x.shape[0]
    _need(x, "norm input")
    _need(weight, "rmsnorm weight", torch.float32, (n,))
    _need(out, "norm output", x.dtype)
    if out.shape[0] != T:
        raise KernelError(f"rmsnorm_cols: {out.shape[0]} output rows for {T} tokens")
    _check(library().li_rmsnorm_cols(_p(x), _i(_dt(x)), _i(x.shape[1]), _i(col), _i(n), _i(width), _p(weight), _f(eps), _p(out), _i(out.shape[1]),
                                     _i(col_a), _i(col_b), _i(T), _stream(out)), "rmsnorm_cols")


def conv_norm_rope_kv(proj: torch.Tensor, out: torch.Tensor, conv_w: Optional[torch.Tensor], state: Optional[torch.Tensor], state_off: int,
                      q_start: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, q_norm: Optional[torch.Tensor],
                      k_norm: Optional[torch.Tensor], eps: float, norm_width: int, positions: torch.Tensor,
                      denominators: Optional[torch.Tensor], rotary_dim: int, slot_mapping: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, write: bool = True, shift: bool = False,
                      to_cache: bool = True, row_rinv: Optional[torch.Tensor] = None) -> None:
    """What stands between a q|k|v product ``proj`` [T, (heads + 2 kv_heads) head_dim] and attention: a causal convolution
    per channel over the last ``taps`` projected rows (``conv_w`` float32 [channels, taps], the last column the token's own;
    rows before a portion come from ``state[slot, state_off:]`` as [taps - 1, channels], oldest first; one tap is a factor
    per channel and reads no state; None: no convolution), an RMS
    norm per query and key head (``q_norm``, ``k_norm`` [head_dim], the mean over ``norm_width`` elements; None: none), the
    rotation of the first ``rotary_dim`` elements of queries and keys; queries to the q columns of ``out``, keys and values
    into the paged cache.  The state is not changed (:func:`conv_state_shift` moves it on), unless ``shift``: the caller
    promises that every sequence of the step has one token, and the state moves on in the same launch.  ``to_cache`` false:
    keys and values go to their columns of ``out`` instead (:func:`rope_kv_write` with ``rotary_dim`` 0 stores them from there)."""
    T = proj.shape[0]
    N = (num_heads + 2 * num_kv_heads) * head_dim
    _need(proj, "q|k|v projection", None, (T, N))
    _need(out, "q|k|v output", proj.dtype)
    if out.dim() != 2 or out.shape[0] != T or out.shape[1] < N:
        raise KernelError(f"conv_norm_rope_kv: output of shape {tuple(out.shape)} for {T} rows of {N}")
    taps = 1
    if conv_w is not None:
        _need(conv_w, "convolution weight", torch.float32)
        if conv_w.dim() != 2 or conv_w.shape[0] != N:
            raise KernelError(f"conv_norm_rope_kv: convolution weight of shape {tuple(conv_w.shape)} for {N} channels")
        taps = conv_w.shape[1]
    st, stride, off = (_p(None), _l(0), _l(0))
    if taps > 1:
        st, stride, off = _state_args(state, state_off)
        if state_off + (taps - 1) * N > state.shape[1]:
            raise KernelError("conv_norm_rope_kv: the state is too small for the convolution's inputs")
    for t, n, hh in ((q_norm, "query norm weight", num_heads), (k_norm, "key norm weight", num_kv_heads)):
        if t is not None:
            _need(t, n, torch.float32, (head_dim * hh,) if row_rinv is not None else (head_dim,))
    if row_rinv is not None:
        _need(row_rinv, "norm factors of the rows", torch.float32, (T, 2))
    _need(positions, "positions", torch.int32, (T,))
    if rotary_dim:
        _need(denominators, "rope denominators", torch.float32, (rotary_dim // 2,))
    _need(slot_mapping, "slot mapping", torch.int32, (T,))
    _need(q_start, "q_start", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(slots, "state slots", torch.int32)
    _need(k_cache, "key cache", proj.dtype)
    pages, nkv, page_size, dh = k_cache.shape
    _need(v_cache, "value cache", proj.dtype, (pages, nkv, dh, page_size))
    if num_kv_heads == 0:
        if write:
            raise KernelError("conv_norm_rope_kv: a projection of queries alone writes no keys and values")
    elif nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    _check(library().li_conv_norm_rope_kv(
        _p(proj), _p(out), _i(_dt(proj)), _p(conv_w), _i(taps), st, stride, off, _p(q_start), _p(seq_of_token), _p(slots),
        _p(q_norm), _p(k_norm), _f(eps), _i(int(norm_width)), _p(row_rinv), _p(positions), _p(denominators if rotary_dim else None), _i(rotary_dim),
        _p(slot_mapping), _p(k_cache), _p(v_cache), _i(T), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages),
        _i(1 if write else 0), _i(1 if shift else 0), _i(1 if to_cache else 0), _i(out.shape[1]), _stream(out)), "conv_norm_rope_kv")


def latent_rope_post(low: torch.Tensor, col_c: int, col_r: int, q: torch.Tensor, dim: int, weight: torch.Tensor, eps: float,
                     positions: torch.Tensor, denominators: Optional[torch.Tensor], magnitude: float, interleaved: bool, out: torch.Tensor,
                     num_heads: int, rank: int, rot_dim: int, head: int) -> None:
    """Latent attention with a rotated part, per token: ``c = rmsnorm(low[:, col_c : col_c + rank]) * weight`` into the first
    ``rank`` columns of the key head and of the value head of ``out`` [T, (num_heads + 2) head]; the one rotated key part all
    heads share, ``low[:, col_r : col_r + rot_dim]``, rotated, behind c in the key head; every query head's rotated part
    (the last ``rot_dim`` of its ``dim + rot_dim`` columns of ``q``) rotated, behind the head's first ``rank`` columns of
    ``out`` (which are not touched); the rest of every head zeros.  Pair i turns by ``position / denominators[i]``;
    ``interleaved``: the pair is (2i, 2i + 1), else (i, i + rot_dim / 2); cosines and sines are multiplied by ``magnitude``."""
    T = low.shape[0]
    _need(low, "latent projection")
    _need(q, "queries", low.dtype)
    _need(weight, "latent norm weight", torch.float32, (rank,))
    _need(positions, "positions", torch.int32, (T,))
    if rot_dim:
        _need(denominators, "rope denominators", torch.float32, (rot_dim // 2,))
    _need(out, "attention rows", low.dtype, (T, (num_heads + 2) * head))
    if q.shape[0] != T:
        raise KernelError(f"latent_rope_post: {q.shape[0]} query rows for {T} tokens")
    _check(library().li_latent_rope_post(_p(low), _i(_dt(low)), _i(low.shape[1]), _i(int(col_c)), _i(int(col_r)), _p(q), _i(q.shape[1]), _i(int(dim)),
                                         _p(weight), _f(eps), _p(positions), _p(denominators if rot_dim else None), _f(float(magnitude)),
                                         _i(1 if interleaved else 0), _p(out), _i(T), _i(num_heads), _i(rank), _i(rot_dim), _i(head), _stream(out)),
           "latent_rope_post")


def row_rinv(x: torch.Tensor, ranges, eps: float, out: torch.Tensor) -> None:
    """``out[t, j] = 1 / sqrt(sum(x[t, col_j : col_j + n_j]^2) / width_j + eps)`` for one or two ``ranges`` (col, n, width):
    the factor of an RMS norm over a whole projection (``width``: how many of the n columns are real, the rest zero padding)."""
    T = x.shape[0]
    _need(x, "rows")
    _need(out, "norm factors", torch.float32, (T, 2))
    r = [tuple(int(v) for v in rg) for rg in ranges]
    if not 1 <= len(r) <= 2:
        raise KernelError("row_rinv: one or two ranges of columns")
    (c0, n0, w0), (c1, n1, w1) = r[0], (r[1] if len(r) == 2 else (0, 0, 1))
    _check(library().li_row_rinv(_p(x), _i(_dt(x)), _i(x.shape[1]), _i(c0), _i(n0), _i(w0), _i(c1), _i(n1), _i(w1), _f(eps), _p(out), _i(T),
                                 _stream(out)), "row_rinv")


# --------------------------------------------------------------------------
# products in groups; routing of a mixture of experts
# --------------------------------------------------------------------------

def grouped_linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, row_offsets: Optional[torch.Tensor] = None,
                   a_group_cols: int = 0, out_group_cols: int = 0, tile_group: Optional[torch.Tensor] = None,
                   epilogue: Optional[str] = None, epilogue_params: Optional[torch.Tensor] = None) -> None:
    """``weight`` [G, N, K]: a product per group.  With ``row_offsets`` (int32 [G + 1] on the device) group g owns the rows
    ``row_offsets[g] .. row_offsets[g + 1] - 1`` of ``a`` [M, K] and ``out`` [M, N].  Without, every group takes all rows, its
    inputs at column ``g * a_group_cols`` of ``a`` and its outputs at column ``g * out_group_cols`` of ``out`` (a map per head).
    ``tile_group`` (int32 on the device; from :func:`moe_sort` with ``pad`` 128): the group of every tile of 128 rows when
    the groups' runs start at multiples of 128; large bfloat16 products then run on the tcgen05 tiles.
    ``epilogue="swiglu"`` (bfloat16, rows in groups): every group's matrix holds gate and up rows interleaved in eights
    (:func:`interleave_gate_up` per group) and ``out`` [M, N / 2] takes ``up * gate / (1 + exp(-gate))``.
    ``epilogue="glu_clamped"``: the same layout, the gated unit with bounded operands; ``epilogue_params`` holds its (limit,
    alpha), float32 on the device.  Rows that belong to no group (behind ``row_offsets[G]``) are left as they are."""
    G, N, Kd = weight.shape
    if epilogue not in (None,) + GATED:
        raise KernelError(f"grouped_linear: unknown epilogue {epilogue!r}")
    if (epilogue == "glu_clamped") != (epilogue_params is not None):
        raise KernelError("grouped_linear: the bounded unit needs its parameters, the other epilogues take none")
    if epilogue_params is not None:
        _need(epilogue_params, "parameters of the gated unit", torch.float32, (2,))
    if epilogue in GATED:
        if a.dtype != torch.bfloat16 or row_offsets is None or N % 16 or Kd % 8:
            raise KernelError("grouped_linear: a gated epilogue takes bfloat16 rows in groups, K a multiple of 8, N a multiple of 16")
        N_out = N // 2
    else:
        N_out = N
    M = a.shape[0]
    _need(a, "grouped input")
    _need(weight, "grouped weights", a.dtype)
    _need(out, "grouped output", a.dtype)
    if out.shape[0] != M:
        raise KernelError(f"grouped_linear: {out.shape[0]} output rows for {M} input rows")
    if row_offsets is not None:
        _need(row_offsets, "row offsets", torch.int32, (G + 1,))
        if a.shape[1] != Kd or out.shape[1] != N_out or a_group_cols or out_group_cols:
            raise KernelError(f"grouped_linear: rows in groups need a [M, {Kd}] and out [M, {N_out}]")
    elif (G - 1) * a_group_cols + Kd > a.shape[1] or (G - 1) * out_group_cols + N > out.shape[1]:
        raise KernelError("grouped_linear: the groups' columns do not fit the rows")
    if tile_group is not None:
        _need(tile_group, "groups of the row tiles", torch.int32)
        if row_offsets is None or tile_group.numel() * 128 < M:
            raise KernelError("grouped_linear: a table of the tiles' groups goes with row offsets and covers every tile of 128 rows")
    _check(library().li_grouped_linear(_p(a), _i(a.shape[1]), _i(a_group_cols), _p(weight), _p(out), _i(out.shape[1]), _i(out_group_cols),
                                       _p(row_offsets), _p(tile_group), _i(_dt(a)), _i(M), _i(N), _i(Kd), _i(G), _i(EPILOGUES[epilogue]), _p(epilogue_params),
                                       _stream(out)),
           "grouped_linear")


def moe_route(logits: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor, scoring: str = "sigmoid") -> None:
    """``ids``, ``weights`` [T, top]: per token the experts with the largest ``sigmoid(logits)`` (the lower index wins a tie)
    and those scores; ``scoring`` "softmax_chosen": the experts with the largest logits, and the softmax over the chosen
    logits alone."""
    if scoring not in ("sigmoid", "softmax_chosen"):
        raise KernelError(f"moe_route: unknown scoring {scoring!r}")
    T, E = logits.shape
    _need(logits, "router logits", torch.float32)
    _need(ids, "expert ids", torch.int32, (T, top))
    _need(weights, "expert weights", torch.float32, (T, top))
    _check(library().li_moe_route(_p(logits), _i(0 if scoring == "sigmoid" else 1), _i(T), _i(E), _i(top), _p(ids), _p(weights), _stream(ids)),
           "moe_route")


def moe_route_grouped(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int, scale: float,
                      ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Routing over all experts at once: ``s = softmax(logits)``; the choice scores are ``s + correction``; the experts form
    ``groups`` equal groups of neighbours, a group's score is its largest choice score, and only experts of the ``keep`` best
    groups can be chosen; the ``top`` largest choice scores choose (the lower index wins a tie); ``weights`` are the chosen
    experts' s divided by their sum (+ 1e-20), times ``scale``."""
    T, E = logits.shape
    _need(logits, "router logits", torch.float32)
    if correction is not None:
        _need(correction, "correction of the choice scores", torch.float32, (E,))
    _need(ids, "expert ids", torch.int32, (T, top))
    _need(weights, "expert weights", torch.float32, (T, top))
    _check(library().li_moe_route_grouped(_p(logits), _p(correction), _i(T), _i(E), _i(top), _i(int(groups)), _i(int(keep)), _f(float(scale)),
                                          _p(ids), _p(weights), _stream(ids)), "moe_route_grouped")


def sorted_rows(pairs: int, experts: int, pad: int = 1) -> int:
    """How many places the sorted order of ``pairs`` (token, choice) pairs has when every expert's run starts at a multiple of ``pad``."""
    return pairs if pad <= 1 else -(-(pairs + experts * (pad - 1)) // pad) * pad


def moe_sort(ids: torch.Tensor, experts: int, offsets: torch.Tensor, pair_at: torch.Tensor, place_of: torch.Tensor, pad: int = 1,
             tile_group: Optional[torch.Tensor] = None, matrices: Optional[int] = None) -> None:
    """A stable sort of the (token, choice) pairs by expert: ``offsets`` [experts + 1] (where each expert's rows start),
    ``pair_at`` (which pair stands at a sorted place; -1: none), ``place_of`` [n] (the sorted place of a pair).  ``pad`` > 1:
    every expert's run starts at a multiple of it, ``pair_at`` has :func:`sorted_rows` places, and ``tile_group`` (if given, one
    entry per ``pad`` places) says which expert each tile of ``pad`` rows belongs to (-1 behind the last run, and for the
    experts from ``matrices`` on: experts without matrices, whose rows a grouped product leaves as they are)."""
    n = ids.numel()
    R = sorted_rows(n, experts, pad)
    _need(ids, "expert ids", torch.int32)
    _need(offsets, "row offsets", torch.int32, (experts + 1,))
    _need(pair_at, "pair at place", torch.int32, (R,))
    _need(place_of, "place of pair", torch.int32, (n,))
    tiles = 0
    if tile_group is not None:
        tiles = R // pad
        _need(tile_group, "groups of the row tiles", torch.int32, (tiles,))
    _check(library().li_moe_sort(_p(ids), _i(n), _i(experts), _i(experts if matrices is None else int(matrices)), _i(int(pad)), _p(offsets), _p(pair_at), _p(place_of), _p(tile_group), _i(tiles),
                                 _i(R), _stream(ids)), "moe_sort")


def moe_gather(h: torch.Tensor, pair_at: torch.Tensor, weights: Optional[torch.Tensor], top: int, out: torch.Tensor) -> None:
    """``out[r] = h[pair_at[r] // top]``, times ``weights.flatten()[pair_at[r]]`` if given (the weight on the expert's input);
    a row of zeros where ``pair_at[r]`` is negative."""
    T, H = h.shape
    n = pair_at.shape[0]
    _need(h, "feed-forward input")
    _need(pair_at, "pair at place", torch.int32)
    if weights is not None:
        _need(weights, "expert weights", torch.float32, (T, top))
    _need(out, "sorted rows", h.dtype, (n, H))
    _check(library().li_moe_gather(_p(h), _i(_dt(h)), _p(pair_at), _p(weights), _i(n), _i(top), _i(H), _p(out), _stream(out)), "moe_gather")


def moe_combine(rows: torch.Tensor, place_of: torch.Tensor, weights: Optional[torch.Tensor], top: int, y: torch.Tensor) -> None:
    """``y[t] = sum_k rows[place_of[t * top + k]]`` (times ``weights[t, k]`` if given), summed in float32 in the order of k."""
    T, H = y.shape
    _need(rows, "sorted rows", None, (rows.shape[0], H))
    _need(place_of, "place of pair", torch.int32, (T * top,))
    if weights is not None:
        _need(weights, "expert weights", torch.float32, (T, top))
    _need(y, "feed-forward output", rows.dtype)
    _check(library().li_moe_combine(_p(rows), _i(_dt(rows)), _p(place_of), _p(weights), _i(T), _i(top), _i(H), _p(y), _stream(y)), "moe_combine")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """Index of the first maximum of each row."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "argmax output", torch.int32, (R,))
    _check(library().li_argmax(_p(logits), _p(out), _i(R), _i(V), _stream(out)), "argmax")


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row.  ``params`` int32 [R, 6]: temperature (float bits; <= 0
    is argmax), top_k, top_p (float bits), seed low, seed high, output index."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(params, "sampling parameters", torch.int32, (R, 6))
    _need(out, "sample output", torch.int32, (R,))
    _check(library().li_sample(_p(logits), _p(params), _p(out), _i(R), _i(V), _stream(out)), "sample")


# --------------------------------------------------------------------------
# LLAISYS_PROFILE=1: device time per kernel function, keyed by phase, reported at exit
# --------------------------------------------------------------------------
# LitInfer's switch of the same name (src/utils/profiler.cpp:47-104) times every operator call on the CPU and prints
# a table of "phase/op  calls  time(ms)  pct(%)" to standard error when the process ends.  Here an operator call is a
# kernel launch, so the time is the device's: a pair of CUDA events around each call, read when the report is made.
# While the switch is on the step function launches every kernel from the host (no captured graphs: a replayed graph
# runs without passing through these functions).

def _env_on(name: str) -> bool:
    import os

    return os.environ.get(name, "").lower() in ("1", "true", "on")


class Profile:
    def __init__(self) -> None:
        self.enabled = _env_on("LLAISYS_PROFILE")
        self.phase = ""
        self._pending = []                                 # (key, start event, stop event)
        self.total_ms = {}
        self.calls = {}
        if self.enabled:
            import atexit

            atexit.register(self.report)

    def reset(self) -> None:
        self._pending.clear()
        self.total_ms.clear()
        self.calls.clear()

    def wrap(self, name, fn):
        import functools

        @functools.wraps(fn)
        def timed(*args, **kwargs):
            if not self.enabled or not torch.cuda.is_available():
                return fn(*args, **kwargs)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                return fn(*args, **kwargs)
            finally:
                stop.record()
                self._pending.append(((self.phase + "/" + name) if self.phase else name, start, stop))
                if len(self._pending) >= 4096:
                    self.collect()

        return timed

    def collect(self) -> None:
        if self._pending:
            torch.cuda.synchronize()
        for key, start, stop in self._pending:
            self.total_ms[key] = self.total_ms.get(key, 0.0) + start.elapsed_time(stop)
            self.calls[key] = self.calls.get(key, 0) + 1
        self._pending.clear()

    def report(self, out=None) -> None:
        import sys

        out = out or sys.stderr
        self.collect()
        grand = sum(self.total_ms.values())
        print("\n================ LLAISYS PROFILE ================", file=out)
        if grand <= 0.0:
            print("(no profiled operations)\n================================================", file=out)
            return
        print(f"  total op time: {grand:.3f} ms (device time of kernel launches)", file=out)
        print("------------------------------------------------", file=out)
        print("  op                          calls     time(ms)    pct(%)", file=out)
        for key, ms in sorted(self.total_ms.items(), key=lambda kv: -kv[1]):
            print(f"  {key:<28}{self.calls[key]:>8}{ms:>12.3f}{100.0 * ms / grand:>9.2f}", file=out)
        print("================================================", file=out, flush=True)


profile = Profile()
TRACE = _env_on("LLAISYS_TRACE")          # LitInfer's other switch (src/llaisys/models/qwen2.cpp:17-26): a line per call on standard error

_TIMED = ("embedding", "rmsnorm", "add_rmsnorm", "gather_rmsnorm", "residual_add", "linear", "linear_add_scaled", "apply_row_scale",
          "rope_kv_write", "linear_rope_kv", "rope_table", "paged_attention", "swiglu", "argmax", "sample", "gather_rows", "scale_inplace",
          "logit_cap", "glu_clamped", "weighted_sum2", "add_position_rows", "hc_expand", "hc_read_norm", "hc_update", "causal_conv_silu", "conv_state_shift",
          "ssm_scan", "decay_scan", "gated_rmsnorm", "norm_add_norm", "add_row", "rmsnorm_cols", "conv_norm_rope_kv", "grouped_linear", "moe_route",
          "moe_sort", "moe_gather", "moe_combine")
if profile.enabled:
    for _name in _TIMED:
        globals()[_name] = profile.wrap(_name, globals()[_name])
