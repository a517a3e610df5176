"""Python faces of the CUDA kernels.

Every function takes torch tensors on the CUDA device, checks what the kernel
assumes (device, dtype, contiguity), and launches on torch's current stream.
There is no CPU path: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .library import KernelError, check, kernels_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

# how many launches of this package's kernels were made (bench reports it)
launch_count = 0


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16") from None


def _ptr(t, dtype=None, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return c_void_p(t.data_ptr())


def _stream():
    """The current stream of the current device as the kernels' void* (the raw handle: this runs once per launch)."""
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _launched(n=1):
    global launch_count
    launch_count += n


def count_launches(n: int) -> None:
    """Kernels of this package launched by replaying a captured graph."""
    _launched(n)


def embedding(ids, table, h_out, from_last=None, seq_index=None, slots=None, last_tokens=None, pos_table=None,
              positions=None, scale=1.0, rows_out=None):
    """h_out[t] = table[ids[t]] as float32 (the residual stream).  Where from_last[t] is set the id is the one the
    last step's sampling left for the token's sequence: last_tokens[slots[seq_index[t]]].  With ``pos_table`` the
    learned vector of the token's position, pos_table[positions[t]], is added (in float).  ``scale`` multiplies the
    token's row (in float) before anything is added.  ``rows_out`` ([tokens, width] of the table's dtype): the same rows once
    more, for a model that reads the embedding's output again later."""
    lib = kernels_library()
    n, width = h_out.shape
    if rows_out is not None and (rows_out.shape != (n, width) or rows_out.dtype != table.dtype):
        raise KernelError("embedding: rows_out must be [tokens, width] of the table's dtype")
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != width):
        raise KernelError("embedding: the position table must have the token table's dtype and width")
    check(lib.rmx_embedding(_ptr(ids, torch.int32, "ids"), _ptr(table, name="table"), _ptr(h_out, torch.float32, "h"),
                            c_int(n), c_int(width), c_int(table.shape[0]), _ptr(from_last, torch.int32, "from_last"),
                            _ptr(seq_index, torch.int32, "seq_index"), _ptr(slots, torch.int32, "slots"),
                            _ptr(last_tokens, torch.int32, "last_tokens"), _ptr(pos_table, name="pos_table"),
                            _ptr(positions if pos_table is not None else None, torch.int32, "positions"),
                            c_int(pos_table.shape[0] if pos_table is not None else 0), c_float(scale), _ptr(rows_out, name="rows_out"),
                            c_int(dtype_code(table)), _stream()))
    _launched()


def add_rmsnorm(h, delta, weight, eps, x_out, rows=None, write_h=True, delta2=None, mult=1.0, mult2=1.0, weight2=None, x2_out=None):
    """v = h + mult * (delta + mult2 * delta2); h = v (if write_h); x_out = RMSNorm(v; weight, eps).  With ``rows`` the
    rows rows[r] are read, x_out[r] is written and h is left alone.  ``weight2`` and ``x2_out``: a second norm of the same
    rows with a weight of its own (the mean of squares is formed once)."""
    lib = kernels_library()
    n = x_out.shape[0]
    width = h.shape[1]
    if delta is not None and delta.dtype != x_out.dtype:
        raise KernelError("add_rmsnorm: delta and output must have the same dtype")
    if delta2 is not None and (delta is None or delta2.dtype != delta.dtype or delta2.shape != delta.shape):
        raise KernelError("add_rmsnorm: a second delta goes with a first of the same shape and dtype")
    if (weight2 is None) != (x2_out is None) or (x2_out is not None and (x2_out.shape != x_out.shape or x2_out.dtype != x_out.dtype)):
        raise KernelError("add_rmsnorm: a second weight goes with a second output like the first")
    check(lib.rmx_add_rmsnorm(_ptr(h, torch.float32, "h"), _ptr(delta, name="delta"), _ptr(delta2, name="delta2"), c_float(mult), c_float(mult2),
                              _ptr(rows, torch.int32, "rows"),
                              _ptr(weight, torch.float32, "weight"), c_float(eps), _ptr(x_out, name="x"),
                              c_int(n), c_int(width), c_int(1 if (write_h and rows is None) else 0),
                              _ptr(weight2, torch.float32, "weight2"), _ptr(x2_out, name="x2"), c_int(dtype_code(x_out)), _stream()))
    _launched()


def add_residual(h, delta):
    lib = kernels_library()
    check(lib.rmx_add_residual(_ptr(h, torch.float32, "h"), _ptr(delta, name="delta"), c_int(h.shape[0]),
                               c_int(h.shape[1]), c_int(dtype_code(delta)), _stream()))
    _launched()


def add_bias(x, bias):
    """x[t, :] += bias in place (float add, one rounding).  ``x`` may be a view of some columns of wider rows."""
    lib = kernels_library()
    if x.dim() != 2 or x.stride(1) != 1 or bias.shape != (x.shape[1],) or not x.is_cuda:
        raise KernelError("add_bias: x must be [rows, width] with unit column stride on a CUDA device, bias [width]")
    check(lib.rmx_add_bias(c_void_p(x.data_ptr()), _ptr(bias, torch.float32, "bias"), c_int(x.shape[0]), c_int(x.shape[1]),
                           c_int(x.stride(0)), c_int(dtype_code(x)), _stream()))
    _launched()


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamp": 2}
UNARY_ACTIVATIONS = {"relu2": 3, "tanh": 4}     # one-argument activations: the square of max(x, 0) (an expert without a gate), tanh


def activation_args(activation, args=()) -> tuple:
    """(code, limit, alpha) of a gated feed-forward's pointwise part.  "silu" and "gelu_tanh" (out = act(gate) * up) take
    no constants; "swish_clamp" takes ``args`` = (limit, alpha): g = min(gate, limit), u = clamp(up, -limit, limit),
    out = g * sigmoid(alpha * g) * (u + 1)."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}: {sorted(ACTIVATIONS)}")
    if activation == "swish_clamp":
        if len(args) != 2 or not args[0] > 0:
            raise KernelError("activation 'swish_clamp' takes (limit, alpha), limit positive")
        return ACTIVATIONS[activation], float(args[0]), float(args[1])
    return ACTIVATIONS[activation], 0.0, 0.0


def swiglu(gate_up, out, block=0, activation="silu", args=()):
    """out = f(gate, up) number by number, f as ``activation_args`` says.  A row of ``gate_up`` is [gate | up] (block 0) or
    blocks of ``block`` gate numbers each followed by its ``block`` up numbers."""
    lib = kernels_library()
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [tokens, 2 * inter] of the output's dtype")
    code, limit, alpha = activation_args(activation, args)
    check(lib.rmx_swiglu(_ptr(gate_up, name="gate_up"), _ptr(out, name="out"), c_int(n), c_int(inter), c_int(block),
                         c_int(code), c_float(limit), c_float(alpha), c_int(dtype_code(out)), _stream()))
    _launched()


def _rows_view(t, name):
    """[rows, heads, size] with unit stride along ``size`` and heads side by side in a row (a view of [rows, heads * size]
    or of some columns of wider rows): (pointer, row stride, head stride)."""
    if t.dim() != 3 or t.stride(2) != 1 or not t.is_cuda:
        raise KernelError(f"{name} must be [rows, heads, size] on a CUDA device with unit stride along size")
    return c_void_p(t.data_ptr()), t.stride(0), t.stride(1)


def gemm_plain_heads(a, w, out):
    """out[t, h, :] = w[h] . a[t, h, :] for every head h on the FMA units (k ascending): a [rows, heads, K],
    w [heads, N, K] contiguous, out [rows, heads, N]."""
    lib = kernels_library()
    m, heads, k = a.shape
    n = w.shape[1]
    if w.shape != (heads, n, k) or out.shape != (m, heads, n) or a.dtype != w.dtype or not w.is_contiguous():
        raise KernelError(f"gemm_plain_heads: {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    pa, lda, ba = _rows_view(a, "a")
    pc, ldc, bc = _rows_view(out, "out")
    ll = ctypes.c_longlong
    check(lib.rmx_gemm_plain_batched(pa, _ptr(w, name="w"), pc, c_int(m), c_int(n), c_int(k), c_int(lda), c_int(k), c_int(ldc),
                                     c_int(heads), ll(ba), ll(n * k), ll(bc), c_int(dtype_code(a)), c_int(dtype_code(out)), _stream()))
    _launched()


def latent_norms(proj, q_rank, kv_rank, q_weight, kv_weight, eps, cq_out, pool, positions, seq_index, block_table, page_size,
                 status):
    """Rows of ``proj`` are [query latent | key/value latent | ...]: cq_out = RMSNorm(query latent; q_weight), and
    (``pool`` given, kv_rank > 0) RMSNorm(key/value latent; kv_weight) goes into the token's place in ``pool``
    [pages, 1, page_size, kv_rank] through its sequence's block table."""
    lib = kernels_library()
    n = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or cq_out.shape != (n, q_rank) or cq_out.dtype != proj.dtype:
        raise KernelError("latent_norms: proj must be [tokens, columns] with unit column stride, cq_out [tokens, q_rank] of its dtype")
    write = pool is not None and kv_rank > 0
    check(lib.rmx_latent_norms(
        c_void_p(proj.data_ptr()), c_int(proj.stride(0)), c_int(q_rank), c_int(kv_rank if write else 0),
        _ptr(q_weight, torch.float32, "q_weight"), _ptr(kv_weight if write else None, torch.float32, "kv_weight"), c_float(eps),
        _ptr(cq_out, name="cq_out"), _ptr(pool if write else None, proj.dtype, "pool"),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size), c_int(n),
        _ptr(status, torch.int32, "status"), c_int(dtype_code(proj)), _stream()))
    _launched()


def latent_rope(kv_rows, kv_rank, rot, interleaved, kv_weight, eps, q, q_rot_at, heads, q_out, row, cos_sin, pool, positions,
                seq_index, block_table, page_size, status):
    """A latent with a rotated part.  ``kv_rows`` [tokens, >= kv_rank + rot] (columns of wider rows allowed) are
    [latent | key part]: the page row of a token becomes [RMSNorm(latent; kv_weight) | rotate(key part) | zeros] of ``row``
    numbers (``pool`` [pages, 1, page_size, row], or None: nothing is written).  ``q`` [tokens, heads, size] (a view):
    q_out[t, h, kv_rank : kv_rank + rot] = rotate(q[t, h, q_rot_at : q_rot_at + rot]), zeros behind it up to ``row``
    (q_out [tokens, heads * row]; its first kv_rank numbers a head are not touched).  ``cos_sin`` [tokens, rot] float32:
    cosines then sines of the token's rot / 2 angles; pairs are (2j, 2j + 1) if ``interleaved`` else (j, j + rot / 2)."""
    lib = kernels_library()
    n = q.shape[0]
    if q.dim() != 3 or q.shape[1] != heads or q.stride(2) != 1 or q_out.shape != (n, heads * row) or q_out.dtype != q.dtype:
        raise KernelError("latent_rope: q must be [tokens, heads, size] with unit stride along size, q_out [tokens, heads * row] of its dtype")
    write = pool is not None
    if write and (kv_rows.dim() != 2 or kv_rows.stride(1) != 1 or kv_rows.shape[1] < kv_rank + rot or kv_rows.dtype != q.dtype):
        raise KernelError("latent_rope: kv_rows must be [tokens, >= kv_rank + rot] with unit column stride")
    check(lib.rmx_latent_rope(
        c_void_p(kv_rows.data_ptr() if write else 0), c_int(kv_rows.stride(0) if write else 0), c_int(kv_rank), c_int(rot),
        c_int(1 if interleaved else 0), _ptr(kv_weight if write else None, torch.float32, "kv_weight"), c_float(eps),
        c_void_p(q.data_ptr()), c_int(q.stride(0)), c_int(q.stride(1)), c_int(q_rot_at), c_int(heads), _ptr(q_out, name="q_out"),
        c_int(row), _ptr(cos_sin, torch.float32, "cos_sin"), _ptr(pool if write else None, q.dtype, "pool"),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size), c_int(n),
        _ptr(status, torch.int32, "status"), c_int(dtype_code(q)), _stream()))
    _launched()


def stream_concat(h, delta, extra, out, delta2=None, mult=1.0, mult2=1.0, write_h=False):
    """out[t] = [round(h[t] + mult * (delta[t] + mult2 * delta2[t])) | extra[t]]: the stream with what is still to be added
    to it, beside ``extra`` rows of the same width, as one row of 2 * width numbers for a product that reads both.  The
    sum is formed in float; ``write_h`` stores it back into the stream."""
    lib = kernels_library()
    n, width = h.shape
    if extra.shape != (n, width) or out.shape != (n, 2 * width) or out.dtype != extra.dtype:
        raise KernelError("stream_concat: extra must be [tokens, width], out [tokens, 2 * width] of its dtype")
    if delta is not None and (delta.shape != (n, width) or delta.dtype != out.dtype):
        raise KernelError("stream_concat: delta must be [tokens, width] of the output's dtype")
    if delta2 is not None and (delta is None or delta2.shape != delta.shape or delta2.dtype != delta.dtype):
        raise KernelError("stream_concat: a second delta goes with a first of the same shape and dtype")
    check(lib.rmx_stream_concat(_ptr(h, torch.float32, "h"), _ptr(delta, name="delta"), _ptr(delta2, name="delta2"), c_float(mult),
                                c_float(mult2), _ptr(extra, name="extra"), _ptr(out, name="out"), c_int(n), c_int(width),
                                c_int(1 if write_h else 0), c_int(dtype_code(out)), _stream()))
    _launched()


def gate_heads(o, gate, heads, vdim):
    """o[t, h, :] *= sigmoid(gate[t, h]) in place.  ``gate`` may be some columns of wider rows."""
    lib = kernels_library()
    n = o.shape[0]
    if o.shape != (n, heads * vdim) or gate.shape != (n, heads) or gate.stride(1) != 1 or gate.dtype != o.dtype:
        raise KernelError("gate_heads: o must be [tokens, heads * vdim], gate [tokens, heads] of the same dtype")
    check(lib.rmx_gate_heads(_ptr(o, name="o"), c_void_p(gate.data_ptr()), c_int(gate.stride(0)), c_int(n), c_int(heads),
                             c_int(vdim), c_int(dtype_code(o)), _stream()))
    _launched()


def moe_route(x, w_router, top, ids_out, weights_out, logits=None, scoring="softmax", correction=None, groups=1, keep=1,
              route_scale=1.0, normalize=True):
    """Router of a mixture of experts: logits = x . w_router^T in float; per row the ``top`` largest choose the
    experts (ids_out [rows, top] int32), weights_out = softmax over the chosen logits.  ``logits``: [rows, experts]
    floats of scratch (made here if not given).
    ``scoring="sigmoid"``: an expert's score is sigmoid(logit); the choice goes by score + ``correction`` (float32 [experts]
    or None) among the experts of the ``keep`` best of ``groups`` equal groups of neighbours (a group's worth: the sum of its
    two largest corrected scores); the weights are the chosen scores over their sum, times ``route_scale``; with
    ``normalize=False`` (sigmoid scoring) a weight is the chosen score itself, times ``route_scale``."""
    lib = kernels_library()
    n, width = x.shape
    e = w_router.shape[0]
    if not normalize and scoring != "sigmoid":
        raise KernelError("moe_route: weights that are not normalised go with sigmoid scoring")
    if w_router.shape != (e, width) or ids_out.shape != (n, top) or weights_out.shape != (n, top):
        raise KernelError("moe_route: shapes do not fit")
    if logits is None:
        logits = torch.empty((n, e), dtype=torch.float32, device=x.device)
    elif logits.shape != (n, e):
        raise KernelError("moe_route: the logits' scratch must be [rows, experts]")
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route: unknown scoring {scoring!r}")
    if correction is not None and correction.shape != (e,):
        raise KernelError("moe_route: the correction must be [experts]")
    check(lib.rmx_moe_route(_ptr(x, name="x"), _ptr(w_router, torch.float32, "w_router"), c_int(n), c_int(width), c_int(e),
                            c_int(top), _ptr(ids_out, torch.int32, "ids"), _ptr(weights_out, torch.float32, "weights"),
                            _ptr(logits, torch.float32, "logits"), c_int(1 if scoring == "sigmoid" else 0),
                            _ptr(correction, torch.float32, "correction"), c_int(groups), c_int(keep), c_float(route_scale),
                            c_int(1 if normalize else 0), c_int(dtype_code(x)), _stream()))
    _launched(2)


def moe_sort(ids, n_experts, offsets_out, sorted_out, where_out):
    """Group the (row, choice) pairs of ``ids`` [rows, top] by expert: offsets_out [experts + 1], sorted_out[p] = the
    pair at place p, where_out[pair] = its place."""
    lib = kernels_library()
    total = ids.numel()
    if offsets_out.numel() != n_experts + 1 or sorted_out.numel() != total or where_out.numel() != total:
        raise KernelError("moe_sort: shapes do not fit")
    check(lib.rmx_moe_sort(_ptr(ids, torch.int32, "ids"), c_int(total), c_int(n_experts), _ptr(offsets_out, torch.int32, "offsets"),
                           _ptr(sorted_out, torch.int32, "sorted"), _ptr(where_out, torch.int32, "where"), _stream()))
    _launched()


def moe_gemm(a, w, out, offsets, sorted_pairs=None, top=0):
    """out[p] = w[e] . a[row(p)] for every place p of expert e's run (``offsets``).  ``w`` [experts, N, K].  With
    ``sorted_pairs`` and ``top`` the rows are gathered from the layer's input (row(p) = sorted_pairs[p] // top), else
    ``a`` is already in sorted order."""
    lib = kernels_library()
    e, n, k = w.shape
    total = out.shape[0]
    if a.shape[1] != k or out.shape != (total, n) or a.dtype != w.dtype or out.dtype != a.dtype or not w.is_contiguous():
        raise KernelError(f"moe_gemm: {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    if sorted_pairs is None and a.shape[0] != total:
        raise KernelError("moe_gemm: rows in sorted order must be as many as the output's")
    check(lib.rmx_moe_gemm(_ptr(a, name="a"), c_int(a.stride(0)), _ptr(sorted_pairs, torch.int32, "sorted"),
                           c_int(top if sorted_pairs is not None else 0), _ptr(w, name="w"), _ptr(out, name="out"),
                           c_int(out.stride(0)), _ptr(offsets, torch.int32, "offsets"), c_int(e), c_int(total), c_int(n), c_int(k),
                           c_int(dtype_code(a)), _stream()))
    _launched()


def moe_gemm_tcgen05_supported(n: int, k: int) -> bool:
    return bool(kernels_library().rmx_moe_gemm_tcgen05_supports(c_int(n), c_int(k)))


def moe_gather(x, sorted_pairs, top, out):
    """out[p] = x[sorted_pairs[p] // top]: the layer's rows in the order of the experts' runs (bfloat16, 16-byte copies)."""
    lib = kernels_library()
    total, width = out.shape
    if x.shape[1] != width or sorted_pairs.numel() != total or x.dtype != out.dtype:
        raise KernelError("moe_gather: shapes do not fit")
    check(lib.rmx_moe_gather(_ptr(x, torch.bfloat16, "x"), _ptr(sorted_pairs, torch.int32, "sorted"), c_int(top),
                             _ptr(out, torch.bfloat16, "out"), c_int(total), c_int(width), _stream()))
    _launched()


def moe_gemm_tcgen05(a, w, out, offsets, status, gated=False, activation="silu", args=(), unary=None):
    """The experts' products on the tcgen05 tensor cores (bfloat16): out[p] = w[e] . a[p] for every place p of expert
    e's run; ``a`` [places, K] in sorted order, ``w`` [experts, N, K].  ``gated``: an expert's rows come in blocks of 64
    gate rows and their 64 up rows, and out [places, N / 2] = f(gate, up) (``activation_args``).  ``unary`` ("relu2"): out =
    f(product) number by number."""
    lib = kernels_library()
    e, n, k = w.shape
    total = a.shape[0]
    if a.shape[1] != k or out.shape != (total, n // 2 if gated else n) or not w.is_contiguous() or a.stride(1) != 1:
        raise KernelError(f"moe_gemm_tcgen05: {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    code, limit, alpha = activation_args(activation, args)
    epilogue = 1 if gated else 0
    if unary is not None:
        if gated:
            raise KernelError("moe_gemm_tcgen05: a gated product takes no one-argument activation")
        epilogue, code = 2, UNARY_ACTIVATIONS[unary]
    check(lib.rmx_moe_gemm_tcgen05(c_void_p(a.data_ptr()), c_int(a.stride(0)), _ptr(w, torch.bfloat16, "w"), _ptr(out, torch.bfloat16, "out"),
                                   c_int(out.stride(0)), _ptr(offsets, torch.int32, "offsets"), c_int(e), c_int(total), c_int(n),
                                   c_int(k), c_int(epilogue), c_int(code), c_float(limit), c_float(alpha), _ptr(status, torch.int32, "status"),
                                   _stream()))
    _launched()


def moe_combine(y, where, weights, shared_out, out):
    """out[row] = sum over choices of weights[row, choice] * y[where[row, choice]] (+ shared_out[row]), summed in float
    in the order of the choices.  ``weights`` None: every choice counts once (the rows were weighted on their way in)."""
    lib = kernels_library()
    n, width = out.shape
    top = where.numel() // n if weights is None else weights.shape[1]
    if y.shape != (n * top, width) or where.numel() != n * top or (shared_out is not None and shared_out.shape != out.shape):
        raise KernelError("moe_combine: shapes do not fit")
    check(lib.rmx_moe_combine(_ptr(y, out.dtype, "y"), _ptr(where, torch.int32, "where"), _ptr(weights, torch.float32, "weights"),
                              _ptr(shared_out, out.dtype if shared_out is not None else None, "shared"), _ptr(out, name="out"),
                              c_int(n), c_int(top), c_int(width), c_int(dtype_code(out)), _stream()))
    _launched()


def gemm_plain(a, w, out):
    """out[M, N] = a[M, K] . w[N, K]^T on the FMA units, k in ascending order."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or a.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not fit")
    check(lib.rmx_gemm_plain(_ptr(a, name="a"), _ptr(w, name="w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k),
                             c_int(k), c_int(k), c_int(n), c_int(dtype_code(a)), c_int(dtype_code(out)), _stream()))
    _launched()


def rope_table(positions, inv_freq, rotary_dim, out, magnitude=1.0):
    """out[t] = magnitude * [cos(pos_t * inv_freq[j]) for j | sin(...) for j]: the angles of a step's positions, formed once."""
    lib = kernels_library()
    n = positions.shape[0]
    check(lib.rmx_rope_table(_ptr(positions, torch.int32, "positions"), _ptr(inv_freq, torch.float32, "inv_freq"),
                             _ptr(out, torch.float32, "out"), c_int(n), c_int(rotary_dim), c_float(magnitude), _stream()))
    _launched()


def qk_rope_cache(qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table, page_size,
                  k_pool, v_pool, q_out, nq, nkv, hd, write_kv, status, cos_sin=None):
    lib = kernels_library()
    n = qkv.shape[0]
    check(lib.rmx_qk_rope_cache(
        _ptr(qkv, name="qkv"), _ptr(q_norm, torch.float32, "q_norm"), _ptr(k_norm, torch.float32, "k_norm"),
        c_float(eps), _ptr(inv_freq, torch.float32, "inv_freq"), c_int(rotary_dim),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(k_pool, qkv.dtype, "k_pool"), _ptr(v_pool, qkv.dtype, "v_pool"), _ptr(q_out, qkv.dtype, "q_out"),
        c_int(n), c_int(nq), c_int(nkv), c_int(hd), c_int(qkv.shape[1]), c_int(1 if write_kv else 0),
        _ptr(status, torch.int32, "status"), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(dtype_code(qkv)), _stream()))
    _launched()


def attention_plain(q, k_pool, v_pool, positions, seq_index, block_table, page_size, out, nq, nkv, hd, window,
                    scale, status, sinks=None, chunk=0, softcap=0.0):
    """``sinks`` (float32 [nq], or None): a score a query head that enters the softmax's denominator and has no value.
    ``chunk`` > 0: a query reads only keys of its own chunk of that many positions (chunks counted from position 0).
    ``softcap`` > 0: scaled scores go through softcap * tanh(s / softcap)."""
    lib = kernels_library()
    n = q.shape[0]
    check(lib.rmx_attention_plain(
        _ptr(q, name="q"), _ptr(k_pool, q.dtype, "k_pool"), _ptr(v_pool, q.dtype, "v_pool"),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, q.dtype, "out"), c_int(n), c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale),
        _ptr(status, torch.int32, "status"), _ptr(sinks, torch.float32, "sinks"), c_int(chunk), c_float(softcap),
        c_int(dtype_code(q)), _stream()))
    _launched()


def qk_whole_norm_rope_cache(qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table, page_size,
                             k_pool, v_pool, q_out, nq, nkv, dq, dv, hd, write_kv, status, cos_sin=None):
    """Rows of ``qkv`` are [q (nq * dq) | k (nkv * dq) | v (nkv * dv)].  q and k are each RMS-normed over the WHOLE
    projection (weights of the projection's size, or None), split into heads, rotated, and written: q to ``q_out``
    [tokens, nq, hd], k and v into their pages, heads padded with zeros to the cache's ``hd``."""
    lib = kernels_library()
    n = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or q_out.shape != (n, nq * hd):
        raise KernelError("qk_whole_norm_rope_cache: qkv must be [tokens, columns] with unit column stride, q_out [tokens, nq * hd]")
    check(lib.rmx_qk_whole_norm_rope_cache(
        c_void_p(qkv.data_ptr()), c_int(qkv.stride(0)), _ptr(q_norm, torch.float32, "q_norm"), _ptr(k_norm, torch.float32, "k_norm"),
        c_float(eps), _ptr(inv_freq, torch.float32, "inv_freq"), c_int(rotary_dim), _ptr(cos_sin, torch.float32, "cos_sin"),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(k_pool, qkv.dtype, "k_pool"), _ptr(v_pool, qkv.dtype, "v_pool"), _ptr(q_out, qkv.dtype, "q_out"), c_int(n), c_int(nq),
        c_int(nkv), c_int(dq), c_int(dv), c_int(hd), c_int(1 if write_kv else 0), _ptr(status, torch.int32, "status"),
        c_int(dtype_code(qkv)), _stream()))
    _launched()


def sigmoid_gate(o, o_head, gate, out, heads, vdim):
    """out[t, h, :] = o[t, h, :vdim] * sigmoid(gate[t, h, :]): ``o`` [tokens, heads * o_head] (heads padded to o_head
    numbers), ``gate`` some columns of wider rows, ``out`` [tokens, heads * vdim] (may be ``o`` when o_head == vdim)."""
    lib = kernels_library()
    n = o.shape[0]
    if o.shape != (n, heads * o_head) or out.shape != (n, heads * vdim) or gate.shape != (n, heads * vdim) or gate.stride(1) != 1 \
            or gate.dtype != o.dtype or out.dtype != o.dtype:
        raise KernelError("sigmoid_gate: shapes or dtypes do not fit")
    check(lib.rmx_sigmoid_gate(_ptr(o, name="o"), c_int(o_head), c_void_p(gate.data_ptr()), c_int(gate.stride(0)), _ptr(out, name="out"),
                               c_int(n), c_int(heads), c_int(vdim), c_int(dtype_code(o)), _stream()))
    _launched()


def short_conv(x, weight, bias, out, ring, batch, slots, activation=None, residual=False):
    """A causal convolution over time on each channel: out_t = act(bias + sum_j weight[j] * x_(t - taps + 1 + j)) (+ x_t).
    ``x`` and ``out``: [tokens, channels] (columns of wider rows allowed), ``weight`` float32 [taps, channels] (taps-major:
    the transpose of how checkpoints store it; its last row is the current token's), ``ring``
    [slots, max(taps - 1, 1), channels] of x's dtype: every sequence's last taps - 1 inputs, read for what lies before the
    step's tokens and written with the step's last ones."""
    lib = kernels_library()
    n, channels = x.shape
    taps = weight.shape[0]
    if weight.shape != (taps, channels) or out.shape != (n, channels) or x.stride(1) != 1 or out.stride(1) != 1 or out.dtype != x.dtype \
            or ring.dtype != x.dtype or ring.shape[1:] != (max(taps - 1, 1), channels):
        raise KernelError("short_conv: shapes or dtypes do not fit")
    if activation not in (None, "silu"):
        raise KernelError(f"short_conv: unknown activation {activation!r}")
    check(lib.rmx_short_conv(c_void_p(x.data_ptr()), c_int(x.stride(0)), _ptr(weight, torch.float32, "weight"),
                             _ptr(bias, torch.float32, "bias"), c_void_p(out.data_ptr()), c_int(out.stride(0)), _ptr(ring, name="ring"),
                             c_int(channels), c_int(taps), _ptr(batch.positions, torch.int32, "positions"),
                             _ptr(batch.seq_index, torch.int32, "seq_index"), _ptr(slots, torch.int32, "slots"),
                             _ptr(batch.q_start, torch.int32, "q_start"), c_int(n), c_int(batch.n_seqs),
                             c_int(1 if activation == "silu" else 0), c_int(1 if residual else 0),
                             c_int(1 if batch.max_q_len == 1 else 0), c_int(dtype_code(x)), _stream()))
    _launched(1 if batch.max_q_len == 1 or taps == 1 else 2)


def _recurrence_warps(batch, heads, vdim):
    """Warps a block of the recurrence (8 columns of a head's state each; a block's warps share the rows it fetches): as many
    as cover a head's columns while the grid still has two blocks an SM; fewer, so that more blocks run side by side, when
    few sequences step."""
    warps = max(1, min(4, -(-vdim // 8)))      # (measured: 2 to 4 warps a block move a decode step's states fastest, 8 are slower)
    while warps > 1 and batch.n_seqs * heads * -(-vdim // (8 * warps)) < 2 * _sm_count():
        warps //= 2
    return warps


def _cols(t, name):
    if t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
        raise KernelError(f"{name} must be [tokens, columns] on a CUDA device with unit column stride")
    return c_void_p(t.data_ptr()), c_int(t.stride(0))


def _recurrence_scratch(workspace, n, row_heads, heads, k, vector_decay):
    """Float scratch of the recurrence's two kernels: rows of k and q padded as the scan reads them, and either the decays'
    rows (a vector a head) or two scalars a token and head."""
    ws = workspace if workspace is not None else _own_workspace()
    row = kernels_library().rmx_recurrence_row(c_int(k))
    if row < 0:
        raise KernelError(f"recurrence: a state of {k} rows a head is beyond 256")
    kf = ws.get("recurrence_k", (n, row_heads, row), torch.float32)
    qf = ws.get("recurrence_q", (n, row_heads, row), torch.float32)
    if vector_decay:
        return kf, qf, ws.get("recurrence_a", (n, heads, row), torch.float32), None
    return kf, qf, ws.get("recurrence_step", (n, heads), torch.float32), ws.get("recurrence_decay", (n, heads), torch.float32)


def recurrence_ssd(conv, dt, dt_bias, a_log, d_skip, state, out, batch, slots, heads, groups, k, v, workspace=None, warps=None):
    """Per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t, dt = softplus(raw + bias):
    ``conv`` rows [x (heads * v) | B (groups * k) | C (groups * k)], ``dt`` [tokens, heads] raw, ``state`` float32
    [slots, heads, v, k] (read and written; kept transposed), ``out`` float32 [tokens, heads * v]."""
    lib = kernels_library()
    n = conv.shape[0]
    if conv.shape[1] != heads * v + 2 * groups * k or dt.shape != (n, heads) or out.shape != (n, heads * v) or state.shape[1:] != (heads, v, k) \
            or dt.dtype != conv.dtype:
        raise KernelError("recurrence_ssd: shapes do not fit")
    kf, qf, s0, s1 = _recurrence_scratch(workspace, n, groups, heads, k, False)
    p0, l0 = _cols(conv, "conv")
    p1, l1 = _cols(dt, "dt")
    check(lib.rmx_linear_recurrence(c_int(0), _ptr(state, torch.float32, "state"), _ptr(out, torch.float32, "out"),
                                    _ptr(batch.q_start, torch.int32, "q_start"), _ptr(slots, torch.int32, "slots"), c_int(batch.n_seqs),
                                    c_int(n), c_int(heads), c_int(k), c_int(v), p0, l0, p1, l1, c_void_p(0), c_int(0),
                                    _ptr(dt_bias, torch.float32, "dt_bias"), _ptr(a_log, torch.float32, "A_log"),
                                    _ptr(d_skip, torch.float32, "D"), c_int(groups), _ptr(kf), _ptr(qf), _ptr(s0), _ptr(s1),
                                    c_int(warps or _recurrence_warps(batch, heads, v)), c_int(dtype_code(conv)), _stream()))
    _launched(2)


def recurrence_gate(q, f, v, f_bias, lower, state, out, batch, slots, heads, k, vdim, workspace=None, warps=None):
    """Per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T silu(q_t), f = lower + (1 - lower) sigmoid(raw + bias):
    ``q`` and ``f`` [tokens, heads * k] raw projections, ``v`` [tokens, heads * vdim] (columns of wider rows allowed),
    ``state`` float32 [slots, heads, vdim, k] (transposed), ``out`` float32 [tokens, heads * vdim]."""
    lib = kernels_library()
    n = q.shape[0]
    if q.shape != (n, heads * k) or f.shape != (n, heads * k) or v.shape != (n, heads * vdim) or out.shape != (n, heads * vdim) \
            or state.shape[1:] != (heads, vdim, k) or f.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("recurrence_gate: shapes do not fit")
    kf, qf, s0, _ = _recurrence_scratch(workspace, n, heads, heads, k, True)
    p0, l0 = _cols(q, "q")
    p1, l1 = _cols(f, "f")
    p2, l2 = _cols(v, "v")
    check(lib.rmx_linear_recurrence(c_int(1), _ptr(state, torch.float32, "state"), _ptr(out, torch.float32, "out"),
                                    _ptr(batch.q_start, torch.int32, "q_start"), _ptr(slots, torch.int32, "slots"), c_int(batch.n_seqs),
                                    c_int(n), c_int(heads), c_int(k), c_int(vdim), p0, l0, p1, l1, p2, l2,
                                    _ptr(f_bias, torch.float32, "f_bias"), _ptr(lower, torch.float32, "lower"), c_void_p(0), c_int(1),
                                    _ptr(kf), _ptr(qf), _ptr(s0), c_void_p(0),
                                    c_int(warps or _recurrence_warps(batch, heads, vdim)), c_int(dtype_code(q)), _stream()))
    _launched(2)


def group_rmsnorm(y, weight, eps, out, groups, gate=None, out_scale=1.0, gate_after=False):
    """out = RMSNorm of each of a row's ``groups`` equal parts of u = y (* silu(gate)), times ``weight`` (as long as a row,
    or as long as a part and shared by the parts), times ``out_scale``; y float32, out and gate in the compute dtype.
    ``gate_after``: the gate multiplies the normed and weighted numbers instead: norm(y) * weight * silu(gate)."""
    lib = kernels_library()
    n, total = y.shape
    if total % groups or out.shape != (n, total) or out.stride(1) != 1 or weight.numel() not in (total, total // groups) \
            or (gate is not None and (gate.shape != (n, total) or gate.stride(1) != 1 or gate.dtype != out.dtype)):
        raise KernelError("group_rmsnorm: shapes or dtypes do not fit")
    check(lib.rmx_group_rmsnorm(_ptr(y, torch.float32, "y"), c_void_p(gate.data_ptr() if gate is not None else 0),
                                c_int(gate.stride(0) if gate is not None else 0), _ptr(weight, torch.float32, "weight"),
                                c_int(weight.numel()), c_float(eps), c_void_p(out.data_ptr()), c_int(out.stride(0)), c_int(n),
                                c_int(groups), c_int(total // groups), c_float(out_scale), c_int(1 if gate_after else 0), c_int(dtype_code(out)), _stream()))
    _launched()


def add_group_rmsnorm(h, terms, weight, eps, groups, x_out, rows=None, write_h=True, weight2=None, x2_out=None):
    """v = h + va * (m1 * d1 + m2 * d2) + vb * d3; h = v (if write_h); the row is normed in ``groups`` equal consecutive
    parts, each over its own root mean square, and x_out = that * weight (x2_out = that * weight2).  ``terms`` =
    (d1, d2, d3, m1, m2, va, vb): tensors of x_out's dtype or None, factors, float32 vectors of a row's length or None.
    With ``rows`` the rows rows[r] are read, x_out[r] is written and h is left alone."""
    lib = kernels_library()
    d1, d2, d3, m1, m2, va, vb = terms
    n, width = x_out.shape[0], h.shape[1]
    for d in (d1, d2, d3):
        if d is not None and (d.dtype != x_out.dtype or d.shape != h.shape):
            raise KernelError("add_group_rmsnorm: what is added must have the stream's shape and the output's dtype")
    if d1 is None and d2 is not None:
        raise KernelError("add_group_rmsnorm: a second term goes with a first")
    for v in (va, vb, weight, weight2):
        if v is not None and v.shape != (width,):
            raise KernelError("add_group_rmsnorm: vectors and weights are as long as a row")
    if (weight2 is None) != (x2_out is None) or (x2_out is not None and (x2_out.shape != x_out.shape or x2_out.dtype != x_out.dtype)):
        raise KernelError("add_group_rmsnorm: a second weight goes with a second output like the first")
    check(lib.rmx_add_group_rmsnorm(_ptr(h, torch.float32, "h"), _ptr(d1, name="d1"), _ptr(d2, name="d2"), _ptr(d3, name="d3"),
                                    c_float(m1), c_float(m2), _ptr(va, torch.float32, "va"), _ptr(vb, torch.float32, "vb"),
                                    _ptr(rows, torch.int32, "rows"), _ptr(weight, torch.float32, "weight"), c_float(eps),
                                    _ptr(x_out, name="x"), c_int(n), c_int(width), c_int(groups),
                                    c_int(1 if (write_h and rows is None) else 0), _ptr(weight2, torch.float32, "weight2"),
                                    _ptr(x2_out, name="x2"), c_int(dtype_code(x_out)), _stream()))
    _launched()


def unary_act(x, out, activation):
    """out = f(x) number by number (float, one rounding; out may be x); ``activation`` "relu2": the square of max(x, 0), or "tanh"."""
    lib = kernels_library()
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("unary_act: shapes or dtypes do not fit")
    check(lib.rmx_unary_act(_ptr(x, name="x"), _ptr(out, name="out"), ctypes.c_longlong(x.numel()), c_int(UNARY_ACTIVATIONS[activation]),
                            c_int(dtype_code(x)), _stream()))
    _launched()


def moe_gather_scaled(x, sorted_pairs, weights, top, out):
    """out[p] = weights[pair] * x[pair // top] with pair = sorted_pairs[p]: the layer's rows in the order of the experts'
    runs, each times the weight of its (row, choice) pair (float product, one rounding)."""
    lib = kernels_library()
    total, width = out.shape
    if x.shape[1] != width or sorted_pairs.numel() != total or weights.numel() != total or x.dtype != out.dtype:
        raise KernelError("moe_gather_scaled: shapes do not fit")
    check(lib.rmx_moe_gather_scaled(_ptr(x, name="x"), _ptr(sorted_pairs, torch.int32, "sorted"), _ptr(weights, torch.float32, "weights"),
                                    c_int(top), _ptr(out, name="out"), c_int(total), c_int(width), c_int(dtype_code(x)), _stream()))
    _launched()


def heads_rope_cache(qkv, bias, q_norm, k_norm, eps, cos_sin, rot, interleaved, v_cos_sin, v_interleaved, positions, seq_index,
                     block_table, page_size, k_pool, v_pool, q_out, nq, nkv, dq, dv, hd, write_kv, status):
    """Rows of ``qkv`` are [q (nq * dq) | k (nkv * dq) | v (nkv * dv)].  ``bias`` (float32, a row long, or None) is added;
    every q and k head is RMS-normed over its dq numbers with one weight of dq numbers for all heads (None: no norm) and
    rotated over its first ``rot`` numbers by the table ``cos_sin`` [tokens, rot] (pairs (j, j + rot / 2), or neighbours
    with ``interleaved``); with ``v_cos_sin`` [tokens, dv] every value head is rotated over all its numbers too.  q goes
    to ``q_out`` [tokens, nq * hd], k and v into their pages, heads padded with zeros to ``hd``."""
    lib = kernels_library()
    n = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != (nq + nkv) * dq + nkv * dv or q_out.shape != (n, nq * hd):
        raise KernelError("heads_rope_cache: qkv must be [tokens, q | k | v] with unit column stride, q_out [tokens, nq * hd]")
    if bias is not None and bias.shape != (qkv.shape[1],):
        raise KernelError("heads_rope_cache: the bias is as long as a row")
    if (cos_sin is not None and cos_sin.shape != (n, rot)) or (v_cos_sin is not None and v_cos_sin.shape != (n, dv)):
        raise KernelError("heads_rope_cache: a table of angles is [tokens, rotated numbers]")
    check(lib.rmx_heads_rope_cache(
        c_void_p(qkv.data_ptr()), c_int(qkv.stride(0)), _ptr(bias, torch.float32, "bias"), _ptr(q_norm, torch.float32, "q_norm"),
        _ptr(k_norm, torch.float32, "k_norm"), c_float(eps), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(rot if cos_sin is not None else 0),
        c_int(1 if interleaved else 0), _ptr(v_cos_sin, torch.float32, "v_cos_sin"), c_int(1 if v_interleaved else 0),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(k_pool, qkv.dtype, "k_pool"), _ptr(v_pool, qkv.dtype, "v_pool"), _ptr(q_out, qkv.dtype, "q_out"), c_int(n), c_int(nq),
        c_int(nkv), c_int(dq), c_int(dv), c_int(hd), c_int(1 if write_kv else 0), _ptr(status, torch.int32, "status"),
        c_int(dtype_code(qkv)), _stream()))
    _launched()


def unrotate_heads(o, cos_sin, interleaved, out, heads, dv, hd):
    """out[t, h, :dv] = o[t, h, :dv] turned by minus the token's angles (``cos_sin`` [tokens, dv]): o's heads are ``hd``
    numbers apart, out is dense."""
    lib = kernels_library()
    n = o.shape[0]
    if o.shape != (n, heads * hd) or out.shape != (n, heads * dv) or cos_sin.shape != (n, dv) or out.dtype != o.dtype:
        raise KernelError("unrotate_heads: shapes do not fit")
    check(lib.rmx_unrotate_heads(_ptr(o, name="o"), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(1 if interleaved else 0),
                                 _ptr(out, name="out"), c_int(n), c_int(heads), c_int(dv), c_int(hd), c_int(dtype_code(o)), _stream()))
    _launched()


def attention_talk_plain(q, k_pool, v_pool, talk, positions, seq_index, block_table, page_size, out, nq, nkv, hd, dq, dv, window,
                         scale, status, splits=1, workspace=None):
    """Attention whose scaled scores are mixed over the heads before the softmax, s'_h = sum_g talk[h, g] s_g, on the FMA
    units: q [tokens, nq * hd], pools with heads of ``hd`` numbers (keys: the first dq, values: the first dv), talk float32
    [nq, nq], out [tokens, nq * dv].  ``splits`` > 1: a token's keys are shared out over that many blocks whose shares a second
    kernel adds (the order of a row's sums then follows the split: not for the 32-bit path)."""
    lib = kernels_library()
    n = q.shape[0]
    if q.shape != (n, nq * hd) or out.shape != (n, nq * dv) or talk.shape != (nq, nq) or out.dtype != q.dtype:
        raise KernelError("attention_talk_plain: shapes do not fit")
    partial = None
    if splits > 1:
        ws = workspace if workspace is not None else _own_workspace()
        partial = ws.get("talk_partial", (n, splits, nq, dv + 2), torch.float32)
    check(lib.rmx_attention_talk(_ptr(q, name="q"), _ptr(k_pool, q.dtype, "k_pool"), _ptr(v_pool, q.dtype, "v_pool"),
                                 _ptr(talk, torch.float32, "talk"), _ptr(positions, torch.int32, "positions"),
                                 _ptr(seq_index, torch.int32, "seq_index"), _ptr(block_table, torch.int32, "block_table"),
                                 c_int(block_table.shape[1]), c_int(page_size), _ptr(out, name="out"), c_int(n), c_int(nq), c_int(nkv),
                                 c_int(hd), c_int(dq), c_int(dv), c_int(window), c_float(scale), _ptr(status, torch.int32, "status"),
                                 c_int(splits), _ptr(partial), c_int(dtype_code(q)), _stream()))
    _launched(1 if splits == 1 else 2)


def attention_talk_mma_supported(nq: int, nkv: int, hd: int) -> bool:
    return bool(kernels_library().rmx_attention_talk_mma_supports(c_int(nq), c_int(nkv), c_int(hd)))


def attention_talk_mma(q, k_pool, v_pool, talk, batch, block_table, page_size, out, nq, nkv, hd, dv, window, scale, splits=1,
                       workspace=None):
    """The same attention on the tensor cores (bfloat16; mma.sync): a block takes 16 tokens of a sequence with all heads.
    ``splits`` > 1: a tile's keys are shared out over that many blocks whose shares a second kernel adds."""
    lib = kernels_library()
    n = q.shape[0]
    partial = None
    if splits > 1:
        ws = workspace if workspace is not None else _own_workspace()
        partial = ws.get("talk_partial", (n, splits, nq, dv + 2), torch.float32)
    if q.shape != (n, nq * hd) or out.shape != (n, nq * dv) or talk.shape != (nq, nq) or q.dtype != torch.bfloat16 or out.dtype != q.dtype:
        raise KernelError("attention_talk_mma: shapes or dtypes do not fit")
    check(lib.rmx_attention_talk_mma(_ptr(q, name="q"), _ptr(k_pool, q.dtype, "k_pool"), _ptr(v_pool, q.dtype, "v_pool"),
                                     _ptr(talk, torch.float32, "talk"), _ptr(batch.positions, torch.int32, "positions"),
                                     _ptr(batch.q_start, torch.int32, "q_start"), c_int(batch.n_seqs), c_int(n),
                                     _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
                                     _ptr(out, name="out"), c_int(nq), c_int(nkv), c_int(hd), c_int(dv), c_int(window), c_float(scale),
                                     _ptr(batch.status, torch.int32, "status"), c_int(splits), _ptr(partial), _stream()))
    _launched(1 if splits == 1 else 2)


def talk_splits(n_tokens: int, max_seq_len: int, window: int = 0) -> int:
    """Into how many blocks a decoded token's keys are split by the mixed-score attention: a power of two (a decode graph
    is captured anew whenever the number changes: it should change seldom while sequences grow), about two blocks an SM in
    all, no block with fewer than four key tiles of 32 (measured at batch 8 and 2,048 keys: 16 splits 41 us, 32 splits 55 us)."""
    span = min(max_seq_len, window) if window else max_seq_len
    tiles = -(-max(span, 1) // 32)
    most = max(1, min(2 * _sm_count() // max(n_tokens, 1), tiles // 4, 64))
    return 1 << (most.bit_length() - 1)


def token_shift_mix(x, mu, out, last, batch, slots):
    """out[s] = x + (prev - x) * mu[s] for every mix s: ``x`` [tokens, channels], ``mu`` float32 [mixes, channels], ``out``
    [mixes, tokens, channels]; prev is the row of the token before in the same sequence: of this step, or ``last``
    [slots, channels] (what the sequence's last step left; written with the step's last rows), or zeros at position 0."""
    lib = kernels_library()
    n, channels = x.shape
    mixes = mu.shape[0]
    if mu.shape != (mixes, channels) or out.shape != (mixes, n, channels) or out.dtype != x.dtype or last.dtype != x.dtype \
            or last.shape[1:] != (channels,):
        raise KernelError("token_shift_mix: shapes or dtypes do not fit")
    single = batch.max_q_len == 1
    check(lib.rmx_token_shift_mix(_ptr(x, name="x"), _ptr(mu, torch.float32, "mu"), _ptr(out, name="out"), _ptr(last, name="last"),
                                  c_int(channels), c_int(mixes), _ptr(batch.positions, torch.int32, "positions"),
                                  _ptr(batch.seq_index, torch.int32, "seq_index"), _ptr(slots, torch.int32, "slots"),
                                  _ptr(batch.q_start, torch.int32, "q_start"), c_int(n), c_int(batch.n_seqs), c_int(1 if single else 0),
                                  c_int(dtype_code(x)), _stream()))
    _launched(1 if single else 2)


def recurrence_decay(r, k, w, v, w0, u, state, out, batch, slots, heads, kdim, vdim, workspace=None, warps=None):
    """Per head and channel a_t = exp(-exp(w_t + w0)); o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, then
    S_t = diag(a_t) S_(t-1) + k_t v_t^T: ``r``, ``k``, ``w`` [tokens, heads * kdim] (columns of wider rows allowed), ``v``
    [tokens, heads * vdim], ``w0`` and ``u`` float32 [heads * kdim], ``state`` float32 [slots, heads, vdim, kdim]
    (transposed), ``out`` float32 [tokens, heads * vdim]."""
    lib = kernels_library()
    n = r.shape[0]
    hk = heads * kdim
    if r.shape != (n, hk) or k.shape != (n, hk) or w.shape != (n, hk) or v.shape != (n, heads * vdim) or out.shape != (n, heads * vdim) \
            or state.shape[1:] != (heads, vdim, kdim) or w0.numel() != hk or u.numel() != hk or len({r.dtype, k.dtype, w.dtype, v.dtype}) != 1:
        raise KernelError("recurrence_decay: shapes or dtypes do not fit")
    kf, qf, af, _ = _recurrence_scratch(workspace, n, heads, heads, kdim, True)
    ws = workspace if workspace is not None else _own_workspace()
    bonus = ws.get("recurrence_bonus", (n, heads), torch.float32)
    p0, l0 = _cols(r, "r")
    p1, l1 = _cols(k, "k")
    p2, l2 = _cols(w, "w")
    p3, l3 = _cols(v, "v")
    check(lib.rmx_decay_recurrence(_ptr(state, torch.float32, "state"), _ptr(out, torch.float32, "out"),
                                   _ptr(batch.q_start, torch.int32, "q_start"), _ptr(slots, torch.int32, "slots"), c_int(batch.n_seqs),
                                   c_int(n), c_int(heads), c_int(kdim), c_int(vdim), p0, l0, p1, l1, p2, l2, p3, l3,
                                   _ptr(w0, torch.float32, "w0"), _ptr(u, torch.float32, "u"), _ptr(af), _ptr(kf), _ptr(qf), _ptr(bonus),
                                   c_int(warps or _recurrence_warps(batch, heads, vdim)), c_int(dtype_code(r)), _stream()))
    _launched(2)


def sample(logits, temperature, uniform, out, slots=None, last_tokens=None):
    """out[r] = greedy choice (temperature None or 0) or a draw from softmax(logits / temperature); with ``slots``
    and ``last_tokens`` the choice is also left at last_tokens[slots[r]] for the next step's embedding."""
    lib = kernels_library()
    r, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows must be contiguous")
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32 on a CUDA device")
    check(lib.rmx_sample(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), _ptr(temperature, torch.float32, "temperature"),
                         _ptr(uniform, torch.float32, "uniform"), _ptr(out, torch.int32, "out"), c_int(r), c_int(v),
                         _ptr(slots, torch.int32, "slots"), _ptr(last_tokens, torch.int32, "last_tokens"), _stream()))
    _launched()


# ---------------------------------------------------------------------------
# Helpers of the dispatch below that hold no state.

def _mpad(m: int) -> int:
    return 16 if m <= 16 else (32 if m <= 32 else 64)


def _graph_time(fn, calls: int, reps: int = 3) -> float:
    """Microseconds per call of ``fn(i)``, timed on the device inside a captured graph."""
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        g.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps / calls * 1e3


class _Sequences:
    """A run of neighbouring sequences of a batch, with what the attention kernels read of a batch.  Token
    numbers in ``q_start`` stay those of the whole batch, so q, out and positions are passed whole."""

    def __init__(self, batch, first: int, last: int):
        self.q_start = batch.q_start[first:last + 1]
        self.q_start_host = batch.q_start_host[first:last + 1]
        self.n_seqs = last - first
        lens = batch.seq_lens_host[first:last]
        counts = [self.q_start_host[i + 1] - self.q_start_host[i] for i in range(self.n_seqs)]
        self.max_seq_len, self.max_q_len = max(lens), max(counts)
        self.positions, self.status = batch.positions, batch.status
        self.first, self.last = first, last


def _short_and_long(batch, group: int):
    """A mixed step: decoded tokens (rows * group <= 16: the key-split kernel's case) beside prompt portions.  If
    the short sequences are the batch's head or its tail, returns the two runs (short, long), else None."""
    if getattr(batch, "seq_lens_host", None) is None or batch.n_seqs < 2:
        return None
    key = ("short_and_long", group)
    memo = getattr(batch, "per_step", None)
    if memo is not None and key in memo:
        return memo[key]
    starts = batch.q_start_host
    short = [(starts[i + 1] - starts[i]) * group <= 16 for i in range(batch.n_seqs)]
    n_short = sum(short)
    found = None
    if 0 < n_short < batch.n_seqs:
        if all(short[:n_short]):
            found = (_Sequences(batch, 0, n_short), _Sequences(batch, n_short, batch.n_seqs))
        elif all(short[batch.n_seqs - n_short:]):
            found = (_Sequences(batch, batch.n_seqs - n_short, batch.n_seqs), _Sequences(batch, 0, batch.n_seqs - n_short))
    if memo is not None:
        memo[key] = found
    return found


def flash_supported(hd: int, group: int) -> bool:
    return bool(kernels_library().rmx_attention_flash_supports(c_int(hd), c_int(group)))


_SM_COUNT = None


def _sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SM_COUNT


def flash_splits(n_tiles: int, nkv: int, max_seq_len: int) -> int:
    """Few rows and long contexts (decoding): share a tile's keys among blocks so that every
    SM has work.  Up to 8 splits form a thread-block cluster and add their results through shared
    memory, which costs far less than the round through global memory that more splits take.
    Measured on B200 at 8 kv heads: clusters of 2, 4 and 8 are placed readily, of 3 or 6 not; the
    grid should stay a little under two blocks per SM, which the kernels before and after need
    some of; and 4 splits beat 8 as soon as 4 give 128 blocks.  So: the largest of 1, 2, 4, 8 that
    keeps the grid under 7/8 of two blocks per SM, 4 rather than 8 if 4 give 128 blocks; more than
    8 only where each split still has 16 tiles of 64 keys."""
    blocks = n_tiles * nkv
    kv_tiles = -(-max_seq_len // 64)
    room = 2 * _sm_count() - _sm_count() // 4
    if blocks >= room or kv_tiles < 4:
        return 1
    want = max(1, min(room // blocks, kv_tiles // 2, 64))
    if want > 8 and kv_tiles // want >= 16 and blocks * 8 < 128:
        return want
    splits = 8 if want >= 8 else (4 if want >= 4 else (2 if want >= 2 else 1))
    if splits == 8 and blocks * 4 >= 128:
        splits = 4
    return splits


def flash_takes_projection(hd: int, group: int, page_size: int, rotary_dim: int) -> bool:
    """Whether the key-split kernel is built to finish the q/k/v projection of a decoding step at these sizes."""
    return bool(kernels_library().rmx_attention_flash_takes_projection(c_int(hd), c_int(group), c_int(page_size), c_int(rotary_dim)))


def _key_span(max_seq_len: int, chunk: int, rows: int = 1) -> int:
    """The most keys that ``rows`` neighbouring queries of a sequence read between them: the sequence's length, or with
    chunks of ``chunk`` positions at most a chunk and the rows themselves."""
    return min(max_seq_len, chunk + rows - 1) if chunk > 0 else max_seq_len


def attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                    n_splits=None, projection=None, use_tma=True, sinks=None, chunk=0, softcap=0.0):
    """Tensor-core attention over pages for bfloat16 (prompt portions and decoded tokens alike).  ``projection``:
    (qkv rows, q_norm, k_norm, eps, cos_sin, write_kv) for a decoding step whose kernel finishes the projection.
    ``use_tma``: keys and values are fetched by TMA where the kernel is built for it."""
    lib = kernels_library()
    group = nq // nkv
    tq = 64 // group
    starts = batch.q_start_host
    n_tiles = sum(-(-(starts[i + 1] - starts[i]) // tq) for i in range(batch.n_seqs))
    if n_splits is None:
        n_splits = flash_splits(n_tiles, nkv, _key_span(batch.max_seq_len, chunk, tq))
    n = out.shape[0]
    qkv, q_norm, k_norm, eps, cos_sin, write_kv = projection if projection is not None else (None, None, None, 0.0, None, False)
    part_o = part_ml = counters = None
    if n_splits > 1:
        part_o = workspace.get("attn_part_o", (n_splits, n * nq, hd), torch.float32)
        part_ml = workspace.get("attn_part_ml", (n_splits, n * nq, 2), torch.float32)
        counters = workspace.get_zeroed("attn_counters", (max(4096, batch.n_seqs * nkv),), torch.int32)
    check(lib.rmx_attention_flash(
        _ptr(q if qkv is None else None, torch.bfloat16, "q"), _ptr(k_pool, torch.bfloat16, "k_pool"), _ptr(v_pool, torch.bfloat16, "v_pool"),
        _ptr(batch.q_start, torch.int32, "q_start"), _ptr(batch.positions, torch.int32, "positions"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, torch.bfloat16, "out"), _ptr(part_o), _ptr(part_ml), _ptr(counters), c_int(batch.n_seqs), c_int(n),
        c_int(n_tiles),
        c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(n_splits),
        c_int(getattr(batch, "max_q_len", 0)), c_int(k_pool.shape[0] if use_tma else 0),
        _ptr(qkv, torch.bfloat16, "qkv"), c_int(qkv.stride(0) if qkv is not None else 0), _ptr(q_norm, torch.float32, "q_norm"),
        _ptr(k_norm, torch.float32, "k_norm"), c_float(eps), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(1 if write_kv else 0),
        c_int(starts[0]), c_int(starts[batch.n_seqs] - starts[0]), _ptr(sinks, torch.float32, "sinks"), c_int(chunk), c_float(softcap),
        _ptr(batch.status, torch.int32, "status"), _stream()))
    _launched(2 if n_splits > 1 else 1)


_scratch = None


def _own_workspace():
    """Scratch for kernels called without an engine's workspace (tests, single calls)."""
    global _scratch
    if _scratch is None:
        from ..engine.workspace import Workspace
        _scratch = Workspace(torch.device("cuda", torch.cuda.current_device()))
    return _scratch


_supported = {}


def tcgen05_supported(m: int, n: int, k: int) -> bool:
    key = (m, n, k)
    if key not in _supported:
        if len(_supported) > 65536:
            _supported.clear()
        _supported[key] = bool(kernels_library().rmx_gemm_tcgen05_supports(c_int(m), c_int(n), c_int(k)))
    return _supported[key]


def tcgen05_splits(m: int, n: int, k: int) -> int:
    """How many slices of K share a tile of 128 weight rows.  The product is bound by reading the
    weight: what matters is that enough blocks are resident to keep loads in flight on every SM
    (measured on Qwen3-8B shapes), not that the last wave is full.  So: the fewest slices that
    give at least 128 blocks; as many as give 192 blocks where each slice then still has 24
    k-blocks of 64 (long reductions: the down projection); at most 8 (a cluster), each slice
    keeping at least 4 k-blocks."""
    tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    if tiles >= 128:
        return 1
    splits = -(-128 // tiles)
    more = -(-192 // tiles)
    if more <= 8 and k_blocks // more >= 24:
        splits = more
    return max(1, min(splits, 8, k_blocks // 4))


def gemm_tcgen05(a, w, out, workspace=None, status=None, splits=None, cluster=True, dependent=False, swiglu=False,
                 activation="silu"):
    """out[M, N] = a[M, K] . w[N, K]^T for M <= 64 on the tcgen05 tensor cores (bfloat16 in,
    float accumulation, bfloat16 or float out).  ``cluster``: split-K slices of a tile form a
    thread-block cluster and add their sums through distributed shared memory (up to 8 slices),
    else through scratch in global memory.  ``dependent``: launch as a programmatic dependent of
    the kernel before it on the stream, so that its weight loads start while that kernel ends."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    # swiglu: w's rows come in blocks of 64 gate rows and their 64 up rows; out is act(gate) * up, [m, n / 2]
    if activation not in ("silu", "gelu_tanh"):
        raise KernelError(f"gemm_tcgen05: the gated epilogue takes silu and gelu_tanh, not {activation!r}")
    want_shape = (m, n // 2) if swiglu else (m, n)
    if w.shape[1] != k or out.shape != want_shape or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} of {a.dtype}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05: the result is bfloat16 or float32")
    ws = workspace if workspace is not None else _own_workspace()
    if splits is None:
        splits = tcgen05_splits(m, n, k)
        if cluster:
            splits = min(splits, 8)
    partial = counters = None
    if splits > 1:
        need = lib.rmx_gemm_tcgen05_scratch_floats(c_int(m), c_int(n), c_int(splits))
        partial = ws.get("gemm_partial", (need,), torch.float32)
        counters = ws.get_zeroed("gemm_counters", (max(4096, -(-n // 128)),), torch.int32)
    if status is None:
        status = ws.get_zeroed("gemm_status", (1,), torch.int32)
    check(lib.rmx_gemm_tcgen05(
        _ptr(a, name="a"), _ptr(w, name="w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0), c_int(splits),
        _ptr(partial), _ptr(counters), _ptr(status, torch.int32, "status"),
        c_int((1 if cluster else 0) | (2 if dependent else 0) | (4 if swiglu else 0) | (8 if ACTIVATIONS[activation] == 1 else 0)),
        _stream()))
    _launched()
    return status


def gemm_tcgen05_wait_probe(a, w, out, status, splits=1, cluster=True, swiglu=False, spin_limit=1000, workspace=None):
    """For tests: the tcgen05 product's kernel launched so that its waits run out (no tile is ever copied, every
    wait gives up after ``spin_limit`` polls).  It must return, leave status 3 in ``status`` and ``out`` untouched."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    ws = workspace if workspace is not None else _own_workspace()
    partial = counters = None
    if splits > 1:
        partial = ws.get("gemm_partial", (lib.rmx_gemm_tcgen05_scratch_floats(c_int(m), c_int(n), c_int(splits)),), torch.float32)
        counters = ws.get_zeroed("gemm_counters", (max(4096, -(-n // 128)),), torch.int32)
    check(lib.rmx_gemm_tcgen05_wait_probe(
        _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k),
        c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0),
        c_int(splits), _ptr(partial), _ptr(counters), _ptr(status, torch.int32, "status"),
        c_int((1 if cluster else 0) | (4 if swiglu else 0)), c_int(spin_limit), _stream()))
    _launched()
    return counters


def tcgen05_attention_supported(hd: int, group: int, page_size: int) -> bool:
    return bool(kernels_library().rmx_attention_tcgen05_supports(c_int(hd), c_int(group), c_int(page_size)))


def tcgen05_attention_shape(counts: list, nkv: int, group: int, max_seq_len: int) -> tuple:
    """(query tiles a block, runs of keys) for prompt portions of ``counts`` tokens.  Measured on 148 SMs: a grid of
    about one block an SM (not more) is fastest; two neighbouring tiles of 128 rows a block, which share the key and
    value tiles it fetches, win once a sequence has some 2,000 keys, one tile a block below that; where whole tiles
    leave SMs without work, every tile's keys go in as many runs as fill them (at most 8, each of at least 4 key
    tiles of 64), whose shares a second kernel adds."""
    tile = 128 // group
    sms = _sm_count()
    pairs = sum(-(-c // (2 * tile)) for c in counts) * nkv
    singles = sum(-(-c // tile) for c in counts) * nkv
    key_tiles = -(-max_seq_len // 64)
    if 4 * pairs >= 3 * sms:
        return 2, 1
    long_keys = max_seq_len >= 2048
    if 4 * singles >= 3 * sms:   # one tile a block would fill the SMs
        return (2, max(1, min(sms // pairs, 8, key_tiles // 4))) if long_keys else (1, 1)
    if long_keys:
        return 2, max(1, min(sms // pairs, 8, key_tiles // 4))
    return 1, max(1, min(sms // singles, 8, key_tiles // 4))


def attention_tcgen05(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, per_block=None,
                      n_splits=None, workspace=None, sinks=None, chunk=0, softcap=0.0):
    """Prompt portions: S = Q K^T and O += P V as tcgen05 MMAs with accumulators in tensor memory (see
    ``tcgen05_attention_shape`` for how the work is divided; ``per_block`` and ``n_splits`` override it)."""
    lib = kernels_library()
    tile = 128 // (nq // nkv)
    starts = batch.q_start_host
    counts = [starts[i + 1] - starts[i] for i in range(batch.n_seqs)]
    if per_block is None and n_splits is None:
        per_block, n_splits = tcgen05_attention_shape(counts, nkv, nq // nkv, _key_span(batch.max_seq_len, chunk, 2 * tile))
        if workspace is None:
            n_splits = 1
    per_block = 2 if per_block is None else per_block
    n_splits = 1 if n_splits is None else n_splits
    n_tiles = sum(-(-c // (per_block * tile)) for c in counts)
    part_o = part_ml = None
    if n_splits > 1:
        ws = workspace if workspace is not None else _own_workspace()
        part_o = ws.get("attn_part_o", (n_splits, q.shape[0] * nq, hd), torch.float32)
        part_ml = ws.get("attn_part_ml", (n_splits, q.shape[0] * nq, 2), torch.float32)
    check(lib.rmx_attention_tcgen05(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_pool, torch.bfloat16, "k_pool"), _ptr(v_pool, torch.bfloat16, "v_pool"),
        _ptr(batch.q_start, torch.int32, "q_start"), _ptr(batch.positions, torch.int32, "positions"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, torch.bfloat16, "out"), c_int(batch.n_seqs), c_int(q.shape[0]), c_int(n_tiles), c_int(per_block),
        c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(k_pool.shape[0]), c_int(n_splits),
        _ptr(part_o), _ptr(part_ml), c_int(starts[0]), c_int(starts[-1] - starts[0]), _ptr(sinks, torch.float32, "sinks"),
        c_int(chunk), c_float(softcap), _ptr(batch.status, torch.int32, "status"), _stream()))
    _launched(2 if n_splits > 1 else 1)


# Whether this package's kernels are launched as programmatic dependents of the kernel before them (a switch of the
# loaded library, so of the process: see ``set_dependent_launch``).
dependent_launch = True


def set_dependent_launch(on: bool) -> None:
    """Programmatic dependent launch of this package's kernels (on by default): a kernel's blocks may take their
    places while the kernel before it drains, and the tcgen05 product fetches weights meanwhile."""
    global dependent_launch
    dependent_launch = bool(on)
    kernels_library().rmx_set_dependent_launch(c_int(1 if on else 0))


# ---------------------------------------------------------------------------
# Dispatch: which kernel serves a call.  float32 always takes the plain kernels (fixed order of summation, no
# tensor cores); bfloat16 takes the fast ones where they apply.  The choices that can be switched or tuned belong
# to a ``Kernels`` object: every engine has its own and hands it to its parts, so two engines in one process
# neither share tuning results nor see each other's switches.

class Kernels:
    """The kernels as one engine sees them: its switches, what its tuning measured, and the dispatch that reads
    both.  Everything else (the plain faces of the kernels above) is reached through it by name.

    ``policy``: which products of few rows (up to 64) take this package's tcgen05 kernel rather than the library's
    product: "auto" (whichever was faster when the engine timed both on the model's own weights, see
    ``autotune_linears``; shapes that were not timed follow "measured"), "measured" (the output head and long
    reductions, where it won on Qwen3-8B shapes: a fixed rule, the same bits on every start), "all" (every product
    the kernel supports), "none"; or a table that ``tuning_table`` returned earlier (the choices of that run again).
    """

    def __init__(self, policy="measured"):
        self.tuned = {}          # (n, k, padded rows[, "swiglu"]) -> True if the tcgen05 kernel was faster
        self.tuned_splits = {}   # (n, k, padded rows) -> the number of K slices that was fastest
        if isinstance(policy, dict):
            self.load_tuning_table(policy)
            policy = "auto"
        if policy not in ("auto", "measured", "all", "none"):
            raise KernelError(f"unknown kernel policy {policy!r}: auto, measured, all, none or a tuning table")
        self.tcgen05_policy = policy
        self.use_tma = True                 # decoding fetches keys and values by TMA where the kernel is built for it
        self.fused_decode_rope = True       # a decoding attention norms and rotates its own token while it waits for keys
        self.fused_swiglu = True            # the gate/up product of few rows forms silu(gate) * up in its epilogue
        self.use_tcgen05_attention = True   # prompt portions at head size 128 run on the tcgen05 tensor cores
        self.use_tcgen05_experts = True     # a routed feed-forward's products run on the tcgen05 tensor cores (bfloat16)
        self._splits_memo = {}

    def __getattr__(self, name):
        # the faces of the kernels that hold no state
        try:
            return globals()[name]
        except KeyError:
            raise AttributeError(name) from None

    @property
    def dependent_launch(self) -> bool:
        return dependent_launch

    # ---- tuning ---------------------------------------------------------------------------------------------
    def tuning_table(self) -> dict:
        """What the tuning chose, in a form that JSON takes and ``Kernels(policy=table)`` reads back."""
        key = lambda k: "x".join(str(p) for p in k)   # noqa: E731
        return {"policy": self.tcgen05_policy, "tcgen05": {key(k): bool(v) for k, v in sorted(self.tuned.items(), key=str)},
                "slices": {key(k): int(v) for k, v in sorted(self.tuned_splits.items(), key=str)}}

    def load_tuning_table(self, table: dict) -> None:
        def key(text):
            return tuple(int(p) if p.lstrip("-").isdigit() else p for p in text.split("x"))
        self.tuned = {key(k): bool(v) for k, v in (table.get("tcgen05") or {}).items()}
        self.tuned_splits = {key(k): int(v) for k, v in (table.get("slices") or {}).items()}

    def prefers_tcgen05(self, m: int, n: int, k: int) -> bool:
        if self.tcgen05_policy == "none" or not tcgen05_supported(m, n, k):
            return False
        if self.tcgen05_policy == "all":
            return True
        if self.tcgen05_policy == "auto" and (n, k, _mpad(m)) in self.tuned:
            return self.tuned[(n, k, _mpad(m))]
        return n * k >= (1 << 28) or (k >= 8192 and m <= 32)

    def autotune_linears(self, weights: list, workspace=None, rows=(8, 32, 64), log=None, min_bytes: float = 256e6) -> dict:
        """Time the tcgen05 product against the library's on the model's own bfloat16 weights, per
        shape and per padded row count, and remember the faster.  Weights of one shape take turns so
        that none is served from L2 (a lone small weight would be: its timing then says little and
        the rule of "measured" stands for it; ``min_bytes`` is how much a shape's weights must hold
        together to be timed)."""
        groups = {}
        for w in weights:
            if w is not None and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_cuda:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (n, k), ws in groups.items():
            if not tcgen05_supported(1, n, k) or len(ws) * n * k * 2 < min_bytes:
                continue
            for m in rows:
                key = (n, k, _mpad(m))
                if key in self.tuned:
                    continue
                a = torch.randn(m, k, device=ws[0].device).to(torch.bfloat16)
                out = torch.empty(m, n, dtype=torch.bfloat16, device=ws[0].device)
                calls = max(4, min(len(ws), 12))
                # the kernel's own choice first: how many slices of K share a tile (from one less than the rule's count up to
                # what a cluster takes: more slices mean fewer k-blocks for each block to stream, and a longer reduction)
                most = 8
                rule = min(tcgen05_splits(m, n, k), most)
                best = None
                for splits in range(max(1, rule - 1), most + 1):
                    if splits > max(1, -(-k // 64) // 4):
                        continue
                    t = _graph_time(lambda i: gemm_tcgen05(a, ws[i % len(ws)], out, workspace, splits=splits, dependent=True), calls)
                    if best is None or t < best[0]:
                        best = (t, splits)
                mine, self.tuned_splits[key] = best
                lib = _graph_time(lambda i: torch.mm(a, ws[i % len(ws)].t(), out=out), calls)
                self.tuned[key] = mine < lib
                if log is not None:
                    log(f"product [{m} x {k}] . [{n} x {k}]^T: tcgen05 {mine:.1f} us with {best[1]} slices of K, library {lib:.1f} us")
        return dict(self.tuned)

    def autotune_fused_swiglu(self, weights: list, workspace=None, rows=(8, 32, 64), log=None, min_bytes: float = 256e6) -> dict:
        """The same for gate/up weights in blocks of 64: the tcgen05 product with the SwiGLU epilogue
        against the library's product followed by the pointwise kernel."""
        groups = {}
        for w in weights:
            if w is not None and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_cuda and w.shape[0] % 128 == 0:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (n, k), ws in groups.items():
            if not tcgen05_supported(1, n, k) or len(ws) * n * k * 2 < min_bytes:
                continue
            for m in rows:
                key = (n, k, _mpad(m), "swiglu")
                if key in self.tuned:
                    continue
                a = torch.randn(m, k, device=ws[0].device).to(torch.bfloat16)
                gu = torch.empty(m, n, dtype=torch.bfloat16, device=ws[0].device)
                act = torch.empty(m, n // 2, dtype=torch.bfloat16, device=ws[0].device)
                calls = max(4, min(len(ws), 12))
                best = None
                for splits in range(1, 4):    # (a weight with this many tiles seldom gains from slices of K; it is asked, not assumed)
                    if splits > max(1, -(-k // 64) // 4):
                        continue
                    t = _graph_time(lambda i: gemm_tcgen05(a, ws[i % len(ws)], act, workspace, swiglu=True, splits=splits, dependent=True), calls)
                    if best is None or t < best[0]:
                        best = (t, splits)
                mine, self.tuned_splits[key] = best

                def lib_pair(i):
                    torch.mm(a, ws[i % len(ws)].t(), out=gu)
                    swiglu(gu, act, 64)
                lib = _graph_time(lib_pair, calls)
                # inside a step the fused product also spares a kernel's start and end, which this timing of the pair
                # alone does not show: it is taken unless the pair is clearly faster
                self.tuned[key] = mine < lib * 1.05
                if log is not None:
                    log(f"gate/up [{m} x {k}] . [{n} x {k}]^T + SwiGLU: fused tcgen05 {mine:.1f} us with {best[1]} slices of K, library + pointwise {lib:.1f} us")
        return dict(self.tuned)

    def prefers_fused_swiglu(self, m: int, n: int, k: int) -> bool:
        """The fused product saves a kernel and the round trip of the [m, n] intermediate; it is taken
        wherever the tcgen05 kernel runs at all, unless timing said the library's product plus the
        pointwise kernel is faster for this shape."""
        if not self.fused_swiglu or self.tcgen05_policy == "none" or not tcgen05_supported(m, n, k) or n % 128:
            return False
        return self.tuned.get((n, k, _mpad(m), "swiglu"), True)

    # ---- products -------------------------------------------------------------------------------------------
    def linear(self, x, w, out, workspace=None, status=None):
        """out = x . w^T.  w is [out_features, in_features] as stored in the checkpoint."""
        if x.dtype == torch.float32:
            gemm_plain(x, w, out)
        else:
            self.linear_bf16(x, w, out, workspace, status)

    def linear_bf16(self, x, w, out, workspace=None, status=None):
        """bfloat16 operands, float accumulation; the result in bfloat16 or (for logits) float32."""
        m, k = x.shape
        if self.prefers_tcgen05(m, w.shape[0], k) and x.stride(1) == 1 and w.stride(1) == 1:
            self.gemm_tcgen05(x, w, out, workspace, status, dependent=dependent_launch)
        elif out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)

    def linear_heads(self, a, w, out):
        """out[t, h, :] = w[h] . a[t, h, :]: every head's rows with that head's own matrix.  a [rows, heads, K] and out
        [rows, heads, N] are views with the heads side by side in a row; w [heads, N, K].  float32: the plain kernel
        (k ascending); bfloat16: the library's batched product with float accumulation, on the strided views as
        they are."""
        if a.dtype == torch.float32:
            gemm_plain_heads(a, w, out)
        else:
            torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))

    def gemm_tcgen05(self, a, w, out, workspace=None, status=None, splits=None, cluster=True, dependent=False, swiglu=False,
                     activation="silu"):
        """The tcgen05 product with the number of K slices that this engine's tuning found best for the shape."""
        if splits is None:
            key = (w.shape[0], a.shape[1], _mpad(a.shape[0])) + (("swiglu",) if swiglu else ())
            splits = self.tuned_splits.get(key)
            if splits is not None and cluster:
                splits = min(splits, 8)
        return gemm_tcgen05(a, w, out, workspace, status, splits, cluster, dependent, swiglu, activation)

    # ---- attention ------------------------------------------------------------------------------------------
    def decode_takes_projection(self, batch, dtype, hd: int, group: int, page_size: int, rotary_dim: int, cos_sin) -> bool:
        """Whether this step's attention may be handed the q/k/v projection's rows as they come: every sequence brings
        one token, heads of 128 all rotated, bfloat16, pages the TMA kernel takes."""
        return (self.fused_decode_rope and self.use_tma and dtype == torch.bfloat16 and cos_sin is not None
                and getattr(batch, "max_q_len", 0) == 1 and batch.n_seqs == batch.positions.shape[0]
                and flash_takes_projection(hd, group, page_size, rotary_dim))

    def attention_flash(self, *args, **kwargs):
        kwargs.setdefault("use_tma", self.use_tma)
        return attention_flash(*args, **kwargs)

    def attention(self, q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace=None,
                  projection=None, sinks=None, chunk=0, softcap=0.0):
        """Picks the attention kernel for the dtype, head size and shape of the step.  A step that mixes decoded
        tokens with prompt portions runs as two launches, each kind with the kernel made for it.  ``projection``
        (see ``decode_takes_projection``): the q/k/v rows before norm and rotation, which the decoding kernel then
        finishes itself; ``q`` is not read.  ``chunk``, ``softcap``: see ``attention_plain``."""
        group = nq // nkv
        if projection is not None:
            self.attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                                 projection=projection)
            return
        if q.dtype == torch.bfloat16 and workspace is not None and flash_supported(hd, group):
            runs = _short_and_long(batch, group)
            if runs is not None:
                for run in runs:
                    self._attention_bf16(q, k_pool, v_pool, run, block_table[run.first:run.last], page_size, out, nq, nkv, hd,
                                         window, scale, workspace, sinks, chunk, softcap)
                return
        self._attention_bf16(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace, sinks,
                             chunk, softcap)

    def _attention_bf16(self, q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                        sinks=None, chunk=0, softcap=0.0):
        group = nq // nkv
        if (q.dtype == torch.bfloat16 and self.use_tcgen05_attention and getattr(batch, "max_q_len", 0) * group > 16
                and tcgen05_attention_supported(hd, group, page_size)):
            attention_tcgen05(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace=workspace,
                              sinks=sinks, chunk=chunk, softcap=softcap)
            return
        if q.dtype == torch.bfloat16 and workspace is not None and flash_supported(hd, nq // nkv):
            self.attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                                 sinks=sinks, chunk=chunk, softcap=softcap)
            return
        attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, block_table, page_size, out, nq, nkv, hd,
                        window, scale, batch.status, sinks, chunk, softcap)

    def attention_talk(self, q, k_pool, v_pool, talk, batch, block_table, page_size, out, nq, nkv, hd, dq, dv, window, scale,
                       workspace=None):
        """Attention whose scores are mixed over the heads before the softmax, over one step's batch: in bfloat16 steps with
        prompt portions take the tensor-core kernel (where it is built for the sizes: otherwise the FMA kernel), and so do steps
        of decoded tokens alone, with every sequence's keys split over several blocks whose shares a second kernel adds; the
        32-bit path takes the FMA kernel unsplit (a fixed order of every sum)."""
        splits = 1
        if q.dtype == torch.bfloat16 and getattr(batch, "max_q_len", 1) == 1:
            splits = talk_splits(q.shape[0], batch.max_seq_len, window)
        elif q.dtype == torch.bfloat16:
            # prompt portions: a causal prompt's tiles of 16 tokens are unequal (the last one walks all keys), and fewer than two
            # an SM leave SMs idle behind the heaviest: then every tile's keys go to up to four blocks (while their shares
            # stay a small buffer)
            tiles = -(-q.shape[0] // 16) + batch.n_seqs
            splits = max(1, min(4, -(-2 * _sm_count() // tiles)))
            if q.shape[0] * splits * nq * (dv + 2) * 4 > (64 << 20):
                splits = 1
        if q.dtype == torch.bfloat16 and attention_talk_mma_supported(nq, nkv, hd):
            attention_talk_mma(q, k_pool, v_pool, talk, batch, block_table, page_size, out, nq, nkv, hd, dv, window, scale, splits, workspace)
            return
        if getattr(batch, "max_q_len", 1) > 1:
            splits = 1      # (the FMA kernel splits the keys of decoded tokens only)
        attention_talk_plain(q, k_pool, v_pool, talk, batch.positions, batch.seq_index, block_table, page_size, out, nq, nkv, hd,
                             dq, dv, window, scale, batch.status, splits, workspace)

    def decode_attention_splits(self, n_seqs: int, nkv: int, hd: int, group: int, max_seq_len: int, dtype, chunk: int = 0) -> int:
        """How many blocks share the keys of a (sequence, kv head) when ``n_seqs`` sequences decode one token each:
        the one shape of a decode step's launches that follows the sequences' lengths."""
        # (asked once a layer and step: remembered by what the answer depends on, the length only through its key tiles)
        max_seq_len = _key_span(max_seq_len, chunk, max(1, 64 // group))
        key = (n_seqs, nkv, hd, group, -(-max_seq_len // 64), dtype)
        found = self._splits_memo.get(key)
        if found is None:
            if len(self._splits_memo) > 4096:
                self._splits_memo.clear()
            found = 1 if dtype != torch.bfloat16 or not flash_supported(hd, group) else flash_splits(n_seqs, nkv, max_seq_len)
            self._splits_memo[key] = found
        return found


# Calls without an engine (tests of single kernels, parts bound by hand) take this one: the fixed rule, no tuning.
default = Kernels("measured")
linear, linear_bf16, attention = default.linear, default.linear_bf16, default.attention
prefers_tcgen05, prefers_fused_swiglu = default.prefers_tcgen05, default.prefers_fused_swiglu
decode_takes_projection = default.decode_takes_projection
