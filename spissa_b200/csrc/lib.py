"""ctypes bindings of the CUDA libraries: tensors in, a launch on the current stream.

Every function here launches a hand-written kernel; there is no CPU or library
fallback. A tensor that is not on a CUDA device, a library that cannot be built or a
size that a kernel refuses raises ``KernelError`` with the kernel's own words.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_float, c_longlong

import torch

from . import build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dt_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, got {t.dtype}") from None


_LIBS: dict = {}
_LOADED_PATHS: dict = {}


def load(module: str) -> ctypes.CDLL:
    """Build (if needed) and load one kernel library; cached per process."""
    lib = _LIBS.get(module)
    if lib is None:
        path = build.build_module(module)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load kernel library {path}: {e}") from None
        getattr(lib, f"sp_{module}_last_error").restype = ctypes.c_char_p
        if module == "seqmix":
            lib.sp_retention_chunked_scratch_floats.restype = c_longlong
        if module == "hybrid":
            lib.sp_gla_chunked_scratch_floats.restype = c_longlong
        _LIBS[module] = lib
        _LOADED_PATHS[module] = str(path)
        checked = getattr(lib, f"sp_{module}_range_checked", None)
        _RANGE_CHECKED[module] = bool(checked()) if checked is not None else False
    return lib


_RANGE_CHECKED: dict = {}


def range_checked(module: str) -> bool:
    """Whether ``module`` is loaded as the debug build whose kernels check table entries (see common.cuh)."""
    load(module)
    return _RANGE_CHECKED[module]


def _declare_bounds(module: str, lib, n_pages: int, n_rows: int, device) -> None:
    """Debug build only: the bounds the next launches of ``module`` check page and row indices against."""
    if _RANGE_CHECKED.get(module):
        getattr(lib, f"sp_{module}_set_bounds")(int(n_pages), int(n_rows), c_void_p(_ptr(status_word(device))))


def _table_rows(meta, pt) -> int:
    declared = getattr(meta, "declared_rows", None)
    return int(declared) if declared is not None else int(pt.shape[0])


def _pool_pages(meta, k_pool) -> int:
    """Pages of the pools; a harness may declare fewer than it allocated (``meta.declared_pages``) to see a check fire
    on an index that still lies inside allocated memory."""
    declared = getattr(meta, "declared_pages", None)
    return int(declared) if declared is not None else (int(k_pool.shape[0]) if k_pool is not None else 0)


def loaded_libraries() -> dict:
    return dict(_LOADED_PATHS)


def _check(module: str, rc: int) -> None:
    if rc != 0:
        msg = getattr(_LIBS[module], f"sp_{module}_last_error")()
        raise KernelError(msg.decode() if msg else f"kernel library {module} returned {rc}")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return t.data_ptr()


launches = 0          # kernels launched through these bindings since import (bench.py reports the difference)


# the current stream's handle without building a Stream object for every launch (a fifth of a launch's host time)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    global launches
    launches += 1
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need_contig(*ts):
    for t in ts:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


# ------------------------------------------------------------------ generic
def embed_gather(table, ids, out, status=None, scale: float = 1.0):
    """out[t,:] (float32) = table[ids[t],:] · scale; an id outside the table zeroes the row and sets ``status``."""
    lib = load("generic")
    T, H = out.shape
    _need_contig(table, ids, out)
    _check("generic", lib.sp_embed_gather(
        c_void_p(_ptr(table)), dt_code(table), c_void_p(_ptr(ids)), c_void_p(_ptr(out)),
        T, H, table.shape[0], c_void_p(_ptr(status)), c_float(scale), c_void_p(_stream())))


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r,:] = x[rows[r] or r,:] / sqrt(mean(x²)+eps) · weight; ``x`` is float32."""
    lib = load("generic")
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the 32-bit residual stream")
    _need_contig(x, weight, out, rows)
    n_rows, H = out.shape
    _check("generic", lib.sp_rmsnorm(
        c_void_p(_ptr(x)), c_void_p(_ptr(weight)), dt_code(weight), c_void_p(_ptr(out)), dt_code(out),
        c_void_p(_ptr(rows)), n_rows, H, c_float(eps), c_void_p(_stream())))


def gemm_generic(a, w, out, accumulate=False):
    """out[M,N] (+)= a[M,K] · w[N,K]ᵀ with 32-bit FFMA accumulation, any sizes."""
    lib = load("generic")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm shapes do not match: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm operands must have unit stride in their last dimension")
    _check("generic", lib.sp_gemm_generic(
        c_void_p(_ptr(a)), dt_code(a), c_void_p(_ptr(w)), dt_code(w), c_void_p(_ptr(out)), dt_code(out),
        M, N, K, a.stride(0), w.stride(0), out.stride(0), int(bool(accumulate)), c_void_p(_stream())))


def rope_kv_write(qkv, q_out, k_pool, v_pool, meta, inv_freq, nh, nkv, hd, rd, write_kv=True):
    """Rotate q and k of ``qkv`` [T, (nh+2·nkv)·hd], store q to ``q_out`` and k, v into the paged cache.

    ``meta`` carries ``token_seq``, ``positions``, ``seq_slot`` and the group's ``page_table``
    and ``page_size``. ``rd`` = 0 writes without rotating.
    """
    lib = load("generic")
    T = qkv.shape[0]
    _need_contig(qkv, q_out)
    pt = meta.page_table
    if pt is not None:
        _declare_bounds("generic", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), qkv.device)
    _check("generic", lib.sp_rope_kv_write(
        c_void_p(_ptr(qkv)), dt_code(qkv), c_void_p(_ptr(q_out)), dt_code(q_out),
        c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool) if k_pool is not None else 0,
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1] if pt is not None else 0, meta.page_size,
        c_void_p(_ptr(inv_freq)), T, nh, nkv, hd, rd, int(bool(write_kv)), c_void_p(_stream())))


def _dist_bias_args(dist_bias, nh):
    """(pointer, last distance with an entry of its own) of a per-head table of scores by distance, float32
    [nh, entries]: a key at distance n takes entry min(n, entries − 1)."""
    if dist_bias is None:
        return c_void_p(None), 0
    if dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[0] != nh or not dist_bias.is_contiguous():
        raise KernelError("attention: the distance bias is a contiguous float32 table [heads, distances]")
    return c_void_p(_ptr(dist_bias)), int(dist_bias.shape[1]) - 1


def attention_generic(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, scale, vd=None, sink=None, dist_bias=None):
    """Causal attention of every token of the step over its sequence's cached keys; ``vd``: the size of a value row
    when it differs from a key row's (``out`` is then [T, nh·vd]). ``sink`` (float32 [nh]): per head a score that joins
    the softmax's denominator once and has no value. ``dist_bias`` (float32 [nh, entries]): a score added by the
    distance between query and key, beyond the scale."""
    lib = load("generic")
    bias_ptr, bias_cap = _dist_bias_args(dist_bias, nh)
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nh):
        raise KernelError("attention: the sinks are one float32 per query head")
    T = q.shape[0]
    _need_contig(q, out)
    pt = meta.page_table
    _declare_bounds("generic", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("generic", lib.sp_attention_generic(
        c_void_p(_ptr(q)), dt_code(q), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool),
        c_void_p(_ptr(out)), c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        T, nh, nkv, hd, int(vd or hd), int(window or 0), c_float(scale), c_void_p(_ptr(sink)), bias_ptr, bias_cap,
        c_void_p(_stream())))


def softcap(x, cap: float):
    """x ← cap · tanh(x / cap), element by element, in place (float32)."""
    lib = load("generic")
    if x.dtype != torch.float32:
        raise KernelError("softcap works on float32 values")
    _need_contig(x)
    _check("generic", lib.sp_softcap(c_void_p(_ptr(x)), c_longlong(x.numel()), c_float(cap), c_void_p(_stream())))


def scale_rows_sigmoid(x, z):
    """x[r, :] ← x[r, :] · sigmoid(z[r]) in place; ``z`` float32 [rows] (a gate with one number per token)."""
    lib = load("generic")
    if z.dtype != torch.float32 or z.numel() != x.shape[0]:
        raise KernelError("scale_rows_sigmoid takes one float32 gate per row")
    _need_contig(x, z)
    _check("generic", lib.sp_scale_rows_sigmoid(c_void_p(_ptr(x)), dt_code(x), c_void_p(_ptr(z)), x.shape[0], x.shape[1],
                                                c_void_p(_stream())))


def silu_mul(gu, out):
    """out[r,:] = silu(gu[r,:I]) ⊙ gu[r,I:]."""
    lib = load("generic")
    rows, I = out.shape
    _need_contig(gu, out)
    if gu.dtype != out.dtype or gu.shape[1] != 2 * I:
        raise KernelError("silu_mul wants gu [rows, 2·I] and out [rows, I] of one dtype")
    _check("generic", lib.sp_silu_mul(c_void_p(_ptr(gu)), c_void_p(_ptr(out)), dt_code(out), rows, I,
                                      c_void_p(_stream())))


def add_inplace(dst, src):
    """dst (float32) += src."""
    lib = load("generic")
    _need_contig(dst, src)
    if dst.dtype != torch.float32 or dst.numel() != src.numel():
        raise KernelError("add_inplace wants a float32 destination and equal sizes")
    _check("generic", lib.sp_add_inplace(c_void_p(_ptr(dst)), c_void_p(_ptr(src)), dt_code(src),
                                         c_longlong(dst.numel()), c_void_p(_stream())))


def gather_i32(src, idx, dst):
    """dst[i] = src[idx[i]] for int32 tensors on the device (indices outside ``src`` give 0)."""
    lib = load("generic")
    _need_contig(src, idx, dst)
    if src.dtype != torch.int32 or idx.dtype != torch.int32 or dst.dtype != torch.int32 or idx.numel() < dst.numel():
        raise KernelError("gather_i32 takes int32 tensors and one index per output")
    _check("generic", lib.sp_gather_i32(c_void_p(_ptr(src)), c_void_p(_ptr(idx)), c_void_p(_ptr(dst)), dst.numel(),
                                        src.numel(), c_void_p(_stream())))


def header_note(header, seq_slot, seq_len, tokens):
    """header[seq_slot[b]] = (seq_len[b], draws + 1, tokens[b], .) for every sequence b of a step."""
    lib = load("generic")
    _need_contig(header, seq_slot, seq_len, tokens)
    if any(t.dtype != torch.int32 for t in (header, seq_slot, seq_len, tokens)) or header.dim() != 2 or header.shape[1] != 4:
        raise KernelError("header_note takes int32 tensors and a header of four words per slot")
    n = tokens.numel()
    if seq_slot.numel() < n or seq_len.numel() < n:
        raise KernelError("header_note needs a slot and a length for every token")
    _check("generic", lib.sp_header_note(c_void_p(_ptr(header)), header.shape[0], c_void_p(_ptr(seq_slot)),
                                         c_void_p(_ptr(seq_len)), c_void_p(_ptr(tokens)), n, c_void_p(_stream())))


def wait_runs_out(device, code: int, limit_us: int, waited_ns=None):
    """Launch a kernel whose only wait, on a barrier nobody arrives on, gives up after ``limit_us`` microseconds and
    records ``code`` in the device's status word: how a bounded wait ends, for tests of the fault path."""
    lib = load("generic")
    _check("generic", lib.sp_wait_runs_out(c_void_p(_ptr(status_word(device))), int(code), c_longlong(int(limit_us)),
                                           c_void_p(_ptr(waited_ns)), c_void_p(_stream())))


def argmax_rows(logits, out):
    """out[r] = index of the first maximum of logits[r,:] (float32)."""
    lib = load("generic")
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax wants float32 logits with unit column stride")
    _check("generic", lib.sp_argmax_rows(c_void_p(_ptr(logits)), c_void_p(_ptr(out)), rows, V,
                                         logits.stride(0), c_void_p(_stream())))


# ------------------------------------------------------------------ the greedy head: no logits
HEAD_ARGMAX_TOKENS = 64


def head_argmax_candidates(M: int, N: int) -> int:
    """Candidates per token that ``head_argmax`` needs room for (pairs of float32 and int32), 0 when it does not take M."""
    if M <= 16:
        return int(load("gemv").sp_gemv_argmax_candidates(int(N)))
    if M <= HEAD_ARGMAX_TOKENS:
        return int(load("tc_stream").sp_tc_stream_argmax_candidates(int(N)))
    return 0


def head_argmax_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    M = x.shape[0]
    if M <= 16:
        return gemv_supported(x, w)
    return M <= HEAD_ARGMAX_TOKENS and tc_stream_supported(x, w, 3)


def head_argmax(x, w, cand, out, note=None):
    """out[m] = argmax_n x[m]·w[n] (int32) without the logits: the product keeps one (value, row) candidate per tile
    of ``w`` and token in ``cand`` (float32 [M, head_argmax_candidates, 2] viewed as pairs), a second kernel takes the
    best of each row; the lowest row wins among equal values. ``note`` (an engine's ``step_note()``): the tokens also
    go into the headers of the step's sequences. Two kernels."""
    M, K = x.shape
    N = w.shape[0]
    n_cand = head_argmax_candidates(M, N)
    if n_cand == 0 or cand.dtype != torch.float32 or cand.numel() < M * n_cand * 2 or not cand.is_contiguous():
        raise KernelError(f"head_argmax: {M} tokens x {N} rows need a float32 table of {M}x{n_cand}x2")
    if out.dtype != torch.int32 or out.numel() < M:
        raise KernelError("head_argmax: the tokens go to an int32 tensor with one entry per row")
    if M <= 16:
        _check("gemv", load("gemv").sp_gemv_argmax(
            c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(cand)), M, N, K, x.stride(0), w.stride(0), n_cand,
            c_void_p(_stream())))
    else:
        _check("tc_stream", load("tc_stream").sp_tc_stream(
            c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(cand)), F32, M, N, K, x.stride(0), w.stride(0),
            n_cand, 3, 0, c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))
    header = note.header if note is not None else None
    _check("generic", load("generic").sp_argmax_candidates(
        c_void_p(_ptr(cand)), M, n_cand, n_cand, c_void_p(_ptr(out)), c_void_p(_ptr(header)),
        header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None), c_void_p(_stream())))


# ------------------------------------------------------------------ sampling
def sample_scratch_keys(rows: int, V: int) -> int:
    lib = load("sampling")
    lib.sp_sample_scratch_keys.restype = c_longlong
    return int(lib.sp_sample_scratch_keys(rows, V))


def sample_rows(logits, temperature, top_k, top_p, u, scratch, out):
    """Temperature / top-k / top-p sampling of each row with the uniform numbers ``u``."""
    lib = load("sampling")
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sampling wants float32 logits with unit column stride")
    _check("sampling", lib.sp_sample_rows(
        c_void_p(_ptr(logits)), logits.stride(0), rows, V, c_float(temperature), int(top_k), c_float(top_p),
        c_void_p(_ptr(u)), c_void_p(_ptr(scratch)), c_longlong(scratch.numel()), c_void_p(_ptr(out)),
        c_void_p(_stream())))


# ------------------------------------------------------------------ tensor-core matrix product
_STATUS: dict = {}

STATUS_TEXT = {101: "the TMA loader waited too long for a free pipeline stage",
               102: "the MMA issuer waited too long for a loaded pipeline stage",
               103: "the epilogue waited too long for the accumulator",
               104: "the MMA issuer waited too long for a free accumulator",
               121: "tc_stream: the TMA loader waited too long for a free pipeline stage",
               122: "tc_stream: the MMA issuer waited too long for operands",
               123: "tc_stream: the epilogue warps waited too long for the accumulator",
               201: "decode layers: the copy warp waited too long for a free stage of the weight ring",
               202: "decode layers: a consumer warp waited too long for a weight tile",
               203: "decode layers: a CTA waited too long at the grid barrier",
               204: "decode layers: the split of the keys read from the device is outside what the scratch holds",
               205: "decode layers: a CTA waited too long for its partner's partial attention results",
               111: "attention: the loader waited too long for a free key/value stage",
               112: "attention: the MMA issuer waited too long for the queries",
               113: "attention: the MMA issuer waited too long for keys and values",
               114: "attention: the MMA issuer waited too long for the probabilities",
               115: "attention: the softmax warps waited too long for the scores",
               116: "attention: the softmax warps waited too long for the previous block's output",
               117: "attention: the softmax warps waited too long for the last block's output",
               301: "embedding: a token id outside the vocabulary",
               401: "range check: a page index from a page table lies beyond the pools",
               402: "range check: a sequence's row lies beyond the page table",
               403: "range check: a position lies beyond the page table's width",
               900: "a wait that was meant to run out (test of the fault path)"}


def status_word(device) -> torch.Tensor:
    """The int32 word in which kernels with bounded waits record that a wait ran out (0 = all well)."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS[key]


def check_status(device) -> None:
    """Synchronises and raises ``KernelError`` if a kernel gave up a wait since the last check."""
    key = torch.device(device).index or 0
    if key in _STATUS:
        code = int(_STATUS[key].item())
        if code:
            _STATUS[key].zero_()
            raise KernelError(f"a kernel gave up a bounded wait (code {code}: {STATUS_TEXT.get(code, 'unknown')})")


def tc_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``tc_gemm`` takes these operands (bfloat16, K-major, rows a multiple of 16 bytes)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.shape[1] != w.shape[1]:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


TC_STORE, TC_ACCUMULATE, TC_SILU_MUL = 0, 1, 2


def tc_gemm(a, w, out, mode=TC_STORE, bn=128):
    """out = a · wᵀ on the tcgen05 tensor cores (bfloat16 operands, float32 accumulation).

    ``mode`` TC_STORE writes ``out`` (bfloat16 or float32), TC_ACCUMULATE adds into a float32 ``out``,
    TC_SILU_MUL takes a weight whose rows interleave gate and up in blocks of ``bn``/2 and writes
    silu(gate)·up into ``out`` [M, N/2].
    """
    lib = load("tc_gemm")
    M, K = a.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"tc_gemm: out {tuple(out.shape)} does not fit a {tuple(a.shape)}, w {tuple(w.shape)}")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("tc_gemm takes bfloat16 operands")
    _check("tc_gemm", lib.sp_tc_gemm(
        c_void_p(_ptr(a)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K,
        a.stride(0), w.stride(0), out.stride(0), int(mode), int(bn), c_void_p(_ptr(status_word(a.device))),
        c_void_p(_stream())))


class _EpiArgs(ctypes.Structure):
    """Mirror of ``EpiArgs`` in tc_gemm.cu."""
    _fields_ = [("row_ssq", c_void_p), ("n_ssq", c_int), ("norm_width", c_int), ("eps", c_float), ("pad0", c_int),
                ("xw", c_void_p), ("next_w", c_void_p), ("ssq_out", c_void_p),
                ("cs", c_void_p), ("tok_page", c_void_p), ("positions", c_void_p),
                ("q_out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("page_size", c_int)]


TC_QKV_ROPE = 3


def tc_gemm_splits(M: int, N: int, K: int, bn: int) -> int:
    """CTAs that share a tile along K when ``tc_gemm`` (the plain epilogues) runs these sizes; 1: K is not split."""
    return int(load("tc_gemm").sp_tc_gemm_splits(int(M), int(N), int(K), int(bn)))


def tc_gemm_n_tiles(N: int, bn: int) -> int:
    return (int(N) + int(bn) - 1) // int(bn)


def tc_gemm_fused(a, w, out, mode, bn, row_ssq=None, norm_width=0, eps=0.0, xw=None, next_w=None, ssq_out=None,
                  rope=None):
    """``tc_gemm`` with an epilogue that saves a pass over a prompt's activations.

    ``row_ssq`` [M, n] float32: ``a`` holds x ⊙ w of an RMS norm over ``norm_width`` columns without its 1/rms; the
    result is multiplied by 1/sqrt(sum(row_ssq[m]) / norm_width + eps).
    ``xw``, ``next_w``, ``ssq_out`` (mode TC_ACCUMULATE): besides out += a·wᵀ, xw = new out ⊙ next_w (bfloat16) and
    ssq_out[m, tile] = the new row's sum of squares over each tile's columns ([M, tc_gemm_n_tiles(N, bn)]).
    ``rope`` (mode TC_QKV_ROPE; ``out`` None): dict(cs, tok_page, positions, q_out, k_pool, v_pool, nh, nkv, hd,
    page_size): q and k are rotated with the (cos, sin) table, q stored, k and v written into the paged cache.
    """
    _fused_product("tc_gemm", a, w, out, mode, int(bn), tc_gemm_n_tiles(w.shape[0], bn), row_ssq, norm_width, eps, xw,
                   next_w, ssq_out, rope)


def tc_stream_max_tokens() -> int:
    """Tokens up to which ``tc_stream`` and ``tc_stream_fused`` are built."""
    return 128


def tc_stream_n_tiles(N: int) -> int:
    """Sums of squares per token that ``tc_stream_fused`` writes when it prepares the next norm (tiles of 128 columns)."""
    return (int(N) + 127) // 128


def tc_stream_fused(a, w, out, mode, pair=0, row_ssq=None, norm_width=0, eps=0.0, xw=None, next_w=None, ssq_out=None,
                    rope=None):
    """``tc_stream`` (17 to 128 tokens) with the epilogues of ``tc_gemm_fused``; ``ssq_out`` is
    [M, tc_stream_n_tiles(N)] here and ``pair`` the block of gate rows for TC_SILU_MUL."""
    _fused_product("tc_stream", a, w, out, mode, int(pair), tc_stream_n_tiles(w.shape[0]), row_ssq, norm_width, eps, xw,
                   next_w, ssq_out, rope)


def _fused_product(module, a, w, out, mode, width, n_tiles, row_ssq, norm_width, eps, xw, next_w, ssq_out, rope):
    lib = load(module)
    M, K = a.shape
    N = w.shape[0]
    ep = _EpiArgs()
    if row_ssq is not None:
        if row_ssq.dtype != torch.float32 or row_ssq.dim() != 2 or row_ssq.shape[0] < M or not row_ssq.is_contiguous():
            raise KernelError(f"{module}_fused: the row statistics are a contiguous float32 [M, n] tensor")
        ep.row_ssq, ep.n_ssq, ep.norm_width, ep.eps = _ptr(row_ssq), row_ssq.shape[1], int(norm_width), float(eps)
    if xw is not None:
        if (xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, N) or not xw.is_contiguous() or next_w.dtype != torch.bfloat16
                or next_w.numel() != N or ssq_out.dtype != torch.float32 or tuple(ssq_out.shape) != (M, n_tiles)
                or not ssq_out.is_contiguous()):
            raise KernelError(f"{module}_fused: xw [M, N] and next_w [N] are bfloat16, ssq_out float32 [M, {n_tiles}]")
        ep.xw, ep.next_w, ep.ssq_out = _ptr(xw), _ptr(next_w), _ptr(ssq_out)
    code = int(mode)
    if mode == TC_QKV_ROPE:
        r = rope
        _need_contig(r["cs"], r["tok_page"], r["positions"], r["q_out"])
        if r["q_out"].dtype != torch.bfloat16 or r["k_pool"].dtype != torch.bfloat16 or r["cs"].dtype != torch.float32:
            raise KernelError(f"{module}_fused: q and the cache are bfloat16, the angle table float32")
        ep.cs, ep.tok_page, ep.positions = _ptr(r["cs"]), _ptr(r["tok_page"]), _ptr(r["positions"])
        ep.q_out, ep.kpool, ep.vpool = _ptr(r["q_out"]), _ptr(r["k_pool"]), _ptr(r["v_pool"])
        ep.nh, ep.nkv, ep.hd, ep.page_size = int(r["nh"]), int(r["nkv"]), int(r["hd"]), int(r["page_size"])
        _declare_bounds(module, lib, r.get("declared_pages", r["k_pool"].shape[0]), 0, a.device)
        c_ptr, c_dt, ldc = None, BF16, 0
        if module == "tc_stream":
            code = 4                                   # 3 is the greedy head's mode there
    else:
        want_cols = N // 2 if mode == TC_SILU_MUL else N
        if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
            raise KernelError(f"{module}_fused: out {tuple(out.shape)} does not fit a {tuple(a.shape)}, w {tuple(w.shape)}")
        c_ptr, c_dt, ldc = _ptr(out), dt_code(out), out.stride(0)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"{module} takes bfloat16 operands")
    fn = lib.sp_tc_gemm_fused if module == "tc_gemm" else lib.sp_tc_stream_fused
    _check(module, fn(
        c_void_p(_ptr(a)), c_void_p(_ptr(w)), c_void_p(c_ptr), c_dt, M, N, K, a.stride(0), w.stride(0), ldc,
        code, width, ctypes.byref(ep), c_void_p(_ptr(status_word(a.device))), c_void_p(_stream())))


def rope_table(meta, inv_freq, half, cs, tok_page):
    """cs[t, i] = (cos, sin)(position[t] · inv_freq[i]) and tok_page[t] = the cache page of token t's position."""
    lib = load("generic")
    T = cs.shape[0]
    pt = meta.page_table
    _need_contig(cs, tok_page, inv_freq)
    _declare_bounds("generic", lib, _pool_pages(meta, getattr(meta, "k_pool", None)), _table_rows(meta, pt), cs.device)
    _check("generic", lib.sp_rope_table(
        c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, c_void_p(_ptr(inv_freq)), int(half), T, c_void_p(_ptr(cs)),
        c_void_p(_ptr(tok_page)), c_void_p(_stream())))


def norm_prepare(x, w, xw, ssq):
    """xw = x ⊙ w (bfloat16) and ssq[r] = sum of x[r]² for the float32 residual ``x`` [T, H]."""
    lib = load("generic")
    T, H = x.shape
    _need_contig(x, w, xw, ssq)
    if x.dtype != torch.float32 or w.dtype != torch.bfloat16 or xw.dtype != torch.bfloat16 or ssq.dtype != torch.float32:
        raise KernelError("norm_prepare: float32 residual and sums, bfloat16 weight and output")
    _check("generic", lib.sp_norm_prepare(c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(xw)), c_void_p(_ptr(ssq)),
                                          T, H, c_void_p(_stream())))


# ------------------------------------------------------------------ flash attention (bfloat16)
def flash_supported(q: torch.Tensor, k_pool: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this shape; else the generic kernel runs."""
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        return False
    return bool(load("attention").sp_flash_supported(int(hd), int(nh), int(nkv), int(page_size)))


def flash_query_tile() -> int:
    """Query rows per CTA of ``flash_prefill``: a step has sum over sequences of ceil(new tokens / this) tiles."""
    return int(load("attention").sp_flash_query_tile())


def flash_tc_query_tile() -> int:
    """The same for ``flash_prefill_tc``."""
    return int(load("flash_tc").sp_flash_tc_query_tile())


def query_tiles(new_counts, tile: int) -> int:
    return sum((int(n) + tile - 1) // tile for n in new_counts)


def _sink_ptr(sink, nh):
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nh or not sink.is_contiguous()):
        raise KernelError("attention: the sinks are one float32 per query head")
    return c_void_p(_ptr(sink))


def flash_prefill(q, k_pool, v_pool, out, meta, seq_start, n_seqs, n_q_tiles, nh, nkv, hd, window, scale, sink=None,
                  dist_bias=None):
    """Causal attention of a step's tokens (any number per sequence) over the paged cache. ``sink`` (float32 [nh]):
    per head a score that joins the softmax's denominator once and has no value. ``dist_bias`` (float32 [nh, entries]): a
    score added by the distance between query and key, beyond the scale.

    ``seq_start`` [B+1] int32 on the device; ``n_q_tiles`` = sum over sequences of ceil(new tokens /
    ``flash_query_tile()``).
    """
    lib = load("attention")
    _need_contig(q, out)
    pt = meta.page_table
    _declare_bounds("attention", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    bias_ptr, bias_cap = _dist_bias_args(dist_bias, nh)
    _check("attention", lib.sp_flash_prefill_bias(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_void_p(_ptr(seq_start)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, int(n_seqs), int(n_q_tiles), nh, nkv, hd,
        int(window or 0), c_float(scale), _sink_ptr(sink, nh), bias_ptr, bias_cap, c_void_p(_stream())))


def flash_decode_plan(n_seqs: int, nkv: int, max_len: int, page_size: int = 64) -> tuple:
    """(tiles per chunk, chunks) for the split-key decode attention.

    Measured on B200 (head 64, 8 kv heads, 512 to 4096 keys): about 256 CTAs in all run fastest; with
    more than 256 (sequence, kv head) pairs two chunks beat one once there are 16 tiles or more.
    """
    tiles = max(1, (max_len + page_size - 1) // page_size)
    base = max(1, n_seqs * nkv)
    if base <= 256:
        n_chunks = min(8, max(1, round(256 / base)))
    else:
        n_chunks = 2 if tiles >= 16 else 1
    n_chunks = min(n_chunks, tiles)
    chunk_tiles = -(-tiles // n_chunks)
    n_chunks = -(-tiles // chunk_tiles)
    return chunk_tiles, n_chunks


def flash_decode_scratch_floats(n_seqs: int, nh: int, hd: int, n_chunks: int) -> int:
    return n_seqs * nh * n_chunks * (hd + 2)


def flash_decode(q, k_pool, v_pool, out, meta, seq_len, nh, nkv, hd, window, scale, chunk_tiles, n_chunks, scratch,
                 counters=None, sink=None, dist_bias=None):
    """One query token per sequence: keys split into chunks over CTAs, partial results combined in order.

    ``seq_len`` [B] int32: each sequence's length including the query token. ``scratch``: float32,
    at least ``flash_decode_scratch_floats`` elements. ``counters``: int32, n_seqs·nkv zeros that the kernel
    hands back as zeros; with them the last CTA of each (sequence, kv head) combines, else a second kernel.
    """
    global launches
    lib = load("attention")
    _need_contig(q, out)
    pt = meta.page_table
    n_seqs = q.shape[0]
    if counters is not None and (counters.dtype != torch.int32 or counters.numel() < n_seqs * nkv):
        raise KernelError("flash_decode: counters must be int32 with a word per (sequence, kv head)")
    _declare_bounds("attention", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    bias_ptr, bias_cap = _dist_bias_args(dist_bias, nh)
    _check("attention", lib.sp_flash_decode_bias(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_void_p(_ptr(seq_len)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        n_seqs, nh, nkv, hd, int(window or 0), c_float(scale), int(chunk_tiles), int(n_chunks),
        c_void_p(_ptr(scratch)), c_longlong(scratch.numel()), c_void_p(_ptr(counters)), _sink_ptr(sink, nh),
        bias_ptr, bias_cap, c_void_p(_stream())))
    if counters is None:
        launches += 1        # two kernels: the chunks and the combine


# ------------------------------------------------------------------ skinny products for decoding
GEMV_MAX_TOKENS = 64


def gemv_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    K = x.shape[1]
    return (0 < x.shape[0] <= GEMV_MAX_TOKENS and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv(x, w, out, mode=TC_STORE, pair=0):
    """out = x · wᵀ for up to 64 tokens, streaming ``w`` once. Modes as ``tc_gemm``; for TC_SILU_MUL
    ``pair`` is the number of gate rows before the matching up rows in the interleaved weight."""
    lib = load("gemv")
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"gemv: out {tuple(out.shape)} does not fit x {tuple(x.shape)}, w {tuple(w.shape)}")
    _check("gemv", lib.sp_gemv(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K,
        x.stride(0), w.stride(0), out.stride(0), int(mode), int(pair), c_void_p(_stream())))


def gemv_qkv_rope(x, w, q_out, k_pool, v_pool, meta, inv_freq, nh, nkv, hd):
    """The QKV product of a few tokens with rotate-half and the cache write in its epilogue.

    ``x`` bfloat16 [M, K]; ``w`` = [Wq; Wk; Wv]; q goes to ``q_out`` (bfloat16), k and v into the paged
    bfloat16 cache at each token's position.
    """
    lib = load("gemv")
    M, K = x.shape
    pt = meta.page_table
    if q_out.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemv_qkv_rope works on bfloat16 weights, queries and cache")
    _declare_bounds("gemv", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), x.device)
    _check("gemv", lib.sp_gemv_qkv_rope(
        c_void_p(_ptr(x)), x.stride(0), c_void_p(_ptr(w)), w.stride(0), M, K, nh, nkv, hd, c_void_p(_ptr(q_out)),
        c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.token_seq)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, c_void_p(_ptr(inv_freq)),
        c_void_p(_stream())))


# ------------------------------------------------------------------ prefill attention on tcgen05
def flash_tc_supported(q: torch.Tensor, k_pool: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int, window) -> bool:
    """Whether the tcgen05 prefill attention takes this shape (head 64 or 128, pages of 64, bfloat16; any window)."""
    return (q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and k_pool.is_contiguous()
            and bool(load("flash_tc").sp_flash_tc_supported(int(hd), int(nh), int(nkv), int(page_size), int(window or 0))))


def flash_prefill_tc(q, k_pool, v_pool, out, meta, seq_start, n_seqs, n_q_tiles, nh, nkv, hd, window, scale, sink=None,
                     dist_bias=None):
    """Causal attention of a step's tokens over the paged cache on the tcgen05 tensor cores. ``dist_bias`` (float32
    [nh, entries]): a score added by the distance between query and key, beyond the scale.

    ``n_q_tiles`` = sum over sequences of ceil(new tokens / ``flash_tc_query_tile()``). S, P and O live in tensor memory.
    """
    lib = load("flash_tc")
    _need_contig(q, out, k_pool, v_pool)
    pt = meta.page_table
    _declare_bounds("flash_tc", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    bias_ptr, bias_cap = _dist_bias_args(dist_bias, nh)
    _check("flash_tc", lib.sp_flash_prefill_tc_bias(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_longlong(k_pool.shape[0]), q.shape[0], c_void_p(_ptr(seq_start)), c_void_p(_ptr(meta.positions)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, int(n_seqs), int(n_q_tiles),
        nh, nkv, hd, int(window or 0), c_float(scale), c_void_p(_ptr(status_word(q.device))), _sink_ptr(sink, nh),
        bias_ptr, bias_cap, c_void_p(_stream())))


FLASH_TC_ROW_SIZES = ((64, 64), (128, 128), (192, 128))      # (key row, value row) per head that the kernel is built for


def flash_tc_rows_supported(dtype, nh: int, nkv: int, hd: int, vd: int | None = None) -> bool:
    """Whether ``flash_prefill_tc_rows`` takes queries, keys and values of this type and shape (``vd``: the size of a
    value row when it differs from a key row's)."""
    if dtype != torch.bfloat16 or (int(hd), int(vd or hd)) not in FLASH_TC_ROW_SIZES:
        return False                              # (asked before the library: a model of other sizes never builds it)
    return bool(load("flash_tc").sp_flash_tc_rows_supported(int(hd), int(vd or hd), int(nh), int(nkv)))


def flash_prefill_tc_rows(q, k, v, out, step, n_q_tiles, nh, nkv, hd, window, scale, sink=None, vd=None):
    """The tcgen05 prefill attention over keys and values that lie in no cache: ``k`` [T, nkv·hd] and ``v`` [T, nkv·vd]
    bfloat16 are the step's own tokens, and EVERY sequence of the step starts at its position 0 (the caller has
    checked). ``out`` is [T, nh·vd]."""
    lib = load("flash_tc")
    _need_contig(q, out, k, v)
    T = q.shape[0]
    vd = int(vd or hd)
    if k.shape != (T, nkv * hd) or v.shape != (T, nkv * vd) or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise KernelError("flash_tc: keys and values as rows are bfloat16 [tokens, kv heads x row size]")
    if out.shape != (T, nh * vd) or q.shape[1] != nh * hd:
        raise KernelError("flash_tc: queries are [tokens, heads x key size], the output [tokens, heads x value size]")
    _check("flash_tc", lib.sp_flash_prefill_tc_rows_kv(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k)), c_void_p(_ptr(v)), T, c_void_p(_ptr(step.seq_start)),
        c_void_p(_ptr(step.positions)), int(step.n_seqs), int(n_q_tiles), nh, nkv, hd, vd, int(window or 0), c_float(scale),
        c_void_p(_ptr(status_word(q.device))), _sink_ptr(sink, nh), c_void_p(_stream())))


# ------------------------------------------------------------------ all layers of a decode step in one kernel
def decode_layers_ctas() -> int:
    return int(load("decode_layers").sp_decode_layers_ctas())


def decode_layers_max_chunks() -> int:
    return int(load("decode_layers").sp_decode_layers_max_chunks())


def decode_layers_max_pages() -> int:
    """Pages of the longest sequence that the kernel's split of the keys can hold."""
    return int(load("decode_layers").sp_decode_layers_max_pages())


def decode_layers_desc_bytes() -> int:
    return int(load("decode_layers").sp_decode_layers_desc_bytes())


def decode_layers_supported(T: int, H: int, hd: int, page_size: int, max_heads_per_kv: int) -> bool:
    return bool(load("decode_layers").sp_decode_layers_supported(int(T), int(H), int(hd), int(page_size),
                                                                 int(max_heads_per_kv)))


def decode_layers_encode_map(w: torch.Tensor, pair: int) -> bytes:
    """The TMA view of weight ``w`` [N, K] for the decode kernel's tile walk (rows in pairs ``pair`` apart; 0: plain)."""
    lib = load("decode_layers")
    _need_contig(w)
    n = int(lib.sp_decode_layers_map_bytes())
    buf = ctypes.create_string_buffer(n)
    _check("decode_layers", lib.sp_decode_layers_encode_map(buf, c_void_p(_ptr(w)), w.shape[0], w.shape[1], int(pair)))
    return buf.raw


def decode_layers(table, maps, n_layers, T, H, hd, x, q, attn, act, xw, ssq, part_o, part_ml, positions, seq_row, page_table,
                  page_size, len_pages, max_nkv, max_heads_per_kv, sync, plan=None, n_pages=0):
    """Every layer of a decode step (one token per sequence, T ≤ 16) on the residual ``x`` [T, H] float32, in place.

    ``table``: the layers' descriptors on the device (``decode_layers_desc_bytes()`` each). One cooperative launch;
    counts as one kernel. ``plan`` (two int32 on the device, from ``decode_layers_plan``) overrides the split of
    the keys that ``len_pages`` would give: a captured launch reads it anew at every replay.
    """
    lib = load("decode_layers")
    _need_contig(x, q, attn, act, page_table)
    if x.dtype != torch.float32 or x.shape[0] != T or x.shape[1] != H:
        raise KernelError(f"decode_layers: the residual must be float32 [{T}, {H}], got {x.dtype} {tuple(x.shape)}")
    _declare_bounds("decode_layers", lib, n_pages, page_table.shape[0], x.device)
    _check("decode_layers", lib.sp_decode_layers(
        c_void_p(_ptr(table)), c_void_p(_ptr(maps)), int(n_layers), int(T), int(H), int(hd), c_void_p(_ptr(x)), c_void_p(_ptr(q)),
        c_void_p(_ptr(attn)), c_void_p(_ptr(act)), c_void_p(_ptr(xw)), c_void_p(_ptr(ssq)), c_void_p(_ptr(part_o)), c_void_p(_ptr(part_ml)),
        c_void_p(_ptr(positions)), c_void_p(_ptr(seq_row)), c_void_p(_ptr(page_table)), page_table.shape[1],
        int(page_size), int(len_pages), int(max_nkv), int(max_heads_per_kv),
        c_void_p(_ptr(plan) if plan is not None else 0), c_void_p(_ptr(sync)),
        c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))


def decode_layers_set_head(mode: int, w, norm_w, eps: float, out, ld: int) -> None:
    """The output head of the NEXT ``decode_layers`` call: ``mode`` 1 writes logits [T, ld] (float32), 2 one (value,
    row) candidate per token and CTA [T, ld] (pairs of float32 and int32, for ``argmax_candidates``). The final norm
    (weight ``norm_w``, ``eps``) is folded into the product; the head's tensor map follows the layers' in ``maps``."""
    lib = load("decode_layers")
    _need_contig(w, norm_w, out)
    _check("decode_layers", lib.sp_decode_layers_set_head(
        int(mode), c_void_p(_ptr(w)), c_void_p(_ptr(norm_w)), c_float(eps), int(w.shape[0]), c_void_p(_ptr(out)), int(ld)))


def decode_layers_set_embedding(table, ids) -> None:
    """For the NEXT ``decode_layers`` call: the kernel fills the residual itself from the bfloat16 embedding ``table``
    [rows, H] and the token ``ids`` (int32 on the device); an id outside the table: a zero row and code 301."""
    lib = load("decode_layers")
    _need_contig(table, ids)
    if table.dtype != torch.bfloat16 or ids.dtype != torch.int32:
        raise KernelError("decode_layers: a bfloat16 embedding table and int32 token ids")
    _check("decode_layers", lib.sp_decode_layers_set_embedding(c_void_p(_ptr(table)), int(table.shape[0]), c_void_p(_ptr(ids))))


def decode_layers_set_greedy_out(tokens, note=None) -> None:
    """With head mode 2, for the NEXT ``decode_layers`` call: the kernel's last CTA also takes the best of each token's
    candidates and writes the tokens (int32 [T]); with ``note`` they also go into the headers of the step's sequences."""
    lib = load("decode_layers")
    header = note.header if note is not None else None
    _check("decode_layers", lib.sp_decode_layers_set_greedy_out(
        c_void_p(_ptr(tokens)), c_void_p(_ptr(header)), header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None)))


def argmax_candidates(cand, rows: int, n_cand: int, out, note=None) -> None:
    """out[r] = the row of the best of ``cand[r, :n_cand]`` ((value, row) pairs; the lowest row among equal values);
    with ``note`` the tokens also go into the headers of the step's sequences."""
    header = note.header if note is not None else None
    _check("generic", load("generic").sp_argmax_candidates(
        c_void_p(_ptr(cand)), int(rows), int(n_cand), int(cand.shape[1]), c_void_p(_ptr(out)), c_void_p(_ptr(header)),
        header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None), c_void_p(_stream())))


def decode_layers_plan(T: int, hd: int, len_pages: int, max_nkv: int) -> tuple:
    """(pages per chunk, chunks) of the keys for ``T`` sequences of at most ``len_pages`` pages."""
    lib = load("decode_layers")
    out = (ctypes.c_int * 2)()
    _check("decode_layers", lib.sp_decode_layers_plan(int(T), int(hd), int(len_pages), int(max_nkv), out))
    return int(out[0]), int(out[1])


# ------------------------------------------------------------------ weight-streaming tensor-core product (17..128 tokens)
def tc_stream_supported(x: torch.Tensor, w: torch.Tensor, mode=TC_STORE, pair: int = 0) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    return load("tc_stream").sp_tc_stream_supported(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0),
        int(mode), int(pair)) == 0


def tc_stream(x, w, out, mode=TC_STORE, pair=0):
    """out = x · wᵀ for up to 128 tokens on the tensor cores with the rows of ``w`` as the instruction's M: every SM
    streams its share of ``w``; K is cut over the CTAs of a cluster, whose pieces are added in a fixed order. Modes as ``tc_gemm``; for
    TC_SILU_MUL ``pair`` is the number of gate rows before the matching up rows in the interleaved weight."""
    lib = load("tc_stream")
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"tc_stream: out {tuple(out.shape)} does not fit x {tuple(x.shape)}, w {tuple(w.shape)}")
    _check("tc_stream", lib.sp_tc_stream(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K, x.stride(0), w.stride(0),
        out.stride(0), int(mode), int(pair), c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))


# ------------------------------------------------------------------ seqmix: other mixers, their norm and activation
def _w_dt(*ts):
    """The one storage type of a part's small tensors (they come from one checkpoint)."""
    codes = {dt_code(t) for t in ts if t is not None}
    if len(codes) != 1:
        raise KernelError("a part's small tensors must share one storage type")
    return codes.pop()


def dyt_norm(x, weight, bias, alpha, out, rows=None):
    """out[r,:] = tanh(alpha · x[rows[r] or r,:]) ⊙ weight + bias; ``x`` is the float32 residual stream."""
    lib = load("seqmix")
    if x.dtype != torch.float32:
        raise KernelError("dyt_norm reads the 32-bit residual stream")
    _need_contig(x, weight, bias, alpha, out, rows)
    n_rows, H = out.shape
    _check("seqmix", lib.sp_dyt_norm(
        c_void_p(_ptr(x)), c_void_p(_ptr(weight)), c_void_p(_ptr(bias)), c_void_p(_ptr(alpha)), _w_dt(weight, bias, alpha),
        c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(rows)), n_rows, H, c_void_p(_stream())))


def token_shift(x, mu, state, out, step, dyt=None):
    """out[t] = h[t] + (h[t-1] − h[t]) ⊙ mu with h = ``x`` itself, or dyt(x) when ``dyt`` = (weight, bias, alpha) and
    ``x`` is the float32 residual stream. h[-1] of a step's first token comes from ``state[slot]`` (float32
    [slots, H]), which then takes the sequence's last h."""
    lib = load("seqmix")
    T, H = out.shape
    _need_contig(x, mu, state, out)
    if state.dtype != torch.float32 or state.shape[-1] != H:
        raise KernelError("token_shift keeps a float32 state of the stream's width per slot")
    w, b, a = dyt if dyt is not None else (None, None, None)
    global launches
    if not step.all_single and (dyt is None or H % 4):
        launches += 1                                  # the state is stored by a second launch behind the first
    _check("seqmix", lib.sp_token_shift(
        c_void_p(_ptr(x)), dt_code(x), c_void_p(_ptr(w)), c_void_p(_ptr(b)), c_void_p(_ptr(a)),
        _w_dt(w, b, a) if dyt is not None else 0, c_void_p(_ptr(mu)), dt_code(mu), c_void_p(_ptr(state)), state.shape[0],
        c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.token_seq)), c_void_p(_ptr(step.seq_start)),
        c_void_p(_ptr(step.seq_slot)), T, step.n_seqs, H, int(bool(step.all_single)), c_void_p(_stream())))


def diff_qkv_store(qkv, bias, q_out, k_pool, v_pool, meta, inv_freq, nq, nk, G, d, vd, rd, residual=None, residual_bias=None):
    """Add ``bias``, rotate neighbouring pairs over the first ``rd`` dims of each of the nq + nk sub-heads of size d,
    store q to ``q_out`` and k (rows of nk/G·d per kv head) and v (rows of vd) into the paged cache. With ``residual``
    (float32 [T, W]) and ``residual_bias`` [W] every token's row of the stream also takes that bias (the output
    projection's, ahead of the product that accumulates into the stream)."""
    lib = load("seqmix")
    if qkv.dtype != torch.float32:
        raise KernelError("diff_qkv_store reads 32-bit projections")
    _need_contig(qkv, bias, q_out, residual, residual_bias)
    if residual is not None and (residual.dtype != torch.float32 or residual_bias is None or bias is None
                                 or residual_bias.dtype != bias.dtype or residual_bias.numel() != residual.shape[1]):
        raise KernelError("diff_qkv_store adds a bias of the projections' storage type to a float32 stream")
    T = qkv.shape[0]
    pt = meta.page_table
    _declare_bounds("seqmix", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), qkv.device)
    _check("seqmix", lib.sp_diff_qkv_store(
        c_void_p(_ptr(qkv)), c_void_p(_ptr(bias)), dt_code(bias) if bias is not None else 0, c_void_p(_ptr(q_out)),
        dt_code(q_out), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool), c_void_p(_ptr(meta.token_seq)),
        c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        c_void_p(_ptr(inv_freq)), T, nq, nk, G, d, vd, rd, c_void_p(_ptr(residual)), c_void_p(_ptr(residual_bias)),
        residual.shape[1] if residual is not None else 0, c_void_p(_stream())))


def diff_attention(q, k_pool, v_pool, out, meta, H, G, d, vd, window, keep_first, scale, softcap, lam, eps, out_scale):
    """Two softmax maps per head over one set of values, a1 − lam·a2, unit rms per head, times ``out_scale``."""
    lib = load("seqmix")
    _need_contig(q, out)
    T = q.shape[0]
    pt = meta.page_table
    _declare_bounds("seqmix", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("seqmix", lib.sp_diff_attention(
        c_void_p(_ptr(q)), dt_code(q), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool), c_void_p(_ptr(out)),
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)),
        pt.shape[1], meta.page_size, T, H, G, d, vd, int(window or 0), int(keep_first or 0), c_float(scale),
        c_float(softcap or 0.0), c_float(lam), c_float(eps), c_float(out_scale), c_void_p(_stream())))


def retention(proj, state, decay, out, step, H, d, vd, eps):
    """proj rows [q | k | v | g] (float32); state float32 [slots, H, d, vd]; out [T, H·vd]."""
    lib = load("seqmix")
    if proj.dtype != torch.float32 or state.dtype != torch.float32 or decay.dtype != torch.float32:
        raise KernelError("retention runs on 32-bit projections, state and decays")
    _need_contig(proj, state, decay, out)
    global launches
    if not step.all_single and step.max_new >= CHUNKED_FROM and retention_chunked_supported(d, vd):
        # a prompt: chunks of 64 tokens in parallel (FFMA tiles), their start states by a short scan
        launches += 3
        n_chunks, T = _chunks(step), proj.shape[0]
        need = lib.sp_retention_chunked_scratch_floats(n_chunks, T, H, d, vd)
        scratch = torch.empty(need, dtype=torch.float32, device=proj.device)
        _check("seqmix", lib.sp_retention_chunked(
            c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(decay)),
            c_void_p(_ptr(scratch)), c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)),
            c_void_p(_ptr(step.seq_slot)), step.n_seqs, T, n_chunks, H, d, vd, c_float(eps), c_void_p(_stream())))
        return
    if step.all_single and d <= 4096:
        # a decode step: the states are streamed once, straight from and to global memory
        launches += 1
        o_raw = torch.empty(proj.shape[0] * H * vd, dtype=torch.float32, device=proj.device)
        _check("seqmix", lib.sp_retention_step(
            c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(decay)),
            c_void_p(_ptr(o_raw)), c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)),
            c_void_p(_ptr(step.seq_slot)), step.n_seqs, H, d, vd, c_float(eps), c_void_p(_stream())))
        return
    _check("seqmix", lib.sp_retention(
        c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(decay)),
        c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), step.n_seqs,
        H, d, vd, c_float(eps), c_void_p(_stream())))


CHUNK_TOKENS = 64            # tokens per chunk of the chunked recurrences
CHUNKED_FROM = 32            # a step's longest portion from which the recurrences run in chunks


def _chunks(step) -> int:
    return query_tiles(step.host["new_counts"], CHUNK_TOKENS)


def retention_chunked_supported(d: int, vd: int) -> bool:
    return bool(load("seqmix").sp_retention_chunked_supported(d, vd))


def mingru(proj, z_bias, x_bias, state, out, step, W):
    """proj rows [z | x | g] (float32, biases not yet added); state float32 [slots, W]; out [T, W]."""
    lib = load("seqmix")
    if proj.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("mingru runs on 32-bit projections and state")
    _need_contig(proj, z_bias, x_bias, state, out)
    if not step.all_single and step.max_new >= CHUNKED_FROM:
        # a prompt: chunks of 64 tokens in parallel, their start states by a short scan
        global launches
        launches += 2
        n_chunks = query_tiles(step.host["new_counts"], int(lib.sp_mingru_chunk_tokens()))
        scratch = torch.empty(n_chunks * W * 2, dtype=torch.float32, device=proj.device)
        _check("seqmix", lib.sp_mingru_chunked(
            c_void_p(_ptr(proj)), c_void_p(_ptr(z_bias)), c_void_p(_ptr(x_bias)), _w_dt(z_bias, x_bias),
            c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(scratch)), c_void_p(_ptr(out)), dt_code(out),
            c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), step.n_seqs, n_chunks, W, c_void_p(_stream())))
        return
    _check("seqmix", lib.sp_mingru(
        c_void_p(_ptr(proj)), c_void_p(_ptr(z_bias)), c_void_p(_ptr(x_bias)), _w_dt(z_bias, x_bias), c_void_p(_ptr(state)),
        state.shape[0], c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)),
        step.n_seqs, W, c_void_p(_stream())))


def polynorm(z, coef, out, eps):
    """out = a·N(z) + b·N(z²) + c·N(z³) + e per row of ``z`` (float32), (a, b, c, e) = ``coef``."""
    lib = load("seqmix")
    if z.dtype != torch.float32:
        raise KernelError("polynorm reads 32-bit pre-activations")
    _need_contig(z, coef, out)
    T, F = z.shape
    _check("seqmix", lib.sp_polynorm(c_void_p(_ptr(z)), c_void_p(_ptr(coef)), dt_code(coef), c_void_p(_ptr(out)),
                                     dt_code(out), T, F, c_float(eps), c_void_p(_stream())))


def add_bias(x, bias):
    """Every row of ``x`` (float32 [T, N]) += ``bias`` [N]."""
    lib = load("seqmix")
    if x.dtype != torch.float32 or bias.numel() != x.shape[1]:
        raise KernelError("add_bias wants a float32 matrix and one bias per column")
    _need_contig(x, bias)
    _check("seqmix", lib.sp_add_bias(c_void_p(_ptr(x)), c_void_p(_ptr(bias)), dt_code(bias), x.shape[0], x.shape[1],
                                     c_void_p(_stream())))


# ------------------------------------------------------------------ diff_flash: differential attention of prompt steps
def diff_flash_supported(d: int, vd: int, H: int, G: int, page_size: int) -> bool:
    return bool(load("diff_flash").sp_diff_flash_supported(d, vd, H, G, page_size))


def diff_flash_query_tile() -> int:
    return int(load("diff_flash").sp_diff_flash_query_tile())


def diff_flash_prefill(q, k_pool, v_pool, out, meta, seq_start, n_seqs, n_q_tiles, H, G, d, vd, window, keep_first,
                       scale, softcap, lam, eps, out_scale):
    """``diff_attention`` for the tokens of prompts (bfloat16 q and cache), 64 queries per CTA on the tensor cores."""
    lib = load("diff_flash")
    _need_contig(q, out)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("diff_flash_prefill takes bfloat16 queries, cache and output")
    pt = meta.page_table
    _declare_bounds("diff_flash", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("diff_flash", lib.sp_diff_flash_prefill(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), c_void_p(_ptr(seq_start)),
        c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        n_seqs, n_q_tiles, H, G, d, vd, int(window or 0), int(keep_first or 0), c_float(scale), c_float(softcap or 0.0),
        c_float(lam), c_float(eps), c_float(out_scale), c_void_p(_stream())))


# ------------------------------------------------------------------ hybrid: several streams, a convolved windowed
# attention, gated linear attention, routed experts
def streams_norm(x, S, W, out=None, weight=None, eps=0.0, y=None, mix=None, out_coef=None, in_coef=None, rows=None):
    """The streams ``x`` (float32 [T, S·W]) take a sublayer's output ``y`` (float32 [T, W], left zeroed) in:
    X_t ← Σ_s mix[s,t] X_s + out_coef[t]·y (``mix`` None: every stream keeps itself, ``out_coef`` None: ones); then
    ``out`` [rows, W] = layer norm (mean and variance, ``weight``, no bias) of Σ_s in_coef[s] X_s (``in_coef`` None:
    the plain sum). Either half may be left out (``y`` None / ``weight`` None). ``rows`` gathers (without ``y``)."""
    lib = load("hybrid")
    if x.dtype != torch.float32 or (y is not None and y.dtype != torch.float32):
        raise KernelError("streams_norm works on the 32-bit residual streams")
    for c in (mix, out_coef, in_coef):
        if c is not None and c.dtype != torch.float32:
            raise KernelError("streams_norm takes its coefficients as float32")
    _need_contig(x, y, mix, out_coef, in_coef, weight, out, rows)
    n_rows = out.shape[0] if out is not None else x.shape[0]
    _check("hybrid", lib.sp_streams_norm(
        c_void_p(_ptr(x)), c_void_p(_ptr(y)), c_void_p(_ptr(mix)), c_void_p(_ptr(out_coef)), c_void_p(_ptr(in_coef)),
        c_void_p(_ptr(weight)), dt_code(weight) if weight is not None else 0, c_void_p(_ptr(out)),
        dt_code(out) if out is not None else 0, c_void_p(_ptr(rows)), n_rows, int(S), int(W), c_float(eps),
        c_void_p(_stream())))


def streams_expand(h, x, S):
    """x [T, S·W] (float32): every stream a copy of ``h`` [T, W]."""
    lib = load("hybrid")
    _need_contig(h, x)
    T, W = h.shape
    _check("hybrid", lib.sp_streams_expand(c_void_p(_ptr(h)), c_void_p(_ptr(x)), T, int(S), W, c_void_p(_stream())))


def conv_qk_store(qkv, conv, taps, state, q_out, k_pool, v_pool, meta, step, inv_freq, nh, nkv, d, vd, rd, eps,
                  v_scale=1.0, unit_rms=True, v_from_k=False):
    """``qkv`` rows [q | k | v] (float32): a causal convolution of ``taps`` taps over time on every channel (``conv``
    [C, taps]; ``state`` float32 [slots, taps−1, C] holds each sequence's last inputs), rotation of dim i with dim
    i + rd/2 over the first ``rd`` dims of each q and k head, unit rms per head, q to ``q_out``, k and v (times
    ``v_scale``) into the paged cache. ``v_from_k``: rows are [q | k] only and a token's values are its keys as they
    leave the convolution, before their rotation."""
    lib = load("hybrid")
    if qkv.dtype != torch.float32 or (state is not None and state.dtype != torch.float32):
        raise KernelError("conv_qk_store reads 32-bit projections and keeps a 32-bit state")
    _need_contig(qkv, conv, state, q_out)
    T = qkv.shape[0]
    pt = meta.page_table
    _declare_bounds("hybrid", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), qkv.device)
    global launches
    if taps > 1 and not step.all_single:
        launches += 1                                  # the state is stored by a second launch behind the first
    _check("hybrid", lib.sp_conv_qk_store(
        c_void_p(_ptr(qkv)), qkv.shape[1], c_void_p(_ptr(conv)), dt_code(conv) if conv is not None else 0, int(taps),
        c_void_p(_ptr(state)), state.shape[0] if state is not None else 0, c_void_p(_ptr(inv_freq)), int(rd),
        c_void_p(_ptr(q_out)), dt_code(q_out), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool),
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)),
        pt.shape[1], meta.page_size, c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), T, step.n_seqs,
        nh, nkv, d, vd, c_float(eps), c_float(v_scale), int(bool(unit_rms)), int(bool(step.all_single)),
        int(bool(v_from_k)), c_void_p(_stream())))


def gla(proj, state, a2, a2_bias, norm_weight, out, step, H, d, vd, rank, tau, eps, out_scale=1.0):
    """Gated linear attention. proj rows [q | k | v | g | r] (float32, r the low-rank input of the decays); state
    float32 [slots, H, d, vd]; out [T, H·vd] = rms norm (``norm_weight`` [vd]) of the heads' outputs ⊙ silu(g) ·
    ``out_scale``."""
    lib = load("hybrid")
    if proj.dtype != torch.float32 or state.dtype != torch.float32:
        raise KernelError("gla runs on 32-bit projections and state")
    _need_contig(proj, state, a2, a2_bias, norm_weight, out)
    o_raw, mode = None, 0
    global launches
    if not step.all_single and step.max_new >= CHUNKED_FROM and lib.sp_gla_chunked_supported(d, vd, rank):
        # a prompt: chunks of 64 tokens in parallel (FFMA tiles), their start states by a short scan
        launches += 4
        T = proj.shape[0]
        n_chunks = query_tiles(step.host["new_counts"], int(lib.sp_gla_chunk_tokens()))
        need = lib.sp_gla_chunked_scratch_floats(n_chunks, T, H, d, vd)
        scratch = torch.empty(need, dtype=torch.float32, device=proj.device)
        _check("hybrid", lib.sp_gla_chunked(
            c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(a2)),
            c_void_p(_ptr(a2_bias)), c_void_p(_ptr(norm_weight)), _w_dt(a2, a2_bias, norm_weight), c_void_p(_ptr(scratch)),
            c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), step.n_seqs,
            T, n_chunks, H, d, vd, rank, c_float(tau), c_float(eps), c_float(out_scale), c_void_p(_stream())))
        return
    if step.all_single and d <= 2048:
        launches += 1                                  # the states streamed once, then the norm and the gate
        o_raw = torch.empty(proj.shape[0] * H * vd, dtype=torch.float32, device=proj.device)
        mode = 1
    _check("hybrid", lib.sp_gla(
        c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(state)), state.shape[0], c_void_p(_ptr(a2)),
        c_void_p(_ptr(a2_bias)), c_void_p(_ptr(norm_weight)), _w_dt(a2, a2_bias, norm_weight), c_void_p(_ptr(o_raw)),
        c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), step.n_seqs,
        H, d, vd, rank, c_float(tau), c_float(eps), c_float(out_scale), mode, c_void_p(_stream())))


def gelu_tanh(z, out):
    """out = ½ z (1 + tanh(√(2/π) (z + 0.044715 z³))), element by element."""
    lib = load("hybrid")
    _need_contig(z, out)
    _check("hybrid", lib.sp_gelu_tanh(c_void_p(_ptr(z)), dt_code(z), c_void_p(_ptr(out)), dt_code(out),
                                      c_longlong(z.numel()), c_void_p(_stream())))


def clamped_glu(gu, out, limit, slope=1.702):
    """gu rows [gate | up]: g = min(gate, limit), u = clamp(up, ±limit), out = g · sigmoid(slope · g) · (u + 1)."""
    lib = load("hybrid")
    rows, F = out.shape
    _need_contig(gu, out)
    if gu.shape[1] != 2 * F:
        raise KernelError("clamped_glu wants gu [rows, 2·F] and out [rows, F]")
    _check("hybrid", lib.sp_clamped_glu(c_void_p(_ptr(gu)), dt_code(gu), c_void_p(_ptr(out)), dt_code(out), rows, F,
                                        c_float(limit), c_float(slope), c_void_p(_stream())))


def moe_select(z, correction, ids, weights, top, n_groups=1, keep=1, softmax=False, weight_scale=1.0, experts=None,
               extra=None):
    """From router logits ``z`` (float32 [T, E]): the ``top`` experts per token by s + correction (s = sigmoid(z), or
    with ``softmax`` the softmax over the row's experts) among the ``keep`` best of ``n_groups`` groups (a group's
    score: its two largest), and their weights s / Σ s · ``weight_scale``. ``experts`` < z's columns: the row's other
    columns are copied to ``extra`` (float32 [T, columns − experts])."""
    lib = load("hybrid")
    if z.dtype != torch.float32 or ids.dtype != torch.int32 or weights.dtype != torch.float32:
        raise KernelError("moe_select takes float32 logits and writes int32 ids and float32 weights")
    _need_contig(z, correction, ids, weights)
    T, ldz = z.shape
    E = int(experts or ldz)
    if (extra is None) != (E == ldz) or (extra is not None and (extra.dtype != torch.float32 or extra.numel() != T * (ldz - E))):
        raise KernelError("moe_select: the columns beyond the experts' need a float32 place to go, and only they")
    _need_contig(extra)
    _check("hybrid", lib.sp_moe_select(
        c_void_p(_ptr(z)), c_void_p(_ptr(correction)), dt_code(correction) if correction is not None else 0,
        c_void_p(_ptr(ids)), c_void_p(_ptr(weights)), T, E, ldz, int(top), int(n_groups or 1), int(keep or 1),
        int(bool(softmax)), c_float(weight_scale), c_void_p(_ptr(extra)), c_void_p(_stream())))


def moe_tile_rows() -> int:
    return int(load("hybrid").sp_moe_tile_rows())


TC_EXPERT_PAIRS = 512        # from this many (token, expert) pairs on, and 8 per expert, whole 128-row tiles pay off


def moe_experts(x, ids, weights, w_gate_up, w_down, y, top, limit, slope=1.702, glu_block=0):
    """y (float32 [T, W]) += Σ_k weights[t,k] · expert_{ids[t,k]}(x[t]) with clamped-GLU experts: ``w_gate_up``
    [E, 2F, W] (an expert's gate rows, then its up rows; with ``glu_block`` = b: blocks of b gate rows, each followed by
    the b up rows of the same outputs), ``w_down`` [E, W, F]. The (token, expert) pairs are sorted by expert on the
    device; nothing comes back to the host. Many pairs in the block layout: the products run as grouped products of the
    tcgen05 tile kernel over rows gathered into 128-row tiles of one expert each."""
    lib = load("hybrid")
    _need_contig(x, ids, weights, w_gate_up, w_down, y)
    T, W = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    n_pairs = T * top
    dev = x.device
    if ids.dtype != torch.int32 or weights.dtype != torch.float32 or y.dtype != torch.float32:
        raise KernelError("moe_experts takes int32 ids, float32 weights and adds into a float32 matrix")
    global launches
    if (glu_block and n_pairs >= max(TC_EXPERT_PAIRS, 8 * E) and W % 128 == 0 and F % 8 == 0 and W % 4 == 0
            and tc_gemm_supported(x, w_gate_up[0]) and w_down.dtype == torch.bfloat16):
        tc = load("tc_gemm")
        max_tiles = (n_pairs + 127) // 128 + E
        rows = max_tiles * 128
        book = torch.empty(E + rows + n_pairs + 5 * max_tiles, dtype=torch.int32, device=dev)
        counts, order, pos = book[:E], book[E:E + rows], book[E + rows:E + rows + n_pairs]
        rest = book[E + rows + n_pairs:]
        tiles, tab_up, tab_down = rest[:3 * max_tiles], rest[3 * max_tiles:4 * max_tiles], rest[4 * max_tiles:]
        xs = torch.empty(rows, W, dtype=torch.bfloat16, device=dev)
        act = torch.empty(rows, F, dtype=torch.bfloat16, device=dev)
        out_rows = torch.empty(rows, W, dtype=torch.float32, device=dev)
        launches += 6
        _check("hybrid", lib.sp_moe_plan_tiles(
            c_void_p(_ptr(x)), c_void_p(_ptr(ids)), T, int(top), W, E, 2 * F, W, c_void_p(_ptr(counts)), c_void_p(_ptr(order)),
            c_void_p(_ptr(pos)), c_void_p(_ptr(tiles)), c_void_p(_ptr(tab_up)), c_void_p(_ptr(tab_down)), max_tiles,
            c_void_p(_ptr(xs)), c_void_p(_stream())))
        status = c_void_p(_ptr(status_word(dev)))
        _check("tc_gemm", tc.sp_tc_gemm_grouped(
            c_void_p(_ptr(xs)), c_void_p(_ptr(w_gate_up)), c_void_p(_ptr(act)), dt_code(act), rows, 2 * F, W, W, W, E * 2 * F, F,
            TC_SILU_MUL, 2 * int(glu_block), c_void_p(_ptr(tab_up)), c_float(limit), c_float(slope), status, c_void_p(_stream())))
        _check("tc_gemm", tc.sp_tc_gemm_grouped(
            c_void_p(_ptr(act)), c_void_p(_ptr(w_down)), c_void_p(_ptr(out_rows)), dt_code(out_rows), rows, W, F, F, F, E * W, W,
            TC_STORE, 256 if W % 256 == 0 else 128, c_void_p(_ptr(tab_down)), c_float(0.0), c_float(0.0), status,
            c_void_p(_stream())))
        _check("hybrid", lib.sp_moe_combine_rows(c_void_p(_ptr(out_rows)), c_void_p(_ptr(pos)), c_void_p(_ptr(weights)),
                                                 c_void_p(_ptr(y)), T, int(top), W, c_void_p(_stream())))
        return
    tm = moe_tile_rows()
    max_tiles = (n_pairs + tm - 1) // tm + E
    book = torch.empty(E + n_pairs + 3 * max_tiles, dtype=torch.int32, device=dev)
    counts, order, tiles = book[:E], book[E:E + n_pairs], book[E + n_pairs:]
    act = torch.empty(n_pairs, F, dtype=x.dtype, device=dev)
    out_pairs = torch.empty(n_pairs, W, dtype=torch.float32, device=dev)
    launches += 4
    _check("hybrid", lib.sp_moe_experts(
        c_void_p(_ptr(x)), dt_code(x), c_void_p(_ptr(ids)), c_void_p(_ptr(w_gate_up)), c_void_p(_ptr(w_down)),
        _w_dt(w_gate_up, w_down), E, c_void_p(_ptr(counts)), c_void_p(_ptr(order)), c_void_p(_ptr(tiles)), max_tiles,
        c_void_p(_ptr(weights)), c_void_p(_ptr(act)), c_void_p(_ptr(out_pairs)), c_void_p(_ptr(y)), T, int(top), W, F,
        c_float(limit), c_float(slope), int(glu_block), c_void_p(_stream())))


# ------------------------------------------------------------------ latent: attention through a cached low-rank latent
def latent_norm_store(proj, q_rank, rank, wq, wc, eps, cq_out, pool, meta, rows_out=None):
    """``proj`` rows (float32) = [q part: ``q_rank`` | latent part: ``rank``]: each part's RMS norm with its weight; the
    q part to ``cq_out`` [T, q_rank], the latent into its page row of ``pool`` ([pages, 1, page_size, rank]; None: the
    rows carry no latent part). ``rows_out`` [T, rank] of ``cq_out``'s type also receives the latents, token by token."""
    lib = load("latent")
    if proj.dtype != torch.float32:
        raise KernelError("latent_norm_store reads 32-bit projections")
    _need_contig(proj, wq, wc, cq_out, rows_out)
    if rows_out is not None and (pool is None or rows_out.dtype != cq_out.dtype or rows_out.shape != (proj.shape[0], int(rank))):
        raise KernelError("latent_norm_store: the latents as rows are [tokens, rank] of the q part's type, beside a pool")
    pt = meta.page_table
    if pool is not None:
        _declare_bounds("latent", lib, _pool_pages(meta, pool), _table_rows(meta, pt), proj.device)
    _check("latent", lib.sp_latent_norm_store(
        c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(wq)), c_void_p(_ptr(wc)), _w_dt(*[w for w in (wq, wc) if w is not None]),
        c_void_p(_ptr(cq_out)), dt_code(cq_out), c_void_p(_ptr(pool)), dt_code(pool) if pool is not None else 0,
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)),
        pt.shape[1], meta.page_size, proj.shape[0], int(q_rank), int(rank), c_float(eps), c_void_p(_ptr(rows_out)),
        c_void_p(_stream())))


HEADWISE_SMALL_TOKENS = 16      # up to this many tokens a stack stored [H·N, K] in bfloat16 is streamed row by row, a warp per row


def headwise_product(a, w, out, H, K_, N, w_rows_are_k):
    """out[t, h, :] = a[t, h, :] · W_h with ``a`` [T, H·K], ``out`` [T, H·N] and ``w`` the heads' matrices one after
    another: [H·K, N] (``w_rows_are_k``) or [H·N, K]."""
    lib = load("latent")
    _need_contig(a, w, out)
    if a.shape[1] != H * K_ or out.shape[1] != H * N or w.numel() != H * K_ * N:
        raise KernelError("headwise_product: the operands' sizes do not fit together")
    _check("latent", lib.sp_headwise_product(c_void_p(_ptr(a)), dt_code(a), c_void_p(_ptr(w)), dt_code(w), c_void_p(_ptr(out)),
                                             dt_code(out), a.shape[0], int(H), int(K_), int(N), int(bool(w_rows_are_k)),
                                             c_void_p(_stream())))


def latent_flash_supported(rank: int, page_size: int) -> bool:
    return bool(load("latent").sp_latent_flash_supported(int(rank), int(page_size)))


def latent_flash(qc, pool, out, meta, step, H, rank, window, scale, sink=None, max_len=None):
    """Attention over cached latents on the tensor cores (bfloat16): ``qc`` [T, H·rank] are the queries in the latent's
    space, ``pool`` [pages, 1, 64, rank] the cached rows (key and value at once), ``out`` [T, H·rank] the weighted sums
    of rows. Window, sink and scale as for the other attention kernels. ``max_len``: no sequence of a decode step is
    longer (the step's longest, or its bucket when the launch is captured in a graph); with it the step's keys are
    shared out over several blocks per sequence."""
    lib = load("latent")
    _need_contig(qc, out, pool)
    if qc.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("latent_flash runs on bfloat16 queries and cached rows")
    pt = meta.page_table
    _declare_bounds("latent", lib, _pool_pages(meta, pool), _table_rows(meta, pt), qc.device)
    decode = bool(step.all_single)
    tiles = 0 if decode else query_tiles(step.host["new_counts"], int(lib.sp_latent_flash_rows()))
    scratch, need = None, 0
    if decode and max_len:
        lib.sp_latent_flash_scratch_floats.restype = c_longlong
        need = int(lib.sp_latent_flash_scratch_floats(int(step.n_seqs), int(H), int(rank), int(window or 0), int(max_len)))
        if need:
            scratch = torch.empty(need, dtype=torch.float32, device=qc.device)
    _check("latent", lib.sp_latent_flash(
        c_void_p(_ptr(qc)), c_void_p(_ptr(out)), c_void_p(_ptr(pool)), c_void_p(_ptr(step.seq_start)),
        c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        int(step.n_seqs), int(tiles), int(decode), int(H), int(rank), int(window or 0), c_float(scale), _sink_ptr(sink, H),
        int(max_len or 0), c_void_p(_ptr(scratch)), c_longlong(need), c_void_p(_stream())))
    if need:
        global launches
        launches += 1        # two kernels: the shares and their combination


# ------------------------------------------------------------------ sandwich: sublayers between two norms, gated attention rows
def pair_embed(table, pairs, step, state, out, buckets, mul_prev, mul_cur, scale, status=None):
    """out[t,:] (float32) = table[id_t,:] · scale + pairs[(id_{t−1} · mul_prev + id_t · mul_cur) mod buckets, :]; a
    sequence's first token takes row ``buckets``. ``state`` int32 [slots]: the token before a step's first one; the
    kernel leaves the step's last token there."""
    lib = load("sandwich")
    T, W = out.shape
    _need_contig(table, pairs, out, state)
    if table.dtype != pairs.dtype or pairs.shape != (int(buckets) + 1, W) or state.dtype != torch.int32:
        raise KernelError("pair_embed: the pair table is [buckets + 1, width] of the token table's type, the state int32")
    _check("sandwich", lib.sp_pair_embed(
        c_void_p(_ptr(table)), c_void_p(_ptr(pairs)), dt_code(table), c_void_p(_ptr(step.tokens)), c_void_p(_ptr(step.positions)),
        c_void_p(_ptr(step.token_seq)), c_void_p(_ptr(step.seq_start)), c_void_p(_ptr(step.seq_slot)), c_void_p(_ptr(state)),
        state.numel(), c_void_p(_ptr(out)), T, W, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), c_float(scale),
        c_void_p(_ptr(status)), c_void_p(_stream())))


def stream_norm_add(x, y, w_post, mult, eps, w_next=None, out=None, raw=False):
    """x ← x + mult · y / sqrt(mean(y²) + eps) ⊙ w_post, row by row, and y ← 0 (x, y float32 [T, W]; the weights
    float32 as they multiply). ``out`` [T, W] then receives the next reader's input: the RMS norm of the new x with
    ``w_next``, or with ``raw`` the new x itself."""
    lib = load("sandwich")
    if x.dtype != torch.float32 or y.dtype != torch.float32 or w_post.dtype != torch.float32 or x.shape != y.shape:
        raise KernelError("stream_norm_add works on two float32 buffers of one shape and float32 weights")
    _need_contig(x, y, w_post, w_next, out)
    mode = 0 if out is None else (2 if raw else 1)
    if mode == 1 and (w_next is None or w_next.dtype != torch.float32):
        raise KernelError("stream_norm_add: the next norm needs a float32 weight")
    _check("sandwich", lib.sp_stream_norm_add(
        c_void_p(_ptr(x)), c_void_p(_ptr(y)), c_void_p(_ptr(w_post)), c_void_p(_ptr(w_next)), c_void_p(_ptr(out)),
        dt_code(out) if out is not None else 0, mode, x.shape[0], x.shape[1], c_float(mult), c_float(eps), c_void_p(_stream())))


def gated_qkv_store(proj, bias, q_out, k_pool, v_pool, meta, gates, freq, nh, nkv, d, vd, rd, write_kv=True, rot_mult=1.0,
                    temp_coef=0.0, temp_every=1):
    """``proj`` rows (float32) = [q: nh·d | k: nkv·d | v: nkv·vd | gates: nh]: add ``bias`` (over q, k, v), multiply q by
    1 + temp_coef · ln(floor((position + 1) / temp_every) + 1), rotate neighbouring pairs over the first ``rd`` dims of
    every q and k head by position · freq[i] (cos and sin times ``rot_mult``), store q to ``q_out``, k and v into their
    page rows and the gates' arguments to ``gates`` (float32 [T, nh], or None)."""
    lib = load("sandwich")
    if proj.dtype != torch.float32:
        raise KernelError("gated_qkv_store reads 32-bit projections")
    _need_contig(proj, bias, q_out, gates, freq)
    pt = meta.page_table
    _declare_bounds("sandwich", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), proj.device)
    _check("sandwich", lib.sp_gated_qkv_store(
        c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(bias)), dt_code(bias) if bias is not None else 0, c_void_p(_ptr(q_out)),
        dt_code(q_out), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool), c_void_p(_ptr(gates)), c_void_p(_ptr(freq)),
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)),
        pt.shape[1], meta.page_size, proj.shape[0], int(nh), int(nkv), int(d), int(vd), int(rd), int(bool(write_kv)),
        c_float(rot_mult), c_float(temp_coef), int(temp_every), c_void_p(_stream())))


def latent_rot_store(proj, wc, q_out, pool, meta, gates, freq, H, d, rd, rank, rot_mult, eps, rows_out=None):
    """``proj`` rows (float32) = [q: H·(d + rd) | row: rank | key part: rd | gates: H] (``pool`` None: no row and no key
    part). The row's RMS norm with ``wc`` and the key part with its neighbouring pairs rotated go into ONE page row
    [rank + rd] of ``pool``; every head's last ``rd`` query dims are rotated the same way; q to ``q_out``, the gates'
    arguments to ``gates`` (float32 [T, H]). ``rows_out`` [T, rank + rd] also receives the page rows token by token."""
    lib = load("sandwich")
    if proj.dtype != torch.float32:
        raise KernelError("latent_rot_store reads 32-bit projections")
    _need_contig(proj, wc, q_out, gates, freq, rows_out)
    pt = meta.page_table
    if pool is not None:
        _declare_bounds("sandwich", lib, _pool_pages(meta, pool), _table_rows(meta, pt), proj.device)
    _check("sandwich", lib.sp_latent_rot_store(
        c_void_p(_ptr(proj)), proj.shape[1], c_void_p(_ptr(wc)), dt_code(wc) if wc is not None else 0, c_void_p(_ptr(q_out)),
        dt_code(q_out), c_void_p(_ptr(pool)), dt_code(pool) if pool is not None else 0, c_void_p(_ptr(rows_out)),
        c_void_p(_ptr(gates)), c_void_p(_ptr(freq)), c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, proj.shape[0], int(H), int(d), int(rd),
        int(rank), c_float(rot_mult), c_float(eps), c_void_p(_stream())))


def gelu_gather_mul(z, table, ids, out, offset):
    """out[t, j] = gelu_tanh(z[t, j]) · table[ids[t], offset + j] for z, out [T, C]."""
    lib = load("sandwich")
    _need_contig(z, table, ids, out)
    if z.shape != out.shape or z.dtype != out.dtype:
        raise KernelError("gelu_gather_mul: input and output are one shape and type")
    _check("sandwich", lib.sp_gelu_gather_mul(
        c_void_p(_ptr(z)), dt_code(z), c_void_p(_ptr(table)), dt_code(table), c_void_p(_ptr(ids)), c_void_p(_ptr(out)),
        z.shape[0], z.shape[1], table.shape[1], int(offset), table.shape[0], c_void_p(_stream())))
