"""Python face of the kernel library: torch tensors in, kernel launches on the current stream.

Each function checks dtypes, shapes and contiguity, passes raw device pointers through
ctypes, and raises `KernelError` with the library's message when a size is refused or a
launch fails.  Nothing here computes on the host or falls back to another implementation:
without the library, or without a device of compute capability 10.x, importing the ops
raises.
"""
import ctypes
import os
import threading

import torch

from . import build as _build

F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
PAGE = 64  # tokens per cache page, as in common.cuh

ERR_BITS = {1: "a token id outside the vocabulary", 2: "a position beyond the position table",
            4: "a page id outside the cache", 8: "a device-side wait ran out"}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()


def lib():
    """The loaded kernel library (built at the first call if needed)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.library_path()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as e:  # pragma: no cover
                    raise KernelError(f"edgelm_b200: cannot load the kernel library {path}: {e}") from e
                loaded.edgelm_last_error.restype = ctypes.c_char_p
                if os.environ.get("EDGELM_PDL") is not None:
                    loaded.edgelm_set_pdl(int(os.environ["EDGELM_PDL"]))
                _lib = loaded
    return _lib


def require_device():
    """Fail loudly unless a Blackwell-class CUDA device is current; there is no other path."""
    if not torch.cuda.is_available():
        raise KernelError("edgelm_b200 runs on a CUDA device (sm_100a) only; torch sees none")
    arch = lib().edgelm_device_arch()
    if arch // 10 != 10:
        raise KernelError(f"edgelm_b200's kernels are built for sm_100a; the current device reports sm_{arch}")


LAUNCHES = 0  # kernels launched through this module since import (a graph replay counts what it captured)


def count_launches(n):
    global LAUNCHES
    LAUNCHES += n


def _check(rc, launches=1):
    if rc != 0:
        raise KernelError(lib().edgelm_last_error().decode())
    count_launches(launches)


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}")


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _i32(t, name):
    _need(t.dtype == torch.int32 and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous int32 CUDA tensor")


def embed_gather(ids, table, x, err, scale=1.0):
    """x[t, :] = table[ids[t], :] * scale as float32; ids outside the table set bit 1 of `err`."""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous() and x.dtype == torch.float32 and x.is_contiguous(), "embed_gather: layout")
    _need(x.shape == (ids.numel(), table.shape[1]), "embed_gather: x has the wrong shape")
    _check(lib().edgelm_embed_gather(_p(ids), _p(table), _dt(table), _p(x), ids.numel(), table.shape[1], table.shape[0],
                                     ctypes.c_float(scale), _p(err), _stream()))


def rmsnorm(x, w, eps, out, rows_idx=None):
    """out[r] = x[rows_idx[r] or r] * rsqrt(mean(x^2) + eps) * w; x and w float32, out float32 or bfloat16."""
    _need(x.dtype == torch.float32 and w.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous(), "rmsnorm: layout")
    rows = out.shape[0]
    dim = x.shape[1]
    _need(out.shape[1] == dim and w.numel() == dim, "rmsnorm: widths differ")
    if rows_idx is not None:
        _i32(rows_idx, "rows_idx")
        _need(rows_idx.numel() == rows, "rmsnorm: one source row per output row")
    else:
        _need(x.shape[0] == rows, "rmsnorm: row counts differ")
    _check(lib().edgelm_rmsnorm(_p(x), _p(w), _p(out), _dt(out), _p(rows_idx), rows, dim, ctypes.c_float(eps), _stream()))


def gemm_simt(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, force_kernel=0):
    """out = a @ w.T (+ epilogue) with float32 accumulation on the CUDA cores."""
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm: 2-D operands")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous(), "gemm: rows must be contiguous")
    _need(a.dtype == w.dtype and (w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous())), "gemm: weight dtypes")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemm: residual layout")
    _check(lib().edgelm_gemm_simt(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), _p(residual), M, N, K,
                                  _dt(a), _dt(out), epilogue, force_kernel, _stream()))


def gemv_takes(a, w, w2=None, normed=False):
    """Whether the vector few-rows kernel takes these operands (K a multiple of a 16-byte vector, aligned rows).
    With `normed`, `a` is the float32 residual stream and the weights give the compute dtype."""
    if not w.is_contiguous() or a.stride(1) != 1:
        return False
    if normed and (a.dtype != torch.float32 or not a.is_contiguous()):
        return False
    if not normed and a.dtype != w.dtype:
        return False
    return bool(lib().edgelm_gemv_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[1], _dt(w), 1 if normed else 0))


def gemv(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, norm_weight=None, eps=0.0, n_sms=0):
    """out = act @ w.T (+ epilogue) for a few rows.  act = a, or RMSNorm(a) * norm_weight rounded to
    w's dtype when norm_weight is given (a is then the float32 residual stream)."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemv: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(out.stride(1) == 1 and w.is_contiguous(), "gemv: rows must be contiguous")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemv: second weight")
    if norm_weight is not None:
        _need(a.dtype == torch.float32 and a.is_contiguous() and norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "gemv: norm operands")
    else:
        _need(a.dtype == w.dtype and a.stride(1) == 1, "gemv: activation dtype")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemv: residual layout")
    _check(lib().edgelm_gemv(_p(a), a.stride(0), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(w2), _p(out), out.stride(0),
                             _p(residual), M, N, K, _dt(w), _dt(out), epilogue, int(n_sms), _stream()))


def gemv_mma_takes(a, w, w2=None, normed=False):
    """Whether the tensor-core few-rows kernel takes these operands: bfloat16 weights, at most 16 rows,
    K a multiple of 8, aligned rows.  With `normed`, `a` is the float32 residual stream."""
    if w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    if normed and (a.dtype != torch.float32 or not a.is_contiguous()):
        return False
    if not normed and a.dtype != torch.bfloat16:
        return False
    return bool(lib().edgelm_gemv_mma_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[0], a.shape[1], 1 if normed else 0))


def gemv_mma(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, norm_weight=None, eps=0.0, prefetch=()):
    """out = act @ w.T (+ epilogue) for at most 16 rows on mma.sync tensor cores; act = a, or
    RMSNorm(a) * norm_weight rounded to bfloat16 when norm_weight is given.  `prefetch`: up to two
    contiguous tensors (the weights the step reads next) that the kernel's blocks ask the L2 cache for."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemv_mma: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(out.stride(1) == 1 and w.is_contiguous() and w.dtype == torch.bfloat16, "gemv_mma: weight layout")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemv_mma: second weight")
    if norm_weight is not None:
        _need(a.dtype == torch.float32 and a.is_contiguous() and norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "gemv_mma: norm operands")
    else:
        _need(a.dtype == torch.bfloat16 and a.stride(1) == 1, "gemv_mma: activation dtype")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemv_mma: residual layout")
    if prefetch:
        _need(len(prefetch) <= 2 and all(t.is_contiguous() for t in prefetch), "gemv_mma: prefetch takes up to two contiguous tensors")
        regions = [(_p(t), ctypes.c_ulonglong(t.numel() * t.element_size())) for t in prefetch] + [(ctypes.c_void_p(0), ctypes.c_ulonglong(0))]
        _check(lib().edgelm_gemv_mma_prefetch_next(regions[0][0], regions[0][1], regions[1][0], regions[1][1]), launches=0)
    _check(lib().edgelm_gemv_mma(_p(a), a.stride(0), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(w2), _p(out), out.stride(0),
                                 _p(residual), M, N, K, _dt(out), epilogue, _stream()))


def gemv_mma_walk(on):
    """Whether few-rows products with wide outputs (at least 296 groups of 16 columns, K up to 4,096) run on the
    kernel whose blocks walk several column groups (default) or on the one of a block per group."""
    lib().edgelm_gemv_mma_walk(int(bool(on)))


def gemm_tc_takes(a, w, out, w2=None):
    """Whether the tensor-core kernel takes these operands: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or not w.is_contiguous():
        return False
    return bool(lib().edgelm_gemm_tc_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[1]))


SPLITK_SCRATCH_BYTES = 32 << 20
_splitk_scratch = None


def _splitk_ready():
    """The scratch that lets products of few tiles and long K spread over the device (split-K): allocated once, at
    the first product outside of a graph capture, and handed to the library."""
    global _splitk_scratch
    if _splitk_scratch is None and not torch.cuda.is_current_stream_capturing():
        _splitk_scratch = torch.empty(SPLITK_SCRATCH_BYTES // 4, dtype=torch.float32, device="cuda")
        lib().edgelm_gemm_tc_splitk.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        lib().edgelm_gemm_tc_splitk(_p(_splitk_scratch), SPLITK_SCRATCH_BYTES, 1)


def gemm_tc(a, w, out, err, epilogue=EPI_STORE, w2=None, residual=None, glu=None, glu_bias=None):
    """out = a @ w.T (+ epilogue) on the tcgen05 tensor cores: bfloat16 operands, float32 accumulation.  `glu` (limit, alpha,
    shift) with the gated epilogue: out = g sigmoid(alpha g) (v + shift), g = min(a @ w.T, limit), v = clamp(a @ w2.T, -limit, limit)
    (limit 0: no clamps); `glu_bias` [2 N] float32: the two branches' biases, added before the unit."""
    _splitk_ready()
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm_tc: 2-D operands")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm_tc: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc: bfloat16 operands")
    _need(a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous(), "gemm_tc: rows must be contiguous")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemm_tc: second weight")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemm_tc: residual layout")
    if glu is not None or glu_bias is not None:
        glu = glu if glu is not None else GLU_SWIGLU
        _need(epilogue == EPI_SWIGLU and w2 is not None and residual is None and glu[0] >= 0, "gemm_tc: the general gated epilogue needs both weights")
        _need(glu_bias is None or (glu_bias.dtype == torch.float32 and glu_bias.is_cuda and glu_bias.is_contiguous() and glu_bias.numel() == 2 * N), "gemm_tc: the gated unit's biases")
        _check(lib().edgelm_gemm_tc_glu(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), M, N, K, _dt(out), ctypes.c_float(glu[0]),
                                        ctypes.c_float(glu[1]), ctypes.c_float(glu[2]), _p(glu_bias), _p(err), _stream()), launches=0)
    else:
        _check(lib().edgelm_gemm_tc(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), _p(residual), M, N, K, _dt(out),
                                    epilogue, _p(err), _stream()), launches=0)
    count_launches(lib().edgelm_gemm_tc_last_launches())


def gemm_tc_rope_takes(a, w, qkv, kcache, vcache, cos, sin, hd):
    """Whether the stacked q, k, v projection can rotate and append in its epilogue (`gemm_tc_rope`)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        return False
    if a.stride(1) != 1 or qkv.stride(1) != 1 or not w.is_contiguous() or not (kcache.is_contiguous() and vcache.is_contiguous()):
        return False
    return bool(lib().edgelm_gemm_tc_rope_takes(_p(a), a.stride(0), _p(w), _p(qkv), qkv.stride(0), a.shape[1], int(hd),
                                                _p(kcache), _p(vcache), _p(cos), _p(sin)))


def gemm_tc_rope(a, w, qkv, tok_pos, tok_seq, seq_slot, page_table, cos, sin, kcache, vcache, nh, nkv, hd, err):
    """The stacked q, k, v projection of a prompt step with rotation and cache append in its epilogue:
    qkv[:, :nh hd] = rotated query heads of a @ w.T; the rotated keys and the values go to each token's place in the
    cache pages.  The k and v columns of `qkv` are left as they were."""
    _splitk_ready()
    M, K = a.shape
    _need(w.shape == ((nh + 2 * nkv) * hd, K) and qkv.shape == (M, (nh + 2 * nkv) * hd), "gemm_tc_rope: shapes")
    _need(gemm_tc_rope_takes(a, w, qkv, kcache, vcache, cos, sin, hd), "gemm_tc_rope: these operands are not taken (bfloat16, head size 64 or 128, aligned)")
    _need(kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "gemm_tc_rope: cache layout")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "gemm_tc_rope: table layout")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (seq_slot, "seq_slot"), (page_table, "page_table")):
        _i32(t, n)
    _need(tok_pos.numel() == M and tok_seq.numel() == M, "gemm_tc_rope: one position and one sequence index per token")
    _check(lib().edgelm_gemm_tc_rope(_p(a), a.stride(0), _p(w), _p(qkv), qkv.stride(0), M, K, _p(tok_pos), _p(tok_seq), _p(seq_slot),
                                     _p(page_table), page_table.stride(0), kcache.shape[0], _p(cos), _p(sin), cos.shape[0],
                                     _p(kcache), _p(vcache), nh, nkv, hd, _p(err), _stream()), launches=0)
    count_launches(lib().edgelm_gemm_tc_last_launches())


def gemm_tc_last_kernel():
    """Which kernel the last `gemm_tc` call took: {"tile_columns", "persistent", "deep_ring", "k_splits"}."""
    v = int(lib().edgelm_gemm_tc_last_kernel())
    return {"tile_columns": v & 0xFFF, "persistent": bool(v >> 12 & 1), "deep_ring": bool(v >> 13 & 1), "k_splits": v >> 16}


def rope_kv_append(qkv, tok_pos, tok_seq, seq_slot, page_table, cos, sin, kcache, vcache, nh, nkv, hd, err):
    """Rotate q and k of the fused projection output in float32; write k and v into their pages."""
    T = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd, "rope_kv_append: qkv layout")
    _need(kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous() and vcache.is_contiguous(), "rope_kv_append: cache dtype")
    _need(kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "rope_kv_append: cache shape")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "rope_kv_append: table layout")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (seq_slot, "seq_slot"), (page_table, "page_table")):
        _i32(t, n)
    _need(tok_pos.numel() >= T and tok_seq.numel() >= T, "rope_kv_append: one position per token")
    _check(lib().edgelm_rope_kv_append(_p(qkv), _dt(qkv), _p(tok_pos), _p(tok_seq), _p(seq_slot), _p(page_table),
                                       page_table.stride(0), kcache.shape[0], _p(cos), _p(sin), cos.shape[0], _p(kcache),
                                       _p(vcache), T, nh, nkv, hd, _p(err), _stream()))


def attn_prefill(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                 max_tile_tokens, nh, nkv, hd, scale, window=0):
    """Causal attention of new tokens (any number per sequence) over the paged cache.  `window` > 0: a token sees
    the last `window` keys only, its own included."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                     _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq), _p(tile_tok0),
                                     _p(tile_ntok), _p(tile_pos0), n_tiles, max_tile_tokens, nh, nkv, hd,
                                     ctypes.c_float(scale), int(window or 0), _stream()))


MMA_PREFILL_TILE = 64  # new tokens per tile of the tensor-core prefill kernel (PM_ROWS in attention_mma.cu)


def attn_prefill_mma_takes(dtype, hd):
    """Whether the tensor-core prefill attention takes this dtype and head size (bfloat16; 32, 64, 96, 128)."""
    return dtype == torch.bfloat16 and bool(lib().edgelm_attn_prefill_mma_takes(int(hd)))


def attn_prefill_mma(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                     nh, nkv, hd, scale, max_keys=0, force_groups=0):
    """Causal attention of new tokens over the paged cache on mma.sync tensor cores; tiles of at most 64 tokens."""
    _need(qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16 and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill_mma: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill_mma(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache),
                                         _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq), _p(tile_tok0),
                                         _p(tile_ntok), _p(tile_pos0), n_tiles, nh, nkv, hd, ctypes.c_float(scale), int(max_keys),
                                         int(force_groups), _stream()))


TC_PREFILL_TILE = 128  # new tokens per tile of the tcgen05 prefill kernel (AT_ROWS in attention_tc.cu)


def attn_prefill_tc_takes(dtype, hd):
    """Whether the tcgen05 prefill attention takes this dtype and head size (bfloat16, 64)."""
    return dtype == torch.bfloat16 and bool(lib().edgelm_attn_prefill_tc_takes(int(hd)))


def attn_prefill_tc(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                    nh, nkv, hd, scale, err):
    """Causal attention of new tokens over the paged cache on tcgen05 tensor cores; tiles of at most 128 tokens."""
    _need(qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16 and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill_tc: layout")
    _need(kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "attn_prefill_tc: cache layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill_tc(_p(qkv), qkv.stride(0), qkv.shape[0], _p(out), out.stride(0), _p(kcache), _p(vcache),
                                        kcache.shape[0], _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq),
                                        _p(tile_tok0), _p(tile_ntok), _p(tile_pos0), n_tiles, nh, nkv, hd, ctypes.c_float(scale),
                                        _p(err), _stream()))


ATTN_PREFILL_TC_TRACE_SHAPE = (2 * 64 + 1, 8)


def attn_prefill_tc_trace(buffer):
    """The next launches of the tcgen05 prefill attention stamp the clock of one softmax warp per group of the
    grid's first block into `buffer` (int64, ATTN_PREFILL_TC_TRACE_SHAPE: [group * 64 + block][before / after the
    wait for the scores, after the exponentials, after the wait for the last P V, after a rescaling, after the
    arrival], and a last row for the block as a whole: entry, tensor memory there, the kernel before done, key
    blocks done, accumulator read, row stored, block done); None stops it."""
    if buffer is not None:
        _need(buffer.dtype == torch.int64 and buffer.is_contiguous() and tuple(buffer.shape) == ATTN_PREFILL_TC_TRACE_SHAPE, "attn_prefill_tc_trace: buffer")
    lib().edgelm_attn_prefill_tc_trace(_p(buffer))


def attn_decode(qkv, out, kcache, vcache, page_table, seq_slot, seq_pos, n_seqs, nh, nkv, hd, scale, n_splits=1,
                part_o=None, part_ml=None, err=None, window=0, meta_ready=False):
    """Attention of one new token per sequence over the paged cache, pages dealt to `n_splits` blocks.
    `err`: the device error word that a copy which never arrives is reported to.  `window` > 0: the token sees the
    last `window` keys only (the CUDA-core kernel then, whatever the dtype).  `meta_ready`: the caller vouches that
    positions, slots and page table were complete before the kernel that precedes this call on the stream started."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_decode: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_pos, "seq_pos")):
        _i32(t, n)
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32 and part_o.numel() >= n_seqs * nh * n_splits * hd, "attn_decode: part_o too small")
        _need(part_ml is not None and part_ml.dtype == torch.float32 and part_ml.numel() >= n_seqs * nh * n_splits * 2, "attn_decode: part_ml too small")
    _check(lib().edgelm_attn_decode(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                    _p(page_table), page_table.stride(0), _p(seq_slot), _p(seq_pos), n_seqs, nh, nkv, hd,
                                    ctypes.c_float(scale), n_splits, _p(part_o), _p(part_ml), int(window or 0), 1 if meta_ready else 0,
                                    _p(err), _stream()),
           launches=0)
    count_launches(lib().edgelm_attn_decode_last_launches())


def attn_decode_rope(qkv, out, kcache, vcache, page_table, seq_slot, seq_pos, cos, sin, n_seqs, nh, nkv, hd, scale,
                     n_splits=1, part_o=None, part_ml=None, err=None, window=0, meta_ready=False):
    """Decode attention with RoPE and the cache append fused in: `qkv` holds the raw projections of one
    new token per sequence; the rotated keys and the values are written into the cache pages."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_decode_rope: layout")
    _need(qkv.shape[1] == (nh + 2 * nkv) * hd and kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "attn_decode_rope: shapes")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "attn_decode_rope: table layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_pos, "seq_pos")):
        _i32(t, n)
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32 and part_o.numel() >= n_seqs * nh * n_splits * hd, "attn_decode_rope: part_o too small")
        _need(part_ml is not None and part_ml.dtype == torch.float32 and part_ml.numel() >= n_seqs * nh * n_splits * 2, "attn_decode_rope: part_ml too small")
    _check(lib().edgelm_attn_decode_rope(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                         _p(page_table), page_table.stride(0), _p(seq_slot), _p(seq_pos), _p(cos), _p(sin),
                                         cos.shape[0], n_seqs, nh, nkv, hd, ctypes.c_float(scale), n_splits, _p(part_o),
                                         _p(part_ml), int(window or 0), 1 if meta_ready else 0, _p(err), _stream()),
           launches=0)
    count_launches(lib().edgelm_attn_decode_last_launches())


def attn_set_error_word(err):
    """The device int32 that decode attention calls which name no error word of their own (the entry point that
    allocates nothing) report a copy that never arrived to (bit 8)."""
    _check(lib().edgelm_attn_set_error_word(_p(err)), launches=0)


def argmax_rows(logits, out):
    """out[r] = index of the first maximum of logits[r]."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "argmax_rows: float32 rows")
    _i32(out, "out")
    _check(lib().edgelm_argmax_rows(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(out), _stream()))


def sample_topk(logits, temperature, top_k, rng_state, out, state_index=None, scratch=None):
    """Temperature + top-k draw per row; rng_state (int64 xorshift64 states) advances by one draw.
    Row r uses state state_index[r] when given (a sequence's slot), else state r.  `scratch` (int32, a word per
    row) lets rows with at most 1,024 kept tokens and a vocabulary of at most 49,152 take the fast kernel (the row
    in registers, no histograms); without it every row takes the general one.  Same choices either way."""
    if scratch is not None:
        _i32(scratch, "scratch")
        _need(scratch.numel() >= logits.shape[0], "sample_topk: a scratch word per row")
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "sample_topk: float32 rows")
    _need(rng_state.dtype == torch.int64 and rng_state.is_contiguous(), "sample_topk: rng_state")
    if state_index is None:
        _need(rng_state.numel() >= logits.shape[0], "sample_topk: one state per row")
    else:
        _i32(state_index, "state_index")
    _i32(out, "out")
    _check(lib().edgelm_sample_topk(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1],
                                    ctypes.c_float(temperature), int(top_k), _p(rng_state), _p(state_index), _p(out),
                                    _p(scratch), _stream()), launches=1 if scratch is None else 2)


def read_error_word(err):
    """Host-side reading of the device error word; raises when a kernel reported bad input."""
    v = int(err.item())
    if v:
        what = [m for b, m in ERR_BITS.items() if v & b]
        err.zero_()
        raise KernelError("a kernel reported: " + "; ".join(what))



# ---------------------------------------------------------------------------------------------------------------------
# Mixers with a fixed-size state (recurrent.cu) and the sliding-window attention with pooled blocks (attention_pooled.cu).
# `seq_tok0`: int32 [n_seqs + 1], the packed row of each sequence's first token, closed by the step's token count;
# `seq_slot`: the row of each sequence's state.  States are float32 tensors [slots, ...].

def _f32(t, name):
    _need(t.dtype == torch.float32 and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous float32 CUDA tensor")


def shift_mix(inp, state, mu, out, tok_seq, seq_tok0, seq_slot, move_state=False):
    """out[m, t] = a + (prev - a) * mu[m] with a = inp[t] and prev the row before it, or the sequence's state row for
    the first token that the sequence brings to this step.  inp [T, D] float32 or bfloat16; mu [M, D]; out [M, T, D].
    With `move_state` the state rows then receive each sequence's last row of this step (what `save_last_rows` does)."""
    T, D = inp.shape
    M = mu.shape[0]
    _f32(state, "state"); _f32(mu, "mu")
    _need(inp.is_contiguous() and out.is_contiguous() and out.shape == (M, T, D) and mu.shape == (M, D) and state.shape[1] == D, "shift_mix: shapes")
    for t, n in ((tok_seq, "tok_seq"), (seq_tok0, "seq_tok0"), (seq_slot, "seq_slot")):
        _i32(t, n)
    _check(lib().edgelm_shift_mix(_p(inp), _dt(inp), _p(state), _p(mu), _p(out), _dt(out), _p(tok_seq), _p(seq_tok0), _p(seq_slot),
                                  T, D, M, 1 if move_state else 0, _stream()))


def save_last_rows(inp, state, seq_tok0, seq_slot, n_seqs):
    """state[slot of s] = inp[last row of sequence s], as float32."""
    _f32(state, "state")
    _need(inp.is_contiguous() and inp.dim() == 2 and state.shape[1] == inp.shape[1], "save_last_rows: shapes")
    _check(lib().edgelm_save_last_rows(_p(inp), _dt(inp), _p(state), _p(seq_tok0), _p(seq_slot), int(n_seqs), inp.shape[1], _stream()))


def conv_silu(u, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, n_seqs, update_state=True):
    """Causal convolution over the channels u[:, off : off + C] with taps w [C, taps] and bias b, then silu; the inputs
    before the step come from state [slots, taps - 1, C], which is then moved on to the step's last inputs (with
    `update_state` False that is left to the caller: `ssm_scan` does it when it is handed the state)."""
    conv_act(u, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, n_seqs, update_state=update_state, act="silu")


def conv_act(u, off, w, b, state, out, tok_seq, seq_tok0, seq_slot, n_seqs, update_state=True, in_bias=None, act=None):
    """`conv_silu` with its options: `b` may be None (no bias on the result); `in_bias` [C] is added to every input that `u`
    brings before the convolution (a projection's bias: the state then keeps inputs with it, and what lies before a
    sequence's start stays zero); `act` None (the sum itself) or "silu"."""
    for t, n in ((u, "u"), (w, "w"), (state, "state"), (out, "out")):
        _f32(t, n)
    T, C = out.shape
    taps = w.shape[1]
    _need(act in (None, "silu"), "conv_act: activation")
    _need(u.shape[0] == T and w.shape[0] == C and tuple(state.shape[1:]) == (taps - 1, C), "conv_act: shapes")
    for t, n in ((b, "b"), (in_bias, "in_bias")):
        _need(t is None or (t.dtype == torch.float32 and t.is_cuda and t.is_contiguous() and t.numel() == C), f"conv_act: {n}")
    _check(lib().edgelm_conv_act(_p(u), u.stride(0), int(off), _p(w), _p(b), _p(state), _p(out), _p(tok_seq), _p(seq_tok0), _p(seq_slot),
                                 T, int(n_seqs), C, taps, 1 if update_state else 0, _p(in_bias), 1 if act == "silu" else 0, _stream()),
           launches=2 if taps > 1 and update_state and T != int(n_seqs) else 1)      # (one token a sequence: the tail moves on in the same launch)


def ssm_scan(xbc, u, dt_off, dt_bias, a_log, d, state, y, seq_tok0, seq_slot, n_seqs, heads, groups, n_state, head_dim,
             conv_state=None, conv_off=0, scratch=None):
    """The selective state-space recurrence over the step's tokens.  xbc [T, H P + 2 G N] (x | B | C after the
    convolution), the raw step sizes at u[:, dt_off + h]; state [slots, H, P, N]; y [T, H P].  `conv_state`: the tail
    [slots, taps - 1, channels] of the convolution that made xbc from u[:, conv_off:]; the kernel moves it on.
    `scratch`: float32 room for 2 T H values (the step sizes and decays, computed once per token and head by a launch
    of its own); taken from torch when not given."""
    for t, n in ((xbc, "xbc"), (u, "u"), (dt_bias, "dt_bias"), (a_log, "A_log"), (d, "D"), (state, "state"), (y, "y")):
        _f32(t, n)
    inner = heads * head_dim
    _need(xbc.shape[1] == inner + 2 * groups * n_state and y.shape == (xbc.shape[0], inner) and u.shape[0] == xbc.shape[0], "ssm_scan: shapes")
    _need(tuple(state.shape[1:]) == (heads, head_dim, n_state) and dt_bias.numel() == heads and a_log.numel() == heads and d.numel() == heads, "ssm_scan: state or per-head vectors")
    if conv_state is not None:
        _f32(conv_state, "conv_state")
        _need(conv_state.dim() == 3 and conv_state.shape[2] == xbc.shape[1] and conv_off + xbc.shape[1] <= u.shape[1], "ssm_scan: the convolution's tail")
    T = xbc.shape[0]
    if scratch is None:
        scratch = torch.empty(2 * T * heads, dtype=torch.float32, device=xbc.device)
    _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= 2 * T * heads, "ssm_scan: scratch too small")
    _check(lib().edgelm_ssm_scan(_p(xbc), xbc.shape[1], inner, groups, n_state, _p(u), u.stride(0), int(dt_off), _p(dt_bias), _p(a_log),
                                 _p(d), _p(state), _p(y), _p(seq_tok0), _p(seq_slot), int(n_seqs), heads, head_dim, _p(conv_state), int(conv_off),
                                 (conv_state.shape[1] + 1) if conv_state is not None else 1, _p(scratch), T, _stream()), launches=2)


def wkv_scan(r, k, v, w, bonus, state, o, seq_tok0, seq_slot, n_seqs, heads, head_dim):
    """o_t = (S + diag(bonus) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T, per head.  r, k, v, w, o: [T, H K]
    float32; state [slots, H, K (value), K (key)]."""
    for t, n in ((r, "r"), (k, "k"), (v, "v"), (w, "w"), (bonus, "bonus"), (state, "state"), (o, "o")):
        _f32(t, n)
    _need(r.shape == k.shape == v.shape == w.shape == o.shape and r.shape[1] == heads * head_dim, "wkv_scan: shapes")
    _need(tuple(state.shape[1:]) == (heads, head_dim, head_dim) and bonus.numel() == heads * head_dim, "wkv_scan: state or bonus")
    _check(lib().edgelm_wkv_scan(_p(r), _p(k), _p(v), _p(w), _p(bonus), _p(state), _p(o), _p(seq_tok0), _p(seq_slot), int(n_seqs),
                                 heads, head_dim, r.shape[0], _stream()))


def lowrank_decay(a, w2, w0, out):
    """out = exp(-exp(w0 + tanh(a) @ w2.T)) in float32; a [T, L] float32, w2 [C, L] float32 or bfloat16."""
    _f32(a, "a"); _f32(w0, "w0"); _f32(out, "out")
    T, L = a.shape
    C = w2.shape[0]
    _need(w2.is_contiguous() and w2.shape == (C, L) and w0.numel() == C and out.shape == (T, C), "lowrank_decay: shapes")
    _check(lib().edgelm_lowrank_decay(_p(a), _p(w2), _dt(w2), _p(w0), _p(out), T, C, L, _stream()))


def gated_group_norm(y, gate, w, out, groups, eps, gate_first, gate_act="silu"):
    """RMS norm of y [T, inner] in `groups` equal parts with weight w, gated by act(gate) before the norm
    (`gate_first`) or after it; `gate_act` "silu" or "sigmoid".  gate: float32 rows of any stride."""
    _need(gate_act in ("silu", "sigmoid"), "gated_group_norm: the gate's activation")
    _f32(y, "y"); _f32(w, "w")
    T, inner = y.shape
    _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (T, inner) and out.is_contiguous() and out.shape == (T, inner), "gated_group_norm: shapes")
    _check(lib().edgelm_gated_group_norm(_p(y), _p(gate), gate.stride(0), _p(w), _p(out), _dt(out), T, inner, int(groups),
                                         ctypes.c_float(eps), 1 if gate_first else 0, 1 if gate_act == "sigmoid" else 0, _stream()))


def rmsnorm_add(x, y1, w, eps, a=1.0, y2=None, b=0.0, cast=None):
    """x += rmsnorm(a y1 + b y2) * w, all float32; `cast` (optional, [T, D] in the compute dtype) receives the new x too."""
    _f32(x, "x"); _f32(y1, "y1"); _f32(w, "w")
    _need(y1.shape == x.shape and (y2 is None or (y2.shape == x.shape and y2.dtype == torch.float32 and y2.is_contiguous())), "rmsnorm_add: shapes")
    _need(cast is None or (cast.shape == x.shape and cast.is_contiguous()), "rmsnorm_add: the copy's layout")
    _check(lib().edgelm_rmsnorm_add(_p(x), _p(y1), ctypes.c_float(a), _p(y2), ctypes.c_float(b), _p(w), _p(cast),
                                    _dt(cast) if cast is not None else F32, x.shape[0], x.shape[1], ctypes.c_float(eps), _stream()))


def scaled_sum(y1, a, y2, b, out, add=False):
    """out = a y1 + b y2 (float32, equal shapes); with `add`, out += a y1 + b y2."""
    _f32(y1, "y1"); _f32(y2, "y2"); _f32(out, "out")
    _need(y1.shape == y2.shape == out.shape, "scaled_sum: shapes")
    _check(lib().edgelm_scaled_sum(_p(y1), ctypes.c_float(a), _p(y2), ctypes.c_float(b), _p(out), ctypes.c_longlong(out.numel()), 1 if add else 0, _stream()))


def _pooled_cache_check(kcache, vcache, nkv, dk, dv, what):
    _need(kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == vcache.dtype, f"{what}: cache layout")
    _need(tuple(kcache.shape[1:]) == (nkv, PAGE, dk) and tuple(vcache.shape[1:]) == (nkv, PAGE, dv) and vcache.shape[0] == kcache.shape[0], f"{what}: cache shape")


def qk_rope_norm_append(qkv, bias, q_out, tok_pos, tok_seq, page_table, kcache, vcache, nh, nkv, dk, dv, rot, freq, eps, unit_norm, err):
    """qkv [T, nh dk + nkv dk + nkv dv] float32 (+ bias): rotate the first `rot` dimensions of every query and key
    head by position * freq (float64 frequencies; pairs i, i + rot/2), divide each head by its root mean square (`unit_norm`), write the
    queries to q_out [T, nh dk] and the keys and values to their places in the cache pages."""
    _f32(qkv, "qkv")
    T = qkv.shape[0]
    _need(qkv.shape[1] == (nh + nkv) * dk + nkv * dv and q_out.shape == (T, nh * dk) and q_out.is_contiguous() and q_out.dtype == kcache.dtype, "qk_rope_norm_append: shapes")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == qkv.shape[1]), "qk_rope_norm_append: bias")
    _need(rot == 0 or (freq is not None and freq.dtype == torch.float64 and freq.numel() == rot // 2 and freq.is_contiguous()), "qk_rope_norm_append: frequencies")
    _pooled_cache_check(kcache, vcache, nkv, dk, dv, "qk_rope_norm_append")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (page_table, "page_table")):
        _i32(t, n)
    _check(lib().edgelm_qk_rope_norm_append(_p(qkv), _p(bias), _p(q_out), _dt(q_out), _p(tok_pos), _p(tok_seq), _p(page_table),
                                            page_table.stride(0), kcache.shape[0], _p(kcache), _p(vcache), T, nh, nkv, dk, dv, int(rot),
                                            _p(freq), ctypes.c_float(eps), 1 if unit_norm else 0, _p(err), _stream()))


def pool_blocks(tok_pos, tok_seq, page_table, kcache, vcache, pooled_k, pooled_v, n_tokens, nkv, dk, dv, pool, err):
    """For every token of the step that ends a block of `pool` positions: the block's mean key and value, from the
    cache pages into the pooled rows."""
    _pooled_cache_check(kcache, vcache, nkv, dk, dv, "pool_blocks")
    _f32(pooled_k, "pooled_k"); _f32(pooled_v, "pooled_v")
    rows = pooled_k.shape[2]
    _need(tuple(pooled_k.shape) == (kcache.shape[0], nkv, rows, dk) and tuple(pooled_v.shape) == (kcache.shape[0], nkv, rows, dv), "pool_blocks: pooled layout")
    _check(lib().edgelm_pool_blocks(_p(tok_pos), _p(tok_seq), _p(page_table), page_table.stride(0), kcache.shape[0], _p(kcache), _p(vcache),
                                    _dt(kcache), _p(pooled_k), _p(pooled_v), int(n_tokens), nkv, dk, dv, int(pool), rows, _p(err), _stream()))


def pooled_window_attn(q, out, kcache, vcache, pooled_k, pooled_v, tok_pos, tok_seq, page_table, nh, nkv, dk, dv, scale, window, pool):
    """Attention of every token of the step over the last `window` keys and one pooled key per block of `pool`
    positions wholly before the window (`pool` 0 or None: the window alone), one softmax over both."""
    T = q.shape[0]
    _need(q.is_contiguous() and out.is_contiguous() and q.shape == (T, nh * dk) and out.shape == (T, nh * dv) and q.dtype == out.dtype == kcache.dtype, "pooled_window_attn: shapes")
    _pooled_cache_check(kcache, vcache, nkv, dk, dv, "pooled_window_attn")
    rows = 0
    if pool:
        _f32(pooled_k, "pooled_k"); _f32(pooled_v, "pooled_v")
        rows = pooled_k.shape[2]
        _need(tuple(pooled_k.shape) == (kcache.shape[0], nkv, rows, dk) and tuple(pooled_v.shape) == (kcache.shape[0], nkv, rows, dv), "pooled_window_attn: pooled layout")
    _check(lib().edgelm_pooled_window_attn(_p(q), _p(out), _p(kcache), _p(vcache), _dt(q), _p(pooled_k) if pool else _p(None),
                                           _p(pooled_v) if pool else _p(None), _p(tok_pos), _p(tok_seq), _p(page_table), page_table.stride(0),
                                           kcache.shape[0], T, nh, nkv, dk, dv, ctypes.c_float(scale), int(window), int(pool or 0), rows, _stream()))


def pooled_window_attn_tiled(q, out, kcache, vcache, pooled_k, pooled_v, page_table, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                             max_tile_tokens, nh, nkv, dk, dv, scale, window, pool):
    """`pooled_window_attn` for prompt steps: the step's tokens come as tiles (runs of at most `max_tile_tokens` consecutive
    tokens of one sequence: `tile_seq` the row of the page table, `tile_tok0` the first packed row, `tile_ntok`, `tile_pos0`
    the first position); a page of keys and values is staged once for all the rows of a tile."""
    T = q.shape[0]
    _need(q.is_contiguous() and out.is_contiguous() and q.shape == (T, nh * dk) and out.shape == (T, nh * dv) and q.dtype == out.dtype == kcache.dtype, "pooled_window_attn_tiled: shapes")
    _pooled_cache_check(kcache, vcache, nkv, dk, dv, "pooled_window_attn_tiled")
    for t, n in ((page_table, "page_table"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"), (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    rows = 0
    if pool:
        _f32(pooled_k, "pooled_k"); _f32(pooled_v, "pooled_v")
        rows = pooled_k.shape[2]
        _need(tuple(pooled_k.shape) == (kcache.shape[0], nkv, rows, dk) and tuple(pooled_v.shape) == (kcache.shape[0], nkv, rows, dv), "pooled_window_attn_tiled: pooled layout")
    _check(lib().edgelm_pooled_window_attn_tiled(_p(q), _p(out), _p(kcache), _p(vcache), _dt(q), _p(pooled_k) if pool else _p(None),
                                                 _p(pooled_v) if pool else _p(None), _p(page_table), page_table.stride(0), kcache.shape[0],
                                                 _p(tile_seq), _p(tile_tok0), _p(tile_ntok), _p(tile_pos0), int(n_tiles), int(max_tile_tokens),
                                                 nh, nkv, dk, dv, ctypes.c_float(scale), int(window), int(pool or 0), rows, _stream()))


# ----------------------------------------------------------------------------- attention with a key range per query
MASK_CAUSAL, MASK_WINDOW, MASK_CHUNK = 0, 1, 2


def _masked_cache_check(kcache, vcache, nkv, dk, dv, what):
    _need(kcache.is_contiguous() and tuple(kcache.shape[1:]) == (nkv, PAGE, dk), f"{what}: key cache shape")
    if vcache is not None:
        _need(vcache.is_contiguous() and vcache.dtype == kcache.dtype and tuple(vcache.shape) == (kcache.shape[0], nkv, PAGE, dv), f"{what}: value cache shape")
    else:
        _need(dv <= dk, f"{what}: values of {dv} dimensions inside keys of {dk}")


def rotate_append(qkv, bias, q_out, tok_pos, tok_seq, page_table, kcache, vcache, nh, nkv, dk, dv, rot, interleaved, freq, err,
                  maps=1, q_norm=None, k_norm=None, eps=0.0, conv_w=None, conv_state=None, seq_tok0=None, seq_slot=None, n_seqs=0):
    """qkv [T, nh dk + nkv dk + nkv dv] float32 (+ bias): the first `rot` dimensions of every query and key head are rotated
    by position * freq (float64 frequencies; pairs (2i, 2i + 1) if `interleaved`, else (i, i + rot/2)); queries go to q_out
    [T, nh dk] float32, keys and values to their places in the cache pages.  `maps` > 1: a head of dk dimensions is `maps`
    runs of dk / maps side by side, each rotated (its first `rot` dimensions) by itself.  `q_norm` / `k_norm` (float32
    [dk / maps]): every run is first divided by its root mean square (`eps` inside the root) and multiplied by the weight.
    `conv_w` (float32 [columns, taps]): every column of qkv + bias first passes a causal filter over time, as `conv_act` computes
    it (inputs from before the step out of `conv_state` [slots, taps - 1, columns], which is moved on to the step's last
    inputs: in the same launch when every sequence brings one token, by a second launch otherwise); `seq_tok0`, `seq_slot`,
    `n_seqs` as for `conv_act`."""
    _need(qkv.dtype == torch.float32 and qkv.is_cuda and qkv.dim() == 2 and qkv.stride(1) == 1, "rotate_append: qkv must be float32 rows")
    _f32(q_out, "q_out")
    T = qkv.shape[0]
    _need(qkv.shape[1] == (nh + nkv) * dk + nkv * dv and qkv.stride(0) >= qkv.shape[1] and q_out.shape == (T, nh * dk), "rotate_append: shapes")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == qkv.shape[1]), "rotate_append: bias")
    _need(rot == 0 or (freq is not None and freq.dtype == torch.float64 and freq.numel() == rot // 2 and freq.is_contiguous()), "rotate_append: frequencies")
    _masked_cache_check(kcache, vcache, nkv, dk, dv, "rotate_append")
    _need(vcache is not None, "rotate_append: values need a cache of their own")
    _need(maps >= 1 and dk % maps == 0 and rot <= dk // maps, "rotate_append: the maps of a head")
    for w, n in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        _need(w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous() and w.numel() == dk // maps), f"rotate_append: {n}")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (page_table, "page_table")):
        _i32(t, n)
    taps, single = 0, False
    if conv_w is not None:
        _f32(conv_w, "conv_w")
        taps = conv_w.shape[1]
        _need(conv_w.shape[0] == qkv.shape[1] and seq_tok0 is not None and seq_slot is not None and n_seqs > 0, "rotate_append: the filter's shapes")
        _need(taps == 1 or (conv_state is not None and conv_state.dtype == torch.float32 and conv_state.is_contiguous() and
                            tuple(conv_state.shape[1:]) == (taps - 1, qkv.shape[1])), "rotate_append: the filter's tails")
        _i32(seq_tok0, "seq_tok0"); _i32(seq_slot, "seq_slot")
        single = T == int(n_seqs)
    _check(lib().edgelm_rotate_append(_p(qkv), _p(bias), _p(q_out), _p(tok_pos), _p(tok_seq), _p(page_table), page_table.stride(0),
                                      kcache.shape[0], _p(kcache), _p(vcache), _dt(kcache), T, nh, nkv, dk, dv, int(rot),
                                      1 if interleaved else 0, _p(freq), _p(err), int(maps), _p(q_norm), _p(k_norm), ctypes.c_float(eps),
                                      qkv.stride(0), _p(conv_w), int(taps), _p(conv_state if taps > 1 else None), _p(seq_tok0), _p(seq_slot),
                                      1 if single else 0, _stream()))
    if conv_w is not None and taps > 1 and not single:
        _check(lib().edgelm_conv_tail_update(_p(qkv), qkv.stride(0), 0, _p(conv_state), _p(seq_tok0), _p(seq_slot), int(n_seqs), qkv.shape[1], int(taps),
                                             _p(bias), _stream()))


def latent_prepare(u, kv_off, has_kv, q_out, q_pitch, q_off, copy_q, norm_w, eps, tok_pos, tok_seq, page_table, kcache, nh, d, rd, r, freq, err,
                   row_out=None):
    """u [T, *] float32: nh query heads of [d | rd] from column 0 and, with `has_kv`, the latent's row [r | rd] from column
    `kv_off`.  The rotated part of every query head (pairs (i, i + rd/2)) goes to q_out[t, h * q_pitch + q_off :], with
    `copy_q` the unrotated part to q_out[t, h * q_pitch :]; the latent, RMS-normed with `norm_w`, and the rotated shared key
    part become the token's cache row [r + rd], and row t of `row_out` [T, r + rd] (optional, the cache's type)."""
    _f32(u, "u"); _f32(q_out, "q_out")
    T = u.shape[0]
    _need(q_out.shape == (T, nh * q_pitch), "latent_prepare: q_out shape")
    _need(rd == 0 or (freq is not None and freq.dtype == torch.float64 and freq.numel() == rd // 2 and freq.is_contiguous()), "latent_prepare: frequencies")
    if has_kv:
        _f32(norm_w, "norm_w")
        _need(norm_w.numel() == r, "latent_prepare: the norm's weight")
        _masked_cache_check(kcache, None, 1, r + rd, r, "latent_prepare")
        _i32(page_table, "page_table")
        _need(row_out is None or (row_out.dtype == kcache.dtype and row_out.is_contiguous() and row_out.shape == (T, r + rd)), "latent_prepare: row_out")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq")):
        _i32(t, n)
    _check(lib().edgelm_latent_prepare(_p(u), u.stride(0), int(kv_off), 1 if has_kv else 0, _p(q_out), int(q_pitch), int(q_off), 1 if copy_q else 0,
                                       _p(norm_w) if has_kv else _p(None), ctypes.c_float(eps), _p(tok_pos), _p(tok_seq),
                                       _p(page_table) if has_kv else _p(None), page_table.stride(0) if has_kv else 0, kcache.shape[0] if has_kv else 0,
                                       _p(kcache) if has_kv else _p(None), _p(row_out) if has_kv else _p(None), _dt(kcache) if has_kv else F32,
                                       T, nh, d, rd, r, _p(freq), _p(err), _stream()))


def latent_expand_keys(kn, rows, kx, nh, d, rd, r):
    """kx[t, h] = [kn[t, h, :d] | rows[t, r:]]: the step's keys per head, the shared rotated part repeated."""
    T = rows.shape[0]
    _need(kn.dtype == rows.dtype == kx.dtype and kn.is_contiguous() and rows.is_contiguous() and kx.is_contiguous(), "latent_expand_keys: layout")
    _need(kn.shape == (T, nh * d) and rows.shape == (T, r + rd) and kx.shape == (T, nh * (d + rd)), "latent_expand_keys: shapes")
    _check(lib().edgelm_latent_expand_keys(_p(kn), _p(rows), _p(kx), _dt(kx), T, nh, d, rd, r, _stream()))


def head_matmul(a, a_head_stride, w, out, out_head_stride):
    """out[t, h * out_head_stride + n] = sum_k a[t, h * a_head_stride + k] * w[h, n, k]: one small product per head.
    a float32 rows; w [heads, N, K] float32 or bfloat16; out float32 or the weights' type."""
    _f32(a, "a")
    _need(w.dim() == 3 and w.is_contiguous() and out.stride(1) == 1 and a.stride(1) == 1, "head_matmul: layout")
    H, N, K = w.shape
    _need((H - 1) * a_head_stride + K <= a.shape[1] and (H - 1) * out_head_stride + N <= out.shape[1] and out.shape[0] == a.shape[0], "head_matmul: shapes")
    _check(lib().edgelm_head_matmul(_p(a), a.stride(0), int(a_head_stride), _p(w), _dt(w), _p(out), _dt(out), out.stride(0), int(out_head_stride),
                                    a.shape[0], H, K, N, _stream()))


def add_row_bias(x, b):
    """x[t, :] += b."""
    _f32(x, "x"); _f32(b, "b")
    _need(x.dim() == 2 and b.numel() == x.shape[1], "add_row_bias: shapes")
    _check(lib().edgelm_add_row_bias(_p(x), _p(b), x.shape[0], x.shape[1], _stream()))


def _head_gate_check(gate, T, nh, what):
    _need(gate is None or (gate.dtype == torch.float32 and gate.is_cuda and gate.shape == (T, nh) and gate.stride(1) == 1), f"{what}: the heads' gate")


def masked_attn(q, out, kcache, vcache, tok_pos, tok_seq, page_table, nh, nkv, dk, dv, scale, mask, mask_size, sink, max_keys, maps=1, gate=None,
                n_splits=1, part=None):
    """Attention of every token of the step over the keys lo .. its position (`mask`: MASK_CAUSAL lo = 0; MASK_WINDOW the
    last `mask_size` keys; MASK_CHUNK the keys of its own chunk of `mask_size` positions).  q [T, nh dk] float32; out
    [T, nh dv] float32 or the cache's type; `vcache` None: a value is the first dv dimensions of its key row.  `sink`
    (float32 [nh] or None): one more term exp(sink_h) in the denominator.  `max_keys`: the most keys a token sees.
    `maps` > 1: every query head and key row holds `maps` runs of dk dimensions, each an attention of its own over the
    head's values: q [T, nh maps dk], key rows of maps dk, out [T, nh maps dv] (no sink then).  `gate` (float32 [T, nh], rows of
    any pitch): head h's output is multiplied by sigmoid(gate[t, h]) before it is rounded.  `n_splits` > 1: a token's keys are
    dealt to so many blocks, whose partial results go through `part` (float32, T nh maps n_splits (2 + dv) values) and are
    merged by a second launch: for steps of few tokens over long sequences."""
    _f32(q, "q")
    T = q.shape[0]
    _head_gate_check(gate, T, nh, "masked_attn")
    _need(n_splits == 1 or (part is not None and part.dtype == torch.float32 and part.is_contiguous() and part.numel() >= T * nh * maps * n_splits * (2 + dv)),
          "masked_attn: room for the splits' partial results")
    _need(q.shape == (T, nh * maps * dk) and out.is_contiguous() and out.shape == (T, nh * maps * dv), "masked_attn: shapes")
    _need(maps == 1 or (sink is None and vcache is not None), "masked_attn: several maps take no sink and values of their own")
    _masked_cache_check(kcache, vcache, nkv, dk * maps, dv, "masked_attn")
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh), "masked_attn: sink")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (page_table, "page_table")):
        _i32(t, n)
    _check(lib().edgelm_masked_attn(_p(q), _p(out), _dt(out), _p(kcache), _p(vcache), _dt(kcache), _p(tok_pos), _p(tok_seq), _p(page_table),
                                    page_table.stride(0), kcache.shape[0], T, nh, nkv, dk, dv, ctypes.c_float(scale), int(mask), int(mask_size or 0),
                                    _p(sink), int(max_keys), int(maps), _p(gate), gate.stride(0) if gate is not None else 0, int(n_splits), _p(part), _stream()),
           launches=2 if n_splits > 1 else 1)


def masked_attn_tiled(q, out, kcache, vcache, page_table, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, max_tile_tokens, nh, nkv,
                      dk, dv, scale, mask, mask_size, sink, n_splits=1, part=None, maps=1, gate=None):
    """`masked_attn` for prompt steps: the step's tokens come as tiles (runs of at most `max_tile_tokens` consecutive tokens of
    one sequence); a page of keys and values is staged once for all the rows of a tile.  `page_table` None: `kcache` [T, nkv dk]
    and `vcache` [T, nkv dv] are the step's own keys and values, and every sequence of the step starts at position 0.
    `n_splits` > 1: the pages that a tile sees are dealt to so many blocks, whose partial results go through `part` (float32,
    T nh n_splits (2 + dv) values) and are merged by a second launch: for steps of few tokens over long sequences.
    `maps` and `gate` as in `masked_attn` (then `part` holds T nh maps n_splits (2 + dv) values)."""
    _f32(q, "q")
    T = q.shape[0]
    _head_gate_check(gate, T, nh, "masked_attn_tiled")
    _need(q.shape == (T, nh * maps * dk) and out.is_contiguous() and out.shape == (T, nh * maps * dv), "masked_attn_tiled: shapes")
    _need(maps == 1 or (sink is None and vcache is not None), "masked_attn_tiled: several maps take no sink and values of their own")
    if page_table is not None:
        _masked_cache_check(kcache, vcache, nkv, dk * maps, dv, "masked_attn_tiled")
        _i32(page_table, "page_table")
    else:
        _need(vcache is not None and kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == vcache.dtype and
              kcache.shape == (T, nkv * dk * maps) and vcache.shape == (T, nkv * dv), "masked_attn_tiled: the step's own keys and values")
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == nh), "masked_attn_tiled: sink")
    _need(n_splits == 1 or (part is not None and part.dtype == torch.float32 and part.is_contiguous() and part.numel() >= T * nh * maps * n_splits * (2 + dv)),
          "masked_attn_tiled: room for the splits' partial results")
    for t, n in ((tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"), (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_masked_attn_tiled(_p(q), _p(out), _dt(out), _p(kcache), _p(vcache), _dt(kcache), _p(page_table),
                                          page_table.stride(0) if page_table is not None else 0, kcache.shape[0] if page_table is not None else 0,
                                          _p(tile_seq), _p(tile_tok0), _p(tile_ntok), _p(tile_pos0), int(n_tiles),
                                          int(max_tile_tokens), nh, nkv, dk, dv, ctypes.c_float(scale), int(mask), int(mask_size or 0), _p(sink),
                                          int(n_splits), _p(part), T, int(maps), _p(gate), gate.stride(0) if gate is not None else 0, _stream()),
           launches=2 if n_splits > 1 else 1)


SPLIT_PREFILL_TILE = 64  # new tokens per tile of the split-precision tensor-core prefill kernel (SP_ROWS in attention_mma_split.cu)


def attn_prefill_split_takes(dtype, dk, dv):
    """Whether the tensor-core prompt attention with float32 scores and weights takes this cache type and these head sizes."""
    return dtype == torch.bfloat16 and dk == dv and dk in (32, 64, 96, 128)


def attn_prefill_split(q, out, kcache, vcache, page_table, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, hd, scale, gate=None,
                       max_keys=0):
    """Causal attention of a prompt step over the paged bfloat16 cache on the tensor cores with float32 scores and softmax
    weights: the float32 operand of each product (queries; weights) goes as three bfloat16 terms.  q [T, nh hd] float32; out
    [T, nh hd] bfloat16; tiles of at most SPLIT_PREFILL_TILE tokens; `page_table` rows are the step's sequences; `gate` as in
    `masked_attn`."""
    _f32(q, "q")
    T = q.shape[0]
    _need(q.shape == (T, nh * hd) and out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (T, nh * hd), "attn_prefill_split: shapes")
    _masked_cache_check(kcache, vcache, nkv, hd, hd, "attn_prefill_split")
    _need(vcache is not None and kcache.dtype == torch.bfloat16, "attn_prefill_split: a bfloat16 cache with values of their own")
    _head_gate_check(gate, T, nh, "attn_prefill_split")
    for t, n in ((page_table, "page_table"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"), (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill_split(_p(q), q.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _p(page_table), page_table.stride(0),
                                           _p(tile_seq), _p(tile_tok0), _p(tile_ntok), _p(tile_pos0), int(n_tiles), nh, nkv, hd, ctypes.c_float(scale),
                                           _p(gate), gate.stride(0) if gate is not None else 0, int(max_keys), _stream()))


# ----------------------------------------------------------------------------- gated delta rule
def delta_prepare(qkv, u, b_off, a_off, a_log, dt_bias, bg, heads, kv_heads, d, e, unit_eps, q_scale):
    """qkv [T, G d | G d | H e] float32, in place: every query and key head becomes x / sqrt(sum(x^2) + unit_eps), queries
    also times q_scale.  bg [T, 2 H] receives beta = sigmoid(u[:, b_off + h]) and the decay exp(-exp(A_log_h)
    softplus(u[:, a_off + h] + dt_bias_h))."""
    for t, n in ((qkv, "qkv"), (a_log, "A_log"), (dt_bias, "dt_bias"), (bg, "bg")):
        _f32(t, n)
    _need(u.dtype == torch.float32 and u.stride(1) == 1 and u.shape[0] == qkv.shape[0] and bg.numel() >= 2 * heads * qkv.shape[0], "delta_prepare: shapes")
    _need(a_log.numel() == heads and dt_bias.numel() == heads, "delta_prepare: per-head vectors")
    _check(lib().edgelm_delta_prepare(_p(qkv), qkv.shape[1], _p(u), u.stride(0), int(b_off), int(a_off), _p(a_log), _p(dt_bias), _p(bg),
                                      qkv.shape[0], heads, kv_heads, d, e, ctypes.c_float(unit_eps), ctypes.c_float(q_scale), _stream()))


def delta_scan(qkv, bg, state, o, seq_tok0, seq_slot, n_seqs, heads, kv_heads, d, e):
    """Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, over the step's tokens of every sequence.
    qkv [T, G d | G d | H e] (prepared), bg [T, 2 H] (beta, decay), state [slots, H, e, d] float32, o [T, H e]."""
    for t, n in ((qkv, "qkv"), (bg, "bg"), (state, "state"), (o, "o")):
        _f32(t, n)
    T = qkv.shape[0]
    _need(tuple(state.shape[1:]) == (heads, e, d) and o.shape == (T, heads * e), "delta_scan: state or output shape")
    _check(lib().edgelm_delta_scan(_p(qkv), qkv.shape[1], _p(bg), _p(state), _p(o), _p(seq_tok0), _p(seq_slot), int(n_seqs), T, heads,
                                   kv_heads, d, e, _stream()))


# ----------------------------------------------------------------------------- mixture of experts
def moe_tile_rows(tensor_cores=False):
    """Rows of a tile of the grouped products: every expert's rows start at a multiple of it (the CUDA-core kernels'
    tile, or the tcgen05 kernel's 128)."""
    return 128 if tensor_cores else int(lib().edgelm_moe_tile_rows())


def moe_max_tiles(n_pairs, n_experts, tile_rows):
    """Row tiles that `n_pairs` (token, choice) pairs grouped by expert take at most."""
    return max(1, min(n_pairs, n_pairs // tile_rows + n_experts))


def moe_route(h, wr, br, idx, wts, top):
    """Router logits h @ wr.T + br in float32; idx [T, top] the experts with the largest logits (first maximum on ties),
    wts [T, top] the softmax over the chosen logits."""
    _f32(wr, "router weight"); _f32(br, "router bias"); _f32(wts, "wts"); _i32(idx, "idx")
    T, D = h.shape
    E = wr.shape[0]
    _need(h.is_contiguous() and wr.shape == (E, D) and br.numel() == E and idx.shape == (T, top) and wts.shape == (T, top), "moe_route: shapes")
    _check(lib().edgelm_moe_route(_p(h), _dt(h), _p(wr), _p(br), _p(idx), _p(wts), T, D, E, int(top), _stream()))


def moe_route_scored(h, wr, correction, idx, wts, top, n_experts, groups=1, keep=1, scale=1.0, extra=None):
    """The router that scores every expert: s = softmax(wr[:n_experts] h) over all experts (float32); the `top` experts with the
    largest s + correction are chosen (first of equal ones), with `groups` > 1 only among the `keep` groups of neighbouring
    experts whose best corrected score is largest (the others count as minus infinity: when the kept groups hold fewer than `top`
    experts, the left-out ones follow in the order of their numbers); wts = s of the chosen over their sum (+ 1e-20), times
    `scale`.  Rows of `wr` after the first `n_experts` give `extra` [T, rows] = sigmoid(row . h).  idx of a choice that could not
    be made (scores that are not numbers): -1."""
    _f32(wr, "router weight"); _f32(wts, "wts"); _i32(idx, "idx")
    T, D = h.shape
    n_extra = wr.shape[0] - n_experts
    _need(h.is_contiguous() and wr.shape[1] == D and n_extra >= 0 and idx.shape == (T, top) and wts.shape == (T, top), "moe_route_scored: shapes")
    _need(correction is None or (correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == n_experts), "moe_route_scored: correction")
    _need((n_extra == 0) == (extra is None) and (extra is None or (extra.dtype == torch.float32 and extra.is_contiguous() and extra.shape == (T, n_extra))), "moe_route_scored: extra rows")
    _check(lib().edgelm_moe_route_scored(_p(h), _dt(h), _p(wr), _p(correction), _p(idx), _p(wts), _p(extra), T, D, int(n_experts), int(n_extra), int(top),
                                         int(groups), int(keep), ctypes.c_float(scale), _stream()))


def moe_plan(idx, n_experts, tile_rows, row_pair, pair_row, tile_expert):
    """Group the pairs of idx [T, top] by expert: row_pair [max_tiles * tile_rows] (pair or -1), pair_row [T * top] (each
    pair's row), tile_expert [max_tiles] (the expert of a tile of rows, or -1)."""
    _i32(idx, "idx"); _i32(row_pair, "row_pair"); _i32(pair_row, "pair_row"); _i32(tile_expert, "tile_expert")
    max_tiles = tile_expert.numel()
    _need(row_pair.numel() == max_tiles * tile_rows and pair_row.numel() == idx.numel(), "moe_plan: sizes of the maps")
    _check(lib().edgelm_moe_plan(_p(idx), idx.numel(), int(n_experts), int(tile_rows), max_tiles, _p(row_pair), _p(pair_row), _p(tile_expert), _stream()))


def moe_gather_rows(h, a, row_pair, top):
    """a[row] = h[row_pair[row] // top], zeros for a row without a pair."""
    _i32(row_pair, "row_pair")
    _need(h.dtype == a.dtype and h.is_contiguous() and a.is_contiguous() and a.shape == (row_pair.numel(), h.shape[1]), "moe_gather_rows: shapes")
    _check(lib().edgelm_moe_gather_rows(_p(h), _p(a), _p(row_pair), row_pair.numel(), int(top), h.shape[1], _dt(h), _stream()))


GLU_SWIGLU = (0.0, 1.0, 0.0)     # (limit, alpha, shift) of the gated unit g sigmoid(alpha g) (v + shift); limit 0: no clamps


def moe_gate_up(h, w_gate, w_up, mid, row_pair, tile_expert, top, glu=GLU_SWIGLU):
    """mid[row] = unit(w_gate[e] h[t], w_up[e] h[t]) for every row of the plan (t = row_pair[row] // top, e the row's tile's
    expert), on the CUDA cores.  The unit is silu(g) * v, or with `glu` (limit, alpha, shift) g sigmoid(alpha g) (v + shift) with
    g = min(g, limit) and v = clamp(v, -limit, limit) when limit > 0."""
    E, N, K = w_gate.shape
    _need(h.dtype == w_gate.dtype == w_up.dtype == mid.dtype and h.is_contiguous() and w_gate.is_contiguous() and w_up.is_contiguous() and mid.is_contiguous(), "moe_gate_up: layout")
    _need(h.shape[1] == K and w_up.shape == w_gate.shape and mid.shape == (row_pair.numel(), N), "moe_gate_up: shapes")
    _need(row_pair.numel() == tile_expert.numel() * moe_tile_rows(), "moe_gate_up: the plan's row tile is not this kernel's")
    _check(lib().edgelm_moe_gemm(_p(h), h.stride(0), _p(w_gate), _p(w_up), _p(mid), mid.stride(0), _p(row_pair), _p(tile_expert),
                                 tile_expert.numel(), int(top), K, N, _dt(h), 1, ctypes.c_float(glu[0]), ctypes.c_float(glu[1]), ctypes.c_float(glu[2]), _stream()))


def moe_down(mid, w_down, y, row_pair, tile_expert, top):
    """y[row] = w_down[e] mid[row] (float32) for every row of the plan, on the CUDA cores."""
    E, N, K = w_down.shape
    _f32(y, "y")
    _need(mid.dtype == w_down.dtype and mid.is_contiguous() and w_down.is_contiguous() and mid.shape == (row_pair.numel(), K) and y.shape == (row_pair.numel(), N), "moe_down: shapes")
    _need(row_pair.numel() == tile_expert.numel() * moe_tile_rows(), "moe_down: the plan's row tile is not this kernel's")
    _check(lib().edgelm_moe_gemm(_p(mid), mid.stride(0), _p(w_down), _p(None), _p(y), y.stride(0), _p(row_pair), _p(tile_expert),
                                 tile_expert.numel(), int(top), K, N, _dt(mid), 0, ctypes.c_float(0.0), ctypes.c_float(1.0), ctypes.c_float(0.0), _stream()))


def gemm_tc_grouped_takes(a, w, w2=None):
    """Whether the grouped tcgen05 product takes these operands: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    return bool(lib().edgelm_gemm_tc_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[1]))


def gemm_tc_grouped(a, w, out, tile_group, err, epilogue=EPI_STORE, w2=None, glu=GLU_SWIGLU):
    """out[row] = a[row] @ w[g].T (+ epilogue) with g = tile_group[row // 128] (negative: a tile without rows): a [M, K]
    bfloat16 with M a multiple of 128, w (and w2 for the gated unit) [groups, N, K] bfloat16, out [M, N] float32 or bfloat16.
    `glu`: the gated unit's form, as in `moe_gate_up`."""
    _i32(tile_group, "tile_group")
    G, N, K = w.shape
    M = a.shape[0]
    _need(a.shape == (M, K) and out.shape == (M, N) and out.stride(1) == 1 and tile_group.numel() * 128 == M, "gemm_tc_grouped: shapes")
    _need(w2 is None or (w2.shape == w.shape and w2.is_contiguous() and w2.dtype == w.dtype), "gemm_tc_grouped: second weight")
    _check(lib().edgelm_gemm_tc_grouped(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), M, N, K, G, _p(tile_group), _dt(out), int(epilogue),
                                        ctypes.c_float(glu[0]), ctypes.c_float(glu[1]), ctypes.c_float(glu[2]), _p(err), _stream()))


def moe_combine(x, y, wts, pair_row, idx=None, n_real=0, h=None, shared=None, gate=None):
    """x[t] += sum_k wts[t, k] * y[pair_row[t * top + k]].  With `idx` [T, top], `n_real` and `h` [T, D]: a pair whose expert
    number is at least `n_real` belongs to an identity expert, whose output is the token's input h[t].  With `shared`
    [T, D] float32 (and `gate` [T] float32, else 1): x[t] += gate[t] * shared[t] as well."""
    _f32(x, "x"); _f32(y, "y"); _f32(wts, "wts"); _i32(pair_row, "pair_row")
    T, top = wts.shape
    D = x.shape[1]
    _need(x.shape[0] == T and y.shape[1] == D and pair_row.numel() == T * top, "moe_combine: shapes")
    if idx is not None:
        _i32(idx, "idx")
        _need(idx.numel() == T * top and h is not None and h.is_contiguous() and h.shape == (T, D), "moe_combine: identity experts need the tokens' inputs")
    if shared is not None:
        _f32(shared, "shared")
        _need(shared.shape == (T, D) and (gate is None or (gate.dtype == torch.float32 and gate.is_contiguous() and gate.numel() == T)), "moe_combine: the shared term")
    _check(lib().edgelm_moe_combine(_p(x), _p(y), y.stride(0), _p(wts), _p(pair_row), T, top, D, _p(idx), int(n_real), _p(h if idx is not None else None),
                                    _dt(h) if idx is not None else F32, _p(shared), _p(gate if shared is not None else None), _stream()))


# ----------------------------------------------------------------------------- several residual streams
def streams_fill(x, xs):
    """xs[t, s] = x[t] for every stream s.  x [T, D], xs [T, S, D], float32."""
    _f32(x, "x"); _f32(xs, "xs")
    T, S, D = xs.shape
    _need(x.shape == (T, D), "streams_fill: shapes")
    _check(lib().edgelm_streams_fill(_p(x), _p(xs), T, S, D, _stream()))


def streams_update(xs, y=None, mix=None, w_out=None, w_in=None, norm_w=None, eps=0.0, h=None):
    """A residual stream kept as S copies xs [T, S, D] (float32).  With `y` [T, D]: every stream is rewritten from the old
    ones, xs'[t] = sum_s mix[s, t] xs[s] + w_out[t] y.  With `w_in` [S]: u = sum_s w_in[s] xs'[s] is read out, into `h` as
    float32, or with `norm_w` [D] as u / sqrt(mean(u^2) + eps) * norm_w in h's type.  Both at once: one pass over xs."""
    _f32(xs, "xs")
    T, S, D = xs.shape
    if y is not None:
        _f32(y, "y"); _f32(mix, "mix"); _f32(w_out, "w_out")
        _need(y.shape == (T, D) and mix.shape == (S, S) and w_out.numel() == S, "streams_update: the write's shapes")
    if w_in is not None:
        _f32(w_in, "w_in")
        _need(w_in.numel() == S and h is not None and h.is_contiguous() and h.shape == (T, D), "streams_update: the read's shapes")
        _need(norm_w is None or (norm_w.dtype == torch.float32 and norm_w.is_contiguous() and norm_w.numel() == D), "streams_update: norm weight")
    _check(lib().edgelm_streams_update(_p(xs), _p(y), _p(mix), _p(w_out), _p(w_in), _p(norm_w), ctypes.c_float(eps), _p(h),
                                       _dt(h) if h is not None else 0, T, S, D, _stream()))


# ----------------------------------------------------------------------------- real-gated linear recurrent unit
RGLRU_SEG = 64        # tokens of a prompt step that one block of the scan composes (RG_SEG in rglru.cu)


def rglru_scratch_floats(n_tokens, n_seqs, W):
    """Floats of scratch that a prompt step of the scan needs: a map (two rows of W) per segment."""
    return 2 * ((n_tokens + RGLRU_SEG - 1) // RGLRU_SEG) * W


def rglru_scan(gates, br, bi, u, c, y, by, state, out, seq_tok0, seq_slot, n_seqs, single, tok_seq=None, scratch=None):
    """S_t = a S_(t-1) + sqrt(1 - a^2) i u with a = exp(c r), r = sigmoid(gates[:, :W] + br), i = sigmoid(gates[:, W:] + bi);
    out = S_t gelu_tanh(y + by).  gates [T, 2 W], u [T, W] and y (a view of W columns) float32 rows; c, br, bi, by [W];
    state [slots, W] float32, read and moved on; `single`: every sequence of the step brings one token.  Other steps name
    every token's sequence (`tok_seq` [T] int32), bring `scratch`, float32 of `rglru_scratch_floats` elements, and leave
    decays and inputs in `gates`."""
    for t, n in ((gates, "gates"), (br, "br"), (bi, "bi"), (c, "c"), (by, "by"), (state, "state")):
        _f32(t, n)
    T, W = out.shape
    _need(u.dtype == y.dtype == torch.float32 and u.stride(1) == 1 and y.stride(1) == 1 and out.is_contiguous(), "rglru_scan: layout")
    _need(gates.shape == (T, 2 * W) and u.shape == (T, W) and y.shape == (T, W) and state.shape[1] == W and
          br.numel() == bi.numel() == c.numel() == by.numel() == W, "rglru_scan: shapes")
    _i32(seq_tok0, "seq_tok0"); _i32(seq_slot, "seq_slot")
    if not single:
        _i32(tok_seq, "tok_seq"); _f32(scratch, "scratch")
        _need(tok_seq.numel() >= T and scratch.numel() >= rglru_scratch_floats(T, int(n_seqs), W), "rglru_scan: tok_seq and scratch sizes")
    _check(lib().edgelm_rglru_scan(_p(gates), gates.stride(0), _p(br), _p(bi), _p(u), u.stride(0), _p(c), _p(y), y.stride(0), _p(by), _p(state),
                                   _p(out), _dt(out), _p(seq_tok0), _p(seq_slot), _p(tok_seq) if not single else None,
                                   _p(scratch) if not single else None, int(n_seqs), T, W, 1 if single else 0, _stream()),
           launches=1 if single else 2)


def rglru_gates(u, w_ra, w_ri, gates, blocks):
    """gates[:, :W] and gates[:, W:] <- the block-diagonal products of u [T, W] float32 with w_ra and w_ri [blocks, W / blocks,
    W / blocks] ([out, in] per block), float32 sums.  bfloat16 matrices run on the tensor cores with the input split into three
    bfloat16 terms (exact products, float32 sums); float32 matrices take the plain float32 kernel, a matrix at a time."""
    _f32(u, "u"); _f32(gates, "gates")
    T, W = u.shape
    bw = W // blocks
    _need(W % blocks == 0 and gates.shape == (T, 2 * W) and w_ra.shape == w_ri.shape == (blocks, bw, bw) and w_ra.dtype == w_ri.dtype and
          w_ra.is_contiguous() and w_ri.is_contiguous() and u.stride(1) == 1, "rglru_gates: shapes")
    if w_ra.dtype == torch.bfloat16:
        _check(lib().edgelm_rglru_gates(_p(u), u.stride(0), _p(w_ra), _p(w_ri), _p(gates), gates.stride(0), T, W, int(blocks), _stream()))
    else:
        head_matmul(u, bw, w_ra, gates[:, :W], bw)
        head_matmul(u, bw, w_ri, gates[:, W:], bw)


def clamped_glu(gu, mid, limit, alpha, shift=1.0, bias=None, x=None, x_bias=None):
    """mid = g sigmoid(alpha g) (v + shift) with g = min(gate, limit), v = clamp(up, -limit, limit) (limit 0: no clamps);
    gu [T, 2 F] float32 = gate | up, `bias` [2 F] float32 added to it first.  limit 0, alpha 1, shift 0: silu(gate) * up.
    With `x` [T, D] float32 and `x_bias` [D]: x += x_bias in the same launch (the bias of the projection that follows, whose
    epilogue adds to x)."""
    _f32(gu, "gu")
    T, F = mid.shape
    _need(gu.shape == (T, 2 * F) and mid.is_contiguous(), "clamped_glu: shapes")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_cuda and bias.is_contiguous() and bias.numel() == 2 * F), "clamped_glu: bias")
    _need((x is None) == (x_bias is None) and (x is None or (x.dtype == torch.float32 and x.is_contiguous() and x.shape[0] == T and x_bias.dtype == torch.float32 and
                                                             x_bias.is_contiguous() and x_bias.numel() == x.shape[1])), "clamped_glu: the rows that take a bias")
    _check(lib().edgelm_clamped_glu(_p(gu), _p(mid), _dt(mid), T, F, ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift), _p(bias),
                                    _p(x), _p(x_bias), x.shape[1] if x is not None else 0, _stream()))


def diff_combine(a, out, lam, eps, post, w=None):
    """Two attention maps of a head into one: a [T, H, 2, dv] float32; o = a_1 - lam a_2, divided by its root mean square over
    dv (`eps` inside the root), times `post` (and `w` [dv], if given); out [T, H dv]."""
    _f32(a, "a")
    T = a.shape[0]
    dv = a.shape[-1]
    _need(a.dim() == 4 and a.shape[2] == 2 and out.is_contiguous() and out.shape == (T, a.shape[1] * dv), "diff_combine: shapes")
    _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == dv), "diff_combine: weight")
    _check(lib().edgelm_diff_combine(_p(a), _p(out), _dt(out), ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(post), _p(w),
                                     T * a.shape[1], dv, _stream()))


# ----------------------------------------------------------------------------- linear attention with a constant decay per head
def silu_columns(u, off, n):
    """u[:, off : off + n] <- silu(.) in place (float32 rows of any pitch)."""
    _need(u.dtype == torch.float32 and u.is_cuda and u.dim() == 2 and u.stride(1) == 1 and 0 <= off and off + n <= u.shape[1], "silu_columns: layout")
    _check(lib().edgelm_silu_columns(_p(u), u.stride(0), int(off), int(n), u.shape[0], _stream()))


def decay_scan(u, q_off, k_off, v_off, decay, state, o, seq_tok0, seq_slot, n_seqs, heads, k_dim, v_dim, act=None):
    """Per head S <- decay_h S + k_t v_t^T, then o_t = S^T q_t, over the step's tokens in order.  q, k (heads x k_dim) and v
    (heads x v_dim) are columns of u [T, *] float32 from q_off, k_off, v_off; decay [heads] float32; state [slots, heads,
    v_dim, k_dim] float32; o [T, heads v_dim] float32.  `act` "silu": q, k and v pass it as they are read (every warp of a head
    again: for steps of few tokens, where that is cheaper than `silu_columns` ahead)."""
    _f32(decay, "decay"); _f32(state, "state"); _f32(o, "o")
    _i32(seq_tok0, "seq_tok0"); _i32(seq_slot, "seq_slot")
    T = u.shape[0]
    _need(u.dtype == torch.float32 and u.is_cuda and u.stride(1) == 1, "decay_scan: u must be float32 rows")
    _need(max(q_off, k_off) + heads * k_dim <= u.shape[1] and v_off + heads * v_dim <= u.shape[1] and o.shape == (T, heads * v_dim), "decay_scan: shapes")
    _need(decay.numel() == heads and tuple(state.shape[1:]) == (heads, v_dim, k_dim), "decay_scan: decay or state")
    _check(lib().edgelm_decay_scan(_p(u), u.stride(0), int(q_off), int(k_off), int(v_off), _p(decay), _p(state), _p(o), _p(seq_tok0), _p(seq_slot),
                                   int(n_seqs), int(heads), int(k_dim), int(v_dim), T, 1 if act == "silu" else 0, _stream()))


DECAY_CHUNK = 64        # tokens of a chunk of the chunked form (LC in linear_attention.cu)


def decay_chunked_takes(k_dim, v_dim):
    """Whether the chunked form takes heads of k_dim x v_dim (its tiles must fit in shared memory)."""
    c = DECAY_CHUNK     # (the rule of `edgelm_decay_chunked_takes`, answered without the library: plans are made on hosts without a device too)
    smem = 4 * (2 * c * (k_dim + 1) + c * (v_dim + 1) + k_dim * (v_dim + 1) + c * (c + 1) + c + 1)
    return 1 <= k_dim <= 128 and 1 <= v_dim <= 128 and smem <= 200 * 1024


def decay_chunked_scratch_floats(n_tiles, heads, k_dim, v_dim):
    return int(n_tiles) * heads * k_dim * v_dim


def decay_powers(decay):
    """The table of the chunked form: decay_h^0 .. decay_h^DECAY_CHUNK for every head, computed in float64 and rounded once
    (float32 [heads, DECAY_CHUNK + 1], on the CPU; the caller moves it to the device)."""
    d = torch.as_tensor(decay, dtype=torch.float64).reshape(-1, 1)
    return (d ** torch.arange(DECAY_CHUNK + 1, dtype=torch.float64).reshape(1, -1)).to(torch.float32).contiguous()


def decay_chunked(u, q_off, k_off, v_off, powers, state, o, seq_tok0, seq_slot, n_seqs, tile_tok0, tile_ntok, n_tiles, heads, k_dim, v_dim,
                  act="silu", scratch=None):
    """`decay_scan` for prompt steps, chunk by chunk (three launches): the step's tokens come as tiles of at most DECAY_CHUNK
    consecutive tokens of one sequence, in the sequences' order, each sequence cut from its first row of the step.  `powers`:
    the table of `decay_powers` on the device.  `act`:
    "silu" (q, k, v pass it as they are read) or None.  `scratch`: float32 room for `decay_chunked_scratch_floats` values."""
    _f32(powers, "powers"); _f32(state, "state"); _f32(o, "o")
    for t, n in ((seq_tok0, "seq_tok0"), (seq_slot, "seq_slot"), (tile_tok0, "tile_tok0"), (tile_ntok, "tile_ntok")):
        _i32(t, n)
    T = u.shape[0]
    _need(u.dtype == torch.float32 and u.is_cuda and u.stride(1) == 1, "decay_chunked: u must be float32 rows")
    _need(max(q_off, k_off) + heads * k_dim <= u.shape[1] and v_off + heads * v_dim <= u.shape[1] and o.shape == (T, heads * v_dim), "decay_chunked: shapes")
    _need(tuple(powers.shape) == (heads, DECAY_CHUNK + 1) and tuple(state.shape[1:]) == (heads, v_dim, k_dim) and act in ("silu", None), "decay_chunked: powers, state or activation")
    need = decay_chunked_scratch_floats(n_tiles, heads, k_dim, v_dim)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=u.device)
    _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need, "decay_chunked: scratch too small")
    _check(lib().edgelm_decay_chunked(_p(u), u.stride(0), int(q_off), int(k_off), int(v_off), _p(powers), _p(state), _p(o), _p(seq_tok0), _p(seq_slot),
                                      int(n_seqs), _p(tile_tok0), _p(tile_ntok), int(n_tiles), int(heads), int(k_dim), int(v_dim), 1 if act == "silu" else 0,
                                      _p(scratch), _stream()), launches=3)


def rmsnorm_pair(x, w1, eps, y1, w2=None, y2=None, add=None):
    """y1 = norm(x) * w1 and y2 = norm(x) * w2 with the rows' statistics computed once; with `add` [T, D] float32, x += add first
    (written back).  x float32 [T, D]; y1, y2 in the compute dtype."""
    _f32(x, "x"); _f32(w1, "w1")
    _need(y1.shape == x.shape and y1.is_contiguous() and w1.numel() == x.shape[1], "rmsnorm_pair: shapes")
    _need((w2 is None) == (y2 is None) and (w2 is None or (w2.dtype == torch.float32 and w2.is_contiguous() and w2.numel() == x.shape[1] and
                                                            y2.shape == x.shape and y2.is_contiguous() and y2.dtype == y1.dtype)), "rmsnorm_pair: the second norm")
    _need(add is None or (add.dtype == torch.float32 and add.is_contiguous() and add.shape == x.shape), "rmsnorm_pair: the rows to add")
    _check(lib().edgelm_rmsnorm_pair(_p(x), _p(add), _p(w1), _p(w2), _p(y1), _p(y2), _dt(y1), x.shape[0], x.shape[1], ctypes.c_float(eps), _stream()))


def softcap(z, cap):
    """z <- cap * tanh(z / cap), in place (float32)."""
    _f32(z, "z")
    _check(lib().edgelm_softcap(_p(z), ctypes.c_longlong(z.numel()), ctypes.c_float(cap), _stream()))
