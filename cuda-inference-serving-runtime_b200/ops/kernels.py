"""Python face of the CUDA kernels: one function per kernel entry point.

Every function checks shapes, types and contiguity, passes raw device pointers and
the current CUDA stream to the C entry point, and raises `KernelError` on a
non-zero status.  Nothing here falls back to a library or to the CPU: without a
CUDA device or without the compiled kernels these functions fail.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
GEMM_WORKSPACE_BYTES = 64 << 20


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"storage type {dtype} is not supported (float32 and bfloat16 only)") from None


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  Every launch asks for it, so it takes the short way where torch has one (a tenth of
    the time of building a Stream object, which showed in steps that launch hundreds of kernels from the host)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_pdl_state = {"on": False}
LAUNCHES = {"own": 0, "library": 0}   # kernels launched so far: this package's own, and vendor-library products


def _check(status: int, what: str, own: int = 1, library: int = 0) -> None:
    LAUNCHES["own"] += own
    LAUNCHES["library"] += library
    if status != 0:
        detail = {-2: "invalid argument", -3: "shared memory need exceeds the device limit"}.get(status, "")
        raise KernelError(f"{what} failed with status {status} {detail}".rstrip())


def _need(t: torch.Tensor, dtype, name: str, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


# ------------------------------------------------------------------ elementwise library
def _elementwise():
    lib = load_library("elementwise.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_embedding.restype = ctypes.c_int
        lib.cisr_add_rmsnorm.restype = ctypes.c_int
        lib.cisr_swiglu.restype = ctypes.c_int
        lib.cisr_rotary_tables.restype = ctypes.c_int
        lib.cisr_rope_store.restype = ctypes.c_int
        lib.cisr_page_copy.restype = ctypes.c_int
        lib.cisr_table_update.restype = ctypes.c_int
        lib.cisr_stream_add.restype = ctypes.c_int
        lib.cisr_scale.restype = ctypes.c_int
        lib.cisr_activation.restype = ctypes.c_int
        lib._typed = True
    return lib


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float, times `scale`."""
    _need(table, None, "table", 2); _need(ids, torch.int32, "ids", 1); _need(out, torch.float32, "out", 2)
    tokens, hidden = out.shape
    if ids.numel() != tokens or table.shape[1] != hidden:
        raise KernelError("embedding: shapes of ids, table and out disagree")
    _check(_elementwise().cisr_embedding(_p(table), dtype_code(table.dtype), _p(ids), _p(out), tokens, hidden,
                                         table.shape[0], ctypes.c_float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, write_back: bool = True,
                delta_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += delta (when given; times the per-channel `delta_scale` when that is given), out = rmsnorm(x) * weight;
    `rows` selects which rows of x become rows of out."""
    _need(x, torch.float32, "x", 2); _need(weight, None, "weight", 1); _need(out, None, "out", 2)
    hidden = x.shape[1]
    if delta is not None:
        _need(delta, torch.float32, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError("add_rmsnorm: delta and x differ in shape")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one row index per output row is needed")
    elif n_rows != x.shape[0]:
        raise KernelError("add_rmsnorm: out and x differ in rows")
    if weight.numel() != hidden or out.shape[1] != hidden:
        raise KernelError("add_rmsnorm: width mismatch")
    if delta_scale is not None:
        _need(delta_scale, torch.float32, "delta_scale", 1)
        if delta_scale.numel() != hidden:
            raise KernelError("add_rmsnorm: one scale per channel is needed")
    _check(_elementwise().cisr_add_rmsnorm(_p(x), _p(delta), _p(weight), dtype_code(weight.dtype), _p(out),
                                           dtype_code(out.dtype), _p(rows), n_rows, hidden, ctypes.c_float(eps),
                                           int(write_back), _p(delta_scale if delta is not None else None), _stream()),
           "add_rmsnorm")
    return out


def stream_add(x: torch.Tensor, delta: Optional[torch.Tensor] = None, delta_scale: Optional[torch.Tensor] = None,
               vector: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t, :] += delta[t, :] * delta_scale + vector, in place; each of the three may be absent."""
    _need(x, torch.float32, "x", 2)
    tokens, hidden = x.shape
    if delta is not None:
        _need(delta, torch.float32, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError("stream_add: delta and x differ in shape")
    for name, t in (("delta_scale", delta_scale), ("vector", vector)):
        if t is not None:
            _need(t, torch.float32, name, 1)
            if t.numel() != hidden:
                raise KernelError(f"stream_add: {name} must have one value per channel")
    _check(_elementwise().cisr_stream_add(_p(x), _p(delta), _p(delta_scale if delta is not None else None), _p(vector), tokens,
                                          hidden, _stream()), "stream_add")
    return x


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x *= scale, in place (float)."""
    _need(x, torch.float32, "x")
    _check(_elementwise().cisr_scale(_p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(scale), _stream()), "scale")
    return x


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need(gate_up, torch.float32, "gate_up", 2); _need(out, None, "out", 2)
    tokens, inter = out.shape
    if gate_up.shape != (tokens, 2 * inter):
        raise KernelError("swiglu: gate_up must be [tokens, 2 * intermediate]")
    _check(_elementwise().cisr_swiglu(_p(gate_up), _p(out), dtype_code(out.dtype), tokens, inter, _stream()), "swiglu")
    return out


ACTIVATIONS = {"relu_squared": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out[:, :n] = act(x) for float x [tokens, n]; columns of out beyond n (padding of the next product's K) get zeros."""
    _need(x, torch.float32, "x", 2); _need(out, None, "out", 2)
    if kind not in ACTIVATIONS:
        raise KernelError(f"unknown activation {kind!r}; known: {', '.join(sorted(ACTIVATIONS))}")
    if out.shape[0] != x.shape[0] or out.shape[1] < x.shape[1]:
        raise KernelError("activation: out must have x's rows and at least its columns")
    _check(_elementwise().cisr_activation(_p(x), _p(out), dtype_code(out.dtype), x.shape[0], x.shape[1], out.shape[1],
                                          ACTIVATIONS[kind], _stream()), "activation")
    return out


def rotary_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  magnitude: float = 1.0) -> None:
    """cos, sin [tokens, pairs] = magnitude * cos / sin(position * inv_freq), angles in float64."""
    _need(positions, torch.int32, "positions", 1); _need(inv_freq, torch.float64, "inv_freq", 1)
    _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
    tokens, half = cos.shape
    if positions.numel() != tokens or inv_freq.numel() != half or sin.shape != cos.shape:
        raise KernelError("rotary_tables: shapes disagree")
    _check(_elementwise().cisr_rotary_tables(_p(positions), _p(inv_freq), _p(cos), _p(sin), tokens, half,
                                             ctypes.c_double(magnitude), _stream()),
           "rotary_tables")


def rope_store(proj: torch.Tensor, k_col: int, v_col: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               rot_half: int, interleaved: bool, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], token_req: torch.Tensor, positions: torch.Tensor,
               req_slot: torch.Tensor, block_table: torch.Tensor, page_size: int, hq: int, hkv: int, dim: int) -> None:
    """Rotate q (and k), write q to q_out and k, v into their cache pages (k_col < 0: queries only)."""
    _need(proj, torch.float32, "proj", 2); _need(q_out, None, "q_out")
    tokens = proj.shape[0]
    if rot_half:
        _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
        if cos.shape != (tokens, rot_half) or sin.shape != cos.shape:
            raise KernelError("rope_store: rotary tables must be [tokens, rot_half]")
    if q_out.numel() != tokens * hq * dim:
        raise KernelError("rope_store: q_out must hold [tokens, heads, head_dim]")
    cache_code = F32
    if k_col >= 0:
        _need(k_cache, None, "k_cache", 4); _need(v_cache, k_cache.dtype, "v_cache", 4)
        if tuple(k_cache.shape[1:]) != (hkv, page_size, dim) or v_cache.shape != k_cache.shape:
            raise KernelError("rope_store: cache must be [pages, kv_heads, page_size, head_dim]")
        if proj.shape[1] < v_col + hkv * dim or proj.shape[1] < k_col + hkv * dim:
            raise KernelError("rope_store: projection row is too short for its key and value columns")
        cache_code = dtype_code(k_cache.dtype)
    _need(token_req, torch.int32, "token_req", 1); _need(positions, torch.int32, "positions", 1)
    _need(block_table, torch.int32, "block_table", 2); _need(req_slot, torch.int32, "req_slot", 1)
    _check(_elementwise().cisr_rope_store(
        _p(proj), proj.shape[1], k_col, v_col, _p(cos if rot_half else None), _p(sin if rot_half else None), rot_half,
        int(interleaved), _p(q_out), dtype_code(q_out.dtype), _p(k_cache), _p(v_cache), cache_code, _p(token_req),
        _p(positions), _p(req_slot), _p(block_table), block_table.shape[1], page_size, hq, hkv, dim, tokens, _stream()),
        "rope_store")


def page_copy(pool: torch.Tensor, pairs: torch.Tensor, n_planes: int, plane_bytes: int, page_bytes: int) -> None:
    """Copy pages (src, dst) in every plane of a pool laid out [planes, pages, page bytes]."""
    _need(pairs, torch.int32, "pairs", 2)
    _check(_elementwise().cisr_page_copy(_p(pool), _p(pairs), pairs.shape[0], n_planes, ctypes.c_longlong(plane_bytes),
                                         ctypes.c_longlong(page_bytes), _stream()), "page_copy")


def table_update(table: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """table.view(-1)[idx[i]] = val[i] for every i with idx[i] >= 0."""
    _need(table, torch.int32, "table"); _need(idx, torch.int32, "idx", 1); _need(val, torch.int32, "val", 1)
    _check(_elementwise().cisr_table_update(_p(table), _p(idx), _p(val), idx.numel(), _stream()), "table_update")


# ------------------------------------------------------------------ attention (one library per head size and storage)
_attention_libs = {}
TENSOR_CORE_MAX_HEAD_DIM = 128


def _attention_source(head_dim: int, dtype: torch.dtype, kind: str):
    """bfloat16 heads up to 128 wide run on the tensor cores; float, and wider heads, on the CUDA cores."""
    if kind not in ("auto", "simt"):
        raise KernelError(f"unknown attention kernel kind {kind!r}")
    if kind == "auto" and dtype == torch.bfloat16 and head_dim <= TENSOR_CORE_MAX_HEAD_DIM:
        return "attention_mma.cu", {"HEAD_DIM": head_dim}
    return "attention.cu", {"HEAD_DIM": head_dim, "STORAGE_BF16": dtype_code(dtype)}


def attention_library(head_dim: int, dtype: torch.dtype, kind: str = "auto"):
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 from 16 to 256, not {head_dim}")
    source, defines = _attention_source(head_dim, dtype, kind)
    key = (source, head_dim, dtype)
    lib = _attention_libs.get(key)
    if lib is None:
        lib = load_library(source, defines)
        for name in ("cisr_attn_prefill", "cisr_attn_decode", "cisr_attn_head_dim", "cisr_attn_prefill_tile"):
            getattr(lib, name).restype = ctypes.c_int
        assert lib.cisr_attn_head_dim() == head_dim
        lib._tensor_core = source == "attention_mma.cu"
        lib._tensor_maps = False
        if lib._tensor_core:
            lib.cisr_attn_set_pdl(int(_pdl_state["on"]))
            lib.cisr_attn_decode_tma_ok.restype = ctypes.c_int
            if head_dim % 64 == 0:          # the variant whose tiles arrive by tensor-map copies
                lib.cisr_attn_tma_init.restype = ctypes.c_int
                lib.cisr_attn_decode_tma.restype = ctypes.c_int
                lib.cisr_attn_decode_tma_launches.restype = ctypes.c_int
                lib.cisr_attn_set_clusters(int(_cluster_state["on"]))
                _check(lib.cisr_attn_tma_init(_p(_error_flag())), "attention tensor-map init", own=0)
                lib._tensor_maps = True
        _attention_libs[key] = lib
    return lib


_error_state = {}
_cluster_state = {"on": os.environ.get("CISR_CLUSTERS", "0") not in ("", "0")}


def set_clusters(on: bool) -> None:
    """Whether the decode attention merges the key ranges of a request inside thread-block clusters, or writes every
    range's partial sum for the merge kernel (the default: inside a chain of kernels that start early, clusters of 16
    did not all become resident at once and the step was slower; CISR_CLUSTERS=1 in the environment turns them on)."""
    _cluster_state["on"] = bool(on)
    for lib in _attention_libs.values():
        if lib._tensor_maps:
            lib.cisr_attn_set_clusters(int(on))


def _error_flag() -> torch.Tensor:
    """One int on the device that a kernel sets when one of its bounded waits ran out."""
    flag = _error_state.get("flag")
    if flag is None:
        flag = _error_state["flag"] = torch.zeros(1, dtype=torch.int32, device="cuda")
    return flag


def attention_jobs(head_dim: int, dtype: torch.dtype):
    """The build job of the attention library for this head size and storage type."""
    source, defines = _attention_source(head_dim, dtype, "auto")
    return (source, defines, ())


def attention_tcgen05_jobs(head_dim: int, dtype: torch.dtype):
    """The build jobs of the tcgen05 prompt attention, where this head size and storage type have one."""
    if dtype == torch.bfloat16 and head_dim in TCGEN05_HEAD_DIMS:
        return [("attention_tcgen05.cu", {"HEAD_DIM": head_dim}, ())]
    return []


TCGEN05_HEAD_DIMS = (64, 128)
WIDE_TILE = 128                  # queries per tile of the tcgen05 prompt attention
_attention_tcgen05_libs = {}


def _attention_tcgen05(head_dim: int):
    lib = _attention_tcgen05_libs.get(head_dim)
    if lib is None:
        lib = load_library("attention_tcgen05.cu", {"HEAD_DIM": head_dim})
        for name in ("cisr_attn_prefill_tcgen05", "cisr_attn_tcgen05_init", "cisr_attn_tcgen05_ok", "cisr_attn_tcgen05_tile"):
            getattr(lib, name).restype = ctypes.c_int
        assert lib.cisr_attn_tcgen05_tile() == WIDE_TILE
        _check(lib.cisr_attn_tcgen05_init(_p(_error_flag())), "tcgen05 attention init", own=0)
        lib.cisr_attn_tcgen05_set_pdl(int(_pdl_state["on"]))
        _attention_tcgen05_libs[head_dim] = lib
    return lib


def attn_prefill_wide_ok(q: torch.Tensor, k_cache: torch.Tensor, page_size: int) -> bool:
    """Whether the tcgen05 prompt attention takes these tensors: bfloat16, head size 64 or 128, a page size that is a
    multiple of 8 and divides 128 or is a multiple of it, 16-byte aligned contiguous buffers."""
    dim = k_cache.shape[-1]
    return (k_cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 and dim in TCGEN05_HEAD_DIMS
            and page_size % 8 == 0 and (128 % page_size == 0 or page_size % 128 == 0)
            and k_cache.is_contiguous() and q.is_contiguous() and q.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0
            and k_cache.shape[0] * k_cache.shape[1] * page_size < 2 ** 31)


def _sink(sink, hq: Optional[int] = None) -> tuple:
    """A softmax sink as the kernels take it: one more term exp(sink) in the denominator that carries no value.  None:
    none; a number: the same for every query head; a float tensor [hq]: one per query head.  Returns the two arguments
    (the number, -inf where there is none; the per-head array or null)."""
    if isinstance(sink, torch.Tensor):
        _need(sink, torch.float32, "sink", 1)
        if hq is not None and sink.numel() != hq:
            raise KernelError("a per-head sink needs one number per query head")
        return ctypes.c_float(float("-inf")), _p(sink)
    return ctypes.c_float(float("-inf") if sink is None else float(sink)), _p(None)


def attn_prefill_wide(q, out, k_cache, v_cache, req_slot, block_table, wide_req, wide_q0, q_start, q_len, ctx_len, hq, hkv,
                      page_size, scale, window, sink=None, keep_first: int = 0) -> None:
    """Attention of portions on tcgen05: q, out [tokens, hq, D]; tiles of 128 queries as (request, first query).
    `sink`: see `_sink`.  `keep_first`: the sequence's first keys that stay in sight behind a window."""
    dim = k_cache.shape[-1]
    _need(q, torch.bfloat16, "q", 3); _need(out, torch.bfloat16, "out", 3); _need(k_cache, torch.bfloat16, "k_cache", 4)
    _need(v_cache, torch.bfloat16, "v_cache", 4)
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("wide_req", wide_req), ("wide_q0", wide_q0),
                    ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if not attn_prefill_wide_ok(q, k_cache, page_size):
        raise KernelError("attn_prefill_wide: not a head size, page size or buffer for the tcgen05 attention")
    lib = _attention_tcgen05(dim)
    _check(lib.cisr_attn_prefill_tcgen05(_p(q), _p(out), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(req_slot),
                                         _p(block_table), block_table.shape[1], _p(wide_req), _p(wide_q0), wide_req.numel(),
                                         _p(q_start), _p(q_len), _p(ctx_len), hq, hkv, page_size, ctypes.c_float(scale),
                                         int(window or 0), int(keep_first or 0), *_sink(sink, hq), _stream()), "attn_prefill_wide")


PREFILL_TILE = 64


def attn_prefill(q, out, k_cache, v_cache, req_slot, block_table, tile_req, tile_q0, q_start, q_len, ctx_len, hq, hkv,
                 page_size, scale, window, kind: str = "auto", sink=None, keep_first: int = 0) -> None:
    """Attention of portions: q, out [tokens, hq, D]; tiles list (request, first query of the tile).  Query i sees key
    j <= i when window is None or i - j < window or j < keep_first."""
    dim = k_cache.shape[-1]
    _need(q, k_cache.dtype, "q"); _need(out, k_cache.dtype, "out"); _need(k_cache, None, "k_cache", 4)
    _need(v_cache, k_cache.dtype, "v_cache", 4)
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("tile_req", tile_req), ("tile_q0", tile_q0), ("q_start", q_start),
                    ("q_len", q_len), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    lib = attention_library(dim, k_cache.dtype, kind)
    _check(lib.cisr_attn_prefill(_p(q), _p(out), _p(k_cache), _p(v_cache), _p(req_slot), _p(block_table), block_table.shape[1],
                                 _p(tile_req), _p(tile_q0), tile_req.numel(), _p(q_start), _p(q_len), _p(ctx_len),
                                 hq, hkv, page_size, ctypes.c_float(scale), int(window or 0), int(keep_first or 0), *_sink(sink, hq),
                                 _stream()), "attn_prefill")


def attn_decode(q, out, k_cache, v_cache, req_slot, block_table, dec_req, n_dec, q_start, ctx_len, partial, stats, hq, hkv,
                page_size, scale, window, split_size, n_splits, kind: str = "auto", staging: str = "auto", merge: bool = True,
                sink=None, keep_first: int = 0) -> None:
    """Attention of single new tokens, split over key ranges of `split_size`, merged into out.  `keep_first`: the
    sequence's first keys that stay in sight behind a window.

    `merge=False` (tensor-core kernels only) leaves the ranges' partial sums in `partial` and `stats` and does not write
    `out`: the caller merges them itself (`merge_out_proj`).

    `staging` picks how the tensor-core kernel brings key and value tiles in: "tensor_map" (one bulk copy per
    page), "gather" (a 16-byte copy per thread), or "auto": tensor maps where the head size (a multiple of 64), the
    page size (a multiple of 8 that divides 64 or is a multiple of it) and the range size allow them."""
    dim = k_cache.shape[-1]
    _need(q, k_cache.dtype, "q"); _need(out, k_cache.dtype, "out"); _need(k_cache, None, "k_cache", 4)
    _need(v_cache, k_cache.dtype, "v_cache", 4); _need(partial, torch.float32, "partial"); _need(stats, torch.float32, "stats")
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("dec_req", dec_req), ("q_start", q_start), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if partial.numel() < n_dec * hq * n_splits * dim or stats.numel() < n_dec * hq * n_splits * 2:
        raise KernelError("attn_decode: scratch for partial sums is too small")
    lib = attention_library(dim, k_cache.dtype, kind)
    tail = [_p(req_slot), _p(block_table), block_table.shape[1], _p(dec_req), n_dec, _p(q_start), _p(ctx_len), _p(partial),
            _p(stats), hq, hkv, page_size, ctypes.c_float(scale), int(window or 0), int(keep_first or 0), split_size, n_splits]
    if lib._tensor_core:
        tail.append(int(merge))
    elif not merge:
        raise KernelError("attn_decode: only the tensor-core kernels leave the merge to the caller")
    if sink is not None and not merge:
        raise KernelError("attn_decode: the sink is added by the merge kernel; a caller that merges itself cannot ask for one")
    tail.extend(_sink(sink, hq))
    tail.append(_stream())
    if staging not in ("auto", "tensor_map", "gather"):
        raise KernelError(f"unknown staging {staging!r}")
    tensor_maps = (lib._tensor_maps and lib.cisr_attn_decode_tma_ok(page_size, split_size) and k_cache.is_contiguous()
                   and v_cache.is_contiguous() and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0
                   and k_cache.shape[0] * hkv * page_size < 2 ** 31)
    if staging == "tensor_map" and not tensor_maps:
        raise KernelError("attn_decode: tensor-map staging does not take this head size, page size, range size or cache")
    if tensor_maps and staging != "gather":
        status = lib.cisr_attn_decode_tma(_p(q), _p(out), _p(k_cache), _p(v_cache), k_cache.shape[0], *tail)
        _check(status, "attn_decode", own=lib.cisr_attn_decode_tma_launches() if status == 0 else 0)
    else:
        _check(lib.cisr_attn_decode(_p(q), _p(out), _p(k_cache), _p(v_cache), *tail), "attn_decode",
               own=-(-(hq // hkv) // 16) + (1 if merge else 0))


# ------------------------------------------------------------------ merge of the key ranges + output projection (decode steps)
_merge_proj_state = {}


def _merge_proj():
    lib = _merge_proj_state.get("lib")
    if lib is None:
        lib = load_library("merge_proj.cu")
        lib.cisr_merge_proj.restype = ctypes.c_int
        lib.cisr_merge_proj_heads_per_cta.restype = ctypes.c_int
        lib.cisr_merge_proj_set_pdl(int(_pdl_state["on"]))
        _merge_proj_state["lib"] = lib
    return lib


def merge_proj_jobs():
    return [("merge_proj.cu", {}, ())]


MERGE_PROJ_MAX_BYTES = 8 << 20     # larger output projections are bandwidth-bound: the streaming product serves them, and the merge kernel is small beside it


def merge_out_proj_ok(n_dec: int, hq: int, dim: int, w: torch.Tensor) -> bool:
    """Whether `merge_out_proj` takes the shape: bfloat16 weights [N, hq * dim] of a latency-bound size, at most 16 tokens,
    head slices of at most 256 columns in at most 16 CTAs; and thread-block clusters in the attention kernel off."""
    return (0 < n_dec <= 16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == hq * dim and w.numel() * 2 < MERGE_PROJ_MAX_BYTES
            and not _cluster_state["on"] and os.environ.get("CISR_MERGE_PROJ", "1") != "0"
            and _merge_proj().cisr_merge_proj_heads_per_cta(n_dec, hq, dim, w.shape[1]) > 0)


def merge_out_proj(partial: torch.Tensor, stats: torch.Tensor, n_splits: int, dec_req: torch.Tensor, q_start: torch.Tensor,
                   n_dec: int, hq: int, dim: int, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[row of request i] (float [tokens, N]) = (log-sum-exp merge of request i's key ranges, rounded to bfloat16) @ w^T:
    the merge kernel and the output projection of a decode step in one launch of a thread-block cluster.  With
    `accumulate` the product is added to what `out` holds (the residual stream)."""
    _need(partial, torch.float32, "partial"); _need(stats, torch.float32, "stats"); _need(w, torch.bfloat16, "w", 2)
    _need(out, torch.float32, "out", 2); _need(dec_req, torch.int32, "dec_req", 1); _need(q_start, torch.int32, "q_start", 1)
    if partial.numel() < n_dec * hq * n_splits * dim or stats.numel() < n_dec * hq * n_splits * 2 or out.shape[1] != w.shape[0]:
        raise KernelError("merge_out_proj: shapes disagree")
    status = _merge_proj().cisr_merge_proj(_p(partial), _p(stats), n_splits, _p(dec_req), _p(q_start), n_dec, hq, dim, _p(w),
                                           w.shape[0], w.shape[1], _p(out), int(bool(accumulate)), _stream())
    _check(status, "merge_out_proj")
    return out


# ------------------------------------------------------------------ several residual streams (hyper-connections) and their norm
_hyper_state = {}
NORM_KINDS = {"layer": 0, "rms": 1}


def _hyper():
    lib = _hyper_state.get("lib")
    if lib is None:
        lib = load_library("hyper.cu")
        for name in ("cisr_hyper_mix_norm", "cisr_hyper_sum", "cisr_hyper_max_streams"):
            getattr(lib, name).restype = ctypes.c_int
        lib.cisr_hyper_set_pdl(int(_pdl_state["on"]))
        _hyper_state["lib"] = lib
    return lib


def hyper_jobs():
    return [("hyper.cu", {}, ())]


HYPER_MAX_STREAMS = 16


def hyper_mix_norm(source: torch.Tensor, streams: torch.Tensor, n_streams: int, *, y: Optional[torch.Tensor] = None,
                   bias: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None,
                   in_w: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                   norm_kind: str = "layer", h: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                   store: bool = True) -> Optional[torch.Tensor]:
    """One pass over the residual streams of every token (see csrc/hyper.cu): with `y` (float [tokens, hidden], plus the
    per-channel `bias`) the streams become x'_t = sum_s mix[s, t] x_s + out_w[t] * (y + bias); then h = norm(sum_t in_w[t]
    x'_t) * norm_w.  `source` is float [tokens, n_streams, hidden], or [tokens, hidden] read as every stream; `streams`
    [tokens, n_streams, hidden] receives x' when `store` (it may be `source`).  mix None: identity; out_w, in_w None:
    ones.  `rows` picks the tokens that become rows of h; h None: the streams only."""
    _need(source, torch.float32, "source"); _need(streams, torch.float32, "streams", 3)
    tokens, s_count, hidden = streams.shape
    if s_count != n_streams or not 1 <= n_streams <= HYPER_MAX_STREAMS:
        raise KernelError(f"hyper_mix_norm: streams must be [tokens, {n_streams}, hidden] with at most {HYPER_MAX_STREAMS} streams")
    source_is_row = source.dim() == 2
    if tuple(source.shape) not in ((tokens, hidden), (tokens, n_streams, hidden)):
        raise KernelError("hyper_mix_norm: source must be [tokens, hidden] or [tokens, streams, hidden]")
    for name, t, n in (("y", y, tokens * hidden), ("bias", bias, hidden), ("mix", mix, n_streams * n_streams),
                       ("out_w", out_w, n_streams), ("in_w", in_w, n_streams)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != n:
                raise KernelError(f"hyper_mix_norm: {name} has {t.numel()} elements, {n} are needed")
    if bias is not None and y is None:
        raise KernelError("hyper_mix_norm: a bias without an output to add it to")
    if norm_kind not in NORM_KINDS:
        raise KernelError(f"unknown norm kind {norm_kind!r}")
    n_rows = tokens
    if h is not None:
        _need(h, None, "h", 2); _need(norm_w, None, "norm_w", 1)
        if norm_w.numel() != hidden or h.shape[1] != hidden:
            raise KernelError("hyper_mix_norm: width mismatch")
        n_rows = h.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
        if h is None or rows.numel() != n_rows:
            raise KernelError("hyper_mix_norm: one row index per row of h is needed")
    elif n_rows != tokens:
        raise KernelError("hyper_mix_norm: h and the streams differ in rows")
    _check(_hyper().cisr_hyper_mix_norm(
        _p(source), int(source_is_row), _p(streams), _p(y), _p(bias), _p(mix), _p(out_w), _p(in_w), _p(norm_w),
        dtype_code(norm_w.dtype) if norm_w is not None else 0, _p(h), dtype_code(h.dtype) if h is not None else 0, _p(rows), n_rows,
        n_streams, hidden, ctypes.c_float(eps), NORM_KINDS[norm_kind], int(bool(store)), _stream()), "hyper_mix_norm")
    return h


def hyper_sum(streams: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = the sum of token t's streams."""
    _need(streams, torch.float32, "streams", 3); _need(out, torch.float32, "out", 2)
    tokens, n_streams, hidden = streams.shape
    if out.shape != (tokens, hidden):
        raise KernelError("hyper_sum: out must be [tokens, hidden]")
    _check(_hyper().cisr_hyper_sum(_p(streams), _p(out), tokens, n_streams, hidden, _stream()), "hyper_sum")
    return out


# ------------------------------------------------------------------ differential attention: row kernels around the paged attention
_diff_state = {}


def _diff():
    lib = _diff_state.get("lib")
    if lib is None:
        lib = load_library("diff_attention.cu")
        for name in ("cisr_diff_rows", "cisr_diff_rope_rows", "cisr_conv_keep", "cisr_diff_combine"):
            getattr(lib, name).restype = ctypes.c_int
        lib.cisr_diff_set_pdl(int(_pdl_state["on"]))
        _diff_state["lib"] = lib
    return lib


def diff_jobs():
    return [("diff_attention.cu", {}, ())]


def diff_rows(proj: torch.Tensor, conv_w: torch.Tensor, taps: int, state: torch.Tensor, *, token_req, req_slot, q_start, positions,
              q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], block_table, page_size: int,
              hq: int, hkv: int, key_dim: int, value_dim: int) -> None:
    """Per token of a step: the causal convolution over time (taps weights per channel, tap by tap: conv_w float [taps,
    channels], the last row the current token's; inputs before the portion from `state` [slots, taps - 1, channels], zeros before the
    sequence) of the first columns of proj (float [tokens, cols]: q [hq * 2 * key_dim], then, when caches are given, k
    [hkv * 2 * key_dim] and v [hkv * value_dim]); the two maps of head h become query rows 2 h and 2 h + 1 of q_out
    [tokens, 2 hq, D] (map m at columns [m * key_dim, (m + 1) * key_dim), zeros elsewhere), a key row [k1 | k2 | 0] and a
    value row [v | 0] go into the token's place in the pages [pages, hkv, page, D]."""
    _need(proj, torch.float32, "proj", 2); _need(conv_w, torch.float32, "conv_w", 2); _need(state, torch.float32, "state")
    _need(q_out, None, "q_out", 3)
    tokens, width = q_out.shape[0], q_out.shape[2]
    write = k_cache is not None
    channels = hq * 2 * key_dim + ((hkv * 2 * key_dim + hkv * value_dim) if write else 0)
    if (proj.shape[0] != tokens or proj.shape[1] < channels or tuple(conv_w.shape) != (taps, channels) or q_out.shape[1] != 2 * hq
            or state[0].numel() != max(taps - 1, 0) * channels and taps > 1):
        raise KernelError("diff_rows: shapes disagree")
    if write:
        _need(k_cache, q_out.dtype, "k_cache", 4); _need(v_cache, q_out.dtype, "v_cache", 4)
        if k_cache.shape[1:] != (hkv, page_size, width) or v_cache.shape != k_cache.shape:
            raise KernelError("diff_rows: the cache is not [pages, kv_heads, page, D]")
    for name, t in (("token_req", token_req), ("req_slot", req_slot), ("q_start", q_start), ("positions", positions), ("block_table", block_table)):
        _need(t, torch.int32, name)
    _check(_diff().cisr_diff_rows(_p(proj), proj.shape[1], _p(conv_w), taps, _p(state), ctypes.c_longlong(state[0].numel()),
                                  _p(token_req), _p(req_slot), _p(q_start), _p(positions), _p(q_out), _p(k_cache), _p(v_cache),
                                  dtype_code(q_out.dtype), _p(block_table), block_table.shape[1], page_size, tokens, hq, hkv, key_dim,
                                  value_dim, width, int(write), _stream()), "diff_rows")


def diff_rope_rows(proj: torch.Tensor, k_col: int, v_col: int, *, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_half: int,
                   interleaved: bool, token_req, req_slot, positions, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                   v_cache: Optional[torch.Tensor], block_table, page_size: int, hq: int, hkv: int, key_dim: int, value_dim: int) -> None:
    """Per token of a step, without a convolution: the first 2 * rot_half coordinates of each map of q and k turn by the
    step's rotary tables (cos, sin float [tokens, rot_half]; rot_half 0: nothing turns).  proj float [tokens, cols] holds q
    [hq * 2 * key_dim] from column 0 and, when caches are given, k [hkv * 2 * key_dim] from `k_col` and v [hkv * value_dim]
    from `v_col`.  Rows are laid out as `diff_rows` lays them out: query rows 2 h and 2 h + 1 of q_out [tokens, 2 hq, D],
    a key row [k1 | k2 | 0] and a value row [v | 0] in the token's place in the pages [pages, hkv, page, D]."""
    _need(proj, torch.float32, "proj", 2); _need(q_out, None, "q_out", 3)
    tokens, width = q_out.shape[0], q_out.shape[2]
    write = k_cache is not None
    if rot_half:
        _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
        if cos.shape != (tokens, rot_half) or sin.shape != cos.shape:
            raise KernelError("diff_rope_rows: rotary tables must be [tokens, rot_half]")
    if (proj.shape[0] != tokens or q_out.shape[1] != 2 * hq or proj.shape[1] < hq * 2 * key_dim
            or (write and (k_col + hkv * 2 * key_dim > proj.shape[1] or v_col + hkv * value_dim > proj.shape[1]))):
        raise KernelError("diff_rope_rows: shapes disagree")
    if write:
        _need(k_cache, q_out.dtype, "k_cache", 4); _need(v_cache, q_out.dtype, "v_cache", 4)
        if k_cache.shape[1:] != (hkv, page_size, width) or v_cache.shape != k_cache.shape:
            raise KernelError("diff_rope_rows: the cache is not [pages, kv_heads, page, D]")
    for name, t in (("token_req", token_req), ("req_slot", req_slot), ("positions", positions), ("block_table", block_table)):
        _need(t, torch.int32, name)
    _check(_diff().cisr_diff_rope_rows(_p(proj), proj.shape[1], k_col, v_col, _p(cos if rot_half else None), _p(sin if rot_half else None),
                                       rot_half, int(interleaved), _p(token_req), _p(req_slot), _p(positions), _p(q_out), _p(k_cache),
                                       _p(v_cache), dtype_code(q_out.dtype), _p(block_table), block_table.shape[1], page_size, tokens, hq,
                                       hkv, key_dim, value_dim, width, int(write), _stream()), "diff_rope_rows")


def conv_keep(proj: torch.Tensor, state: torch.Tensor, req_slot, q_start, q_len, n_req: int, taps: int, channels: int) -> None:
    """Per request of a step: the last taps - 1 rows of its portion's first `channels` columns of proj (older ones from
    what was kept before, where the portion is shorter) become its kept inputs, state [slots, taps - 1, channels]."""
    if taps <= 1:
        return
    _need(proj, torch.float32, "proj", 2); _need(state, torch.float32, "state")
    _check(_diff().cisr_conv_keep(_p(proj), proj.shape[1], _p(state), ctypes.c_longlong(state[0].numel()), _p(req_slot), _p(q_start),
                                  _p(q_len), n_req, taps, channels, _stream()), "conv_keep")


def diff_combine(mixed: torch.Tensor, gate: Optional[torch.Tensor], gate_col: int, out: torch.Tensor, hq: int, value_dim: int, lam: float,
                 eps: float, out_scale: float) -> torch.Tensor:
    """Per (token, head): o = a1 - lam * a2 from rows 2 h and 2 h + 1 of mixed [tokens, 2 hq, D] (their first value_dim
    columns), o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate), the gate's logits being columns gate_col + h *
    value_dim of the float tensor `gate` (None: no gate); out [tokens, hq * value_dim] in mixed's type."""
    _need(mixed, None, "mixed", 3); _need(out, mixed.dtype, "out", 2)
    tokens, _, width = mixed.shape
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
    if (mixed.shape[1] != 2 * hq or out.shape != (tokens, hq * value_dim)
            or (gate is not None and (gate.shape[0] != tokens or gate.shape[1] < gate_col + hq * value_dim))):
        raise KernelError("diff_combine: shapes disagree")
    _check(_diff().cisr_diff_combine(_p(mixed), _p(gate), gate.shape[1] if gate is not None else 0, gate_col, _p(out), dtype_code(mixed.dtype), tokens, hq, value_dim,
                                     width, ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(out_scale), _stream()), "diff_combine")
    return out


# ------------------------------------------------------------------ depth-weighted average of the residual stream
_depth_state = {}


def _depth():
    lib = _depth_state.get("lib")
    if lib is None:
        lib = load_library("depth.cu")
        lib.cisr_depth_mix_norm.restype = ctypes.c_int
        lib.cisr_depth_set_pdl(int(_pdl_state["on"]))
        _depth_state["lib"] = lib
    return lib


def depth_jobs():
    return [("depth.cu", {}, ())]


def depth_mix_norm(hist: torch.Tensor, x: torch.Tensor, pending: Optional[torch.Tensor], w: torch.Tensor, n_new: int, *,
                   norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, h: Optional[torch.Tensor] = None,
                   mixed_out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None, store: bool = True):
    """The seam between two layers (csrc/depth.cu): entry n_new of hist (float [entries, tokens, hidden]) becomes x +
    pending, x becomes sum_(j <= n_new) w[j] * hist[j], and h = rmsnorm(x) * norm_w.  `rows` picks tokens (nothing is
    stored then); `mixed_out` also receives the sum."""
    _need(hist, torch.float32, "hist", 3); _need(x, torch.float32, "x", 2); _need(w, torch.float32, "w", 1)
    entries, tokens, hidden = hist.shape
    if x.shape != (tokens, hidden) or not 1 <= n_new < entries or w.numel() != n_new + 1:
        raise KernelError("depth_mix_norm: shapes disagree")
    if pending is not None:
        _need(pending, torch.float32, "pending", 2)
        if pending.shape != x.shape:
            raise KernelError("depth_mix_norm: pending and x differ in shape")
    n_rows = tokens if rows is None else rows.numel()
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
        store = False
    if h is not None:
        _need(h, None, "h", 2); _need(norm_w, torch.float32, "norm_w", 1)
        if h.shape != (n_rows, hidden) or norm_w.numel() != hidden:
            raise KernelError("depth_mix_norm: h or norm_w has the wrong shape")
    if mixed_out is not None:
        _need(mixed_out, torch.float32, "mixed_out", 2)
    _check(_depth().cisr_depth_mix_norm(_p(hist), ctypes.c_longlong(tokens * hidden), _p(x), _p(pending), _p(w), n_new,
                                        _p(norm_w if h is not None else None), ctypes.c_float(eps), _p(h),
                                        dtype_code(h.dtype) if h is not None else 0, _p(mixed_out), _p(rows), n_rows, hidden,
                                        int(bool(store)), _stream()), "depth_mix_norm")
    return h


# ------------------------------------------------------------------ feed-forward row kernels (whole-row and gated activations)
_ffn_rows_state = {}


def _ffn_rows():
    lib = _ffn_rows_state.get("lib")
    if lib is None:
        lib = load_library("ffn_rows.cu")
        lib.cisr_polynorm.restype = ctypes.c_int
        lib.cisr_gated_clamp.restype = ctypes.c_int
        lib.cisr_ffn_rows_set_pdl(int(_pdl_state["on"]))
        _ffn_rows_state["lib"] = lib
    return lib


def ffn_rows_jobs():
    return [("ffn_rows.cu", {}, ())]


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[t] = a N(z_t) + b N(z_t^2) + c N(z_t^3) + e, N(u) = u / sqrt(mean(u^2) + eps) over the row, coef = (a, b, c, e)
    float; z float [tokens, ff]; out [tokens, >= ff] (further columns zero)."""
    _need(z, torch.float32, "z", 2); _need(coef, torch.float32, "coef", 1); _need(out, None, "out", 2)
    if coef.numel() != 4 or out.shape[0] != z.shape[0] or out.shape[1] < z.shape[1]:
        raise KernelError("polynorm: shapes disagree")
    _check(_ffn_rows().cisr_polynorm(_p(z), z.shape[1], _p(coef), ctypes.c_float(eps), _p(out), dtype_code(out.dtype), z.shape[0],
                                     z.shape[1], out.shape[1], _stream()), "polynorm")
    return out


GATE_ALPHA = 1.702


def gated_clamp(gate_up: torch.Tensor, ff: int, limit: float, out: torch.Tensor, scale_col: int = -1) -> torch.Tensor:
    """out[t, f] = g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit), g and u columns f
    and ff + f of the float rows of gate_up; with scale_col the row is also multiplied by sigmoid(gate_up[t, scale_col]).
    out [rows, >= ff] (further columns zero)."""
    _need(gate_up, torch.float32, "gate_up", 2); _need(out, None, "out", 2)
    if gate_up.shape[1] < 2 * ff or out.shape[0] != gate_up.shape[0] or out.shape[1] < ff or scale_col >= gate_up.shape[1]:
        raise KernelError("gated_clamp: shapes disagree")
    _check(_ffn_rows().cisr_gated_clamp(_p(gate_up), gate_up.shape[1], ff, ctypes.c_float(limit), ctypes.c_float(GATE_ALPHA), scale_col,
                                        _p(out), dtype_code(out.dtype), out.shape[0], out.shape[1], _stream()), "gated_clamp")
    return out


# ------------------------------------------------------------------ the rows of a stacked q | k | v projection
_rows_state = {}


def _attention_rows():
    lib = _rows_state.get("lib")
    if lib is None:
        lib = load_library("attention_rows.cu")
        lib.cisr_attention_rows.restype = ctypes.c_int
        lib.cisr_bias_add.restype = ctypes.c_int
        lib.cisr_attention_rows_set_pdl(int(_pdl_state["on"]))
        _rows_state["lib"] = lib
    return lib


def attention_rows_jobs():
    return [("attention_rows.cu", {}, ())]


def attention_rows(proj: torch.Tensor, k_col: int, v_col: int, *, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor],
                   k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_half: int,
                   interleaved: bool, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, token_req: torch.Tensor,
                   positions: torch.Tensor, req_slot: torch.Tensor, block_table: torch.Tensor, page_size: int, hq: int, hkv: int,
                   key_dim: int, value_dim: int) -> None:
    """proj float [tokens, cols] holds q at column 0, k at `k_col`, v at `v_col` (`v_col` < 0: the values are the keys as
    projected).  Adds `bias` (float [cols]), norms q and k over their whole projection (`q_norm`, `k_norm`: float weights of
    that size, or None), rotates, pads the heads to the cache's width D, writes q_out [tokens, hq, D] and the key and value
    rows into their pages ([pages, hkv, page_size, D]).  See csrc/attention_rows.cu."""
    _need(proj, torch.float32, "proj", 2); _need(q_out, None, "q_out", 3); _need(k_cache, q_out.dtype, "k_cache", 4)
    _need(v_cache, q_out.dtype, "v_cache", 4)
    tokens, cols = proj.shape
    width = k_cache.shape[-1]
    if tuple(q_out.shape) != (tokens, hq, width) or tuple(k_cache.shape[1:]) != (hkv, page_size, width) or v_cache.shape != k_cache.shape:
        raise KernelError("attention_rows: q_out must be [tokens, hq, D] and the caches [pages, hkv, page_size, D]")
    for name, t, n in (("bias", bias, cols), ("q_norm", q_norm, hq * key_dim), ("k_norm", k_norm, hkv * key_dim)):
        if t is not None:
            _need(t, torch.float32, name, 1)
            if t.numel() != n:
                raise KernelError(f"attention_rows: {name} has {t.numel()} elements, {n} are needed")
    if rot_half:
        _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
        if cos.shape != (tokens, rot_half) or sin.shape != cos.shape:
            raise KernelError("attention_rows: rotary tables must be [tokens, rot_half]")
    for name, t in (("token_req", token_req), ("positions", positions), ("req_slot", req_slot), ("block_table", block_table)):
        _need(t, torch.int32, name)
    _check(_attention_rows().cisr_attention_rows(
        _p(proj), cols, k_col, v_col, _p(bias), _p(q_norm), _p(k_norm), ctypes.c_float(eps), _p(cos if rot_half else None),
        _p(sin if rot_half else None), rot_half, int(interleaved), _p(q_out), dtype_code(q_out.dtype), _p(k_cache), _p(v_cache),
        dtype_code(k_cache.dtype), _p(token_req), _p(positions), _p(req_slot), _p(block_table), block_table.shape[1], page_size,
        hq, hkv, key_dim, value_dim, width, tokens, _stream()), "attention_rows")


def bias_add(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[t, :] += bias, in place (float)."""
    _need(out, torch.float32, "out", 2); _need(bias, torch.float32, "bias", 1)
    if bias.numel() != out.shape[1]:
        raise KernelError("bias_add: one bias per column is needed")
    _check(_attention_rows().cisr_bias_add(_p(out), _p(bias), out.shape[0], out.shape[1], _stream()), "bias_add")
    return out


# ------------------------------------------------------------------ the gated delta rule
_delta_state = {}
DELTA_MAX_KEY_DIM = 256
DELTA_CHUNK = 64                                       # tokens per chunk of the chunked recurrence
DELTA_CHUNK_TABLE = 2 * DELTA_CHUNK * DELTA_CHUNK + DELTA_CHUNK   # floats of scratch per (chunk, head)


def _delta():
    lib = _delta_state.get("lib")
    if lib is None:
        lib = load_library("delta.cu")
        for name in ("cisr_delta_prepare", "cisr_delta_keep", "cisr_delta_recurrence", "cisr_delta_output", "cisr_delta_max_key_dim",
                     "cisr_delta_chunks", "cisr_delta_chunk_tokens"):
            getattr(lib, name).restype = ctypes.c_int
        lib.cisr_delta_chunk_table_floats.restype = ctypes.c_longlong
        assert lib.cisr_delta_max_key_dim() == DELTA_MAX_KEY_DIM and lib.cisr_delta_chunk_tokens() == DELTA_CHUNK
        assert lib.cisr_delta_chunk_table_floats() == DELTA_CHUNK_TABLE
        lib.cisr_delta_set_pdl(int(_pdl_state["on"]))
        _delta_state["lib"] = lib
    return lib


def delta_jobs():
    return [("delta.cu", {}, ())]


def delta_prepare(proj, conv_w, taps, state, a_log, dt_bias, token_req, req_slot, q_start, qkv, beta, decay, heads, kv_heads,
                  key_dim, value_dim, norm_eps) -> None:
    """Convolution over time with the request's kept inputs, silu, unit norms of q and k, beta and the decay, per token."""
    _check(_delta().cisr_delta_prepare(_p(proj), proj.shape[1], _p(conv_w), taps, _p(state), ctypes.c_longlong(state.shape[1]),
                                       ctypes.c_longlong(heads * key_dim * value_dim), _p(a_log), _p(dt_bias), _p(token_req),
                                       _p(req_slot), _p(q_start), _p(qkv), _p(beta), _p(decay), heads, kv_heads, key_dim, value_dim,
                                       ctypes.c_float(norm_eps), proj.shape[0], _stream()), "delta_prepare")


def delta_keep(proj, state, req_slot, q_start, q_len, n_req, taps, channels, matrix) -> None:
    """The last taps - 1 convolution inputs of every request of the step become its kept inputs."""
    _check(_delta().cisr_delta_keep(_p(proj), proj.shape[1], _p(state), ctypes.c_longlong(state.shape[1]), ctypes.c_longlong(matrix),
                                    _p(req_slot), _p(q_start), _p(q_len), taps, channels, n_req, _stream()), "delta_keep")


def delta_chunks(qkv, beta, decay, chunk_req, chunk_t0, n_chunks, req_chunk0, state, req_slot, q_start, q_len, o, n_req, heads, kv_heads,
                 key_dim, value_dim, least) -> None:
    """The recurrence for the requests that bring at least `least` tokens, a chunk of DELTA_CHUNK tokens at a time: two
    launches (the chunks' tables, all at once; then the walk from chunk to chunk).  chunk_req, chunk_t0: per chunk its
    request and its first token inside the portion; req_chunk0: per request the index of its first chunk."""
    for name, t in (("chunk_req", chunk_req), ("chunk_t0", chunk_t0), ("req_chunk0", req_chunk0)):
        _need(t, torch.int32, name, 1)
    if chunk_req.numel() < n_chunks or chunk_t0.numel() < n_chunks or req_chunk0.numel() < n_req:
        raise KernelError("delta_chunks: the chunk lists are too short")
    tables = torch.empty((n_chunks, heads, DELTA_CHUNK_TABLE), dtype=torch.float32, device=qkv.device)
    _check(_delta().cisr_delta_chunks(_p(qkv), _p(beta), _p(decay), _p(chunk_req), _p(chunk_t0), n_chunks, _p(req_chunk0), _p(tables),
                                      _p(state), ctypes.c_longlong(state.shape[1]), _p(req_slot), _p(q_start), _p(q_len), _p(o), heads,
                                      kv_heads, key_dim, value_dim, n_req, int(least), _stream()), "delta_chunks", own=2)


def delta_recurrence(qkv, beta, decay, state, req_slot, q_start, q_len, o, n_req, heads, kv_heads, key_dim, value_dim, lanes=0, below=0) -> None:
    """The state's walk over each request's tokens, in order; o [tokens, heads, value_dim] float.  `lanes`: how many lanes
    share a column of the state (4, 8, 16 or 32); 0: chosen by the size of the launch.  `below` > 0: only the requests that
    bring fewer tokens than that (the others are `delta_chunks`')."""
    _check(_delta().cisr_delta_recurrence(_p(qkv), _p(beta), _p(decay), _p(state), ctypes.c_longlong(state.shape[1]), _p(req_slot),
                                          _p(q_start), _p(q_len), _p(o), heads, kv_heads, key_dim, value_dim, n_req, int(lanes), int(below),
                                          _stream()), "delta_recurrence")


def delta_output(o, proj, gate_col, norm_w, eps, out, heads, value_dim) -> None:
    """out = o / rms(o) * norm_w * silu(gate) per head, rounded to out's type."""
    _check(_delta().cisr_delta_output(_p(o), _p(proj), proj.shape[1], gate_col, _p(norm_w), ctypes.c_float(eps), _p(out),
                                      dtype_code(out.dtype), out.shape[1], heads, value_dim, o.shape[0], _stream()), "delta_output")


def delta_step(proj: torch.Tensor, conv_w: torch.Tensor, taps: int, state: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               norm_w: torch.Tensor, eps: float, norm_eps: float, token_req: torch.Tensor, req_slot: torch.Tensor, q_start: torch.Tensor,
               q_len: torch.Tensor, n_req: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, out: torch.Tensor,
               lanes: int = 0, chunks=None) -> torch.Tensor:
    """The gated delta rule for a step's tokens (see csrc/delta.cu).  proj float [tokens, cols]: the stacked projection
    q | k | v | gate | b | a (cols may be padded beyond them); conv_w float [2 * kv_heads * key_dim + heads * value_dim, taps];
    state float [slots, heads * key_dim * value_dim + (taps - 1) * conv channels] is read and advanced for the step's
    requests; out [tokens, >= heads * value_dim] in the operand type of the output projection.  `chunks`: None (every request
    token by token) or (chunk_req, chunk_t0, req_chunk0, n_chunks, n_short, least): the requests with at least `least` tokens
    run chunk by chunk, the `n_short` others token by token."""
    _need(proj, torch.float32, "proj", 2); _need(conv_w, torch.float32, "conv_w", 2); _need(state, torch.float32, "state", 2)
    for name, t in (("a_log", a_log), ("dt_bias", dt_bias), ("norm_w", norm_w)):
        _need(t, torch.float32, name, 1)
    for name, t in (("token_req", token_req), ("req_slot", req_slot), ("q_start", q_start), ("q_len", q_len)):
        _need(t, torch.int32, name, 1)
    _need(out, None, "out", 2)
    tokens, cols = proj.shape
    channels = 2 * kv_heads * key_dim + heads * value_dim
    matrix = heads * key_dim * value_dim
    if (tuple(conv_w.shape) != (channels, taps) or state.shape[1] != matrix + (taps - 1) * channels or a_log.numel() != heads
            or dt_bias.numel() != heads or norm_w.numel() != value_dim or out.shape[0] != tokens or out.shape[1] < heads * value_dim
            or cols < channels + heads * value_dim + 2 * heads or key_dim > DELTA_MAX_KEY_DIM):
        raise KernelError("delta_step: shapes disagree")
    device = proj.device
    qkv = torch.empty((tokens, channels), dtype=torch.float32, device=device)
    beta = torch.empty((tokens, heads), dtype=torch.float32, device=device)
    decay = torch.empty((tokens, heads), dtype=torch.float32, device=device)
    o = torch.empty((tokens, heads, value_dim), dtype=torch.float32, device=device)
    delta_prepare(proj, conv_w, taps, state, a_log, dt_bias, token_req, req_slot, q_start, qkv, beta, decay, heads, kv_heads, key_dim,
                  value_dim, norm_eps)
    if taps > 1:
        delta_keep(proj, state, req_slot, q_start, q_len, n_req, taps, channels, matrix)
    if chunks is not None and chunks[3] > 0:
        chunk_req, chunk_t0, req_chunk0, n_chunks, n_short, least = chunks
        delta_chunks(qkv, beta, decay, chunk_req, chunk_t0, n_chunks, req_chunk0, state, req_slot, q_start, q_len, o, n_req, heads,
                     kv_heads, key_dim, value_dim, least)
        if n_short:
            delta_recurrence(qkv, beta, decay, state, req_slot, q_start, q_len, o, n_req, heads, kv_heads, key_dim, value_dim, lanes, least)
    else:
        delta_recurrence(qkv, beta, decay, state, req_slot, q_start, q_len, o, n_req, heads, kv_heads, key_dim, value_dim, lanes)
    delta_output(o, proj, channels, norm_w, eps, out, heads, value_dim)
    return out


# ------------------------------------------------------------------ lightning attention (linear attention with a fixed decay per head)
_lightning_state = {}
LIGHTNING_MAX_KEY_DIM = 256
LIGHTNING_CHUNK = 64             # tokens per chunk of the chunked recurrence; portions of at least this many tokens run chunk by chunk


def _lightning():
    lib = _lightning_state.get("lib")
    if lib is None:
        lib = load_library("lightning.cu")
        for name in ("cisr_lightning_recurrence", "cisr_lightning_output", "cisr_lightning_chunk_tokens", "cisr_lightning_max_key_dim"):
            getattr(lib, name).restype = ctypes.c_int
        assert lib.cisr_lightning_chunk_tokens() == LIGHTNING_CHUNK and lib.cisr_lightning_max_key_dim() == LIGHTNING_MAX_KEY_DIM
        lib.cisr_lightning_set_pdl(int(_pdl_state["on"]))
        _lightning_state["lib"] = lib
    return lib


def lightning_jobs():
    return [("lightning.cu", {}, ())]


def lightning_recurrence(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
                         req_slot: torch.Tensor, q_start: torch.Tensor, q_len: torch.Tensor, n_req: int, o: torch.Tensor, heads: int,
                         key_dim: int, value_dim: int, least: int = 0, n_short: int = 0, chunks=None, columns_per_cta: int = 0) -> torch.Tensor:
    """Per head S <- decay S + silu(k) silu(v)^T, o = S^T silu(q) over each request's tokens in order.  proj float
    [tokens, columns] holds the projections' sums (q and k: heads x key_dim from `q_col` / `k_col`; v: heads x value_dim
    from `v_col`); state float [slots, heads * value_dim * key_dim] is read and advanced; o float [tokens, heads *
    value_dim].  `least` > 0 with `chunks` = (chunk_req, chunk_t0, req_chunk0, n_chunks): the requests that bring at least
    that many tokens run chunk by chunk (per chunk of LIGHTNING_CHUNK tokens its request and its first token inside the
    portion, per request the index of its first chunk: int32 on the device), the `n_short` others token by token; 0: all
    token by token.  `columns_per_cta` (16, 32, 64; 0: by the size of the launch): value columns a CTA of the chunked form takes."""
    _need(proj, torch.float32, "proj", 2); _need(decay, torch.float32, "decay", 1); _need(state, torch.float32, "state", 2)
    _need(o, torch.float32, "o", 2)
    for name, t in (("req_slot", req_slot), ("q_start", q_start), ("q_len", q_len)):
        _need(t, torch.int32, name, 1)
    tokens, cols = proj.shape
    if (decay.numel() != heads or state.shape[1] != heads * key_dim * value_dim or o.shape != (tokens, heads * value_dim)
            or max(q_col, k_col) + heads * key_dim > cols or v_col + heads * value_dim > cols or key_dim > LIGHTNING_MAX_KEY_DIM):
        raise KernelError("lightning_recurrence: shapes disagree")
    chunk_req = chunk_t0 = req_chunk0 = scratch = None
    n_chunks = 0
    if least > 0 and chunks is not None and chunks[3] > 0:
        chunk_req, chunk_t0, req_chunk0, n_chunks = chunks
        for name, t in (("chunk_req", chunk_req), ("chunk_t0", chunk_t0), ("req_chunk0", req_chunk0)):
            _need(t, torch.int32, name, 1)
        if chunk_req.numel() < n_chunks or chunk_t0.numel() < n_chunks or req_chunk0.numel() < n_req:
            raise KernelError("lightning_recurrence: the chunk lists are too short")
        scratch = torch.empty((n_chunks, heads, key_dim, value_dim), dtype=torch.float32, device=proj.device)
    launches = (3 if n_chunks else 0) + (1 if not n_chunks or n_short else 0)
    _check(_lightning().cisr_lightning_recurrence(_p(proj), cols, q_col, k_col, v_col, _p(decay), _p(state), ctypes.c_longlong(state.shape[1]),
                                                  _p(req_slot), _p(q_start), _p(q_len), _p(o), heads, key_dim, value_dim, n_req,
                                                  int(least if n_chunks else 0), int(n_chunks), int(n_short), _p(chunk_req), _p(chunk_t0),
                                                  _p(req_chunk0), _p(scratch), int(columns_per_cta), _stream()), "lightning_recurrence",
           own=launches)
    return o


def lightning_output(o: torch.Tensor, gate: torch.Tensor, gate_col: int, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[:, :width] = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate[:, gate_col : gate_col + width]) with the mean over
    a token's whole row (all heads at once); float arithmetic, rounded once to out's type.  out may be wider than o (padding
    columns are left as they are)."""
    _need(o, torch.float32, "o", 2); _need(gate, torch.float32, "gate", 2); _need(norm_w, torch.float32, "norm_w", 1); _need(out, None, "out", 2)
    tokens, width = o.shape
    if gate.shape[0] != tokens or gate_col + width > gate.shape[1] or norm_w.numel() != width or out.shape[0] != tokens or out.shape[1] < width:
        raise KernelError("lightning_output: shapes disagree")
    _check(_lightning().cisr_lightning_output(_p(o), _p(gate), gate.shape[1], gate_col, _p(norm_w), ctypes.c_float(eps), _p(out),
                                              dtype_code(out.dtype), out.shape[1], width, tokens, _stream()), "lightning_output")
    return out


# ------------------------------------------------------------------ latent attention: the kernels around its products
_latent_state = {}


def _latent():
    lib = _latent_state.get("lib")
    if lib is None:
        lib = load_library("latent.cu")
        for name in ("cisr_latent_rows", "cisr_latent_query", "cisr_latent_gate", "cisr_latent_absorb", "cisr_latent_values"):
            getattr(lib, name).restype = ctypes.c_int
        lib.cisr_latent_set_pdl(int(_pdl_state["on"]))
        _latent_state["lib"] = lib
    return lib


def latent_jobs():
    return [("latent.cu", {}, ())]


def latent_rows(proj: torch.Tensor, q_col: int, q_rank: int, q_norm_w: Optional[torch.Tensor], cq_out: Optional[torch.Tensor],
                c_col: int, kv_rank: int, c_norm_w: torch.Tensor, eps: float, cos: torch.Tensor, sin: torch.Tensor,
                rot_half: int, interleaved: bool, cache: Optional[torch.Tensor], token_req, positions, req_slot, block_table,
                page_size: int) -> None:
    """From the stacked down projections `proj` (float [tokens, columns]): the unit-normed query latent (`q_rank` columns
    from `q_col`, to `cq_out`; q_rank 0: none) and the token's cache row [unit-normed latent | rotated shared key part | 0]
    written into its page of `cache` [pages, 1, page_size, row width] (None: the row is not written)."""
    _need(proj, torch.float32, "proj", 2); _need(c_norm_w, torch.float32, "c_norm_w", 1)
    _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
    tokens = proj.shape[0]
    if cos.shape != (tokens, rot_half) or sin.shape != cos.shape:
        raise KernelError("latent_rows: rotary tables must be [tokens, rot_half]")
    dtype = None
    if q_rank:
        _need(q_norm_w, torch.float32, "q_norm_w", 1); _need(cq_out, None, "cq_out", 2)
        if cq_out.shape != (tokens, q_rank) or q_norm_w.numel() != q_rank or q_col + q_rank > proj.shape[1]:
            raise KernelError("latent_rows: query latent shapes disagree")
        dtype = cq_out.dtype
    row_width = 0
    if cache is not None:
        _need(cache, dtype, "cache", 4)
        if cache.shape[1] != 1 or cache.shape[2] != page_size:
            raise KernelError("latent_rows: cache must be [pages, 1, page_size, row width]")
        row_width = cache.shape[3]
        dtype = cache.dtype
        if c_col + kv_rank + 2 * rot_half > proj.shape[1] or c_norm_w.numel() != kv_rank:
            raise KernelError("latent_rows: key/value latent shapes disagree")
    for name, t in (("token_req", token_req), ("positions", positions), ("req_slot", req_slot), ("block_table", block_table)):
        _need(t, torch.int32, name)
    _check(_latent().cisr_latent_rows(
        _p(proj), proj.shape[1], q_col, q_rank, _p(q_norm_w), _p(cq_out), c_col, kv_rank, _p(c_norm_w), ctypes.c_float(eps),
        _p(cos), _p(sin), rot_half, int(interleaved), _p(cache), row_width, dtype_code(dtype), _p(token_req), _p(positions),
        _p(req_slot), _p(block_table), block_table.shape[1], page_size, tokens, _stream()), "latent_rows")


def latent_query(q: torch.Tensor, q_col: int, heads: int, plain_dim: int, cos: torch.Tensor, sin: torch.Tensor, rot_half: int,
                 interleaved: bool, plain_out: torch.Tensor, q_rows: torch.Tensor, kv_rank: int) -> None:
    """Split the heads of `q` (float [tokens, columns], heads of [plain | rotated part] from `q_col` on): the plain parts
    go to `plain_out` [tokens, heads, plain_dim]; the rotated parts, turned to the tokens' positions, go to columns
    kv_rank .. of `q_rows` [tokens, heads, row width], the columns behind them are zeroed."""
    _need(q, torch.float32, "q", 2); _need(plain_out, q_rows.dtype, "plain_out", 3); _need(q_rows, None, "q_rows", 3)
    _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
    tokens = q.shape[0]
    if (plain_out.shape != (tokens, heads, plain_dim) or q_rows.shape[:2] != (tokens, heads)
            or q_col + heads * (plain_dim + 2 * rot_half) > q.shape[1] or cos.shape != (tokens, rot_half)):
        raise KernelError("latent_query: shapes disagree")
    _check(_latent().cisr_latent_query(_p(q), q.shape[1], q_col, heads, plain_dim, _p(cos), _p(sin), rot_half, int(interleaved),
                                       _p(plain_out), _p(q_rows), kv_rank, q_rows.shape[2], dtype_code(q_rows.dtype), tokens,
                                       _stream()), "latent_query")


def latent_gate(values: torch.Tensor, gate: Optional[torch.Tensor], gate_col: int, out: torch.Tensor) -> torch.Tensor:
    """out = values * sigmoid(gate[:, gate_col : gate_col + width]) (gate None: out = values), rounded to out's type."""
    _need(values, torch.float32, "values", 2); _need(out, None, "out", 2)
    tokens, width = values.shape
    if out.shape != values.shape:
        raise KernelError("latent_gate: out and values differ in shape")
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
        if gate.shape[0] != tokens or gate_col + width > gate.shape[1]:
            raise KernelError("latent_gate: the gate's columns lie outside its rows")
    _check(_latent().cisr_latent_gate(_p(values), _p(gate), gate.shape[1] if gate is not None else 0, gate_col, _p(out),
                                      dtype_code(out.dtype), tokens, width, _stream()), "latent_gate")
    return out


LATENT_ROW_KERNEL_MAX_TOKENS = 16     # up to here the per-head products run as row kernels, beyond as library products


def latent_absorb(q: torch.Tensor, q_col: int, heads: int, plain_dim: int, cos: torch.Tensor, sin: torch.Tensor, rot_half: int,
                  interleaved: bool, k_up: torch.Tensor, q_rows: torch.Tensor, kv_rank: int) -> torch.Tensor:
    """Few tokens: `latent_query` and the per-head product with k_up ([heads, plain_dim, kv_rank]) in one launch:
    q_rows[t, h] = [k_up[h]^T q_plain[t, h] | rotated part | 0]."""
    _need(q, torch.float32, "q", 2); _need(q_rows, None, "q_rows", 3); _need(k_up, q_rows.dtype, "k_up", 3)
    _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
    tokens = q.shape[0]
    if (k_up.shape != (heads, plain_dim, kv_rank) or q_rows.shape[:2] != (tokens, heads)
            or q_col + heads * (plain_dim + 2 * rot_half) > q.shape[1] or cos.shape != (tokens, rot_half)):
        raise KernelError("latent_absorb: shapes disagree")
    _check(_latent().cisr_latent_absorb(_p(q), q.shape[1], q_col, heads, plain_dim, _p(cos), _p(sin), rot_half, int(interleaved),
                                        _p(k_up), _p(q_rows), kv_rank, q_rows.shape[2], dtype_code(q_rows.dtype), tokens, _stream()),
           "latent_absorb")
    return q_rows


def latent_values(mixed: torch.Tensor, v_up: torch.Tensor, gate: Optional[torch.Tensor], gate_col: int, out: torch.Tensor) -> torch.Tensor:
    """Few tokens: the per-head product with v_up ([heads, value_dim, kv_rank]) over the first kv_rank columns of
    mixed [tokens, heads, row width], times sigmoid(gate[:, gate_col + ...]) when a gate is given, rounded to out's type."""
    _need(mixed, None, "mixed", 3); _need(v_up, mixed.dtype, "v_up", 3); _need(out, mixed.dtype, "out", 2)
    tokens, heads, row_width = mixed.shape
    _, value_dim, kv_rank = v_up.shape
    if v_up.shape[0] != heads or kv_rank > row_width or out.shape != (tokens, heads * value_dim):
        raise KernelError("latent_values: shapes disagree")
    if gate is not None:
        _need(gate, torch.float32, "gate", 2)
        if gate.shape[0] != tokens or gate_col + heads * value_dim > gate.shape[1]:
            raise KernelError("latent_values: the gate's columns lie outside its rows")
    _check(_latent().cisr_latent_values(_p(mixed), heads, row_width, kv_rank, _p(v_up), value_dim, _p(gate),
                                        gate.shape[1] if gate is not None else 0, gate_col, _p(out), dtype_code(out.dtype), tokens,
                                        _stream()), "latent_values")
    return out


# ------------------------------------------------------------------ routed experts
_moe_state = {}


def _moe():
    lib = _moe_state.get("lib")
    if lib is None:
        lib = load_library("moe.cu")
        for name in ("cisr_moe_select", "cisr_moe_rows", "cisr_moe_sort", "cisr_moe_gather", "cisr_moe_combine"):
            getattr(lib, name).restype = ctypes.c_int
        lib.cisr_moe_set_pdl(int(_pdl_state["on"]))
        _moe_state["lib"] = lib
    return lib


def moe_jobs():
    return [("moe.cu", {}, ())]


def moe_select(logits: torch.Tensor, top: int, n_groups: int, keep: int, route_scale: float, chosen: torch.Tensor,
               weight: torch.Tensor, scores: str = "sigmoid", choice_bias: Optional[torch.Tensor] = None,
               renormalize: bool = False) -> None:
    """Per token, from the router's logits (float [tokens, experts]): scores (`scores`: "sigmoid" of each logit, or
    "softmax" over all of them), the open groups, the `top` chosen experts (`chosen`, int32 [tokens, top], best first;
    chosen by score + choice_bias where that is given) and their weights score * route_scale (`weight`, float); with
    `renormalize` the chosen scores are divided by their sum (+ 1e-20) before the scale."""
    _need(logits, torch.float32, "logits", 2); _need(chosen, torch.int32, "chosen", 2); _need(weight, torch.float32, "weight", 2)
    tokens, experts = logits.shape
    if chosen.shape != (tokens, top) or weight.shape != (tokens, top):
        raise KernelError("moe_select: shapes disagree")
    if scores not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_select: unknown scores {scores!r}")
    if choice_bias is not None:
        _need(choice_bias, torch.float32, "choice_bias", 1)
        if choice_bias.numel() != experts:
            raise KernelError("moe_select: one choice bias per router output is needed")
    _check(_moe().cisr_moe_select(_p(logits), tokens, experts, top, n_groups, keep, ctypes.c_float(route_scale),
                                  int(scores == "softmax"), int(renormalize), _p(choice_bias), _p(chosen), _p(weight), _stream()), "moe_select")


def _channel_scale(scale: Optional[torch.Tensor], hidden: int, what: str) -> None:
    if scale is not None:
        _need(scale, torch.float32, "out_scale", 1)
        if scale.numel() != hidden:
            raise KernelError(f"{what}: one output scale per channel is needed")


def moe_rows(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor, weight: torch.Tensor,
             act: torch.Tensor, out: torch.Tensor, out_scale: Optional[torch.Tensor] = None, gate_limit: Optional[float] = None,
             activation: str = "relu_squared") -> torch.Tensor:
    """out (float [tokens, hidden]) = sum over a token's chosen experts of weight * W_down_e a(W_up_e h) (`activation`:
    "relu_squared" max(z, 0)^2 or "gelu" z Phi(z)), a warp per
    output feature; w_up [experts, ff, hidden], w_down [experts, hidden, ff]; `act` [tokens * top, ff] is scratch; `out_scale`
    (float, one per channel) multiplies the sum.  With `gate_limit` the experts are gated: w_up [experts, 2 ff, hidden]
    (gate rows, then up rows) and the activation is `gated_clamp`'s.  A chosen index beyond the experts that have
    matrices is an identity expert: it adds weight * h."""
    _need(h, None, "h", 2); _need(w_up, h.dtype, "w_up", 3); _need(w_down, h.dtype, "w_down", 3); _need(act, h.dtype, "act", 2)
    _need(out, torch.float32, "out", 2); _need(chosen, torch.int32, "chosen", 2); _need(weight, torch.float32, "weight", 2)
    tokens, hidden = h.shape
    experts, ff, _ = w_up.shape
    if gate_limit is not None:
        ff //= 2
    top = chosen.shape[1]
    if (w_up.shape[2] != hidden or w_down.shape != (experts, hidden, ff) or act.shape != (tokens * top, ff)
            or out.shape != (tokens, hidden) or chosen.shape[0] != tokens or weight.shape != chosen.shape):
        raise KernelError("moe_rows: shapes disagree")
    _channel_scale(out_scale, hidden, "moe_rows")
    _check(_moe().cisr_moe_rows(_p(h), _p(w_up), _p(w_down), dtype_code(h.dtype), _p(chosen), _p(weight), tokens, hidden, ff, top,
                                experts, int(gate_limit is not None), ctypes.c_float(gate_limit or 0.0),
                                0 if gate_limit is not None else EXPERT_ACTIVATIONS[activation],
                                _p(act), _p(out_scale), _p(out),
                                _stream()), "moe_rows", own=2)
    return out


EXPERT_ACTIVATIONS = {"relu_squared": 0, "gelu": 1}      # ungated expert activations as the kernels number them
MOE_TILE = 128                   # rows per tile of the grouped product: each expert's rows are padded to whole tiles
MOE_GROUPED_MIN_ROWS = 64        # (token, expert) pairs per expert, on average, from which sorting and the grouped product pay


def moe_grouped_ok(h: torch.Tensor, w_up: torch.Tensor, top: int, gated: bool = False) -> bool:
    """Whether a step's experts run as grouped tcgen05 products: bfloat16, widths whose rows are 16-byte multiples, and
    enough pairs per expert that whole 128-row tiles are mostly real rows."""
    experts, ff, hidden = w_up.shape
    if gated:
        ff //= 2
    return (h.dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0 and h.shape[0] * top >= MOE_GROUPED_MIN_ROWS * experts
            and h.shape[0] >= TCGEN05_MIN_TOKENS)


def moe_sorted_rows(tokens: int, top: int, experts: int) -> int:
    """Rows of the sorted layout: every expert's block padded to whole tiles, in the worst case."""
    pairs = tokens * top
    return max(MOE_TILE, (pairs + min(pairs, experts) * (MOE_TILE - 1)) // MOE_TILE * MOE_TILE)


def moe_sort(chosen: torch.Tensor, experts: int, row_of: torch.Tensor, src_token: torch.Tensor, tile_group: torch.Tensor) -> None:
    """Lay the (token, chosen expert) pairs out expert by expert, each expert's rows padded to whole tiles of MOE_TILE:
    row_of[pair] = its row, src_token[row] = the token of that row (-1: padding), tile_group[tile] = its expert (-1: unused)."""
    _need(chosen, torch.int32, "chosen", 2)
    for name, t in (("row_of", row_of), ("src_token", src_token), ("tile_group", tile_group)):
        _need(t, torch.int32, name, 1)
    tokens, top = chosen.shape
    rows = src_token.numel()
    if row_of.numel() != tokens * top or rows % MOE_TILE or tile_group.numel() != rows // MOE_TILE:
        raise KernelError("moe_sort: shapes disagree")
    _check(_moe().cisr_moe_sort(_p(chosen), tokens, top, experts, MOE_TILE, rows, _p(row_of), _p(src_token), _p(tile_group), _stream()),
           "moe_sort")


def moe_gather(h: torch.Tensor, src_token: torch.Tensor, sorted_h: torch.Tensor) -> torch.Tensor:
    """sorted_h[row] = h[src_token[row]], zeros where src_token[row] < 0 (bfloat16 rows of 16-byte multiples)."""
    _need(h, torch.bfloat16, "h", 2); _need(sorted_h, torch.bfloat16, "sorted_h", 2); _need(src_token, torch.int32, "src_token", 1)
    if sorted_h.shape != (src_token.numel(), h.shape[1]):
        raise KernelError("moe_gather: shapes disagree")
    _check(_moe().cisr_moe_gather(_p(h), _p(src_token), _p(sorted_h), sorted_h.shape[0], h.shape[1], _stream()), "moe_gather")
    return sorted_h


def moe_combine(sorted_out: torch.Tensor, row_of: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                out_scale: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = out_scale * sum over k of weight[t, k] * sorted_out[row_of[t * top + k]], in the order of k; a pair
    without a row (row_of < 0: an identity expert) adds weight[t, k] * h[t] (`h` bfloat16 [tokens, hidden])."""
    if h is not None:
        _need(h, torch.bfloat16, "h", 2)
    _need(sorted_out, torch.float32, "sorted_out", 2); _need(row_of, torch.int32, "row_of", 1); _need(weight, torch.float32, "weight", 2)
    _need(out, torch.float32, "out", 2)
    tokens, top = weight.shape
    if row_of.numel() != tokens * top or out.shape != (tokens, sorted_out.shape[1]):
        raise KernelError("moe_combine: shapes disagree")
    _channel_scale(out_scale, out.shape[1], "moe_combine")
    _check(_moe().cisr_moe_combine(_p(sorted_out), _p(row_of), _p(weight), tokens, top, out.shape[1], _p(h), _p(out_scale), _p(out),
                                   _stream()), "moe_combine")
    return out


def moe_grouped(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor, weight: torch.Tensor,
                out: torch.Tensor, out_scale: Optional[torch.Tensor] = None, gate_limit: Optional[float] = None,
                activation: str = "relu_squared") -> torch.Tensor:
    """The same sum as `moe_rows` for many tokens: pairs sorted by expert on the device, activations gathered into that
    order, both products as grouped tcgen05 products (the activation, relu^2 or the clamped gated form over the stacked
    gate and up rows, as the first one's epilogue), rows summed per token with the router's weights in the router's
    order.  Nothing is read back to the host."""
    _need(w_up, torch.bfloat16, "w_up", 3); _need(w_down, torch.bfloat16, "w_down", 3)
    tokens, hidden = h.shape
    experts, ff, _ = w_up.shape
    if gate_limit is not None:
        ff //= 2
    top = chosen.shape[1]
    if w_up.shape[2] != hidden or w_down.shape != (experts, hidden, ff) or out.shape != (tokens, hidden) or weight.shape != chosen.shape:
        raise KernelError("moe_grouped: shapes disagree")
    rows = moe_sorted_rows(tokens, top, experts)
    device = h.device
    row_of = torch.empty(tokens * top, dtype=torch.int32, device=device)
    src_token = torch.empty(rows, dtype=torch.int32, device=device)
    tile_group = torch.empty(rows // MOE_TILE, dtype=torch.int32, device=device)
    moe_sort(chosen, experts, row_of, src_token, tile_group)
    sorted_h = moe_gather(h, src_token, torch.empty((rows, hidden), dtype=torch.bfloat16, device=device))
    if gate_limit is None:
        act = gemm_tcgen05_grouped(sorted_h, w_up, torch.empty((rows, ff), dtype=torch.bfloat16, device=device), tile_group, tokens * top,
                                   activation=activation)
    else:
        act = gemm_tcgen05_grouped_gated(sorted_h, w_up, torch.empty((rows, ff), dtype=torch.bfloat16, device=device), tile_group,
                                         gate_limit, tokens * top)
    sorted_out = gemm_tcgen05_grouped(act, w_down, torch.empty((rows, hidden), dtype=torch.float32, device=device), tile_group, tokens * top)
    return moe_combine(sorted_out, row_of, weight, out, out_scale, h=h)


# ------------------------------------------------------------------ sampling
def _sampling():
    lib = load_library("sampling.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_sample.restype = ctypes.c_int
        lib.cisr_decode_advance.restype = ctypes.c_int
        lib.cisr_uniform_host.restype = ctypes.c_float
        lib.cisr_uniform_host.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
        lib._typed = True
    return lib


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
           counter: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """Token per row: argmax where temperature <= 0 (or None), else inverse-CDF sampling."""
    _need(logits, torch.float32, "logits", 2); _need(out, torch.int32, "out", 1)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, torch.float32, "temperature", 1); _need(seed, torch.int64, "seed", 1)
        _need(counter, torch.int32, "counter", 1)
    _check(_sampling().cisr_sample(_p(logits), rows, vocab, _p(temperature), _p(seed), _p(counter), _p(out), _stream()),
           "sample")
    return out


def decode_advance(token_ids, positions, ctx_len, counter, sampled, live, ring: Optional[torch.Tensor] = None,
                   step_index: Optional[torch.Tensor] = None) -> None:
    """Feed sampled tokens back as the next inputs of live rows and advance their positions, lengths and counters.

    `ring` (int32 [slots, rows + 1]) with `step_index` (one int32): the sampled tokens and the kernels' error flag also
    go to slot step_index % slots, and step_index moves on by one."""
    for name, t in (("token_ids", token_ids), ("positions", positions), ("ctx_len", ctx_len), ("counter", counter),
                    ("sampled", sampled), ("live", live)):
        _need(t, torch.int32, name, 1)
    slots = 0
    if ring is not None:
        _need(ring, torch.int32, "ring", 2); _need(step_index, torch.int32, "step_index", 1)
        if ring.shape[1] != token_ids.numel() + 1:
            raise KernelError("decode_advance: ring must be [slots, rows + 1]")
        slots = ring.shape[0]
    _check(_sampling().cisr_decode_advance(_p(token_ids), _p(positions), _p(ctx_len), _p(counter), _p(sampled), _p(live),
                                           token_ids.numel(), _p(_error_state.get("flag")), _p(ring), slots, _p(step_index),
                                           _stream()), "decode_advance")


def uniform_host(seed: int, counter: int) -> float:
    """The uniform the device sampler draws for (seed, counter), computed on the host by the same code."""
    return float(_sampling().cisr_uniform_host(seed, counter))


# ------------------------------------------------------------------ library matrix product
_gemm_state = {}


def _gemm_library():
    lib = _gemm_state.get("lib")
    if lib is None:
        lib = load_library("gemm_library.cu", extra=("-lcublas",))
        lib.cisr_gemm_library_init.restype = ctypes.c_int
        lib.cisr_gemm_library.restype = ctypes.c_int
        lib.cisr_gemm_library_batched.restype = ctypes.c_int
        workspace = torch.empty(GEMM_WORKSPACE_BYTES, dtype=torch.uint8, device="cuda")
        _check(lib.cisr_gemm_library_init(_p(workspace), ctypes.c_longlong(GEMM_WORKSPACE_BYTES)), "gemm library init")
        _gemm_state["lib"], _gemm_state["workspace"] = lib, workspace
    return lib


def gemm_library(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T by the vendor library, float accumulation."""
    _need(a, None, "a", 2); _need(w, a.dtype, "w", 2); _need(out, torch.float32, "out", 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_gemm_library().cisr_gemm_library(_p(a), _p(w), dtype_code(a.dtype), _p(out), m, n, k, _stream()), "gemm",
           own=0, library=1)
    return out


def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, w_is_nk: bool) -> torch.Tensor:
    """One product per head by the vendor library: out[:, h, :n] = a[:, h, :k] @ w_h, float accumulation.

    a [M, H, >= k] and out [M, H, >= n] may be wider than the product uses (their last axis is the row of a head, of
    which the first k or n columns take part); w [H, n, k] (`w_is_nk`, the checkpoint's [out, in] layout per head) or
    [H, k, n].  out is float or has the operands' type."""
    _need(w, a.dtype, "w", 3); _need(a, None, "a", 3); _need(out, None, "out", 3)
    heads = w.shape[0]
    n, k = (w.shape[1], w.shape[2]) if w_is_nk else (w.shape[2], w.shape[1])
    m = a.shape[0]
    if a.shape[1] != heads or out.shape[1] != heads or out.shape[0] != m or a.shape[2] < k or out.shape[2] < n:
        raise KernelError(f"gemm_heads: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    if out.dtype not in (torch.float32, a.dtype):
        raise KernelError("gemm_heads: out must be float or of the operands' type")
    lib = _gemm_library()
    _check(lib.cisr_gemm_library_batched(
        _p(a), heads * a.shape[2], ctypes.c_longlong(a.shape[2]), _p(w), w.shape[2], ctypes.c_longlong(w.shape[1] * w.shape[2]),
        int(w_is_nk), dtype_code(a.dtype), _p(out), heads * out.shape[2], ctypes.c_longlong(out.shape[2]), dtype_code(out.dtype),
        m, n, k, heads, _stream()), "gemm_heads", own=0, library=1)
    return out


def gemm_jobs(dtype: torch.dtype):
    """Build jobs of the libraries `gemm` may launch for operands of this dtype."""
    jobs = [("gemm_library.cu", {}, ("-lcublas",))]
    if dtype == torch.bfloat16:
        jobs.append(("gemm_tcgen05.cu", {}, ()))
    return jobs


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T; picks the kernel for the shape and dtype.

    bfloat16 with at least one 128-row tile of tokens: this package's tcgen05 + TMA kernel; float (true 32-bit),
    and shapes that kernel does not take: the vendor library."""
    if tcgen05_ok(a, w):
        return gemm_tcgen05(a, w, out)
    return gemm_library(a, w, out)


# ------------------------------------------------------------------ weight-streaming products for few tokens
SKINNY_MAX_TOKENS = int(os.environ.get("CISR_SKINNY_MAX_TOKENS", "16"))   # most tokens the latency kernels are chosen for (they take up to 64)
SKINNY_NORM_MAX_TOKENS = 16      # beyond this the norm runs once as its own kernel instead of in every CTA
EPI_PLAIN, EPI_SWIGLU, EPI_ROPE = 0, 1, 2


def _skinny():
    lib = load_library("skinny_gemm.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_skinny_gemm.restype = ctypes.c_int
        lib._typed = True
    return lib


def set_pdl(on: bool) -> None:
    """Launch the decode-path kernels with programmatic dependent launch (a kernel may fetch its weights while the
    kernel before it is still running)."""
    _skinny().cisr_skinny_set_pdl(int(on))
    if "lib" in _stream_state:
        _stream_state["lib"].cisr_stream_set_pdl(int(on))
    for lib in _attention_tcgen05_libs.values():
        lib.cisr_attn_tcgen05_set_pdl(int(on))
    if "lib" in _merge_proj_state:
        _merge_proj_state["lib"].cisr_merge_proj_set_pdl(int(on))
    _elementwise().cisr_elementwise_set_pdl(int(on))
    _sampling().cisr_sampling_set_pdl(int(on))
    if "lib" in _latent_state:
        _latent_state["lib"].cisr_latent_set_pdl(int(on))
    if "lib" in _moe_state:
        _moe_state["lib"].cisr_moe_set_pdl(int(on))
    if "lib" in _hyper_state:
        _hyper_state["lib"].cisr_hyper_set_pdl(int(on))
    if "lib" in _rows_state:
        _rows_state["lib"].cisr_attention_rows_set_pdl(int(on))
    if "lib" in _delta_state:
        _delta_state["lib"].cisr_delta_set_pdl(int(on))
    if "lib" in _lightning_state:
        _lightning_state["lib"].cisr_lightning_set_pdl(int(on))
    if "lib" in _diff_state:
        _diff_state["lib"].cisr_diff_set_pdl(int(on))
    if "lib" in _depth_state:
        _depth_state["lib"].cisr_depth_set_pdl(int(on))
    if "lib" in _ffn_rows_state:
        _ffn_rows_state["lib"].cisr_ffn_rows_set_pdl(int(on))
    if "lib" in _tcgen05_state:
        _tcgen05_state["lib"].cisr_gemm_tcgen05_set_pdl(int(on))
    for (source, _, _), lib in list(_attention_libs.items()):
        if source == "attention_mma.cu":
            lib.cisr_attn_set_pdl(int(on))
    _pdl_state["on"] = bool(on)


def skinny_jobs():
    return [("skinny_gemm.cu", {}, ()), ("stream_gemm.cu", {}, ())]


def stream_takes(tokens: int, w: torch.Tensor) -> bool:
    """Whether skinny_gemm(kind="auto") hands this product to the persistent streaming kernel (stream_gemm.cu): a large
    bfloat16 weight matrix, at most 16 tokens, the tokens and at least three 16 KB stages in shared memory.  (The
    epilogues add their own conditions; where they fail the latency kernels take over.)"""
    if w.dtype != torch.bfloat16 or not 0 < tokens <= STREAM_MAX_TOKENS or w.shape[1] % 8 or w.numel() * 2 < STREAM_MIN_BYTES:
        return False
    padded = 8 if tokens <= 8 else 16
    fixed = 1024 + 64 + 4 * 8 * 16 * padded + tokens * (w.shape[1] + 8) * 2
    return fixed + 3 * (16384 + 16) <= 224 * 1024 - 8192          # 8 KB kept for the rotation tables of the ROPE epilogue


def skinny_ok(tokens: int, w: torch.Tensor) -> bool:
    """Shapes the weight-streaming kernels take: bfloat16 weights, at most 16 tokens, K a multiple of 8."""
    if w.dtype != torch.bfloat16 or not 0 < tokens <= SKINNY_MAX_TOKENS or w.shape[1] % 8:
        return False
    if stream_takes(tokens, w):
        return True
    padded = -(-tokens // 8) * 8
    return padded * (w.shape[1] + 8) * 2 + 64 * padded * 4 * 2 <= 200 * 1024     # the tokens and the partial sums fit in shared memory


def skinny_gemm(w: torch.Tensor, tokens: int, *, act: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
                delta: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                x_out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None, epilogue: int = EPI_PLAIN,
                out: Optional[torch.Tensor] = None, rope: Optional[dict] = None, kind: str = "auto",
                accumulate: bool = False, out_mult: float = 1.0) -> None:
    """out = prologue(input) @ w^T with a fused epilogue; see csrc/skinny_gemm.cu and csrc/stream_gemm.cu.

    `kind`: "latency" (skinny_gemm.cu: a CTA per 16 output rows, weights straight to registers), "stream"
    (stream_gemm.cu: persistent CTAs, weights through a ring of tensor-map copies; up to 16 tokens), or "auto": the
    streaming kernel for weight matrices of 8 MB and more where it takes the shape.

    Input is either `act` (bfloat16 [tokens, K]) or the norm prologue (`x`, optional `delta`, `norm_w`, `eps`,
    optional `x_out` receiving x + delta, optional `rows` picking rows of x).  PLAIN writes float `out`
    [tokens, N], or with `accumulate` adds the product to what `out` holds (the residual stream), in both cases times
    `out_mult` (a constant factor of the residual branch); SWIGLU writes bfloat16 `out` [tokens, N / 2]; ROPE takes the `rope` dict (cos, sin, rot_half,
    interleaved, q_out, k_cache, v_cache, positions, token_req, req_slot, block_table, page_size, hq, hkv, dim).
    """
    _need(w, torch.bfloat16, "w", 2)
    n, k = w.shape
    if act is not None:
        _need(act, torch.bfloat16, "act", 2)
        if act.shape[0] < tokens or act.shape[1] != k:
            raise KernelError("skinny_gemm: act must be [tokens, K]")
    else:
        _need(x, torch.float32, "x", 2); _need(norm_w, None, "norm_w", 1)
        if x.shape[1] != k or norm_w.numel() != k:
            raise KernelError("skinny_gemm: x and norm_w must be K wide")
        if delta is not None:
            _need(delta, torch.float32, "delta", 2)
        if x_out is not None:
            _need(x_out, torch.float32, "x_out", 2)
            if x_out.data_ptr() == x.data_ptr():
                raise KernelError("skinny_gemm: x_out must be another buffer than x")
        if rows is not None:
            _need(rows, torch.int32, "rows", 1)
    r = rope or {}
    out_f32 = out if epilogue == EPI_PLAIN else None
    out_b16 = out if epilogue == EPI_SWIGLU else None
    if epilogue == EPI_PLAIN:
        _need(out, torch.float32, "out", 2)
        if out.shape[0] < tokens or out.shape[1] != n:
            raise KernelError("skinny_gemm: out must be float [tokens, N]")
    elif epilogue == EPI_SWIGLU:
        _need(out, torch.bfloat16, "out", 2)
        if out.shape[0] < tokens or out.shape[1] * 2 != n:
            raise KernelError("skinny_gemm: out must be bfloat16 [tokens, N / 2]")
    else:
        for name in ("q_out", "k_cache", "v_cache"):
            _need(r[name], torch.bfloat16, name)
        for name in ("positions", "token_req", "req_slot", "block_table"):
            _need(r[name], torch.int32, name)
        if r["rot_half"]:
            _need(r["cos"], torch.float32, "cos", 2); _need(r["sin"], torch.float32, "sin", 2)
    args = (_p(w), n, k, _p(act), _p(x), _p(delta), _p(norm_w), dtype_code(norm_w.dtype) if norm_w is not None else 0,
            ctypes.c_float(eps), _p(x_out), _p(rows), tokens, epilogue, _p(out_f32), _p(out_b16),
            n // 2 if epilogue == EPI_SWIGLU else 0, _p(r.get("cos")), _p(r.get("sin")), int(r.get("rot_half", 0)),
            int(bool(r.get("interleaved", False))), _p(r.get("q_out")), _p(r.get("k_cache")), _p(r.get("v_cache")),
            _p(r.get("positions")), _p(r.get("token_req")), _p(r.get("req_slot")), _p(r.get("block_table")),
            r["block_table"].shape[1] if rope else 0, int(r.get("page_size", 0)), int(r.get("hq", 0)), int(r.get("hkv", 0)),
            int(r.get("dim", 0)), int(bool(accumulate)), ctypes.c_float(out_mult), _stream())
    if (accumulate or out_mult != 1.0) and epilogue != EPI_PLAIN:
        raise KernelError("skinny_gemm: only the plain epilogue adds into its output or multiplies it")
    if kind not in ("auto", "latency", "stream"):
        raise KernelError(f"unknown kind {kind!r}")
    if kind == "stream" or (kind == "auto" and tokens <= STREAM_MAX_TOKENS and w.numel() * 2 >= STREAM_MIN_BYTES):
        status = _stream_lib().cisr_stream_gemm(*args)
        if status != -2:                  # -2: not a shape for the streaming kernel
            _check(status, "stream_gemm")
            return
        if kind == "stream":
            raise KernelError("stream_gemm does not take this shape")
    _check(_skinny().cisr_skinny_gemm(*args), "skinny_gemm")


STREAM_MAX_TOKENS = 16
STREAM_MIN_BYTES = 8 << 20       # smaller weight matrices are latency-bound: the kernels of skinny_gemm.cu serve them better
_stream_state = {}


def _stream_lib():
    lib = _stream_state.get("lib")
    if lib is None:
        lib = load_library("stream_gemm.cu")
        lib.cisr_stream_gemm.restype = ctypes.c_int
        lib.cisr_stream_init.restype = ctypes.c_int
        _check(lib.cisr_stream_init(_p(_error_flag())), "stream gemm init", own=0)
        lib.cisr_stream_set_pdl(int(_pdl_state["on"]))
        _stream_state["lib"] = lib
    return lib


# ------------------------------------------------------------------ tcgen05 + TMA matrix product
_tcgen05_state = {}
TCGEN05_MIN_TOKENS = int(os.environ.get("CISR_TCGEN05_MIN_TOKENS", "128"))   # below one 128-row tile the weight-streaming kernels or the library serve better


def _tcgen05():
    lib = _tcgen05_state.get("lib")
    if lib is None:
        lib = load_library("gemm_tcgen05.cu")
        lib.cisr_gemm_tcgen05_init.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_swiglu.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_rope.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_grouped.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_grouped_gated.restype = ctypes.c_int
        _check(lib.cisr_gemm_tcgen05_init(_p(_error_flag())), "tcgen05 gemm init", own=0)
        lib.cisr_gemm_tcgen05_set_pdl(int(_pdl_state["on"]))
        _tcgen05_state["lib"] = lib
    return lib


def tcgen05_jobs():
    return [("gemm_tcgen05.cu", {}, ())]


# The product with rotation and cache write as its epilogue replaces two launches (the library's product and the rotate
# kernel), which pays from far fewer tokens on than the plain product does against the library's.
TCGEN05_FUSED_MIN_TOKENS = int(os.environ.get("CISR_TCGEN05_FUSED_MIN_TOKENS", "17"))


def tcgen05_ok(a: torch.Tensor, w: torch.Tensor, fused: bool = False) -> bool:
    least = min(TCGEN05_MIN_TOKENS, TCGEN05_FUSED_MIN_TOKENS) if fused else TCGEN05_MIN_TOKENS
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] >= least
            and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, out_mult: float = 1.0) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T on tcgen05 tensor cores fed by TMA (bfloat16 operands); with
    `accumulate`, out += the product (the residual add as the product's epilogue); `out_mult`: the product is multiplied
    by it first (a constant factor of the residual branch)."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, torch.float32, "out", 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05(_p(a), _p(w), _p(out), m, n, k, int(accumulate), ctypes.c_float(out_mult), _stream()), "gemm_tcgen05")
    return out


def gemm_tcgen05_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out (bfloat16 [M, I]) = silu(a @ w[:I]^T) * (a @ w[I:]^T): the product with SwiGLU as its epilogue."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, torch.bfloat16, "out", 2)
    m, k = a.shape
    inter = out.shape[1]
    if w.shape != (2 * inter, k) or out.shape[0] != m:
        raise KernelError(f"gemm swiglu: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05_swiglu(_p(a), _p(w), _p(out), m, inter, k, _stream()), "gemm_tcgen05_swiglu")
    return out


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor,
                         rows_in_use: Optional[int] = None, activation: str = "relu_squared") -> torch.Tensor:
    """Rows of `a` (bfloat16 [M, K], M a multiple of 128) sorted by group, each 128-row tile with its group's matrix
    w[g] (w bfloat16 [groups, N, K]; tile_group int32 [M / 128], -1: skip the tile).  out float [M, N]: the products;
    out bfloat16 [M, N]: the activation of the products (`activation`: "relu_squared" max(z, 0)^2, "gelu" z Phi(z)).
    `rows_in_use` (how many rows are not padding) only labels measurements."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 3); _need(out, None, "out", 2); _need(tile_group, torch.int32, "tile_group", 1)
    m, k = a.shape
    groups, n, _ = w.shape
    if w.shape[2] != k or out.shape != (m, n) or m % 128 or tile_group.numel() != m // 128 or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm grouped: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05_grouped(_p(a), _p(w), _p(out), m, n, k, groups, _p(tile_group),
                                                1 + EXPERT_ACTIVATIONS[activation] if out.dtype == torch.bfloat16 else 0, _stream()),
           "gemm_tcgen05_grouped")
    return out


def tcgen05_rope_ok(dim: int, rot_half: int, interleaved: bool) -> bool:
    """The rotation epilogue takes heads of 64 or 128 rotated over their whole width in split-half pairs."""
    return dim in (64, 128) and 2 * rot_half == dim and not interleaved


def gemm_tcgen05_grouped_gated(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, limit: float,
                               rows_in_use: Optional[int] = None) -> torch.Tensor:
    """The grouped product of gated experts with the activation as its epilogue: rows of `a` as for `gemm_tcgen05_grouped`,
    w bfloat16 [groups, 2 ff, K] (a group's gate rows, then its up rows), out bfloat16 [M, ff] =
    g' sigmoid(1.702 g') (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit) from the float sums."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 3); _need(out, torch.bfloat16, "out", 2); _need(tile_group, torch.int32, "tile_group", 1)
    m, k = a.shape
    groups, n2, _ = w.shape
    ff = out.shape[1]
    if w.shape[2] != k or n2 != 2 * ff or out.shape[0] != m or m % 128 or tile_group.numel() != m // 128:
        raise KernelError(f"gemm grouped gated: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05_grouped_gated(_p(a), _p(w), _p(out), m, ff, k, groups, _p(tile_group), ctypes.c_float(limit),
                                                      ctypes.c_float(GATE_ALPHA), _stream()), "gemm_tcgen05_grouped_gated")
    return out


def gemm_tcgen05_rope(a: torch.Tensor, w: torch.Tensor, rope: dict) -> None:
    """The stacked q/k/v product with rotation and cache write as its epilogue (`rope` as for skinny_gemm)."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2)
    m, k = a.shape
    hq, hkv, dim = rope["hq"], rope["hkv"], rope["dim"]
    if w.shape != ((hq + 2 * hkv) * dim, k):
        raise KernelError("gemm rope: w must stack the q, k and v heads")
    for name in ("q_out", "k_cache", "v_cache"):
        _need(rope[name], torch.bfloat16, name)
    for name in ("positions", "token_req", "req_slot", "block_table"):
        _need(rope[name], torch.int32, name)
    _need(rope["cos"], torch.float32, "cos", 2); _need(rope["sin"], torch.float32, "sin", 2)
    if rope["cos"].shape != (m, dim // 2):
        raise KernelError("gemm rope: rotary tables must be [tokens, head_dim / 2]")
    _check(_tcgen05().cisr_gemm_tcgen05_rope(
        _p(a), _p(w), m, k, _p(rope["cos"]), _p(rope["sin"]), _p(rope["q_out"]), _p(rope["k_cache"]), _p(rope["v_cache"]),
        _p(rope["positions"]), _p(rope["token_req"]), _p(rope["req_slot"]), _p(rope["block_table"]),
        rope["block_table"].shape[1], rope["page_size"], hq, hkv, dim, _stream()), "gemm_tcgen05_rope")


_GAVE_UP = {1: "a tcgen05 matrix product gave up waiting on a barrier",
            3: "an attention kernel gave up waiting on a tensor-map copy",
            4: "a weight-streaming product gave up waiting on a tensor-map copy",
            5: "the tcgen05 attention gave up waiting on a barrier"}


def error_flag_tensor() -> Optional[torch.Tensor]:
    """The device flag, for callers that copy it to the host behind a step of their own (None before any kernel that
    can give up was loaded)."""
    return _error_state.get("flag")


def raise_for_code(code: int) -> None:
    """The error for a value read from the flag; clears the flag on the device."""
    if code != 0:
        flag = _error_state.get("flag")
        if flag is not None:
            flag.zero_()
        raise KernelError(f"{_GAVE_UP.get(code, _GAVE_UP[1])}; its output is not valid")


def raise_if_kernel_gave_up() -> None:
    """Reads the flag a kernel sets when one of its bounded waits ran out (synchronises the device)."""
    flag = _error_state.get("flag")
    if flag is not None:
        raise_for_code(int(flag.item()))


# ------------------------------------------------------------------ per-launch timing, for measurement only
_timing = {"records": None}


class timed_launches:
    """Inside this context every kernel function of this module is bracketed by two CUDA events on the current stream;
    `records` collects (function name, shape description, begin event, end event).  Used by bench.py for the
    per-kernel figures (launches run one after the other, outside graphs, so these are isolated kernel times); the
    engine never turns it on.  Read the times with `summary()` after a synchronisation."""

    def __enter__(self):
        self.records = []
        _timing["records"] = self.records
        return self

    def __exit__(self, *exc):
        _timing["records"] = None
        return False

    def summary(self) -> dict:
        """(name, shape) -> {"launches", "us"}: total device time between the two events of each launch."""
        torch.cuda.synchronize()
        out = {}
        for name, shape, begin, end in self.records:
            entry = out.setdefault((name, shape), {"launches": 0, "us": 0.0})
            entry["launches"] += 1
            entry["us"] += begin.elapsed_time(end) * 1e3
        return out


def _describe_gemm(a, w, *rest, **kw):
    return (int(a.shape[0]), int(w.shape[0]), int(w.shape[1]))


_DESCRIBE = {
    "embedding": lambda table, ids, out, scale=1.0: (int(out.shape[0]), int(out.shape[1])),
    "add_rmsnorm": lambda x, delta, weight, eps, out, rows=None, write_back=True, delta_scale=None: (int(out.shape[0]), int(out.shape[1]), delta is not None),
    "stream_add": lambda x, *a, **kw: (int(x.shape[0]), int(x.shape[1])),
    "scale_": lambda x, scale: (int(x.numel()),),
    "latent_rows": lambda proj, *a, **kw: (int(proj.shape[0]), int(proj.shape[1])),
    "latent_query": lambda q, *a, **kw: (int(q.shape[0]), int(q.shape[1])),
    "latent_gate": lambda values, *a, **kw: (int(values.shape[0]), int(values.shape[1])),
    "latent_absorb": lambda q, q_col, heads, plain_dim, cos, sin, rot_half, interleaved, k_up, q_rows, kv_rank:
        (int(q.shape[0]), int(heads), int(plain_dim), int(kv_rank)),
    "latent_values": lambda mixed, v_up, *a, **kw: (int(mixed.shape[0]), int(v_up.shape[0]), int(v_up.shape[1]), int(v_up.shape[2])),
    "moe_select": lambda logits, *a, **kw: (int(logits.shape[0]), int(logits.shape[1])),
    "moe_rows": lambda h, w_up, w_down, chosen, *a, **kw: (int(h.shape[0]), int(w_up.shape[0]), int(w_up.shape[1]), int(w_up.shape[2]), int(chosen.shape[1])),
    "moe_sort": lambda chosen, experts, *a: (int(chosen.shape[0]), int(chosen.shape[1]), int(experts)),
    "moe_gather": lambda h, src_token, sorted_h: (int(sorted_h.shape[0]), int(sorted_h.shape[1])),
    "moe_combine": lambda sorted_out, row_of, weight, out, out_scale=None, h=None: (int(out.shape[0]), int(weight.shape[1]), int(out.shape[1])),
    "gemm_tcgen05_grouped": lambda a, w, out, tile_group, rows_in_use=None, activation="relu_squared":
        (int(rows_in_use or a.shape[0]), int(w.shape[0]), int(w.shape[1]), int(w.shape[2]), out.dtype == torch.bfloat16),
    "gemm_tcgen05_grouped_gated": lambda a, w, out, tile_group, limit, rows_in_use=None:
        (int(rows_in_use or a.shape[0]), int(w.shape[0]), int(w.shape[1]), int(w.shape[2])),
    "gemm_heads": lambda a, w, out, w_is_nk: (int(a.shape[0]), int(w.shape[0]), int(w.shape[1]), int(w.shape[2])),
    "swiglu": lambda gate_up, out: (int(out.shape[0]), int(out.shape[1])),
    "rotary_tables": lambda positions, inv_freq, cos, sin, magnitude=1.0: (int(cos.shape[0]), int(cos.shape[1])),
    "hyper_mix_norm": lambda source, streams, n_streams, **kw:
        (int(streams.shape[0] if kw.get("h") is None else kw["h"].shape[0]), int(n_streams), int(streams.shape[2]), kw.get("y") is not None,
         bool(kw.get("store", True)), source.dim() == 2),
    "hyper_sum": lambda streams, out: tuple(int(n) for n in streams.shape),
    "attention_rows": lambda proj, *a, **kw: (int(proj.shape[0]), int(proj.shape[1])),
    "bias_add": lambda out, bias: (int(out.shape[0]), int(out.shape[1])),
    "activation": lambda x, out, kind: (int(x.shape[0]), int(x.shape[1])),
    "delta_prepare": lambda proj, conv_w, taps, *a: (int(proj.shape[0]), int(conv_w.shape[0]), int(taps)),
    "delta_keep": lambda proj, state, req_slot, q_start, q_len, n_req, taps, channels, matrix: (int(n_req), int(channels), int(taps)),
    "delta_chunks": lambda qkv, beta, decay, chunk_req, chunk_t0, n_chunks, req_chunk0, state, req_slot, q_start, q_len, o, n_req, heads,
                           kv_heads, key_dim, value_dim, least: (int(qkv.shape[0]), int(n_req), int(heads), int(kv_heads), int(key_dim), int(value_dim)),
    "delta_recurrence": lambda qkv, beta, decay, state, req_slot, q_start, q_len, o, n_req, heads, kv_heads, key_dim, value_dim, lanes=0, below=0:
        (int(qkv.shape[0]), int(n_req), int(heads), int(kv_heads), int(key_dim), int(value_dim)),
    "delta_output": lambda o, proj, *a: (int(o.shape[0]), int(o.shape[1] * o.shape[2])),
    "diff_rows": lambda proj, conv_w, taps, state, **kw: (int(proj.shape[0]), int(conv_w.shape[1]), int(taps), int(kw["q_out"].shape[1] * kw["q_out"].shape[2]),
                                                         0 if kw.get("k_cache") is None else int(kw["k_cache"].shape[1] * kw["k_cache"].shape[3])),
    "conv_keep": lambda proj, state, req_slot, q_start, q_len, n_req, taps, channels: (int(n_req), int(channels), int(taps)),
    "diff_rope_rows": lambda proj, k_col, v_col, **kw: (int(proj.shape[0]), int(proj.shape[1]), int(kw["q_out"].shape[1] * kw["q_out"].shape[2]),
                                                        0 if kw.get("k_cache") is None else int(kw["k_cache"].shape[1] * kw["k_cache"].shape[3])),
    "lightning_recurrence": lambda proj, q_col, k_col, v_col, decay, state, req_slot, q_start, q_len, n_req, o, heads, key_dim, value_dim, **kw:
        (int(proj.shape[0]), int(n_req), int(heads), int(key_dim), int(value_dim), int(kw["chunks"][3]) if kw.get("chunks") else 0),
    "lightning_output": lambda o, *a, **kw: (int(o.shape[0]), int(o.shape[1])),
    "diff_combine": lambda mixed, gate, gate_col, out, *a: (int(out.shape[0]), int(out.shape[1]), int(mixed.shape[1] * mixed.shape[2])),
    "depth_mix_norm": lambda hist, x, pending, w, n_new, **kw:
        (int(x.shape[0] if kw.get("rows") is None else kw["rows"].numel()), int(n_new), int(x.shape[1]), pending is not None,
         bool(kw.get("store", True)) and kw.get("rows") is None, kw.get("h") is not None),
    "polynorm": lambda z, coef, eps, out: (int(z.shape[0]), int(z.shape[1])),
    "gated_clamp": lambda gate_up, ff, limit, out, scale_col=-1: (int(out.shape[0]), int(ff)),
    "rope_store": lambda proj, *rest, **kw: (int(proj.shape[0]), int(proj.shape[1])),
    "page_copy": lambda *a, **kw: (),
    "table_update": lambda *a, **kw: (),
    # (tokens, query heads, key heads, head width, window or 0); the window is the sixteenth positional argument of both
    "attn_prefill_wide": lambda q, out, k_cache, *rest, **kw: (int(q.shape[0]), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2]), int(rest[12] or 0)),
    "attn_prefill": lambda q, out, k_cache, *rest, **kw: (int(q.shape[0]), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2]), int(rest[12] or 0)),
    "attn_decode": lambda q, out, k_cache, v_cache, req_slot, block_table, dec_req, n_dec, *rest, **kw:
        (int(n_dec), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2]), bool(kw.get("merge", True)), k_cache.data_ptr() == v_cache.data_ptr(),
         int(rest[8] or 0)),
    "merge_out_proj": lambda partial, stats, n_splits, dec_req, q_start, n_dec, hq, dim, w, out, **kw:
        (int(n_dec), int(w.shape[0]), int(w.shape[1]), int(n_splits)),
    "sample": lambda logits, *rest, **kw: (int(logits.shape[0]), int(logits.shape[1])),
    "decode_advance": lambda *a, **kw: (),
    "gemm_library": _describe_gemm,
    "gemm_tcgen05": lambda a, w, out, accumulate=False, out_mult=1.0: _describe_gemm(a, w),
    "gemm_tcgen05_swiglu": _describe_gemm,
    "gemm_tcgen05_rope": _describe_gemm,
    "skinny_gemm": lambda w, tokens, **kw: (int(tokens), int(w.shape[0]), int(w.shape[1]), int(kw.get("epilogue", EPI_PLAIN)),
                                            kw.get("act") is None),
}


def _instrument() -> None:
    import functools

    def wrap(name, describe):
        fn = globals()[name]

        @functools.wraps(fn)
        def launched(*args, **kwargs):
            records = _timing["records"]
            if records is None:
                return fn(*args, **kwargs)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = fn(*args, **kwargs)
            end.record()
            records.append((name, describe(*args, **kwargs), begin, end))
            return result

        globals()[name] = launched

    for name, describe in _DESCRIBE.items():
        wrap(name, describe)


_instrument()
