"""Drop-in replacement for the ops of the reference engine's `kernels.py`.

Same names, positional signatures and semantics as kbwal/inference-engine
qwen3-1.7b/kernels.py (LayerKVCache :11-17, decode_attention :272-361, fused_rope_kv_decode
:483-544, fused_norm_rope_prefill :673-714, quantize_kv_prefill :826-865,
dequantize_kv_prefix :935-970, prefill_attention :1129-1175, silu_mul :1204-1212,
add_rms_norm :1261-1285, sample :1341-1370), backed by hand-written sm_100a CUDA kernels
reached through the C ABI in include/b200kv.h.  There is no Triton, no other backend and no
CPU fallback: without a CUDA device and the built library every op raises.  `linear`
(:1430-1463) is cuBLAS through F.linear unless `tune_linear` (:1465-1485) measured the library's
weight-streaming matmul (`skinny_matmul`, :1373-1428) faster for that weight and row count.

One generalisation: wherever the reference takes `slot_ids [B]` (one contiguous cache row per
sequence), a 2-D int32 block table `[B, max_pages]` is accepted as well, in which case the
cache tensors are read as pages `[num_pages, Hkv, page_size, D]` (page_size a multiple of 16).
The reference layout is the one-page-per-sequence case of the same kernels.
"""
from __future__ import annotations

import ctypes
import functools
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib


@dataclass
class LayerKVCache:
    k: torch.Tensor  # int8  [pool, Hkv, max_len, D]   (paged: [num_pages, Hkv, page_size, D])
    v: torch.Tensor  # int8  [pool, Hkv, max_len, D]
    k_scale: torch.Tensor  # fp32  [pool, Hkv, max_len]
    v_scale: torch.Tensor  # fp32  [pool, Hkv, max_len]
    k_calibration: torch.Tensor  # fp32  [pool, Hkv, 1, D]


def make_layer_cache(num_pages: int, num_kv_heads: int, page_size: int, head_dim: int, device="cuda") -> LayerKVCache:
    """engine.py:472-492: zeroed codes and scales, calibration of ones."""
    return LayerKVCache(
        k=torch.zeros(num_pages, num_kv_heads, page_size, head_dim, device=device, dtype=torch.int8),
        v=torch.zeros(num_pages, num_kv_heads, page_size, head_dim, device=device, dtype=torch.int8),
        k_scale=torch.zeros(num_pages, num_kv_heads, page_size, device=device, dtype=torch.float32),
        v_scale=torch.zeros(num_pages, num_kv_heads, page_size, device=device, dtype=torch.float32),
        k_calibration=torch.ones(num_pages, num_kv_heads, 1, head_dim, device=device, dtype=torch.float32),
    )


# ----------------------------------------------------------------------------- plumbing
@functools.cache
def num_sms(device: torch.device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Device int32 the kernels OR error bits into (bad page id / token position).  Created on
    first use per device, so call any op once before capturing a CUDA graph."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        # a normal tensor even when the first op runs under torch.inference_mode(): check_status clears it in place
        with torch.inference_mode(False):
            t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> int:
    """Read and clear the status word (synchronises).  0 means no device-side error was seen."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = status_word(dev)
    val = int(t.item())
    if val:
        t.zero_()
    return val


_early_start = False


def set_early_start(enabled: bool) -> None:
    """Allow every kernel of this module to be brought up while the kernel enqueued just before it on
    the stream is still running (programmatic dependent launch).  A kernel reads only the step's
    metadata (cu_seqlens, cu_cached, cached_lens, num_decoding, block table, tile_start, seq_ids)
    before it waits for that kernel, and everything else afterwards.  Safe when no kernel that
    directly precedes one of these ops on its stream writes those arrays, which holds for the engine:
    it uploads them once per step, before the first layer (engine.py:347-356), and the ops are
    preceded by GEMMs or by one another (architecture.py:99-198).  Off by default."""
    global _early_start
    _early_start = bool(enabled)
    _lib.load().b200kv_set_chained_launch(1 if enabled else 0)


_workspaces: dict[tuple, torch.Tensor] = {}


def decode_workspace(device: torch.device, B: int, Hq: int, Hkv: int, nbytes: int) -> torch.Tensor:
    """Workspace of decode_attention (split partials + arrival counters) for one (device, batch
    size, head counts), allocated zeroed on first use and reused by every later call of that shape:
    the C ABI wants the counters zero on entry and leaves them zero, and their place in the buffer
    depends on B.  Calls on one device must be stream-ordered (the reference engine is
    single-stream); a new shape allocates, so run each shape once before graph capture (the
    engine's capture_graph warm-up does)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, B, Hq, Hkv)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("decode_attention workspace must exist before CUDA-graph capture: "
                               "run the same call once eagerly first")
        ws = torch.zeros(nbytes, device=torch.device("cuda", idx), dtype=torch.uint8)
        _workspaces[key] = ws
    return ws


_nvtx = False


def set_nvtx(enabled: bool) -> None:
    """Bracket every op of this module in an NVTX range named after it, as the reference's callers do around
    theirs (architecture.py:84,100,115,200).  Off by default: a range costs two host calls per op."""
    global _nvtx
    _nvtx = bool(enabled)


def _ranged(fn):
    """The op inside an NVTX range of its own name while set_nvtx(True) is in force."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        if not _nvtx:
            return fn(*args, **kwargs)
        torch.cuda.nvtx.range_push(fn.__name__)
        try:
            return fn(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()

    return wrapper


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("b200kv ops need CUDA tensors: there is no CPU path")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cache_struct(cache: LayerKVCache) -> _lib.Cache:
    k, v, ks, vs, cal = cache.k, cache.v, cache.k_scale, cache.v_scale, cache.k_calibration
    assert k.stride() == v.stride(), "kernel uses one set of strides for k and v"
    assert ks.stride() == vs.stride()
    assert k.dtype == torch.int8 and v.dtype == torch.int8 and ks.dtype == torch.float32 and cal.dtype == torch.float32
    assert k.stride(3) == 1 and ks.stride(2) == 1 and cal.stride(3) == 1
    return _lib.Cache(
        k.data_ptr(), v.data_ptr(), ks.data_ptr(), vs.data_ptr(), cal.data_ptr(),
        k.stride(0), k.stride(1), k.stride(2), ks.stride(0), ks.stride(1), cal.stride(0), cal.stride(1),
        k.shape[0], k.shape[1], k.shape[2], k.shape[3])


def _table_struct(slot_ids: torch.Tensor) -> _lib.Table:
    assert slot_ids.dtype == torch.int32, "slot ids / block table must be int32"
    if slot_ids.ndim == 1:
        assert slot_ids.numel() <= 1 or slot_ids.stride(0) >= 1
        return _lib.Table(slot_ids.data_ptr(), slot_ids.stride(0) if slot_ids.numel() > 1 else 1, 1)
    assert slot_ids.ndim == 2 and (slot_ids.stride(1) == 1 or slot_ids.shape[1] == 1)
    return _lib.Table(slot_ids.data_ptr(), slot_ids.stride(0), slot_ids.shape[1])


def _i32(t: torch.Tensor) -> int:
    assert t.dtype == torch.int32 and (t.numel() <= 1 or t.stride(-1) == 1)
    return t.data_ptr()


def _row_stride(t: torch.Tensor) -> int:
    """Entry stride of a [N, 1, D/2] or [N, D/2] rope table."""
    assert t.stride(-1) == 1
    return t.stride(0)


# ----------------------------------------------------------------------------- ops
@_ranged
def plan_decode_step(
    cached_lens: torch.Tensor,  # [B]
    slot_ids: torch.Tensor,  # [B] or [B, max_pages]
    num_decoding: torch.Tensor,  # int32 [1]
    kv_cache: LayerKVCache,  # any layer's cache of the step: only its head count and page size are used
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """The work split of decode_attention for one decoder step, computed once (one small kernel) and
    handed to every layer's call as `decode_attention(..., plan=plan)`.  It is a function of
    cached_lens, num_decoding and the block table only, which the engine uploads once per step
    (engine.py:347-356, 461-465) and no layer changes.  Not part of the reference's interface:
    without a plan decode_attention derives the same split inside every launch.  The plan must be
    remade whenever those three arrays change; under a CUDA graph, capture this call at the head of
    the step.  `out`: a uint8 buffer of plan_decode_bytes(device) to reuse."""
    _require_cuda(cached_lens, slot_ids, num_decoding, kv_cache.k)
    lib = _lib.load()
    dev = cached_lens.device
    sms = num_sms(dev)
    nbytes = lib.b200kv_decode_plan_bytes(sms)
    if out is None:
        out = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    assert out.dtype == torch.uint8 and out.numel() >= nbytes and out.is_contiguous()
    ts = _table_struct(slot_ids)
    rc = lib.b200kv_decode_plan(ctypes.byref(ts), _i32(cached_lens), _i32(num_decoding), cached_lens.shape[0],
                                kv_cache.k.shape[1], kv_cache.k.shape[2], sms, out.data_ptr(), out.numel(), _stream())
    _lib.check(rc, "plan_decode_step")
    return out


def plan_decode_bytes(device: torch.device) -> int:
    return int(_lib.load().b200kv_decode_plan_bytes(num_sms(device)))


@_ranged
def decode_attention(
    q: torch.Tensor,  # [B, Hq, D], one new token per sequence
    kv_cache: LayerKVCache,
    cached_lens: torch.Tensor,  # [B], tokens already cached per sequence
    slot_ids: torch.Tensor,  # [B] cache row per sequence, or [B, max_pages] block table
    num_decoding: torch.Tensor,  # int32 [1]
    scale,
    out: torch.Tensor | None = None,  # [>= B, Hq, D]
    variant: int = 0,
    plan: torch.Tensor | None = None,  # from plan_decode_step for this step's metadata (not a reference argument)
):
    _require_cuda(q, kv_cache.k, cached_lens, slot_ids, num_decoding)
    lib = _lib.load()
    B, Hq, D = q.shape
    Hkv = kv_cache.k.shape[1]
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1
    if out is None:
        out = torch.empty(B, Hq, D, device=q.device, dtype=q.dtype)
    assert out.shape[0] >= B and out.shape[1:] == (Hq, D) and out.stride(-1) == 1
    sms = num_sms(q.device)
    if plan is not None:
        # The plan was made for all entries of cached_lens (plan_decode_step), and the kernel checks that.  q and out
        # need only hold the rows of the decoding entries, which come first: a caller that packs tokens (a mixed
        # step with fewer tokens than entries) may pass fewer rows than entries.
        B = cached_lens.shape[0]
    nbytes = lib.b200kv_decode_attn_workspace_bytes(B, Hq, Hkv, D, sms)
    if nbytes == 0:
        raise ValueError("decode_attention: unsupported geometry")
    workspace = decode_workspace(q.device, B, Hq, Hkv, nbytes)
    cs, ts = _cache_struct(kv_cache), _table_struct(slot_ids)
    variant = variant | (4 if _early_start else 0)
    if plan is None:
        rc = lib.b200kv_decode_attn(
            q.data_ptr(), q.stride(0), q.stride(1), ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens),
            _i32(num_decoding), float(scale), out.data_ptr(), out.stride(0), out.stride(1), workspace.data_ptr(),
            workspace.numel(), B, Hq, sms, variant, status_word(q.device).data_ptr(), _stream())
    else:
        assert plan.dtype == torch.uint8 and plan.is_cuda
        rc = lib.b200kv_decode_attn_planned(
            q.data_ptr(), q.stride(0), q.stride(1), ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens),
            _i32(num_decoding), float(scale), out.data_ptr(), out.stride(0), out.stride(1), workspace.data_ptr(),
            workspace.numel(), plan.data_ptr(), plan.numel(), B, Hq, sms, variant,
            status_word(q.device).data_ptr(), _stream())
    _lib.check(rc, "decode_attention")
    return out


@_ranged
def decode_attention_static(q, kv_cache: LayerKVCache, cached_lens, slot_ids, num_decoding, scale, out: torch.Tensor):
    """decode_attention for callers that must not allocate device memory at this point (all of it
    already belongs to their own pool, or an allocator call is not allowed where they run): the
    kernel's scratch is an 8 MiB array built into the library instead of a tensor, and `out` must
    be supplied, so nothing here allocates.  Same result as decode_attention.  Raises ValueError
    when the batch needs more than the built-in scratch.  Calls on one device share that array:
    keep them stream-ordered.  Make the first call on a device outside any graph capture."""
    _require_cuda(q, kv_cache.k, cached_lens, slot_ids, num_decoding, out)
    lib = _lib.load()
    B, Hq, D = q.shape
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1
    assert out.shape[0] >= B and out.shape[1:] == (Hq, D) and out.stride(-1) == 1
    cs, ts = _cache_struct(kv_cache), _table_struct(slot_ids)
    rc = lib.b200kv_decode_attn_static(
        q.data_ptr(), q.stride(0), q.stride(1), ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens),
        _i32(num_decoding), float(scale), out.data_ptr(), out.stride(0), out.stride(1), B, Hq, num_sms(q.device),
        status_word(q.device).data_ptr(), _stream())
    _lib.check(rc, "decode_attention_static")
    return out


@_ranged
def fused_rope_kv_decode(
    q: torch.Tensor,  # (B, Hq, D), one new token per sequence
    k: torch.Tensor,  # (B, Hkv, D)
    v: torch.Tensor,
    q_norm_weight: torch.Tensor,  # (D,)
    k_norm_weight: torch.Tensor,
    cos: torch.Tensor,  # (B, 1, D // 2)
    sin: torch.Tensor,
    slot_ids: torch.Tensor,
    kv_cache: LayerKVCache,
    cached_lens: torch.Tensor,
    num_decoding: torch.Tensor,
    eps: float,
):
    """Returns normed + roped q (times calibration) and writes the new K/V token into the cache."""
    _require_cuda(q, k, v, kv_cache.k)
    lib = _lib.load()
    B, Hq, D = q.shape
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    out = torch.empty(B, Hq, D, device=q.device, dtype=q.dtype)
    cs, ts = _cache_struct(kv_cache), _table_struct(slot_ids)
    rc = lib.b200kv_write_decode(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0),
        v.stride(1), q_norm_weight.data_ptr(), k_norm_weight.data_ptr(), cos.data_ptr(), _row_stride(cos),
        sin.data_ptr(), _row_stride(sin), ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens), _i32(num_decoding),
        out.data_ptr(), out.stride(0), out.stride(1), B, Hq, float(eps), status_word(q.device).data_ptr(), _stream())
    _lib.check(rc, "fused_rope_kv_decode")
    return out


@_ranged
def fused_norm_rope_prefill(
    q: torch.Tensor,  # bf16 [N, Hq, D]
    k: torch.Tensor,  # bf16 [N, Hkv, D]
    q_norm_weight: torch.Tensor,
    k_norm_weight: torch.Tensor,
    cos: torch.Tensor,  # [N, 1, D // 2]
    sin: torch.Tensor,
    eps: float,
) -> tuple[torch.Tensor, torch.Tensor]:
    _require_cuda(q, k)
    lib = _lib.load()
    N, Hq, D = q.shape
    Hkv = k.shape[1]
    assert q.stride(-1) == 1 and k.stride(-1) == 1, "kernel assumes contiguous head_dim"
    assert cos.stride(-1) == 1 and sin.stride(-1) == 1
    q_out = torch.empty(N, Hq, D, device=q.device, dtype=q.dtype)
    k_out = torch.empty(N, Hkv, D, device=k.device, dtype=k.dtype)
    rc = lib.b200kv_norm_rope_prefill(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), q_norm_weight.data_ptr(),
        k_norm_weight.data_ptr(), cos.data_ptr(), _row_stride(cos), sin.data_ptr(), _row_stride(sin), q_out.data_ptr(),
        q_out.stride(0), q_out.stride(1), k_out.data_ptr(), k_out.stride(0), k_out.stride(1), N, Hq, Hkv, D, float(eps),
        _stream())
    _lib.check(rc, "fused_norm_rope_prefill")
    return q_out, k_out


@_ranged
def quantize_kv_prefill(
    k: torch.Tensor,  # bf16 [N, Hkv, D], all sequences packed along N
    v: torch.Tensor,
    cu_seqlens: torch.Tensor,  # int32 [B + 1]
    slot_ids: torch.Tensor,
    cached_lens: torch.Tensor,
    num_decoding: torch.Tensor,
    cache: LayerKVCache,
):
    _require_cuda(k, v, cache.k)
    lib = _lib.load()
    N = k.shape[0]
    assert k.stride(-1) == 1 and v.stride(-1) == 1, "kernel assumes contiguous head_dim"
    cs, ts = _cache_struct(cache), _table_struct(slot_ids)
    rc = lib.b200kv_quantize_prefill(
        k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0), v.stride(1), _i32(cu_seqlens),
        cu_seqlens.shape[0] - 1, ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens), _i32(num_decoding), N,
        status_word(k.device).data_ptr(), _stream())
    _lib.check(rc, "quantize_kv_prefill")


@_ranged
def write_prefill(
    q: torch.Tensor,  # bf16 [N, Hq, D], raw projections, all sequences packed along N
    k: torch.Tensor,  # bf16 [N, Hkv, D]
    v: torch.Tensor,
    q_norm_weight: torch.Tensor,
    k_norm_weight: torch.Tensor,
    cos: torch.Tensor,  # [N, 1, D // 2]
    sin: torch.Tensor,
    cu_seqlens: torch.Tensor,  # int32 [B + 1]
    slot_ids: torch.Tensor,
    cached_lens: torch.Tensor,
    num_decoding: torch.Tensor,
    cache: LayerKVCache,
    eps: float,
) -> tuple[torch.Tensor, torch.Tensor]:
    """fused_norm_rope_prefill followed by quantize_kv_prefill as one call (not a reference function; the
    reference's caller makes the two calls, architecture.py:133-150): returns the same (q_p, k_p) and leaves the
    same bytes in the cache."""
    _require_cuda(q, k, v, cache.k)
    lib = _lib.load()
    N, Hq, D = q.shape
    Hkv = k.shape[1]
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert cos.stride(-1) == 1 and sin.stride(-1) == 1
    q_out = torch.empty(N, Hq, D, device=q.device, dtype=q.dtype)
    k_out = torch.empty(N, Hkv, D, device=k.device, dtype=k.dtype)
    cs, ts = _cache_struct(cache), _table_struct(slot_ids)
    rc = lib.b200kv_write_prefill(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0),
        v.stride(1), q_norm_weight.data_ptr(), k_norm_weight.data_ptr(), cos.data_ptr(), _row_stride(cos), sin.data_ptr(),
        _row_stride(sin), _i32(cu_seqlens), cu_seqlens.shape[0] - 1, ctypes.byref(cs), ctypes.byref(ts), _i32(cached_lens),
        _i32(num_decoding), q_out.data_ptr(), q_out.stride(0), q_out.stride(1), k_out.data_ptr(), k_out.stride(0),
        k_out.stride(1), N, Hq, float(eps), status_word(q.device).data_ptr(), _stream())
    _lib.check(rc, "write_prefill")
    return q_out, k_out


@_ranged
def dequantize_kv_prefix(
    cache: LayerKVCache,
    cu_cached: torch.Tensor,  # int32 [B + 1]
    slot_ids: torch.Tensor,
    k_out: torch.Tensor,  # bf16 [Hkv, >= total_cached, D]
    v_out: torch.Tensor,
):
    _require_cuda(cache.k, k_out, v_out)
    lib = _lib.load()
    assert k_out.stride() == v_out.stride() and k_out.stride(-1) == 1
    cs, ts = _cache_struct(cache), _table_struct(slot_ids)
    rc = lib.b200kv_dequant_prefix(
        ctypes.byref(cs), ctypes.byref(ts), _i32(cu_cached), cu_cached.shape[0] - 1, k_out.data_ptr(), v_out.data_ptr(),
        k_out.stride(0), k_out.stride(1), k_out.shape[1], status_word(k_out.device).data_ptr(), _stream())
    _lib.check(rc, "dequantize_kv_prefix")


@_ranged
def prefill_attention(
    q: torch.Tensor,  # bf16 [N, Hq, D]
    k: torch.Tensor,  # bf16 [N, Hkv, D]
    v: torch.Tensor,
    seq_ids: torch.Tensor,  # [N]
    cu_seqlens: torch.Tensor,  # [B + 1] int32
    tile_start: torch.Tensor,  # [num_tiles] int32
    k_prefix: torch.Tensor,  # bf16 [Hkv, total_cached, D]
    v_prefix: torch.Tensor,
    cu_cached: torch.Tensor,  # [B + 1] int32
    PREFILL_BLOCK_M: int,
    *,
    variant: int = 0,  # 0 = automatic, 1 = mma.sync kernel, 2 = tcgen05 kernel (not a reference argument)
) -> torch.Tensor:
    _require_cuda(q, k, v)
    lib = _lib.load()
    N, Hq, D = q.shape
    Hkv = k.shape[1]
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert k_prefix.stride() == v_prefix.stride() and k_prefix.stride(-1) == 1
    out = torch.empty(N, Hq, D, device=q.device, dtype=q.dtype)
    rc = lib.b200kv_prefill_attn_variant(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(), v.stride(0),
        v.stride(1), _i32(seq_ids), _i32(cu_seqlens), _i32(tile_start), tile_start.shape[0], int(PREFILL_BLOCK_M),
        k_prefix.data_ptr(), v_prefix.data_ptr(), k_prefix.stride(0), k_prefix.stride(1), k_prefix.shape[1],
        _i32(cu_cached), out.data_ptr(), out.stride(0), out.stride(1), N, Hq, Hkv, D, int(variant),
        status_word(q.device).data_ptr(), _stream())
    _lib.check(rc, "prefill_attention")
    return out


# ----------------------------------------------------------------------------- decoder-block ops
# The two element-wise ops between the attention path and the GEMMs, as CUDA kernels behind the same C ABI.
@_ranged
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """kernels.py:1204-1212: bf16 [N, 2D] -> bf16 [N, D] = silu(gate) * up."""
    _require_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.stride(-1) == 1 and gate_up.dtype == torch.bfloat16
    N, two_d = gate_up.shape
    out = torch.empty(N, two_d // 2, device=gate_up.device, dtype=gate_up.dtype)
    rc = _lib.load().b200kv_silu_mul(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), out.stride(0), N, two_d // 2,
                                     _stream())
    _lib.check(rc, "silu_mul")
    return out


@_ranged
def add_rms_norm(residual: torch.Tensor, delta: torch.Tensor, rms_norm: torch.Tensor, eps: float):
    """kernels.py:1261-1285: (residual + delta, rmsnorm(residual + delta) * weight), bf16 [N, D] each."""
    _require_cuda(residual, delta, rms_norm)
    assert residual.dim() == 2 and residual.shape == delta.shape and residual.dtype == torch.bfloat16
    assert residual.stride(-1) == 1 and delta.stride(-1) == 1 and rms_norm.is_contiguous()
    N, D = residual.shape
    new_residual = torch.empty_like(residual)
    normed = torch.empty_like(residual)
    rc = _lib.load().b200kv_add_rms_norm(residual.data_ptr(), residual.stride(0), delta.data_ptr(), delta.stride(0),
                                         rms_norm.data_ptr(), new_residual.data_ptr(), new_residual.stride(0),
                                         normed.data_ptr(), normed.stride(0), N, D, ctypes.c_float(eps), _stream())
    _lib.check(rc, "add_rms_norm")
    return new_residual, normed


# ----------------------------------------------------------------------------- scaffold ops
# The remaining names the reference's architecture.py / engine.py import from kernels.py.  They
# are outside the attention path; plain PyTorch keeps a model built on this module runnable.
@_ranged
def sample(logits: torch.Tensor, tau: float, seed: torch.Tensor) -> torch.Tensor:
    """kernels.py:1341-1370: Gumbel-max sampling (tau = 0: greedy argmax), int64 [B, 1]; `seed` (int64 [1] on
    the device) advances by one."""
    _require_cuda(logits, seed)
    assert logits.dim() == 2 and logits.stride(-1) == 1, "kernel assumes contiguous vocab dim"
    assert logits.dtype in (torch.bfloat16, torch.float32) and seed.dtype == torch.int64
    B, V = logits.shape
    lib = _lib.load()
    nbytes = lib.b200kv_sample_workspace_bytes(B, V)
    ws = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=logits.device)
    out = torch.empty(B, 1, dtype=torch.int64, device=logits.device)
    rc = lib.b200kv_sample(logits.data_ptr(), logits.stride(0), logits.element_size(), seed.data_ptr(), ctypes.c_float(tau),
                           ws.data_ptr(), nbytes, out.data_ptr(), out.stride(0), B, V, _stream())
    _lib.check(rc, "sample")
    return out


def skinny_matmul(x: torch.Tensor, weight: torch.Tensor, splits: int = 1) -> torch.Tensor:
    """kernels.py:1430-1455: [M, K] bf16 @ [N, K] bf16 .T -> [M, N] bf16 for M <= 64, the weight read once from HBM
    (tcgen05 kernel behind b200kv_skinny_linear).  `splits` = CTAs sharing a block of 128 weight rows (1, 2, 4, 8)."""
    _require_cuda(x, weight)
    M, K = x.shape
    N = weight.shape[0]
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert x.stride(-1) == 1 and weight.stride(-1) == 1
    assert M <= 64, "many rows are compute bound: cuBLAS is the tool there"
    y = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
    rc = _lib.load().b200kv_skinny_linear(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), y.data_ptr(),
                                          y.stride(0), M, N, K, int(splits), status_word(x.device).data_ptr(), _stream())
    _lib.check(rc, "skinny_matmul")
    return y


# (N, K, M) -> cluster size with which skinny_matmul beat cuBLAS for that weight shape and row count (0: cuBLAS won).
# Filled by tune_linear before graph capture; anything it never measured uses cuBLAS (kernels.py:1458-1470).
use_skinny: dict[tuple[int, int, int], int] = {}


def skinny_supported(M: int, N: int, K: int) -> list[int]:
    """The cluster sizes b200kv_skinny_linear accepts for this shape ([] = not at all)."""
    if M < 1 or M > 64 or N % 128 or K % 64 or K < 64:
        return []
    T = 16 if M <= 16 else (32 if M <= 32 else 64)
    return [s for s in (1, 2, 4, 8) if s <= T // 2 and s <= K // 64]


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:  # kernels.py:1465
    """[M, K] @ [N, K].T -> [M, N] with whichever of skinny_matmul and cuBLAS (F.linear) tune_linear measured faster
    for this (weight shape, row count); unmeasured shapes go to cuBLAS."""
    if x.dim() == 2 and x.stride(-1) == 1 and weight.stride(-1) == 1:
        s = use_skinny.get((weight.shape[0], weight.shape[1], x.shape[0]), 0)
        if s:
            return skinny_matmul(x, weight, s)
    return F.linear(x, weight)


def tune_linear(weights, rows, min_gain: float = 0.02) -> None:
    """kernels.py:1473-1485: time skinny_matmul (every cluster size the shape allows) against cuBLAS for each weight
    shape at each row count <= 64 and keep the faster; skinny_matmul has to win by `min_gain` to be picked.  L2 is
    flushed before every timed call, as in the model, where each layer's weights come from HBM."""
    if not weights:
        return
    dev = weights[0].device
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)

    def time_us(fn, reps: int = 5) -> float:
        fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return sorted(ts)[len(ts) // 2]

    for weight in weights:
        N, K = weight.shape
        for M in rows:
            if M > 64 or (N, K, M) in use_skinny or weight.dtype != torch.bfloat16 or weight.stride(-1) != 1:
                continue
            options = skinny_supported(M, N, K)
            if not options:
                use_skinny[(N, K, M)] = 0
                continue
            x = torch.randn(M, K, device=dev, dtype=weight.dtype)
            cublas = time_us(lambda: F.linear(x, weight))
            best, best_s = cublas * (1.0 - min_gain), 0
            for s in options:
                t = time_us(lambda: skinny_matmul(x, weight, s))
                if t < best:
                    best, best_s = t, s
            use_skinny[(N, K, M)] = best_s
    check_status(dev)
