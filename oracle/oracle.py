"""CPU restatement of the int8-KV-cache attention path (TEST INFRASTRUCTURE ONLY).

This module is the checker the CUDA kernels are compared against.  It is imported only
by tests, the smoke check and the benchmark's CPU-baseline leg; the product package never
imports it and has no CPU fallback.

Every function restates one function of the reference engine, file qwen3-1.7b/kernels.py
(cited per function as kernels.py:LINES), in numpy float32 with a fixed operation order:
IEEE fp32 add/mul/div/sqrt, no fused multiply-add, and numpy's pairwise order for the
64-element sums.  That is the arithmetic the reference's own Triton kernels perform when
they are executed by Triton's CPU interpreter, which is how this restatement is pinned
(tests/golden/make_golden.py runs the unmodified reference kernels there and stores their
outputs; tests/test_oracle_golden.py compares).

Conventions
-----------
* bf16 tensors are carried as float32 arrays whose values are bf16-representable.
  `bf16_round` rounds float32 to bf16 with round-to-nearest-even (what the GPU does on a
  bf16 store); `bf16_trunc` chops (what Triton's CPU interpreter does) and exists only so
  the restatement can be compared with interpreter output.
* The cache is the reference's LayerKVCache (kernels.py:11-17) generalised to pages:
  k, v int8 [num_pages, Hkv, page_size, D]; k_scale, v_scale fp32 [num_pages, Hkv, page_size];
  k_calibration fp32 [num_pages, Hkv, 1, D].  `table` is either the reference's slot_ids [B]
  (one page per sequence, page_size = max_len) or a block table [B, max_pages].  Token t of
  sequence b lives in page table[b, t // page_size] at row t % page_size; the calibration
  row of a sequence is that of its first page.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------- bf16 helpers
def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    out = r.view(np.float32).copy()
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.nan
    return out.reshape(x.shape)


def bf16_trunc(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 by dropping the low 16 bits (Triton CPU-interpreter behaviour)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32).reshape(x.shape)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """bf16-representable float32 -> uint16 bit patterns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) >> 16).astype(np.uint16).reshape(x.shape)


def from_bf16_bits(u: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(u, dtype=np.uint16)
    return (u.astype(np.uint32) << 16).view(np.float32).reshape(u.shape)


_ROUND = {"rne": bf16_round, "trunc": bf16_trunc}


# --------------------------------------------------------------------------- cache type
@dataclass
class KVCache:
    """LayerKVCache of kernels.py:11-17 with the slot axis read as a page axis."""

    k: np.ndarray  # int8 [num_pages, Hkv, page_size, D]
    v: np.ndarray  # int8 [num_pages, Hkv, page_size, D]
    k_scale: np.ndarray  # fp32 [num_pages, Hkv, page_size]
    v_scale: np.ndarray  # fp32 [num_pages, Hkv, page_size]
    k_calibration: np.ndarray  # fp32 [num_pages, Hkv, 1, D]

    @property
    def page_size(self) -> int:
        return self.k.shape[2]

    def copy(self) -> "KVCache":
        return KVCache(*(a.copy() for a in (self.k, self.v, self.k_scale, self.v_scale, self.k_calibration)))


def make_cache(num_pages: int, Hkv: int, page_size: int, D: int) -> KVCache:
    """engine.py:472-492: zero codes and scales, calibration of ones."""
    return KVCache(
        np.zeros((num_pages, Hkv, page_size, D), np.int8),
        np.zeros((num_pages, Hkv, page_size, D), np.int8),
        np.zeros((num_pages, Hkv, page_size), np.float32),
        np.zeros((num_pages, Hkv, page_size), np.float32),
        np.ones((num_pages, Hkv, 1, D), np.float32),
    )


def _table2d(table: np.ndarray) -> np.ndarray:
    table = np.asarray(table)
    return table[:, None] if table.ndim == 1 else table


def locate(cache: KVCache, table: np.ndarray, b: int, t) -> tuple[np.ndarray, np.ndarray]:
    """(page, row) of token(s) t of sequence b: kernels.py:147,169,455 with a block table."""
    t = np.asarray(t)
    P = cache.page_size
    tab = _table2d(table)
    return tab[b, t // P], t % P


# --------------------------------------------------------------------------- arithmetic atoms
def pairwise_sum64(a: np.ndarray) -> np.ndarray:
    """Sum of the last axis (length 64) in numpy's pairwise order for n < 128:
    eight strided running sums r[j] += a[8i+j] (i ascending), then
    ((r0+r1)+(r2+r3)) + ((r4+r5)+(r6+r7)).  This is what `tl.sum` over 64 lanes evaluates to
    in the interpreter (kernels.py:417,426,594,615)."""
    a = np.asarray(a, dtype=np.float32)
    assert a.shape[-1] == 64
    r = a[..., 0:8].copy()
    for i in range(1, 8):
        r = r + a[..., 8 * i : 8 * i + 8]
    return ((r[..., 0] + r[..., 1]) + (r[..., 2] + r[..., 3])) + ((r[..., 4] + r[..., 5]) + (r[..., 6] + r[..., 7]))


def norm_rope(x: np.ndarray, w: np.ndarray, cos: np.ndarray, sin: np.ndarray, eps: float) -> np.ndarray:
    """Per-head RMSNorm followed by half-split (neox) rotation, all fp32.

    x [T, H, D] (bf16 values), w [D] (bf16 values), cos/sin [T, D/2] (bf16 values).
    kernels.py:410-436 (decode) and :579-633 (prefill) are the same arithmetic:
      rstd = 1 / sqrt((sum(x1^2) + sum(x2^2)) / D + eps);  y = (x * rstd) * w;
      out1 = y1*cos - y2*sin;  out2 = y1*sin + y2*cos
    """
    x = np.asarray(x, np.float32)
    T, H, D = x.shape
    h = D // 2
    assert h == 64, "the pairwise order restated here is for head_dim 128"
    w = np.asarray(w, np.float32)
    x1, x2 = x[..., :h], x[..., h:]
    ss = pairwise_sum64(x1 * x1) + pairwise_sum64(x2 * x2)  # [T, H]
    rstd = F32(1.0) / np.sqrt(ss / F32(D) + F32(eps))
    y1 = (x1 * rstd[..., None]) * w[:h]
    y2 = (x2 * rstd[..., None]) * w[h:]
    c = np.asarray(cos, np.float32).reshape(T, 1, h)
    s = np.asarray(sin, np.float32).reshape(T, 1, h)
    o1 = y1 * c - y2 * s
    o2 = y1 * s + y2 * c
    return np.concatenate([o1, o2], axis=-1).astype(np.float32)


def quantize_rows(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-row absmax int8 quantizer, kernels.py:460-480 and :798-811.

    scale = max(absmax, 1e-6) / 127 (fp32 divide); code = clamp(rint(x / scale), -127, 127).
    x [..., D] fp32 -> (int8 [..., D], fp32 [...])."""
    x = np.asarray(x, np.float32)
    amax = np.max(np.abs(x), axis=-1)
    scale = (np.maximum(amax, F32(1e-6)) / F32(127.0)).astype(np.float32)
    codes = np.clip(np.rint(x / scale[..., None]), F32(-127.0), F32(127.0)).astype(np.int8)
    return codes, scale


# --------------------------------------------------------------------------- write paths
def write_decode(q, k, v, q_norm_w, k_norm_w, cos, sin, table, cache: KVCache, cached_lens,
                 num_decoding: int, eps: float, bf16: str = "rne") -> np.ndarray:
    """fused_rope_kv_decode, kernels.py:364-544.

    For every decoding entry b < num_decoding: normalise + rotate q and k in fp32; q' =
    q * calibration -> bf16 (returned); k / calibration -> int8 + scale written at token
    position cached_lens[b]; v -> int8 + scale at the same position.  Rows b >= num_decoding
    of the returned q' are left as zeros here (the reference leaves them unwritten).
    q [B,Hq,D], k,v [B,Hkv,D], cos,sin [B,1,D/2] or [B,D/2]; mutates `cache`."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    tab = _table2d(table)
    out = np.zeros((B, Hq, D), np.float32)
    nd = int(num_decoding)
    if nd == 0:
        return out
    cos2 = np.asarray(cos, np.float32).reshape(B, D // 2)
    sin2 = np.asarray(sin, np.float32).reshape(B, D // 2)
    qn = norm_rope(q[:nd], q_norm_w, cos2[:nd], sin2[:nd], eps)
    kn = norm_rope(k[:nd], k_norm_w, cos2[:nd], sin2[:nd], eps)
    for b in range(nd):
        cal = cache.k_calibration[tab[b, 0], :, 0, :]  # [Hkv, D]
        out[b] = _ROUND[bf16](qn[b] * np.repeat(cal, G, axis=0))  # kernels.py:440-447
        page, row = locate(cache, table, b, int(cached_lens[b]))
        kc, ks = quantize_rows(kn[b] / cal)  # kernels.py:456-470
        vc, vs = quantize_rows(v[b])  # kernels.py:472-480
        cache.k[page, :, row, :] = kc
        cache.k_scale[page, :, row] = ks
        cache.v[page, :, row, :] = vc
        cache.v_scale[page, :, row] = vs
    return out


def norm_rope_prefill(q, k, q_norm_w, k_norm_w, cos, sin, eps: float, bf16: str = "rne"):
    """fused_norm_rope_prefill, kernels.py:547-714: norm + rope of every packed row,
    outputs rounded to bf16 (q_out [N,Hq,D], k_out [N,Hkv,D])."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    N, _, D = q.shape
    cos2 = np.asarray(cos, np.float32).reshape(N, D // 2)
    sin2 = np.asarray(sin, np.float32).reshape(N, D // 2)
    rnd = _ROUND[bf16]
    return rnd(norm_rope(q, q_norm_w, cos2, sin2, eps)), rnd(norm_rope(k, k_norm_w, cos2, sin2, eps))


def quantize_prefill(k, v, cu_seqlens, table, cached_lens, num_decoding: int, cache: KVCache) -> None:
    """quantize_kv_prefill, kernels.py:717-865.

    For every entry b >= num_decoding with a non-empty chunk: if nothing is cached yet the
    per-channel calibration max(1e-3, max_t |k[t,d]|) is computed from this chunk and stored,
    otherwise it is loaded; then k / calibration and v are quantized row by row into token
    positions cached_lens[b] + t.  k is the bf16 output of norm_rope_prefill."""
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    tab = _table2d(table)
    S = len(cu_seqlens) - 1
    for b in range(int(num_decoding), S):
        s0, s1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if s1 - s0 == 0:
            continue
        c0 = int(cached_lens[b])
        kb, vb = k[s0:s1], v[s0:s1]  # [L, Hkv, D]
        first = tab[b, 0]
        if c0 == 0:
            cal = np.maximum(F32(1e-3), np.max(np.abs(kb), axis=0)).astype(np.float32)  # [Hkv, D]
            cache.k_calibration[first, :, 0, :] = cal
        else:
            cal = cache.k_calibration[first, :, 0, :]
        kc, ks = quantize_rows(kb / cal[None])
        vc, vs = quantize_rows(vb)
        pages, rows = locate(cache, table, b, c0 + np.arange(s1 - s0))
        for t in range(s1 - s0):
            cache.k[pages[t], :, rows[t], :] = kc[t]
            cache.v[pages[t], :, rows[t], :] = vc[t]
            cache.k_scale[pages[t], :, rows[t]] = ks[t]
            cache.v_scale[pages[t], :, rows[t]] = vs[t]


def dequantize_prefix(cache: KVCache, cu_cached, table, k_out: np.ndarray, v_out: np.ndarray,
                      bf16: str = "rne") -> None:
    """dequantize_kv_prefix, kernels.py:868-970: for entry b, rows [cu_cached[b], cu_cached[b+1])
    of k_out/v_out [Hkv, >=total, D] receive bf16((code * k_scale) * calibration) and
    bf16(code * v_scale) of the entry's first cu_cached[b+1]-cu_cached[b] cached tokens."""
    tab = _table2d(table)
    rnd = _ROUND[bf16]
    for b in range(len(cu_cached) - 1):
        o0, o1 = int(cu_cached[b]), int(cu_cached[b + 1])
        n = o1 - o0
        if n <= 0:
            continue
        pages, rows = locate(cache, table, b, np.arange(n))
        cal = cache.k_calibration[tab[b, 0], :, 0, :]  # [Hkv, D]
        kc = cache.k[pages, :, rows, :].astype(np.float32)  # [n, Hkv, D]
        vc = cache.v[pages, :, rows, :].astype(np.float32)
        ks = cache.k_scale[pages, :, rows]  # [n, Hkv]
        vs = cache.v_scale[pages, :, rows]
        kd = (kc * ks[..., None]) * cal[None]
        vd = vc * vs[..., None]
        k_out[:, o0:o1, :] = rnd(kd).transpose(1, 0, 2)
        v_out[:, o0:o1, :] = rnd(vd).transpose(1, 0, 2)


# --------------------------------------------------------------------------- attention
def gather_sequence(cache: KVCache, table, b: int, n: int):
    """Codes and scales of the first n tokens of sequence b: ([n,Hkv,D] int8 x2, [n,Hkv] fp32 x2)."""
    pages, rows = locate(cache, table, b, np.arange(n))
    return (cache.k[pages, :, rows, :], cache.v[pages, :, rows, :],
            cache.k_scale[pages, :, rows], cache.v_scale[pages, :, rows])


def decode_attention(q, cache: KVCache, cached_lens, table, num_decoding: int, scale: float,
                     out: np.ndarray | None = None) -> np.ndarray:
    """decode_attention, kernels.py:272-361, computed the plain way: dequantize, fp32 softmax,
    fp32 P.V, round to bf16.  Entry b attends tokens [0, cached_lens[b]] (the new token was
    written at position cached_lens[b] by write_decode; kernels.py:137-138).  q is the q'
    returned by write_decode (calibration already folded in).  Rows b >= num_decoding are
    left untouched (zeros when `out` is not given)."""
    q = np.asarray(q, np.float32)
    B, Hq, D = q.shape
    Hkv = cache.k.shape[1]
    G = Hq // Hkv
    if out is None:
        out = np.zeros((B, Hq, D), np.float32)
    for b in range(int(num_decoding)):
        n = int(cached_lens[b]) + 1
        kc, vc, ks, vs = gather_sequence(cache, table, b, n)
        kd = kc.astype(np.float32) * ks[..., None]  # [n, Hkv, D]
        vd = vc.astype(np.float32) * vs[..., None]
        for h in range(Hkv):
            qh = q[b, h * G : (h + 1) * G]  # [G, D]
            s = (qh @ kd[:, h, :].T) * F32(scale)  # [G, n]
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True, dtype=np.float32)
            o = (p @ vd[:, h, :]) / l
            out[b, h * G : (h + 1) * G] = bf16_round(o.astype(np.float32))
    return out


def prefill_attention(q, k, v, cu_seqlens, k_prefix, v_prefix, cu_cached, num_decoding: int,
                      out: np.ndarray | None = None) -> np.ndarray:
    """prefill_attention, kernels.py:973-1175, plain fp32 softmax form.

    Packed row r of entry b (b >= num_decoding, rows [cu_seqlens[b], cu_seqlens[b+1])) attends
    the entry's dequantized prefix rows [cu_cached[b], cu_cached[b+1]) of k_prefix/v_prefix
    [Hkv, total, D] in full, then its own chunk rows up to and including r (causal), with
    softmax scale D**-0.5.  q,k,v are bf16 values: q,k from norm_rope_prefill, v raw."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    N, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    if out is None:
        out = np.zeros((N, Hq, D), np.float32)
    sc = F32(D ** -0.5)
    for b in range(int(num_decoding), len(cu_seqlens) - 1):
        s0, s1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if s1 == s0:
            continue
        p0, p1 = int(cu_cached[b]), int(cu_cached[b + 1])
        L, Pn = s1 - s0, p1 - p0
        causal = np.arange(L)[None, :] <= np.arange(L)[:, None]  # [L(query), L(key)]
        for h in range(Hq):
            hk = h // G
            keys = np.concatenate([np.asarray(k_prefix[hk, p0:p1], np.float32), k[s0:s1, hk]], axis=0)
            vals = np.concatenate([np.asarray(v_prefix[hk, p0:p1], np.float32), v[s0:s1, hk]], axis=0)
            s = (q[s0:s1, h] @ keys.T) * sc  # [L, Pn+L]
            mask = np.concatenate([np.ones((L, Pn), bool), causal], axis=1)
            s = np.where(mask, s, F32(-np.inf))
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True, dtype=np.float32)
            out[s0:s1, h] = bf16_round(((p @ vals) / l).astype(np.float32))
    return out


# --------------------------------------------------------------------------- input producers
def rope_tables(positions, D: int = 128, base: float = 1e6):
    """architecture.py:343-354,387-390: inv_freq = base ** (-arange(0,D,2)/D) in fp32,
    angles = positions * inv_freq (fp32), cos/sin rounded to bf16.  Returns [N, D/2] fp32
    arrays holding bf16 values.  Uses torch on the CPU for pow/cos/sin so the table is the one
    the engine would build; the kernels take the table as an input, so their parity does not
    depend on this function."""
    import torch

    inv_freq = float(base) ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    pos = torch.as_tensor(np.asarray(positions)).to(torch.int32)
    ang = pos[:, None] * inv_freq[None, :]
    cos = ang.cos().to(torch.bfloat16).to(torch.float32).numpy()
    sin = ang.sin().to(torch.bfloat16).to(torch.float32).numpy()
    return cos, sin


# --------------------------------------------------------------------------- weight-streaming matmul
def linear(x, weight) -> np.ndarray:
    """skinny_matmul / linear, kernels.py:1386-1470: y = x @ weight.T for bf16 x [M, K] and weight [N, K] (the layout
    of nn.Linear.weight), products and sums in fp32, result rounded to bf16.  The order of the fp32 sums is not part
    of the contract (the reference's depends on its autotuned BLOCK_K), so parity is "within one bf16 step"."""
    x = np.asarray(x, np.float32)
    w = np.asarray(weight, np.float32)
    return bf16_round((x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32))


# --------------------------------------------------------------------------- decoder-block element-wise ops
def silu_mul(gate_up) -> np.ndarray:
    """silu_mul, kernels.py:1178-1212: [N, 2D] bf16 -> [N, D]: bf16((gate * sigmoid(gate)) * up), all in fp32,
    gate = columns [0, D), up = columns [D, 2D)."""
    x = np.asarray(gate_up, np.float32)
    d = x.shape[-1] // 2
    gate, up = x[..., :d], x[..., d:]
    sig = (F32(1.0) / (F32(1.0) + np.exp(-gate, dtype=np.float32))).astype(np.float32)
    return bf16_round(((gate * sig).astype(np.float32) * up).astype(np.float32))


def add_rms_norm(residual, delta, weight, eps: float):
    """add_rms_norm, kernels.py:1215-1285: new_residual = bf16(residual + delta) (fp32 add); normed =
    bf16((new_residual * rsqrt(sum(new_residual^2) / D + eps)) * weight), the sum over the bf16-rounded
    new residual in fp32.  Returns (new_residual, normed) as fp32 arrays holding bf16 values."""
    r = bf16_round((np.asarray(residual, np.float32) + np.asarray(delta, np.float32)).astype(np.float32))
    D = r.shape[-1]
    ss = np.sum((r * r).astype(np.float32), axis=-1, keepdims=True, dtype=np.float32)
    inv = (F32(1.0) / np.sqrt(ss / F32(D) + F32(eps), dtype=np.float32)).astype(np.float32)
    normed = ((r * inv).astype(np.float32) * np.asarray(weight, np.float32)).astype(np.float32)
    return r, bf16_round(normed)


# --------------------------------------------------------------------------- sampler
def philox4x32_10(c0: np.ndarray, key_lo: int, key_hi: int) -> np.ndarray:
    """First output word of Philox-4x32 with ten rounds (Salmon et al., "Parallel random numbers: as easy as
    1, 2, 3", SC'11) for counters (c0, 0, 0, 0) and key (key_lo, key_hi): the generator behind Triton's
    tl.rand(seed, offset), which the reference's sampler calls with offset = row * V + column
    (kernels.py:1310) and the 64-bit seed split into the two key words."""
    M0, M1, W0, W1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), 0x9E3779B9, 0xBB67AE85
    mask = np.uint64(0xFFFFFFFF)
    c0 = c0.astype(np.uint64) & mask
    c1 = np.zeros_like(c0)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = key_lo & 0xFFFFFFFF, key_hi & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2  # 32 x 32 -> 64-bit products
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)) & mask, p1 & mask, \
                         ((p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)) & mask, p0 & mask
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return c0.astype(np.uint32)


def sample(logits, tau: float, seed: int) -> np.ndarray:
    """sample, kernels.py:1286-1370 (Gumbel-max; tau = 0 is argmax): token[b] = the FIRST index attaining
    max_v (logits[b, v] + tau * -log(-log(u))), u = clamp(uniform(seed, b * V + v), 1e-10, 1 - 1e-7), fp32
    throughout, products and sums rounded separately.  The uniform is Triton's: the Philox word as a signed
    int32 x, folded to non-negative (x < 0 -> -x - 1), converted to fp32 and multiplied by 4.6566127342e-10.
    Returns int64 [B]; the caller's seed advances by one per call (kernels.py:1369)."""
    z = np.asarray(logits, np.float32)
    B, V = z.shape
    off = (np.arange(B, dtype=np.int64)[:, None] * V + np.arange(V, dtype=np.int64)[None, :]).astype(np.uint32)
    x = philox4x32_10(off, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF).view(np.int32).astype(np.int64)
    x = np.where(x < 0, -x - 1, x)
    u = (x.astype(np.float32) * F32(4.6566127342e-10)).astype(np.float32)
    u = np.clip(u, F32(1e-10), F32(1.0 - 1e-7))
    gumbel = (-np.log(-np.log(u, dtype=np.float32), dtype=np.float32)).astype(np.float32)
    z = (z + (F32(tau) * gumbel).astype(np.float32)).astype(np.float32)
    return np.argmax(z, axis=1).astype(np.int64)  # numpy's argmax returns the first maximum
