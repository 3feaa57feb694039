"""Generate golden vectors by running the UNMODIFIED reference kernels on the CPU.

The reference (kbwal/inference-engine, qwen3-1.7b/kernels.py) has no tests and no golden
vectors; its kernels are Triton only.  Triton ships a CPU interpreter (TRITON_INTERPRET=1)
that executes a @triton.jit function with numpy, so the reference's own code can produce
known answers without a GPU.  This script imports the reference from a checkout given by
--reference (it is never copied), runs each kernel of the int8-KV-cache attention path on
small seeded inputs and writes inputs + outputs to tests/golden/reference_interp.npz.

Harness-side shims (the reference source is not edited):
  1. kernels.libdevice.rint -> numpy rint (the interpreter has no libdevice externs).
  2. kernels.num_sms -> 148 (it asks the CUDA driver for the SM count; 148 = B200).
  3. autotuned kernels pinned to their first config (the autotuner needs a GPU to time).
  4. bf16 fidelity of the *interpreter* (not of the reference): it keeps bf16 as raw uint16,
     truncates fp32->bf16 and feeds raw bits to dot/int casts.  Patched here to round to
     nearest even on fp32->bf16 (what the GPU does), to convert int->bf16 by value, and to
     widen bf16 operands of tl.dot to fp32 by value.

Run:  python tests/golden/make_golden.py --reference /path/to/inference-engine
bf16 arrays are stored as uint16 bit patterns (suffix _bf16).
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def install_shims(kernels):
    import triton.language as tl
    from triton.runtime import interpreter as interp

    def rint(x):
        h = x.handle
        return tl.tensor(interp.TensorHandle(np.rint(h.data), h.dtype), x.type)

    class _Lib:
        pass

    lib = _Lib()
    lib.rint = rint
    kernels.libdevice = lib
    kernels.num_sms = lambda device: 148
    for name in ("decode_attention_kernel", "prefill_attention_kernel"):
        k = getattr(kernels, name)
        k.configs = k.configs[:1]

    def f32_to_bf16_bits(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16).reshape(a.shape)

    def bf16_bits_to_f32(a):
        return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(a.shape)

    orig_convert = interp._convert_float

    def convert_float(inp, in_t, out_t, rounding):
        if in_t == tl.float32 and out_t == tl.bfloat16:
            return f32_to_bf16_bits(inp)
        if in_t == tl.bfloat16 and out_t == tl.float32:
            return bf16_bits_to_f32(inp)
        return orig_convert(inp, in_t, out_t, rounding)

    interp._convert_float = convert_float
    B = interp.InterpreterBuilder
    orig_cast = B.cast_impl

    def cast_impl(self, src, dst_type):
        s, d = src.dtype.scalar, dst_type.scalar
        if d == tl.bfloat16 and s.is_int():
            return interp.TensorHandle(f32_to_bf16_bits(src.data.astype(np.float32)), d)
        return orig_cast(self, src, dst_type)

    B.cast_impl = cast_impl
    for n in ("create_si_to_fp", "create_ui_to_fp", "create_fp_to_si", "create_fp_to_ui", "create_fp_ext",
              "create_fp_trunc"):
        setattr(B, n, lambda self, src, dst_type: self.cast_impl(src, dst_type))
    orig_dot = B.create_dot

    def create_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
        if a.dtype.scalar == tl.bfloat16:
            a = interp.TensorHandle(bf16_bits_to_f32(a.data), tl.float32)
        if b.dtype.scalar == tl.bfloat16:
            b = interp.TensorHandle(bf16_bits_to_f32(b.data), tl.float32)
        return orig_dot(self, a, b, d, input_precision, max_num_imprecise_acc)

    B.create_dot = create_dot


def rope(pos: torch.Tensor, D: int):
    inv = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = pos[:, None, None] * inv[None, None, :]
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of kbwal/inference-engine (the unmodified reference)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_interp.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "qwen3-1.7b"))
    import kernels

    install_shims(kernels)
    Hq, Hkv, D = 16, 8, 128
    W = (Hq + 2 * Hkv) * D
    bf = torch.bfloat16
    G = {}

    def new_cache(pool, max_len, gen, random_cal=True):
        cal = torch.ones(pool, Hkv, 1, D)
        if random_cal:
            cal = (0.5 + 2.0 * torch.rand(pool, Hkv, 1, D, generator=gen)).float()
        return kernels.LayerKVCache(
            torch.zeros(pool, Hkv, max_len, D, dtype=torch.int8), torch.zeros(pool, Hkv, max_len, D, dtype=torch.int8),
            torch.zeros(pool, Hkv, max_len), torch.zeros(pool, Hkv, max_len), cal)

    def save_cache(prefix, c):
        G[prefix + "k"] = c.k.numpy().copy()
        G[prefix + "v"] = c.v.numpy().copy()
        G[prefix + "k_scale"] = c.k_scale.numpy().copy()
        G[prefix + "v_scale"] = c.v_scale.numpy().copy()
        G[prefix + "k_calibration"] = c.k_calibration.numpy().copy()

    # ---- 1. fused_rope_kv_decode: strided q/k/v views of one [B, 4096] row, like the engine
    gen = torch.Generator().manual_seed(100)
    B = 6
    qkv = torch.randn(B, W, generator=gen).to(bf)
    qkv[4, Hq * D + 3 * D : Hq * D + 4 * D] = 0  # an all-zero K head (scale floor 1e-6/127)
    qkv[4, (Hq + Hkv) * D : (Hq + Hkv) * D + D] = 0  # an all-zero V head
    q, k, v = (t.view(B, -1, D) for t in qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1))
    qw = (1 + 0.02 * torch.randn(D, generator=gen)).to(bf)
    kw = (1 + 0.02 * torch.randn(D, generator=gen)).to(bf)
    cached = torch.tensor([5, 17, 0, 39, 8, 3], dtype=torch.int32)
    cos, sin = rope(cached, D)
    slots = torch.tensor([2, 0, 5, 1, 4, 3], dtype=torch.int32)
    cache = new_cache(7, 40, gen)
    save_cache("wd_in_", cache)
    nd = torch.tensor([5], dtype=torch.int32)  # entry 5 is not decoding: must stay untouched
    out = kernels.fused_rope_kv_decode(q, k, v, qw, kw, cos, sin, slots, cache, cached, nd, 1e-6)
    G.update(wd_qkv_bf16=to_bits(qkv), wd_qw_bf16=to_bits(qw), wd_kw_bf16=to_bits(kw), wd_cos_bf16=to_bits(cos),
             wd_sin_bf16=to_bits(sin), wd_cached=cached.numpy(), wd_slots=slots.numpy(), wd_nd=nd.numpy(),
             wd_out_q_bf16=to_bits(out[:5]))
    save_cache("wd_out_", cache)
    print("fused_rope_kv_decode done")

    # ---- 2. fused_norm_rope_prefill + 3. quantize_kv_prefill + 4. dequantize_kv_prefix + 5. prefill_attention
    gen = torch.Generator().manual_seed(101)
    # entries: 0,1 decoding (1 token each); 2: first chunk of 45 tokens (calibration computed);
    # 3: chunk of 21 tokens on top of 19 cached (calibration loaded); 4: padding on scratch slot
    # (5 tokens); 5: unused entry (0 tokens)
    chunk = [1, 1, 45, 21, 5, 0]
    cached = torch.tensor([9, 30, 0, 19, 0, 0], dtype=torch.int32)
    slots = torch.tensor([3, 1, 0, 2, 4, 4], dtype=torch.int32)
    num_dec = 2
    N = sum(chunk)
    cu = torch.tensor([0] + list(np.cumsum(chunk)), dtype=torch.int32)
    qkv = torch.randn(N, W, generator=gen).to(bf)
    q, k, v = (t.view(N, -1, D) for t in qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1))
    pos = torch.cat([torch.arange(c, c + L) for c, L in zip(cached.tolist(), chunk)]).to(torch.int32)
    seq_ids = torch.cat([torch.full((L,), b) for b, L in enumerate(chunk)]).to(torch.int32)
    cos, sin = rope(pos, D)
    q_p, k_p = kernels.fused_norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
    G.update(pf_qkv_bf16=to_bits(qkv), pf_cos_bf16=to_bits(cos), pf_sin_bf16=to_bits(sin), pf_cu=cu.numpy(),
             pf_cached=cached.numpy(), pf_slots=slots.numpy(), pf_nd=np.array([num_dec], np.int32),
             pf_pos=pos.numpy(), pf_seq_ids=seq_ids.numpy(), pf_q_p_bf16=to_bits(q_p), pf_k_p_bf16=to_bits(k_p))
    print("fused_norm_rope_prefill done")

    cache = new_cache(5, 64, gen)
    # give the slots that already hold tokens (entries 0, 1, 3) plausible contents
    for b in (0, 1, 3):
        s, n = int(slots[b]), int(cached[b])
        cache.k[s, :, :n] = torch.randint(-127, 128, (Hkv, n, D), generator=gen, dtype=torch.int8)
        cache.v[s, :, :n] = torch.randint(-127, 128, (Hkv, n, D), generator=gen, dtype=torch.int8)
        cache.k_scale[s, :, :n] = 0.01 + 0.03 * torch.rand(Hkv, n, generator=gen)
        cache.v_scale[s, :, :n] = 0.01 + 0.03 * torch.rand(Hkv, n, generator=gen)
    save_cache("pf_in_", cache)
    ndt = torch.tensor([num_dec], dtype=torch.int32)
    kernels.quantize_kv_prefill(k_p, v, cu, slots, cached, ndt, cache)
    save_cache("pf_out_", cache)
    print("quantize_kv_prefill done")

    prefix_lens = [0] * num_dec + cached[num_dec:].tolist()
    cu_cached = torch.tensor([0] + list(np.cumsum(prefix_lens)), dtype=torch.int32)
    total = int(cu_cached[-1])
    k_pre = torch.zeros(Hkv, total + 3, D, dtype=bf)
    v_pre = torch.zeros(Hkv, total + 3, D, dtype=bf)
    kernels.dequantize_kv_prefix(cache, cu_cached, slots, k_pre, v_pre)
    G.update(pf_cu_cached=cu_cached.numpy(), pf_k_prefix_bf16=to_bits(k_pre), pf_v_prefix_bf16=to_bits(v_pre))
    print("dequantize_kv_prefix done")

    block_m = 16
    tiles = []
    for b, (s0, L) in enumerate(zip(cu[:-1].tolist(), chunk)):
        if b >= num_dec:
            tiles += list(range(s0, s0 + L, block_m))
    tiles += [-1] * 3
    tile_start = torch.tensor(tiles, dtype=torch.int32)
    out = kernels.prefill_attention(q_p, k_p, v, seq_ids, cu, tile_start, k_pre, v_pre, cu_cached, block_m)
    G.update(pf_tile_start=tile_start.numpy(), pf_block_m=np.array([block_m], np.int32), pf_attn_out_bf16=to_bits(out))
    print("prefill_attention done")

    # ---- 6. decode_attention (split-K + combine) over random codes/scales
    gen = torch.Generator().manual_seed(102)
    cached = torch.tensor([0, 16, 63, 64, 149, 7], dtype=torch.int32)  # n = 1, 17, 64, 65, 150; entry 5 not decoding
    B = cached.numel()
    slots = torch.tensor([4, 2, 0, 5, 1, 3], dtype=torch.int32)
    cache = new_cache(6, 160, gen, random_cal=False)
    for b in range(5):  # only the attended rows get contents, so the fixture compresses
        s, n = int(slots[b]), int(cached[b]) + 1
        cache.k[s, :, :n] = torch.randint(-127, 128, (Hkv, n, D), generator=gen, dtype=torch.int8)
        cache.v[s, :, :n] = torch.randint(-127, 128, (Hkv, n, D), generator=gen, dtype=torch.int8)
        cache.k_scale[s, :, :n] = 0.01 + 0.03 * torch.rand(Hkv, n, generator=gen)
        cache.v_scale[s, :, :n] = 0.01 + 0.03 * torch.rand(Hkv, n, generator=gen)
    qd = torch.randn(B, Hq, D, generator=gen).to(bf)
    nd = torch.tensor([5], dtype=torch.int32)
    out = kernels.decode_attention(qd, cache, cached, slots, nd, D ** -0.5)
    save_cache("da_", cache)
    G.update(da_q_bf16=to_bits(qd), da_cached=cached.numpy(), da_slots=slots.numpy(), da_nd=nd.numpy(),
             da_out_bf16=to_bits(out[:5]))
    print("decode_attention done")

    np.savez_compressed(args.out, **G)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
