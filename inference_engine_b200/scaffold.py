"""Random-init Qwen3-1.7B-shaped decoder around the attention ops, and the host-side planning
of one chunked-prefill + decode step.

This is the caller of the attention path, not part of it: everything outside the attention ops
is plain PyTorch (cuBLAS GEMMs through `kernels.linear`, torch elementwise ops), weights are
~N(0, 0.02) with tied embeddings, token ids are synthetic.  It exists so the attention path is
exercised, checked and timed under the call order and the metadata the reference engine gives
it:

* the per-layer call order of kbwal/inference-engine qwen3-1.7b/architecture.py:85-203
  (`AttentionLayer.forward`: pure decode = write + decode attention; a step with prefill =
  norm+rope, quantize, prefix dequantize, prefill attention, then the decode write and decode
  attention into the first rows of the same output),
* the block / model structure of architecture.py:205-476 (residual + RMSNorm fused add,
  SwiGLU MLP, final norm, last row of each entry, tied lm_head),
* the step metadata of engine.py:262-356 (`fill_inputs`): entries numbered absolutely, the
  decoding ones first with one token each, then the prefilling ones, then one padding entry
  that tops the token count up to the bucket, then unused entries; `tile_start` with -1 for
  idle programs; `cu_cached` laying the prefilling entries' cached prefixes end to end.

The cache is paged: `slot_ids` is a 2-D block table `[entries, max_pages]`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import kernels as K

HIDDEN, FFN, VOCAB, LAYERS = 2048, 6144, 151936, 28
HQ, HKV, D = 16, 8, 128
EPS = 1e-6
ROPE_BASE = 1e6
FUSED_PREFILL_WRITE = True  # attention_ops: kernels.write_prefill instead of fused_norm_rope_prefill + quantize_kv_prefill


@dataclass
class PrefixScratch:
    """architecture.py:19-27: bf16 copy of the prefilling entries' cached tokens."""

    k: torch.Tensor  # bf16 [Hkv, >= total_cached, D]
    v: torch.Tensor
    cu_cached: torch.Tensor  # int32 [entries + 1]


@dataclass
class StepInputs:
    """Device views of one step's metadata (engine.py:243-260 `input_views`)."""

    ids: torch.Tensor  # int32 [N]
    positions: torch.Tensor  # int32 [N]
    seq_ids: torch.Tensor  # int32 [N]
    cu_seqlens: torch.Tensor  # int32 [S + 1]
    cached_lens: torch.Tensor  # int32 [S]
    cu_cached: torch.Tensor  # int32 [S + 1]
    tile_start: torch.Tensor  # int32 [ceil(N / block_m) + S]
    num_decoding: torch.Tensor  # int32 [1]
    block_table: torch.Tensor  # int32 [S, max_pages]
    prefix_tokens: int
    block_m: int


def plan_step(
    decode_cached: list[int],
    prefill: list[tuple[int, int]],
    n_tokens: int,
    num_entries: int,
    block_m: int = 128,
) -> dict[str, list[int]]:
    """Host lists for one step.  `decode_cached[i]` = tokens already cached for decoding entry i
    (it contributes one new token at that position); `prefill[j] = (cached, chunk)` for each
    prefilling entry.  The padding entry takes the tokens missing up to `n_tokens`
    (engine.py:262-356)."""
    nd, npf = len(decode_cached), len(prefill)
    used = nd + sum(c for _, c in prefill)
    assert used <= n_tokens and nd + npf + 1 <= num_entries
    chunk = [1] * nd + [c for _, c in prefill] + [n_tokens - used]
    chunk += [0] * (num_entries - len(chunk))
    cached = list(decode_cached) + [p for p, _ in prefill]
    cached += [0] * (num_entries - len(cached))
    cu = [0]
    for c in chunk:
        cu.append(cu[-1] + c)
    positions: list[int] = []
    seq_ids: list[int] = []
    tiles: list[int] = []
    for b in range(num_entries):
        positions.extend(range(cached[b], cached[b] + chunk[b]))
        seq_ids.extend([b] * chunk[b])
        if b >= nd:
            tiles.extend(range(cu[b], cu[b] + chunk[b], block_m))
    tiles += [-1] * (math.ceil(n_tokens / block_m) + num_entries - len(tiles))
    prefix = [0] * nd + cached[nd:]
    cu_cached = [0]
    for p in prefix:
        cu_cached.append(cu_cached[-1] + p)
    return dict(
        chunk=chunk, cached=cached, cu_seqlens=cu, positions=positions, seq_ids=seq_ids,
        tile_start=tiles, cu_cached=cu_cached, num_decoding=[nd],
    )


def assign_pages(plan: dict[str, list[int]], page_size: int, max_pages: int, generator=None):
    """A block table for the plan's entries: every entry with tokens gets the pages its cached
    + new tokens need, drawn from a random permutation of the pool (the padding entry, when it
    has tokens, is an entry like any other: what it writes lands on pages nobody reads); unused
    entries have no tokens and touch no page.  Returns (table int32 [S, max_pages], pages used)."""
    S = len(plan["chunk"])
    need = [(plan["cached"][b] + plan["chunk"][b] + page_size - 1) // page_size for b in range(S)]
    live = [b for b in range(S) if plan["chunk"][b] > 0]
    total = sum(need[b] for b in live)
    perm = torch.randperm(total, generator=generator).to(torch.int32)
    table = torch.zeros(S, max_pages, dtype=torch.int32)
    at = 0
    for b in live:
        assert need[b] <= max_pages
        table[b, : need[b]] = perm[at : at + need[b]]
        at += need[b]
    return table, total


def upload_step(plan: dict[str, list[int]], table: torch.Tensor, ids: list[int], device, block_m: int = 128) -> StepInputs:
    """All of the step's metadata in one pinned int32 buffer and one host-to-device copy
    (engine.py:72-76, 347-356), returned as views."""
    fields = [ids, plan["positions"], plan["seq_ids"], plan["cu_seqlens"], plan["cached"],
              plan["cu_cached"], plan["tile_start"], plan["num_decoding"], table.reshape(-1).tolist()]
    sizes = [len(f) for f in fields]
    host = torch.tensor([x for f in fields for x in f], dtype=torch.int32).pin_memory()
    dev = host.to(device, non_blocking=True)
    v = dev.split(sizes)
    return StepInputs(
        ids=v[0], positions=v[1], seq_ids=v[2], cu_seqlens=v[3], cached_lens=v[4], cu_cached=v[5],
        tile_start=v[6], num_decoding=v[7], block_table=v[8].view(table.shape),
        prefix_tokens=plan["cu_cached"][-1], block_m=block_m,
    )


def attention_ops(q, k, v, qw, kw, cos, sin, cache, inp: StepInputs | None, cached_lens, slot_ids, num_decoding,
                  prefix: PrefixScratch | None, plan: torch.Tensor | None = None):
    """The attention path of one layer, in the reference's call order (architecture.py:99-198).
    `inp is None` = pure decode.  `plan` = this step's kernels.plan_decode_step result, shared by all
    layers (None: every decode_attention call derives its work split itself).  Returns the attention
    output [N, Hq, D]."""
    scale = D ** -0.5
    if inp is None:
        q_d = K.fused_rope_kv_decode(q, k, v, qw, kw, cos, sin, slot_ids, cache, cached_lens, num_decoding, EPS)
        return K.decode_attention(q_d, cache, cached_lens, slot_ids, num_decoding, scale, plan=plan)
    if FUSED_PREFILL_WRITE:  # norm + rope + quantize-on-write of the chunk rows in one call
        q_p, k_p = K.write_prefill(q, k, v, qw, kw, cos, sin, inp.cu_seqlens, slot_ids, cached_lens, num_decoding, cache, EPS)
    else:  # the two calls the reference's caller makes
        q_p, k_p = K.fused_norm_rope_prefill(q, k, qw, kw, cos, sin, EPS)
        K.quantize_kv_prefill(k_p, v, inp.cu_seqlens, slot_ids, cached_lens, num_decoding, cache)
    K.dequantize_kv_prefix(cache, prefix.cu_cached, slot_ids, prefix.k, prefix.v)
    out = K.prefill_attention(q_p, k_p, v, inp.seq_ids, inp.cu_seqlens, inp.tile_start,
                              prefix.k, prefix.v, prefix.cu_cached, inp.block_m)
    B = slot_ids.shape[0]
    q_d = K.fused_rope_kv_decode(q[:B], k[:B], v[:B], qw, kw, cos[:B], sin[:B], slot_ids, cache,
                                 cached_lens, num_decoding, EPS)
    K.decode_attention(q_d, cache, cached_lens, slot_ids, num_decoding, scale, out=out, plan=plan)
    return out


class DecoderScaffold:
    """Weights of a Qwen3-shaped decoder, ~N(0, std), norm weights 1, tied embeddings
    (architecture.py:478-516 for the 1.7B geometry).  Not an nn.Module: inference only."""

    def __init__(self, device, hidden=HIDDEN, ffn=FFN, vocab=VOCAB, layers=LAYERS, std=0.02, seed=0):
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=device) * std).to(torch.bfloat16)

        self.device, self.hidden, self.vocab, self.num_layers = device, hidden, vocab, layers
        self.embed = w(vocab, hidden)
        self.layers = [
            dict(
                qkv=w((HQ + 2 * HKV) * D, hidden), o=w(hidden, HQ * D), gate_up=w(2 * ffn, hidden), down=w(hidden, ffn),
                ln1=torch.ones(hidden, device=device, dtype=torch.bfloat16),
                ln2=torch.ones(hidden, device=device, dtype=torch.bfloat16),
                qn=torch.ones(D, device=device, dtype=torch.bfloat16),
                kn=torch.ones(D, device=device, dtype=torch.bfloat16),
            )
            for _ in range(layers)
        ]
        self.norm = torch.ones(hidden, device=device, dtype=torch.bfloat16)
        self.plan_steps = True  # one kernels.plan_decode_step per forward, shared by the layers
        self.tau = 0.0  # sampling temperature (0 = greedy) and the sampler's seed, advanced by every step
        self.seed = torch.zeros(1, dtype=torch.int64, device=device)
        self.inv_freq = ROPE_BASE ** (-torch.arange(0, D, 2, dtype=torch.float32, device=device) / D)

    def rope(self, positions: torch.Tensor):
        ang = positions[:, None, None] * self.inv_freq[None, None, :]  # architecture.py:387-390
        return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)

    @torch.inference_mode()
    def forward(self, caches, inp: StepInputs | None, ids, cached_lens, slot_ids, num_decoding,
                prefix: PrefixScratch | None = None):
        """One step: token ids [N] -> sampled next token per entry [entries] (int64; greedy while tau = 0).
        `inp is None` = pure decode (ids has one token per entry, position = cached length)."""
        # the decode-attention work split of this step, once for all layers (it depends on the step's metadata only)
        plan = K.plan_decode_step(cached_lens, slot_ids, num_decoding, caches[0]) if self.plan_steps else None
        x = self.embed[ids.long()]
        cos, sin = self.rope(cached_lens if inp is None else inp.positions)
        N = x.shape[0]
        residual = None
        for L, cache in zip(self.layers, caches):
            if residual is None:
                residual = x
                normed = torch.nn.functional.rms_norm(x, (self.hidden,), L["ln1"], EPS)
            else:
                residual, normed = K.add_rms_norm(residual, x, L["ln1"], EPS)
            q, k, v = K.linear(normed, L["qkv"]).split([HQ * D, HKV * D, HKV * D], dim=-1)
            out = attention_ops(q.view(N, HQ, D), k.view(N, HKV, D), v.view(N, HKV, D), L["qn"], L["kn"], cos, sin,
                                cache, inp, cached_lens, slot_ids, num_decoding, prefix, plan)
            attn = K.linear(out.view(N, HQ * D), L["o"])
            residual, normed = K.add_rms_norm(residual, attn, L["ln2"], EPS)
            x = K.linear(K.silu_mul(K.linear(normed, L["gate_up"])), L["down"])
        _, x = K.add_rms_norm(residual, x, self.norm, EPS)
        if inp is not None:
            x = x[(inp.cu_seqlens[1:] - 1).long()]  # each entry's last row; junk for entries without tokens
        logits = K.linear(x, self.embed)
        return K.sample(logits, self.tau, self.seed).view(-1)
