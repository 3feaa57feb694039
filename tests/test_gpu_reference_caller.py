"""The reference engine's OWN caller code running on this module: the unmodified architecture.py and engine.py of
kbwal/inference-engine (qwen3-1.7b/) are imported with `kernels` resolving to inference_engine_b200.kernels, a
small random-init Qwen3-shaped model is built (real head geometry: 16 q heads, 8 kv heads, head_dim 128), and the
reference Engine constructs itself (tune_matmuls, capture_decode_graphs, capture_prefill_graphs: engine.py:38-117),
serves requests through its CUDA graphs, and is compared with

  * the same engine run eagerly (no graph replays) at the same shapes: identical tokens;
  * the CPU oracle, op by op, on the tensors the reference's AttentionLayer.forward (architecture.py:60-202)
    handed to the six attention ops during recorded eager steps, in its one-row-per-sequence cache layout
    (1-D slot_ids, page_size = max_len): bit-exact caches, rotated q/k and dequantized prefixes, attention
    outputs within the path's tolerance.

The reference checkout is found through the environment variable B200KV_REFERENCE (the directory holding
architecture.py and engine.py, or its parent) or, failing that, under baseline/_ref/ of this repository, where
tests/stage_reference.py puts an unmodified copy; the test is skipped when neither exists."""
import importlib
import os
import sys
import types

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["LayerKVCache", "decode_attention", "fused_rope_kv_decode", "fused_norm_rope_prefill", "quantize_kv_prefill",
         "dequantize_kv_prefix", "prefill_attention", "silu_mul", "add_rms_norm", "linear", "sample", "tune_linear"]
RECORDED = ["decode_attention", "fused_rope_kv_decode", "fused_norm_rope_prefill", "quantize_kv_prefill",
            "dequantize_kv_prefix", "prefill_attention"]


def reference_dir():
    cands = []
    env = os.environ.get("B200KV_REFERENCE")
    if env:
        cands += [env, os.path.join(env, "qwen3-1.7b")]
    cands.append(os.path.join(ROOT, "baseline", "_ref", "qwen3-1.7b"))
    for c in cands:
        if os.path.exists(os.path.join(c, "architecture.py")) and os.path.exists(os.path.join(c, "engine.py")):
            return c
    return None


class Recorder:
    """Wraps the six attention ops: while `on`, every call is logged with copies of its tensor arguments,
    the layer cache before and after, and its results."""

    def __init__(self, K):
        self.K, self.on, self.calls = K, False, []

    def wrap(self, name):
        fn = getattr(self.K, name)

        def wrapper(*args, **kwargs):
            if not self.on or torch.cuda.is_current_stream_capturing():
                return fn(*args, **kwargs)
            cache = next(a for a in args if isinstance(a, self.K.LayerKVCache)) if name != "fused_norm_rope_prefill" and \
                name != "prefill_attention" else None
            snap = lambda c: None if c is None else H.cache_to_numpy(c).copy()
            rec = {"op": name, "args": [a.detach().clone() if isinstance(a, torch.Tensor) else a for a in args],
                   "kwargs": {k: (v.detach().clone() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()},
                   "cache_id": None if cache is None else id(cache.k), "before": snap(cache)}
            res = fn(*args, **kwargs)
            torch.cuda.synchronize()
            rec["after"] = snap(cache)
            if isinstance(res, tuple):
                rec["result"] = tuple(r.detach().clone() for r in res)
            elif isinstance(res, torch.Tensor):
                rec["result"] = res.detach().clone()
            else:
                rec["result"] = None
            if name == "dequantize_kv_prefix":  # its outputs are the scratch tensors it was given
                rec["result"] = (args[3].detach().clone(), args[4].detach().clone())
            self.calls.append(rec)
            return res

        wrapper.__name__ = name
        return wrapper


@pytest.fixture(scope="module")
def ref():
    path = reference_dir()
    if path is None:
        pytest.skip("no reference checkout: set B200KV_REFERENCE or run tests/stage_reference.py --reference PATH")
    from inference_engine_b200 import kernels as K

    rec = Recorder(K)
    shim = types.ModuleType("kernels")
    for n in NAMES:
        setattr(shim, n, rec.wrap(n) if n in RECORDED else getattr(K, n))
    saved = {m: sys.modules.get(m) for m in ("kernels", "architecture", "engine")}
    sys.modules["kernels"] = shim
    for m in ("architecture", "engine"):
        sys.modules.pop(m, None)
    sys.path.insert(0, path)
    try:
        arch = importlib.import_module("architecture")
        eng = importlib.import_module("engine")
        assert os.path.dirname(os.path.abspath(arch.__file__)) == os.path.abspath(path)
        yield types.SimpleNamespace(arch=arch, eng=eng, K=K, rec=rec)
    finally:
        sys.path.remove(path)
        for m, old in saved.items():
            if old is None:
                sys.modules.pop(m, None)
            else:
                sys.modules[m] = old


MAX_BATCH, MAX_LEN, BUDGET = 4, 384, 128
PROMPT_LENS = [5, 40, 150, 70, 17, 33, 200]
NEW_TOKENS = 6


def build_engine(ref):
    torch.manual_seed(1234)
    model = ref.arch.Qwen3_1_7B(model_dim=256, mlp_intermediate_dim=512, head_dim=128, num_q_heads=16, num_kv_heads=8,
                                vocab_size=1000, num_layers=2, tie_word_embeddings=True, prefill_block_m=128, device="cuda")
    with torch.no_grad():
        for blk in model.model.layers:  # non-trivial per-head norm weights, as a trained model has
            blk.self_attn.q_norm.weight.copy_(1 + 0.05 * torch.randn(128, device="cuda"))
            blk.self_attn.k_norm.weight.copy_(1 + 0.05 * torch.randn(128, device="cuda"))
    return ref.eng.Engine(model, max_batch_size=MAX_BATCH, max_len=MAX_LEN, stop_token_id=-1, tau=0.0,
                          max_tokens_per_step=BUDGET, min_first_chunk=16, max_graph_tokens=BUDGET)


def prompts():
    g = torch.Generator().manual_seed(7)
    return [torch.randint(0, 1000, (n,), generator=g).tolist() for n in PROMPT_LENS]


def eager_decode(engine, plan):
    """replay_decode_graph (engine.py:451-470) without the graph: same padded bucket, same tensors, the model and
    the sampler called directly."""
    from kernels import sample  # the shim

    B = len(plan)
    b = next(x for x in engine.graph_buckets if x >= B)
    pad = b - B
    engine.graph_ids[:b].copy_(torch.tensor([t[0] for _, t in plan] + [0] * pad, dtype=torch.int64))
    engine.graph_cached_lens[:b].copy_(torch.tensor([r.cached_len for r, _ in plan] + [0] * pad, dtype=torch.int32))
    engine.graph_slot_ids[:b].copy_(torch.tensor([r.slot for r, _ in plan] + [engine.scratch_slot] * pad, dtype=torch.int32))
    logits = engine.model(engine.graph_ids[:b], engine.kv_cache, num_decoding=engine.graph_num_decoding[b],
                          cached_lens=engine.graph_cached_lens[:b], slot_ids=engine.graph_slot_ids[:b])
    return sample(logits, engine.tau, engine.seed)[:B].view(-1).tolist()


def test_reference_engine_runs_on_this_module(ref):
    K = ref.K
    engine = build_engine(ref)  # constructs = tunes, warms up and captures every decode and prefill bucket
    assert sorted(engine.graphs) == [1, 2, 4] and sorted(engine.prefill_graphs) == [16, 32, 64, 128]
    assert K.check_status() == 0

    with_graphs = [r.output for r in engine.generate(prompts(), NEW_TOKENS)]
    assert K.check_status() == 0
    assert all(len(o) == NEW_TOKENS and all(0 <= t < 1000 for t in o) for o in with_graphs)
    again = [r.output for r in engine.generate(prompts(), NEW_TOKENS)]
    assert again == with_graphs, "graph replays must be reproducible"

    # the same engine without graph replays, at the same shapes, every attention op recorded
    engine.prefill_graphs = {}
    engine.replay_decode_graph = lambda plan: eager_decode(engine, plan)
    ref.rec.on, ref.rec.calls = True, []
    try:
        eager = [r.output for r in engine.generate(prompts(), NEW_TOKENS)]
    finally:
        ref.rec.on = False
    assert K.check_status() == 0
    assert eager == with_graphs, "graph replay and eager execution of the reference engine must give the same tokens"
    check_recorded_calls(ref.rec.calls)


def np32(t):
    return t.detach().float().cpu().numpy()


def ints(t):
    return t.detach().cpu().numpy().astype(np.int32)


def check_recorded_calls(calls):
    """Every recorded call against the oracle on the same inputs (reference layout: slot_ids 1-D)."""
    seen = {n: 0 for n in RECORDED}
    mixed_with_prefix = 0
    for c in calls:
        a, op = c["args"], c["op"]
        seen[op] += 1
        if op == "fused_rope_kv_decode":
            q, k, v, qw, kw, cos, sin, slots, _, cached, nd, eps = a
            cache = c["before"]
            want_q = O.write_decode(np32(q), np32(k), np32(v), np32(qw), np32(kw), np32(cos)[:, 0], np32(sin)[:, 0],
                                    ints(slots), cache, ints(cached), int(nd.item()), float(eps))
            n = int(nd.item())
            assert np.array_equal(H.to_bits(c["result"])[:n], O.bf16_bits(want_q)[:n]), "rotated q (decode write)"
            H.assert_cache_equal(c["after"], cache, "decode write: ")
        elif op == "fused_norm_rope_prefill":
            q, k, qw, kw, cos, sin, eps = a
            q_p, k_p = O.norm_rope_prefill(np32(q), np32(k), np32(qw), np32(kw), np32(cos)[:, 0], np32(sin)[:, 0], float(eps))
            assert np.array_equal(H.to_bits(c["result"][0]), O.bf16_bits(q_p)), "prefill q"
            assert np.array_equal(H.to_bits(c["result"][1]), O.bf16_bits(k_p)), "prefill k"
        elif op == "quantize_kv_prefill":
            k_p, v, cu, slots, cached, nd, _ = a
            cache = c["before"]
            O.quantize_prefill(np32(k_p), np32(v), ints(cu), ints(slots), ints(cached), int(nd.item()), cache)
            H.assert_cache_equal(c["after"], cache, "prefill write: ")
        elif op == "dequantize_kv_prefix":
            _, cu_cached, slots, k_out, v_out = a
            cu = ints(cu_cached)
            live = int(cu[-1])
            mixed_with_prefix += live > 0
            kpre = np.zeros(k_out.shape, np.float32)
            vpre = np.zeros_like(kpre)
            O.dequantize_prefix(c["before"], cu, ints(slots), kpre, vpre)
            got_k, got_v = c["result"]
            assert np.array_equal(H.to_bits(got_k[:, :live]), O.bf16_bits(kpre[:, :live])), "dequantized K prefix"
            assert np.array_equal(H.to_bits(got_v[:, :live]), O.bf16_bits(vpre[:, :live])), "dequantized V prefix"
        elif op == "prefill_attention":
            q_p, k_p, v, seq_ids, cu, tile_start, kpre, vpre, cu_cached, block_m = a
            # which entries prefill: those owning a query tile (tile_start lists them; decoders get none)
            cu_h, seq_h = ints(cu), ints(seq_ids)
            tiles = ints(tile_start)
            starts = tiles[tiles >= 0]
            if len(starts) == 0:
                continue
            nd = int(seq_h[starts.min()])
            want = O.prefill_attention(np32(q_p), np32(k_p), np32(v), cu_h, np32(kpre), np32(vpre), ints(cu_cached), nd)
            lo = int(cu_h[nd])
            mx, mean = H.attn_errors(np32(c["result"])[lo:], want[lo:])
            assert mx <= 2e-2 and mean <= 2e-3, ("prefill attention", mx, mean)
        elif op == "decode_attention":
            q, _, cached, slots, nd, scale = a[:6]
            n = int(nd.item())
            if n == 0:
                continue
            want = O.decode_attention(np32(q), c["before"], ints(cached), ints(slots), n, float(scale))
            got = c["result"] if "out" not in c["kwargs"] else c["result"]
            mx, mean = H.attn_errors(np32(got)[:n], want[:n])
            assert mx <= 2e-2 and mean <= 2e-3, ("decode attention", mx, mean)
    assert all(v > 0 for v in seen.values()), seen
    assert mixed_with_prefix > 0, "no recorded step continued a prompt on a cached prefix"
