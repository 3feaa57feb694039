#!/usr/bin/env python
"""Headline benchmark: int8-KV-cache decode attention at B=64, ctx 4096 (per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one decode pass of the attention path over a stack of LAYERS distinct layer caches
(28, as in Qwen3-1.7B): per layer, quantize-on-write of the B new tokens (fused QK-RMSNorm +
RoPE + int8) then split-K paged decode attention over ctx tokens.  The whole step is one CUDA
graph replay, as in the reference engine.  Metric: algorithmic HBM bytes of the step / time.

With N > 1 (torchrun) every rank holds its own B sequences (sequence sharding, no collective
on the data path: weak scaling); the reported value is all ranks' bytes over the slowest
rank's device time.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, PAGE = 16, 8, 128, 16
CACHE_BYTES_PER_TOKEN = HKV * (2 * D + 8)  # int8 K+V codes and fp32 K+V scales of one token, one layer = 2112
WRITE_BYTES_PER_TOKEN = 14656  # q,k,v,cos,sin read (8448) + q', codes, scales written (6208)


REPEATS = 5  # every timed loop of the headline run is repeated this often; median, min and max are reported


def ncu_traffic(B: int, n: int):
    """dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch of this shape, from the figures
    file kept beside the ncu summary (profiles/decode_attn_B64_ctx4096.json); None for a shape never captured."""
    try:
        with open(os.path.join(ROOT, "profiles", "decode_attn_B64_ctx4096.json")) as f:
            rec = json.load(f)
        if (rec["batch"], rec["ctx"]) == (B, n):
            return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        pass
    return None


def attn_bytes(B: int, n: int) -> int:
    """Algorithmic bytes of one decode_attention call: cache stream + q read + out write."""
    return B * n * CACHE_BYTES_PER_TOKEN + 2 * (B * HQ * D * 2)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU arm
class CpuSample:
    """The CPU port of the reference math (C/OpenMP restatement in oracle/, all host threads) on one
    layer's worth of the workload: decode attention over `seqs` sequences x ctx tokens, repeated
    `passes` times (a step of `passes` layers).  `run()` returns seconds for all passes."""

    def __init__(self, B: int, n: int, seqs: int, passes: int, seed: int = 2):
        from oracle import c_oracle as C
        from oracle import oracle as O

        self.C, self.n, self.seqs, self.passes = C, n, seqs, passes
        rng = np.random.default_rng(seed)
        pages_per_seq = (n + PAGE - 1) // PAGE
        num_pages = seqs * pages_per_seq
        self.cache = O.make_cache(num_pages, HKV, PAGE, D)
        self.cache.k[...] = rng.integers(-127, 128, self.cache.k.shape, dtype=np.int8)
        self.cache.v[...] = rng.integers(-127, 128, self.cache.v.shape, dtype=np.int8)
        self.cache.k_scale[...] = 0.02
        self.cache.v_scale[...] = 0.02
        self.table = rng.permutation(num_pages).astype(np.int32).reshape(seqs, pages_per_seq)
        self.q = O.bf16_round(rng.standard_normal((seqs, HQ, D)).astype(np.float32))
        self.cached = np.full(seqs, n - 1, np.int32)
        self.out = np.zeros((seqs, HQ, D), np.float32)
        C.set_threads(os.cpu_count() or 1)
        self.threads = C.threads()
        self.bytes = passes * attn_bytes(seqs, n)
        self.sample = (f"decode attention, {seqs} of {B} sequences x ctx {n}, {passes} layer passes per step "
                       f"(C/OpenMP port of the reference math, {self.threads} threads; the reference itself is "
                       f"Triton-only and has no CPU path)")

    def run(self) -> float:
        t0 = time.perf_counter()
        for _ in range(self.passes):
            self.C.decode_attention(self.q, self.cache, self.cached, self.table, self.seqs, D ** -0.5, out=self.out)
        return time.perf_counter() - t0


def run_reference(args):
    """--impl reference: the reference publishes no CPU implementation of this path (it is
    Triton-only), so the CPU arm is the oracle port of its math, timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cs = CpuSample(args.batch, args.ctx, max(1, min(args.batch, args.cpu_seqs)), args.layers)
    secs = [cs.run() for _ in range(args.warmup + args.steps)][args.warmup:]
    dt = float(np.mean(secs))
    v = cs.bytes / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "decode_attention_hbm_gbs", "value": round(v, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * dt, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": workload_config(args), "l2": "n/a (CPU)",
        "cpu_baseline": {"value": round(v, 4), "unit": "GB/s", "cores": cs.threads, "kind": "port", "sample": cs.sample},
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": round(cs.seqs / dt, 3),
    }))


def workload_config(args):
    """The same dictionary in both arms (what differs between them is reported beside it, not inside)."""
    return {"workload": f"split-K paged int8 decode attention sweep cell B={args.batch} ctx={args.ctx} "
                        f"(16 Q / 8 KV heads, head_dim 128, 16-token pages, random page table), "
                        f"{args.layers} distinct layer caches per step, quantize-on-write of the new token included",
            "batch_per_gpu": args.batch, "ctx": args.ctx, "layers": args.layers, "page_size": PAGE,
            "sharding": "sequences across GPUs, no collective"}


def oracle_sample_check(K, cache, table_np, lens_np, sample, got_rows, q_rot=None, qkv_rows=None, cos_rows=None,
                        sin_rows=None):
    """Parity of real output rows after a timed region: the sequences `sample` of one layer are recomputed by the
    CPU oracle from the device cache as the step left it (only their pages are copied back) and compared with the
    rows the step produced.  With `qkv_rows` the oracle also redoes the quantize-on-write of their new tokens: the
    step rewrites the same row every time, so the codes and scales it left must equal the oracle's bytes, and the
    oracle's rotated q feeds the attention; otherwise `q_rot` is the query the attention call was given."""
    import torch

    from oracle import c_oracle as C
    from oracle import oracle as O

    sample = [int(x) for x in sample]
    need = [(int(lens_np[s]) + PAGE - 1) // PAGE for s in sample]
    pages = np.concatenate([table_np[s, :k] for s, k in zip(sample, need)]).astype(np.int64)
    idx = torch.from_numpy(pages).to(cache.k.device)
    sub = O.KVCache(*(t.index_select(0, idx).cpu().numpy() for t in (cache.k, cache.v, cache.k_scale, cache.v_scale,
                                                                    cache.k_calibration)))
    tab = np.zeros((len(sample), max(need)), np.int32)
    at = 0
    for i, k in enumerate(need):
        tab[i, :k] = np.arange(at, at + k)
        at += k
    cached = np.array([int(lens_np[s]) - 1 for s in sample], np.int32)
    res = {"rows": len(sample) * HQ, "sequences": sample}
    if qkv_rows is not None:
        x = qkv_rows.float().numpy()
        q = x[:, : HQ * D].reshape(-1, HQ, D)
        k = x[:, HQ * D : (HQ + HKV) * D].reshape(-1, HKV, D)
        v = x[:, (HQ + HKV) * D :].reshape(-1, HKV, D)
        ones = np.ones(D, np.float32)
        before = sub.copy()
        q_rot = O.write_decode(q, k, v, ones, ones, cos_rows.float().numpy().reshape(-1, D // 2),
                               sin_rows.float().numpy().reshape(-1, D // 2), tab, sub, cached, len(sample), 1e-6)
        res["write_bytes_differing"] = int(sum(np.count_nonzero(getattr(before, f).view(np.uint8) != getattr(sub, f).view(np.uint8))
                                               for f in ("k", "v", "k_scale", "v_scale")))
    C.set_threads(os.cpu_count() or 1)
    want = C.decode_attention(np.ascontiguousarray(q_rot, np.float32), sub, cached, tab, len(sample), D ** -0.5)
    # as in the tests: absolute error, taken relative to the reference value where that exceeds 1 (random codes
    # with scales of 0.01-0.04 give outputs of a few units, where one bf16 step is already 2^-6)
    err = np.abs(got_rows.float().numpy() - want) / np.maximum(1.0, np.abs(want))
    res.update({"max_abs": float(err.max()), "mean_abs": float(err.mean()),
                "within_gate": bool(err.max() <= 2e-2 and err.mean() <= 2e-3)})
    return res


# ----------------------------------------------------------------------------- GPU arm
def run_b200(args):
    import torch
    import torch.distributed as dist

    from inference_engine_b200 import kernels as K
    from inference_engine_b200.host_step import HostDecodeStep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    K.set_early_start(not args.no_early_start)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, n, L = args.batch, args.ctx, args.layers
    gen = torch.Generator(device=dev).manual_seed(2 + rank)
    pages_per_seq = (n + PAGE - 1) // PAGE
    num_pages = B * pages_per_seq + 1
    caches = []
    for _ in range(L):
        c = K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev)
        c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device=dev, dtype=torch.int8))
        c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device=dev, dtype=torch.int8))
        c.k_scale.copy_(0.01 + 0.03 * torch.rand(c.k_scale.shape, generator=gen, device=dev))
        c.v_scale.copy_(0.01 + 0.03 * torch.rand(c.v_scale.shape, generator=gen, device=dev))
        caches.append(c)
    table_h = torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(2 + rank)).to(torch.int32)
    table_h = table_h.reshape(B, pages_per_seq).contiguous().pin_memory()
    W = (HQ + 2 * HKV) * D
    g_cpu = torch.Generator().manual_seed(12 + rank)
    qkv_h = torch.randn(L, B, W, generator=g_cpu).to(torch.bfloat16).pin_memory()
    pos = torch.full((B,), n - 1, dtype=torch.int32)  # the new token is token n-1: ctx counts it
    inv_freq = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = pos[:, None, None] * inv_freq[None, None, :]
    cos_h, sin_h = ang.cos().to(torch.bfloat16).pin_memory(), ang.sin().to(torch.bfloat16).pin_memory()
    cached_h = pos.clone().pin_memory()
    nd_h = torch.tensor([B], dtype=torch.int32).pin_memory()
    out_h = torch.empty(L, B, HQ, D, dtype=torch.bfloat16).pin_memory()

    step = HostDecodeStep(caches, B, HQ, HKV, D, tuple(table_h.shape))
    step.use_plan = not args.no_plan
    step.run_host(qkv_h, cos_h, sin_h, cached_h, table_h, nd_h, out_h)  # fills the device inputs
    torch.cuda.synchronize()
    if K.check_status(dev):
        raise SystemExit("device status word reports an inconsistent page table")
    step.capture()

    # a graph of decode_attention calls only (dominant kernel + its reduction), one per layer cache, behind the
    # step's one plan kernel
    q_dev = torch.randn(L, B, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
    attn_out = torch.empty_like(q_dev)
    attn_plan = torch.empty(K.plan_decode_bytes(dev), dtype=torch.uint8, device=dev)

    def attn_only():
        plan = None if args.no_plan else K.plan_decode_step(step.dev_cached, step.dev_table, step.dev_nd, caches[0], out=attn_plan)
        for l in range(L):
            K.decode_attention(q_dev[l], caches[l], step.dev_cached, step.dev_table, step.dev_nd, D ** -0.5, out=attn_out[l],
                               plan=plan)

    # The roofline figure is for the kernel by itself: no early start here, or consecutive attention
    # launches would overlap each other's tails and the per-launch time would flatter the kernel.
    K.set_early_start(False)
    attn_only()
    torch.cuda.synchronize()
    attn_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(attn_graph):
        attn_only()
    K.set_early_start(not args.no_early_start)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """REPEATS timed loops of exactly `steps` calls each, every one between barriers; device time per loop,
        max over ranks.  Returns the list of loop times in ms."""
        out = []
        for _ in range(REPEATS):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            out.append(ms)
        return out

    for _ in range(max(args.warmup, 3)):
        step.run_device()
        attn_graph.replay()
    with ClockSampler(local) as clocks:
        ms_dev = timed(step.run_device, args.steps)
        ms_attn = timed(attn_graph.replay, args.steps)
        ms_e2e = timed(lambda: step.run_host(qkv_h, cos_h, sin_h, cached_h, table_h, nd_h, out_h), args.steps)
    if K.check_status(dev):
        raise SystemExit("device status word set during the timed region")

    step_bytes = L * (attn_bytes(B, n) + B * WRITE_BYTES_PER_TOKEN)
    peak, peak_kind = peaks()
    med = statistics.median
    gbs = lambda ms: world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    value, e2e = gbs(med(ms_dev)), gbs(med(ms_e2e))
    per_call_us = [ms * 1e3 / (args.steps * L) for ms in ms_attn]
    achieved = attn_bytes(B, n) / (med(per_call_us) * 1e-6) / 1e9

    # parity of what the timed regions really produced (rank 0's rows): four sequences of the last layer, from the
    # host-buffer step's output (quantize-on-write + attention) and from the attention-only graph
    parity = None
    if rank == 0 and not args.no_parity:
        sample = sorted({0, B // 3, (2 * B) // 3, B - 1})
        lens_np = np.full(B, n, np.int64)
        p_step = oracle_sample_check(K, caches[L - 1], table_h.numpy(), lens_np, sample, out_h[L - 1][sample].reshape(-1, HQ, D),
                                     qkv_rows=qkv_h[L - 1][sample], cos_rows=cos_h[sample], sin_rows=sin_h[sample])
        p_attn = oracle_sample_check(K, caches[L - 1], table_h.numpy(), lens_np, sample,
                                     attn_out[L - 1][sample].cpu().reshape(-1, HQ, D), q_rot=q_dev[L - 1][sample].float().cpu().numpy())
        parity = {"rows": p_step["rows"] + p_attn["rows"], "max_abs": max(p_step["max_abs"], p_attn["max_abs"]),
                  "mean_abs": max(p_step["mean_abs"], p_attn["mean_abs"]),
                  "within_gate": p_step["within_gate"] and p_attn["within_gate"],
                  "write_bytes_differing": p_step["write_bytes_differing"], "sequences": sample, "layer": L - 1,
                  "what": "rows of the host-buffer step's output and of the attention-only graph, recomputed by the CPU oracle "
                          "from the device cache the timed steps left; gate max-abs 2e-2 / mean-abs 2e-3, write bit-exact"}
        if not parity["within_gate"] or parity["write_bytes_differing"]:
            raise SystemExit(f"parity check failed after the timed region: {parity}")

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cs = CpuSample(B, n, max(1, min(B, args.cpu_seqs)), L)
        cs.run()
        dt = min(cs.run() for _ in range(3))
        cpu = {"value": round(cs.bytes / dt / 1e9, 4), "unit": "GB/s", "cores": cs.threads, "kind": "port",
               "sample": cs.sample, "seconds": round(dt, 2)}
    line = None
    if rank == 0:
        line = {
            "metric": "decode_attention_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(med(ms_dev) / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 codes, fp16 MMA operands, fp32 accumulate",
            "data": "synthetic", "config": workload_config(args),
            "l2": f"step streams {step_bytes / 1e9:.1f} GB per GPU, far above the 126 MB L2",
            "repeats": REPEATS, "value_min": round(gbs(max(ms_dev)), 1), "value_max": round(gbs(min(ms_dev)), 1),
            "pct_of_8TBs": round(100 * value / world / 8000.0, 2),
            "tokens_per_s": round(world * B * args.steps / (med(ms_dev) * 1e-3), 1),
            "roofline": {"bound": "hbm", "kernel": "decode_attn_kernel (tensor-core variant, cross-split reduction fused in): one per "
                                                   "decode_attention call" + ("" if args.no_plan else ", work split read from the step's plan"),
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "peak_kind": peak_kind, "us_per_call": round(med(per_call_us), 2),
                         "us_per_call_min": round(min(per_call_us), 2), "us_per_call_max": round(max(per_call_us), 2),
                         "algorithmic_bytes_per_call": attn_bytes(B, n), "traffic": ncu_traffic(B, n)},
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "ms_per_step": round(med(ms_e2e) / args.steps, 4),
                    "value_min": round(gbs(max(ms_e2e)), 1), "value_max": round(gbs(min(ms_e2e)), 1),
                    "h2d_bytes_per_step": step.h2d_bytes, "d2h_bytes_per_step": step.d2h_bytes},
            "gpu_launches": args.steps * REPEATS * (L * 2 + (0 if args.no_plan else 1)),
            "parity": parity, "cpu_baseline": cpu, "clocks": clocks.summary(),
        }
    # the sequence-sharded configuration on the same ranks, right after the headline step (strong scaling)
    del step, attn_graph, caches, q_dev, attn_out
    torch.cuda.empty_cache()
    if not args.no_sharded:
        rec = sharded_record(args, rank, world, dev)
        if line is not None:
            line["sharded"] = rec
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def sharded_record(args, rank, world, dev, layers=None, model=False):
    """The sequence-sharded decode configuration on the ranks of an initialised run: `--seqs` concurrent sequences
    with contexts drawn log-uniform in [512, 32768] (seed 4), partitioned over the ranks by KV bytes
    (inference_engine_b200.sharding), one process per GPU, no collective on the data path.  Per step every rank
    runs the step's plan kernel, then quantize-on-write + decode attention for its sequences over `layers`
    distinct layer caches (only as many as fit are kept resident: the full 28-layer cache of 2048 such sequences
    is ~940 GB).  After the timed region a fixed sample of sequences (every 128th) is verified: its owner
    recomputes it with the CPU oracle from its device cache, and one NCCL all_gather brings every sequence's
    output row (and the owners' findings) to every rank, where the sample's rows are compared with what the owners
    checked.  Returns the record (identical on all ranks up to the per-rank lists, which rank 0 holds)."""
    import torch
    import torch.distributed as dist

    from inference_engine_b200 import kernels as K
    from inference_engine_b200.host_step import HostDecodeStep
    from inference_engine_b200.sharding import gather_outputs, plan_shards

    K.set_early_start(not args.no_early_start)
    rng = np.random.default_rng(4)
    lens_all = np.exp(rng.uniform(np.log(512), np.log(32768), args.seqs)).astype(np.int64)
    plan = plan_shards(lens_all, world)
    mine = plan.local[rank]
    lens = lens_all[mine]
    B, L = len(mine), (layers if layers is not None else args.sharded_layers)
    pages_per = (lens + PAGE - 1) // PAGE
    num_pages = int(pages_per.sum()) + 1
    max_pages = int(pages_per.max())
    # never ask for more resident layer caches than fit: one layer of this shard is num_pages x 8 heads x 16 tokens
    # x (2 x 128 code bytes + 2 x 4 scale bytes); keep them within 60 % of the device's memory
    layer_bytes = num_pages * HKV * PAGE * (2 * D + 8)
    L = max(1, min(L, int(0.6 * torch.cuda.get_device_properties(dev).total_memory // layer_bytes)))
    table_np = np.full((B, max_pages), 0, np.int32)
    perm = np.random.default_rng(40 + rank).permutation(num_pages - 1).astype(np.int32)
    at = 0
    for i, k in enumerate(pages_per):
        table_np[i, :k] = perm[at:at + k]
        at += int(k)
    gen = torch.Generator(device=dev).manual_seed(4 + rank)
    caches = []
    for _ in range(L):
        c = K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev)
        c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device=dev, dtype=torch.int8))
        c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device=dev, dtype=torch.int8))
        c.k_scale.fill_(0.02)
        c.v_scale.fill_(0.02)
        caches.append(c)
    W = (HQ + 2 * HKV) * D
    qkv_h = torch.randn(L, B, W, generator=torch.Generator().manual_seed(14 + rank)).to(torch.bfloat16).pin_memory()
    pos = torch.from_numpy((lens - 1).astype(np.int32))
    inv_freq = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = pos[:, None, None] * inv_freq[None, None, :]
    cos_h, sin_h = ang.cos().to(torch.bfloat16).pin_memory(), ang.sin().to(torch.bfloat16).pin_memory()
    cached_h, nd_h = pos.clone().pin_memory(), torch.tensor([B], dtype=torch.int32).pin_memory()
    table_h = torch.from_numpy(table_np).pin_memory()
    out_h = torch.empty(L, B, HQ, D, dtype=torch.bfloat16).pin_memory()
    step = HostDecodeStep(caches, B, HQ, HKV, D, tuple(table_h.shape))
    step.use_plan = not args.no_plan
    step.run_host(qkv_h, cos_h, sin_h, cached_h, table_h, nd_h, out_h)
    torch.cuda.synchronize()
    if K.check_status(dev):
        raise SystemExit("device status word reports an inconsistent page table")
    step.capture(groups=1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step.run_device()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step.run_device()
    e1.record()
    barrier()
    my_ms = e0.elapsed_time(e1)
    ms = my_ms
    if world > 1:
        t = torch.tensor([my_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if K.check_status(dev):
        raise SystemExit("device status word set during the sharded run")
    my_bytes = L * (int(lens.sum()) * CACHE_BYTES_PER_TOKEN + B * 8192 + B * WRITE_BYTES_PER_TOKEN)
    my_gbs = my_bytes * args.steps / (my_ms * 1e-3) / 1e9

    # verification, off the timed path
    stride = max(1, args.seqs // 16)
    local_of = {g: i for i, g in enumerate(mine)}
    my_sample = [g for g in range(0, args.seqs, stride) if g in local_of]
    found = {"max_abs": 0.0, "mean_abs": 0.0, "write_bytes_differing": 0, "within_gate": True}
    if my_sample and not args.no_parity:
        loc = [local_of[g] for g in my_sample]
        found = oracle_sample_check(K, caches[L - 1], table_np, lens, loc, step.dev_out[L - 1][loc].cpu().reshape(-1, HQ, D),
                                    qkv_rows=qkv_h[L - 1][loc], cos_rows=cos_h[loc], sin_rows=sin_h[loc])
    stats = torch.tensor([my_gbs, float(lens.sum()), float(B), found["max_abs"], found["mean_abs"],
                          float(found["write_bytes_differing"]), float(len(my_sample))], device=dev)
    parts = [torch.zeros_like(stats) for _ in range(world)]
    if world > 1:
        dist.all_gather(parts, stats)
    else:
        parts = [stats]
    # every sequence's output row of the last resident layer, by NCCL, in global order; column 0 carries the id
    rows = torch.cat([torch.from_numpy(np.asarray(mine, dtype=np.int64)).to(dev).float()[:, None],
                      step.dev_out[L - 1].float().reshape(B, HQ * D)], dim=1)
    got = gather_outputs(rows, plan, rank)
    served_once = bool(torch.equal(got[:, 0].cpu(), torch.arange(args.seqs, dtype=torch.float32)))
    rows_match = True
    if my_sample:  # what came back through the gather for my sample is what I checked against the oracle
        rows_match = bool(torch.equal(got[my_sample, 1:], rows[[local_of[g] for g in my_sample], 1:]))
    flag = torch.tensor([1.0 if rows_match else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    full = None
    if model:
        full = sharded_decoder(args, rank, world, dev, caches, L, B, cached_h, table_h, nd_h, plan, gen, barrier)
    peak, peak_kind = peaks()
    per = [{"rank": r, "gbs": round(float(p[0]), 1), "frac_of_measured_peak": round(float(p[0]) / peak, 4),
            "kv_tokens": int(p[1]), "sequences": int(p[2])} for r, p in enumerate(parts)]
    checked = int(sum(float(p[6]) for p in parts))
    vmax, vmean = max(float(p[3]) for p in parts), max(float(p[4]) for p in parts)
    rec = {
        "metric": "sharded_decode_attention_tokens_per_s", "value": round(args.seqs * args.steps / (ms * 1e-3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
        "data": "synthetic", "config": {"workload": f"{args.seqs} sequences, contexts log-uniform [512, 32768] (seed 4), "
                                                    f"sharded by KV bytes over {world} GPU(s), {L} resident layer caches per step "
                                                    f"(attention path only: plan + write + decode attention)",
                                        "plan_imbalance": round(plan.imbalance(), 4), "resident_layers": L},
        "aggregate_gbs": round(sum(p["gbs"] for p in per), 1),
        "per_gpu_frac_min": min(p["frac_of_measured_peak"] for p in per),
        "per_gpu_frac_max": max(p["frac_of_measured_peak"] for p in per), "peak_kind": peak_kind, "per_gpu": per,
        "verification": {"all_sequences_served_once": served_once, "sequences_checked_against_oracle": checked,
                         "max_abs": vmax, "mean_abs": vmean,
                         "write_bytes_differing": int(sum(float(p[5]) for p in parts)),
                         "gathered_rows_equal_checked_rows": bool(flag.item() > 0),
                         "within_gate": bool(vmax <= 2e-2 and vmean <= 2e-3)},
        "full_decoder": full}
    del step, caches
    torch.cuda.empty_cache()
    return rec


def sharded_decoder(args, rank, world, dev, caches, L, B, cached_h, table_h, nd_h, plan, gen, barrier):
    """--sharded --model: the same shard through the whole random-init decoder (28 layers, GEMMs, sampler): the L
    resident layer caches are used in turn by the 28 layers (each is far larger than L2, so every layer still
    streams its KV bytes from HBM; only their contents repeat)."""
    import torch
    import torch.distributed as dist

    from inference_engine_b200 import scaffold as S
    from inference_engine_b200.sharding import gather_outputs

    model = S.DecoderScaffold(dev, seed=4)
    cyc = [caches[i % L] for i in range(S.LAYERS)]
    ids = torch.randint(0, S.VOCAB, (B,), generator=gen, device=dev, dtype=torch.int32)
    d_cached, d_table, d_nd = cached_h.to(dev), table_h.to(dev), nd_h.to(dev)
    with torch.inference_mode():
        for _ in range(2):
            toks = model.forward(cyc, None, ids, d_cached, d_table, d_nd)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            toks = model.forward(cyc, None, ids, d_cached, d_table, d_nd)
    for _ in range(max(args.warmup, 3)):
        g.replay()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        g.replay()
    f1.record()
    barrier()
    fms = torch.tensor([f0.elapsed_time(f1)], device=dev)
    if world > 1:
        dist.all_reduce(fms, op=dist.ReduceOp.MAX)
    all_toks = gather_outputs(toks.float()[:, None], plan, rank)  # the sampled ids of all sequences, by NCCL
    return {"layers": S.LAYERS, "ms_per_step": round(float(fms.item()) / args.steps, 4),
            "output_tokens_per_s": round(args.seqs * args.steps / (float(fms.item()) * 1e-3), 1),
            "tokens_gathered": int(all_toks.shape[0]),
            "tokens_in_vocabulary": bool(((all_toks >= 0) & (all_toks < S.VOCAB)).all().item())}


def run_sharded(args):
    """--sharded: the sequence-sharded decode configuration alone (see sharded_record), one JSON line on rank 0."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = sharded_record(args, rank, world, dev, layers=args.layers, model=args.model)
    if rank == 0:
        print(json.dumps(rec))
    if world > 1:
        dist.destroy_process_group()


def run_serve(args):
    """--serve: offline serving run of the step loop (inference_engine_b200/engine.py) on the random-init
    Qwen3-1.7B-shaped decoder: 128 requests submitted at once, prompt lengths log-uniform in [32, 1024]
    (synthetic ids), 128 new tokens each (no stop token), at most 64 running requests, 1024 tokens per step,
    rows of 2048 tokens, paged int8 cache.  Wall-clock times (the loop reads the sampled tokens back every
    step, like the reference engine)."""
    import time

    import torch

    from inference_engine_b200 import kernels as K
    from inference_engine_b200 import scaffold as S
    from inference_engine_b200.engine import Engine

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K.set_early_start(not args.no_early_start)
    model = S.DecoderScaffold(dev, seed=5)
    t0 = time.perf_counter()
    eng = Engine(model, max_batch_size=64, max_len=2048, stop_token_id=-1, max_tokens_per_step=1024, min_first_chunk=64,
                 max_graph_tokens=1024)
    torch.cuda.synchronize()
    t_capture = time.perf_counter() - t0
    g = torch.Generator().manual_seed(5)
    n_req, new = 128, 128
    lens = torch.exp(torch.empty(n_req).uniform_(math.log(32), math.log(1024), generator=g)).long().tolist()
    prompts = [torch.randint(0, S.VOCAB, (n,), generator=g).tolist() for n in lens]
    for warm in (True, False):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reqs = [eng.submit_request(p, new) for p in (prompts[:8] if warm else prompts)]
        steps = 0
        while not eng.sched.idle():
            eng.step()
            steps += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    out_tokens = sum(len(r.output) for r in reqs)
    ttft = sorted(r.t_first_token - r.t_submit for r in reqs)
    print(json.dumps({
        "case": "offline serving run of the step loop", "requests": n_req, "prompt_tokens": sum(lens),
        "output_tokens": out_tokens, "steps": steps, "wall_s": round(wall, 3),
        "output_tokens_per_s": round(out_tokens / wall), "total_tokens_per_s": round((out_tokens + sum(lens)) / wall),
        "ttft_s": {"median": round(ttft[len(ttft) // 2], 3), "max": round(ttft[-1], 3)},
        "steps_by_kind": eng.steps_run, "graph_capture_s": round(t_capture, 2),
        "host_seconds_both_runs": {k: round(v, 3) for k, v in eng.seconds.items()},
        "pages": {"pool": eng.pool.capacity, "free_at_end": eng.pool.uncommitted()}, "status": K.check_status(dev),
        "data": "synthetic ids, random-init weights"}), flush=True)


def run_decode_model(args):
    """--decode-model: one pure-decode step of the random-init Qwen3-1.7B-shaped decoder at the headline shape
    (B sequences of ctx cached tokens, one new token each, 28 layers, int8 paged cache, random block table):
    embedding -> 28 x (norm, qkv GEMM, quantize-on-write, decode attention, o GEMM, norm, SwiGLU MLP) -> norm ->
    tied lm_head -> sampler (greedy), captured as one CUDA graph.  Reports step time, tokens/s and the attention path's
    share (a second graph with only the write + attention ops on the same caches)."""
    import torch

    from inference_engine_b200 import kernels as K
    from inference_engine_b200 import scaffold as S

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K.set_early_start(not args.no_early_start)
    B, n = args.batch, args.ctx
    model = S.DecoderScaffold(dev, seed=4)
    gen = torch.Generator(device=dev).manual_seed(4)
    pages_per_seq = (n + PAGE) // PAGE  # room for the new token
    num_pages = B * pages_per_seq
    caches = []
    for _ in range(S.LAYERS):
        c = K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev)
        c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device=dev, dtype=torch.int8))
        c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device=dev, dtype=torch.int8))
        c.k_scale.uniform_(0.01, 0.04, generator=gen)
        c.v_scale.uniform_(0.01, 0.04, generator=gen)
        caches.append(c)
    table = torch.randperm(num_pages, generator=gen, device=dev).to(torch.int32).reshape(B, pages_per_seq)
    cached = torch.full((B,), n - 1, dtype=torch.int32, device=dev)  # the new token is the ctx-th
    nd = torch.tensor([B], dtype=torch.int32, device=dev)
    ids = torch.randint(0, S.VOCAB, (B,), generator=gen, device=dev, dtype=torch.int32)
    qkv = torch.randn(B, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
    q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
    q, k, v = q.view(B, HQ, D), k.view(B, HKV, D), v.view(B, HKV, D)
    cos, sin = model.rope(cached)

    def step():
        return model.forward(caches, None, ids, cached, table, nd)

    def path_only():
        for L, c in zip(model.layers, caches):
            S.attention_ops(q, k, v, L["qn"], L["kn"], cos, sin, c, None, cached, table, nd, None)

    def graph_ms(fn):
        with torch.inference_mode():
            fn()
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                res = fn()
        for _ in range(max(args.warmup, 3)):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts), res

    tuned = None
    if args.tune:
        # what the reference's Engine does before capturing its graphs (engine.py:91-103): each weight shape is timed
        # with both matmuls at this step's row count and the faster is kept
        L0 = model.layers[0]
        K.tune_linear([L0["qkv"], L0["o"], L0["gate_up"], L0["down"], model.embed], [B])
        tuned = {f"{N}x{Kd}": s for (N, Kd, M), s in sorted(K.use_skinny.items()) if M == B}
    step_ms, toks = graph_ms(step)
    path_ms, _ = graph_ms(path_only)
    kv_bytes = S.LAYERS * (B * n * 2112 + B * WRITE_BYTES_PER_TOKEN)
    print(json.dumps({
        "case": "pure decode step of the random-init decoder", "batch": B, "ctx": n, "layers": S.LAYERS,
        "step_ms": round(step_ms, 3), "tokens_per_s": round(B / step_ms * 1e3), "attention_path_ms": round(path_ms, 3),
        "attention_path_share": round(path_ms / step_ms, 3), "attention_path_gbs": round(kv_bytes / path_ms / 1e6, 1),
        "matmul_cluster_size_by_weight (0 = cuBLAS)": tuned,
        "status": K.check_status(dev), "sampled_head": toks[:4].tolist(), "data": "synthetic ids, random-init weights"}), flush=True)


def run_path(args):
    """--path: each op of the mixed step's attention path timed alone (seed 3 shapes: 32 decoding sequences
    with contexts ~U[128,4096] + one 992-row chunk on a prior context of 0 and of 3072 tokens, 34 entries,
    1024 packed rows), then all six in the engine's call order.  CUDA graph of 10 calls on 10 distinct layer
    caches, median of `steps` replays, microseconds per call."""
    import torch

    from inference_engine_b200 import kernels as K
    from inference_engine_b200 import scaffold as S

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K.set_early_start(not args.no_early_start)
    n_dec, chunk, n_tokens, reps = 32, 992, 1024, 10
    for prior in (0, 3072):
        gen = torch.Generator().manual_seed(3)
        dgen = torch.Generator(device=dev).manual_seed(3)
        ctx = torch.randint(128, 4097, (n_dec,), generator=gen).tolist()
        plan = S.plan_step(ctx, [(prior, chunk)], n_tokens, n_dec + 2)
        table, pages = S.assign_pages(plan, PAGE, (4096 + PAGE) // PAGE + 1, generator=gen)
        inp = S.upload_step(plan, table, [0] * n_tokens, dev)
        caches = []
        for _ in range(reps):
            c = K.make_layer_cache(pages, HKV, PAGE, D, device=dev)
            c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=dgen, device=dev, dtype=torch.int8))
            c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=dgen, device=dev, dtype=torch.int8))
            c.k_scale.uniform_(0.01, 0.04, generator=dgen)
            c.v_scale.uniform_(0.01, 0.04, generator=dgen)
            caches.append(c)
        cap = max(prior, 16)
        prefix = S.PrefixScratch(torch.empty(HKV, cap, D, device=dev, dtype=torch.bfloat16),
                                 torch.empty(HKV, cap, D, device=dev, dtype=torch.bfloat16), inp.cu_cached)
        qkv = torch.randn(n_tokens, (HQ + 2 * HKV) * D, generator=dgen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(-1, HQ, D), k.view(-1, HKV, D), v.view(-1, HKV, D)
        qw = torch.ones(D, device=dev, dtype=torch.bfloat16)
        inv = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D)
        ang = inp.positions[:, None, None] * inv[None, None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        E, tab, cl, nd = inp.block_table.shape[0], inp.block_table, inp.cached_lens, inp.num_decoding
        q_p, k_p = K.fused_norm_rope_prefill(q, k, qw, qw, cos, sin, 1e-6)
        out = torch.empty(n_tokens, HQ, D, device=dev, dtype=torch.bfloat16)
        hid = torch.randn(n_tokens, 2048, generator=dgen, device=dev).to(torch.bfloat16)
        hid2 = torch.randn(n_tokens, 2048, generator=dgen, device=dev).to(torch.bfloat16)
        lnw = torch.ones(2048, device=dev, dtype=torch.bfloat16)
        gate_up = torch.randn(n_tokens, 12288, generator=dgen, device=dev).to(torch.bfloat16)
        q_d = K.fused_rope_kv_decode(q[:E], k[:E], v[:E], qw, qw, cos[:E], sin[:E], tab, caches[0], cl, nd, 1e-6)
        ops = {
            "fused_norm_rope_prefill": lambda c: K.fused_norm_rope_prefill(q, k, qw, qw, cos, sin, 1e-6),
            "quantize_kv_prefill": lambda c: K.quantize_kv_prefill(k_p, v, inp.cu_seqlens, tab, cl, nd, c),
            "dequantize_kv_prefix": lambda c: K.dequantize_kv_prefix(c, prefix.cu_cached, tab, prefix.k, prefix.v),
            "prefill_attention": lambda c: K.prefill_attention(q_p, k_p, v, inp.seq_ids, inp.cu_seqlens, inp.tile_start,
                                                               prefix.k, prefix.v, prefix.cu_cached, 128),
            "fused_rope_kv_decode": lambda c: K.fused_rope_kv_decode(q[:E], k[:E], v[:E], qw, qw, cos[:E], sin[:E], tab, c,
                                                                     cl, nd, 1e-6),
            "decode_attention": lambda c: K.decode_attention(q_d, c, cl, tab, nd, D ** -0.5, out=out),
            "all six in the engine's order": lambda c: S.attention_ops(q, k, v, qw, qw, cos, sin, c, inp, cl, tab, nd, prefix),
            # the block's two element-wise ops at this step's sizes (hidden 2048, FFN 6144)
            "add_rms_norm [1024 x 2048]": lambda c: K.add_rms_norm(hid, hid2, lnw, 1e-6),
            "silu_mul [1024 x 12288]": lambda c: K.silu_mul(gate_up),
        }
        line = {"case": "attention path of the mixed step, per op", "prior_context": prior, "us_per_call": {}}
        for name, fn in ops.items():
            def call():
                for c in caches:
                    fn(c)
            call()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                call()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / reps)
            line["us_per_call"][name] = round(statistics.median(ts), 1)
        line["status"] = K.check_status(dev)
        print(json.dumps(line), flush=True)
        del caches
        torch.cuda.empty_cache()


def run_prefill(args):
    """--prefill: the chunked-prefill attention kernel alone (seed 3 shapes): one 992-row chunk on a
    prior context of 0/1024/2048/3072 tokens, 16 q heads over 8 kv heads, block_m 128, bf16 ~N(0,1).
    Both kernels (1 = mma.sync, 2 = tcgen05), CUDA graph of 10 calls, median of `steps` replays.
    FLOPs counted: 4 * D * visible (query, key) pairs * q heads (causal pairs, not padded tiles)."""
    import torch

    from inference_engine_b200 import kernels as K
    from inference_engine_b200 import scaffold as S

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(3)
    chunk, reps = 992, 10
    for prior in (0, 1024, 2048, 3072):
        plan = S.plan_step([], [(prior, chunk)], chunk, 2)
        table, _ = S.assign_pages(plan, PAGE, (prior + chunk) // PAGE + 1)
        inp = S.upload_step(plan, table, [0] * chunk, dev)
        qkv = torch.randn(chunk, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(-1, HQ, D), k.view(-1, HKV, D), v.view(-1, HKV, D)
        kp = torch.randn(HKV, max(prior, 16), D, generator=gen, device=dev).to(torch.bfloat16)
        vp = torch.randn(HKV, max(prior, 16), D, generator=gen, device=dev).to(torch.bfloat16)
        pairs = chunk * prior + chunk * (chunk + 1) // 2
        flops = 4.0 * D * pairs * HQ
        outs = {}
        for variant in (1, 2):
            def call():
                for _ in range(reps):
                    outs[variant] = K.prefill_attention(q, k, v, inp.seq_ids, inp.cu_seqlens, inp.tile_start, kp, vp,
                                                        inp.cu_cached, 128, variant=variant)
            call()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                call()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / reps)
            us = statistics.median(ts)
            print(json.dumps({"case": "prefill_attention", "kernel": {1: "mma.sync", 2: "tcgen05"}[variant],
                              "chunk": chunk, "prior_context": prior, "us_per_call": round(us, 1),
                              "tflops": round(flops / us / 1e6, 1), "status": K.check_status(dev)}), flush=True)
        diff = (outs[1].float() - outs[2].float()).abs().max().item()
        print(json.dumps({"case": "prefill_attention", "prior_context": prior, "max_abs_diff_between_kernels": diff}), flush=True)


def run_mixed(args):
    """--mixed: one chunked-prefill + decode step (seed 3) inside a random-init Qwen3-1.7B-shaped
    decoder (28 layers, hidden 2048, FFN 6144, vocab 151936, tied embeddings, weights ~N(0,0.02)):
    32 decoding sequences (contexts ~U[128,4096]) + one 992-token chunk on a prior context of
    0/1024/2048/3072 tokens = 1024 tokens per step, int8 paged cache (16-token pages, random block
    table).  The step is captured as one CUDA graph (embedding -> 28 layers -> final norm -> tied
    lm_head -> sampler) and replayed; a second graph holds only the attention-path ops of the 28
    layers on the same metadata, to state their share of the step.  One JSON line per prior."""
    import torch

    from inference_engine_b200 import kernels as K
    from inference_engine_b200 import scaffold as S

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    K.set_early_start(not args.no_early_start)
    gen = torch.Generator().manual_seed(3)
    model = S.DecoderScaffold(dev, seed=3)
    n_dec, chunk, n_tokens = 32, 992, 1024
    entries = n_dec + 2
    ctx = torch.randint(128, 4097, (n_dec,), generator=gen).tolist()
    max_pages = (4096 + PAGE) // PAGE + 1
    for prior in (0, 1024, 2048, 3072):
        plan = S.plan_step(ctx, [(prior, chunk)], n_tokens, entries)
        table, pages = S.assign_pages(plan, PAGE, max_pages, generator=gen)
        ids = torch.randint(0, S.VOCAB, (n_tokens,), generator=gen).tolist()
        inp = S.upload_step(plan, table, ids, dev)
        dgen = torch.Generator(device=dev).manual_seed(3)
        caches = []
        for _ in range(S.LAYERS):
            c = K.make_layer_cache(pages, HKV, PAGE, D, device=dev)
            c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=dgen, device=dev, dtype=torch.int8))
            c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=dgen, device=dev, dtype=torch.int8))
            c.k_scale.uniform_(0.01, 0.04, generator=dgen)
            c.v_scale.uniform_(0.01, 0.04, generator=dgen)
            caches.append(c)
        cap = max(prior, 16)
        prefix = S.PrefixScratch(torch.empty(HKV, cap, D, device=dev, dtype=torch.bfloat16),
                                 torch.empty(HKV, cap, D, device=dev, dtype=torch.bfloat16), inp.cu_cached)

        def step():
            return model.forward(caches, inp, inp.ids, inp.cached_lens, inp.block_table, inp.num_decoding, prefix)

        qkv = torch.randn(n_tokens, (HQ + 2 * HKV) * D, generator=dgen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(-1, HQ, D), k.view(-1, HKV, D), v.view(-1, HKV, D)
        cos, sin = model.rope(inp.positions)

        def star_only():
            for L, c in zip(model.layers, caches):
                S.attention_ops(q, k, v, L["qn"], L["kn"], cos, sin, c, inp, inp.cached_lens, inp.block_table,
                                inp.num_decoding, prefix)

        def graph_ms(fn):
            with torch.inference_mode():
                fn()
                fn()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    res = fn()
            for _ in range(max(args.warmup, 3)):
                g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts), res

        step_ms, toks = graph_ms(step)
        star_ms, _ = graph_ms(star_only)
        status = K.check_status(dev)
        print(json.dumps({
            "case": "mixed step: 32 decode (ctx~U[128,4096]) + 992-token chunk", "prior_context": prior,
            "tokens_per_step": n_tokens, "step_ms": round(step_ms, 3), "tokens_per_s": round(n_tokens / step_ms * 1e3),
            "attention_path_ms": round(star_ms, 3), "attention_path_share": round(star_ms / step_ms, 3),
            "decode_kv_tokens": sum(ctx) + n_dec, "status": status, "sampled_head": toks[:4].tolist(),
            "data": "synthetic ids, random-init weights"}), flush=True)
        del caches, prefix
        torch.cuda.empty_cache()


def find_reference(args):
    cands = []
    for base in (args.reference, os.environ.get("B200KV_REFERENCE")):
        if base:
            cands += [base, os.path.join(base, "qwen3-1.7b")]
    cands.append(os.path.join(ROOT, "baseline", "_ref", "qwen3-1.7b"))
    for c in cands:
        if os.path.exists(os.path.join(c, "kernels.py")):
            return c
    return None


def run_vs_triton(args):
    """--vs-triton [--reference PATH]: the reference's own Triton kernels (qwen3-1.7b/kernels.py, imported from PATH,
    from B200KV_REFERENCE or from the staged copy under baseline/_ref; JIT-compiled by the installed Triton for this
    GPU, autotuned during warm-up, outside every timed region) beside this library's kernels, same inputs, in the
    reference's one-row-per-sequence cache layout, which both accept.  CUDA graph of L calls on L distinct caches,
    median of `steps` replays, microseconds per call.  One JSON line per case:
      decode_attention: the 40 cells of the sweep configuration (ours unplanned and with the step's plan);
      fused_rope_kv_decode at T = 1, 64, 1024; fused_norm_rope_prefill + quantize_kv_prefill at T = 64, 1024;
      dequantize_kv_prefix + prefill_attention for a 992-row chunk on 0 / 1024 / 2048 / 3072 cached tokens;
    with the differences between the two implementations' results (bit mismatches for codes, scales and rotated
    q/k; max-abs for attention outputs)."""
    import importlib.util

    import torch

    from inference_engine_b200 import kernels as K

    path = find_reference(args)
    if path is None:
        print(json.dumps({"case": "vs-triton", "unavailable": "no reference checkout: pass --reference PATH"}))
        return
    spec = importlib.util.spec_from_file_location("reference_kernels", os.path.join(path, "kernels.py"))
    R = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(R)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(2)

    def mine(c):
        return K.LayerKVCache(c.k, c.v, c.k_scale, c.v_scale, c.k_calibration)

    def graph_us(fn, reps_in_graph):
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / reps_in_graph)
        return statistics.median(ts)

    def ref_cache(rows, max_len, filled=True):
        shape = (rows, HKV, max_len, D)
        if filled:
            k = torch.randint(-127, 128, shape, generator=gen, device=dev, dtype=torch.int8)
            v = torch.randint(-127, 128, shape, generator=gen, device=dev, dtype=torch.int8)
            ks = 0.01 + 0.03 * torch.rand(shape[:3], generator=gen, device=dev)
            vs = 0.01 + 0.03 * torch.rand(shape[:3], generator=gen, device=dev)
        else:
            k, v = torch.zeros(shape, device=dev, dtype=torch.int8), torch.zeros(shape, device=dev, dtype=torch.int8)
            ks, vs = torch.zeros(shape[:3], device=dev), torch.zeros(shape[:3], device=dev)
        return R.LayerKVCache(k, v, ks, vs, torch.ones(rows, HKV, 1, D, device=dev))

    def bits_differ(a, b):
        return int((a.contiguous().view(torch.uint8) != b.contiguous().view(torch.uint8)).sum().item())

    # ---- decode attention, the 40 cells
    dropped = {(256, 4096), (256, 2048), (128, 4096), (256, 1024), (128, 2048)}
    for B in (1, 2, 4, 8, 16, 32, 64, 128, 256):
        for n in (128, 512, 1024, 2048, 4096):
            if (B, n) in dropped and not args.all_cells:
                continue
            nbytes = attn_bytes(B, n)
            L = int(min(28, max(4, -(-300_000_000 // nbytes))))
            caches = [ref_cache(B + 1, n) for _ in range(L)]
            q = torch.randn(B, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
            cl = torch.full((B,), n - 1, dtype=torch.int32, device=dev)
            slots = torch.randperm(B + 1, generator=gen, device=dev)[:B].to(torch.int32)
            nd = torch.tensor([B], dtype=torch.int32, device=dev)
            outs = {}

            def run_ref():
                for c in caches:
                    outs["ref"] = R.decode_attention(q, c, cl, slots, nd, D ** -0.5)

            def run_mine(planned):
                plan = K.plan_decode_step(cl, slots, nd, mine(caches[0])) if planned else None
                for c in caches:
                    outs["mine"] = K.decode_attention(q, mine(c), cl, slots, nd, D ** -0.5, plan=plan)

            line = {"case": "decode_attention", "B": B, "ctx": n, "layers_in_graph": L, "bytes": nbytes}
            try:
                line["triton_us"] = round(graph_us(run_ref, L), 2)
            except Exception as e:  # noqa: BLE001
                line["triton_error"] = repr(e)[:200]
            line["ours_us"] = round(graph_us(lambda: run_mine(False), L), 2)
            line["ours_planned_us"] = round(graph_us(lambda: run_mine(True), L), 2)
            if "ref" in outs:
                d = (outs["ref"].float() - outs["mine"].float()).abs()
                line.update({"max_abs_diff": float(d.max()), "mean_abs_diff": float(d.mean()),
                             "speedup_vs_triton": round(line["triton_us"] / line["ours_planned_us"], 3)})
            line["status"] = K.check_status(dev)
            print(json.dumps(line), flush=True)
            del caches
            torch.cuda.empty_cache()

    # ---- quantize-on-write, decode flavour: T tokens = T sequences, one row each
    qw = (1 + 0.02 * torch.randn(D, generator=gen, device=dev)).to(torch.bfloat16)
    kw = (1 + 0.02 * torch.randn(D, generator=gen, device=dev)).to(torch.bfloat16)
    inv_freq = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D)
    reps = 10
    for T in (1, 64, 1024):
        max_len = 64
        qkv = torch.randn(T, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(T, HQ, D), k.view(T, HKV, D), v.view(T, HKV, D)
        cl = torch.randint(0, max_len, (T,), generator=gen, device=dev, dtype=torch.int32)
        pos = torch.randint(0, 32768, (T,), generator=gen, device=dev, dtype=torch.int32)
        ang = pos[:, None, None] * inv_freq[None, None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        slots = torch.randperm(T + 1, generator=gen, device=dev)[:T].to(torch.int32)
        nd = torch.tensor([T], dtype=torch.int32, device=dev)
        ca = [ref_cache(T + 1, max_len, filled=False) for _ in range(reps)]
        cb = [ref_cache(T + 1, max_len, filled=False) for _ in range(reps)]
        for c in ca + cb:
            c.k_calibration.copy_(0.5 + torch.rand(c.k_calibration.shape, generator=torch.Generator(device=dev).manual_seed(9), device=dev))
        res = {}

        def w_ref():
            for c in ca:
                res["ref"] = R.fused_rope_kv_decode(q, k, v, qw, kw, cos, sin, slots, c, cl, nd, 1e-6)

        def w_mine():
            for c in cb:
                res["mine"] = K.fused_rope_kv_decode(q, k, v, qw, kw, cos, sin, slots, mine(c), cl, nd, 1e-6)

        line = {"case": "fused_rope_kv_decode", "T": T}
        try:
            line["triton_us"] = round(graph_us(w_ref, reps), 2)
        except Exception as e:  # noqa: BLE001
            line["triton_error"] = repr(e)[:200]
        line["ours_us"] = round(graph_us(w_mine, reps), 2)
        if "ref" in res:
            line.update({"q_bits_differing_elements": int((res["ref"].view(torch.int16) != res["mine"].view(torch.int16)).sum().item()),
                         "code_bytes_differing": bits_differ(ca[0].k, cb[0].k) + bits_differ(ca[0].v, cb[0].v),
                         "scales_differing": int((ca[0].k_scale != cb[0].k_scale).sum().item() + (ca[0].v_scale != cb[0].v_scale).sum().item()),
                         "elements": {"q": T * HQ * D, "codes": 2 * T * HKV * D, "scales": 2 * T * HKV},
                         "speedup_vs_triton": round(line["triton_us"] / line["ours_us"], 3)})
        print(json.dumps(line), flush=True)

    # ---- quantize-on-write, prefill flavour: one first chunk of T rows
    for T in (64, 1024):
        qkv = torch.randn(T, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(T, HQ, D), k.view(T, HKV, D), v.view(T, HKV, D)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        ang = pos[:, None, None] * inv_freq[None, None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        slots = torch.tensor([1], dtype=torch.int32, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        ca = [ref_cache(2, T, filled=False) for _ in range(reps)]
        cb = [ref_cache(2, T, filled=False) for _ in range(reps)]
        res = {}

        def p_ref():
            for c in ca:
                q_p, k_p = R.fused_norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
                R.quantize_kv_prefill(k_p, v, cu, slots, zero, zero, c)
                res["ref"] = (q_p, k_p)

        def p_mine():
            for c in cb:
                q_p, k_p = K.fused_norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
                K.quantize_kv_prefill(k_p, v, cu, slots, zero, zero, mine(c))
                res["mine"] = (q_p, k_p)

        line = {"case": "fused_norm_rope_prefill + quantize_kv_prefill (first chunk)", "T": T}
        try:
            line["triton_us"] = round(graph_us(p_ref, reps), 2)
        except Exception as e:  # noqa: BLE001
            line["triton_error"] = repr(e)[:200]
        line["ours_us"] = round(graph_us(p_mine, reps), 2)
        if "ref" in res:
            line.update({"qk_bits_differing_elements": int(sum((a.view(torch.int16) != b.view(torch.int16)).sum().item()
                                                               for a, b in zip(res["ref"], res["mine"]))),
                         "code_bytes_differing": bits_differ(ca[0].k, cb[0].k) + bits_differ(ca[0].v, cb[0].v),
                         "scales_differing": int((ca[0].k_scale != cb[0].k_scale).sum().item() + (ca[0].v_scale != cb[0].v_scale).sum().item()),
                         "calibration_differing": int((ca[0].k_calibration != cb[0].k_calibration).sum().item()),
                         "speedup_vs_triton": round(line["triton_us"] / line["ours_us"], 3)})
        print(json.dumps(line), flush=True)

    # ---- prefix dequantize + prefill attention: a 992-row chunk on `prior` cached tokens
    chunk = 992
    for prior in (0, 1024, 2048, 3072):
        from inference_engine_b200 import scaffold as S

        plan = S.plan_step([], [(prior, chunk)], chunk, 2)
        inp = S.upload_step(plan, torch.zeros(2, 1, dtype=torch.int32), [0] * chunk, dev)
        slots = torch.tensor([1, 0], dtype=torch.int32, device=dev)
        cache = ref_cache(2, 4096)
        qkv = torch.randn(chunk, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(-1, HQ, D), k.view(-1, HKV, D), v.view(-1, HKV, D)
        cap = max(prior, 16)
        pk = [torch.zeros(HKV, cap, D, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        pv = [torch.zeros(HKV, cap, D, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        res = {}

        def a_ref():
            for _ in range(reps):
                R.dequantize_kv_prefix(cache, inp.cu_cached, slots, pk[0], pv[0])
                res["ref"] = R.prefill_attention(q, k, v, inp.seq_ids, inp.cu_seqlens, inp.tile_start, pk[0], pv[0], inp.cu_cached, 128)

        def a_mine():
            for _ in range(reps):
                K.dequantize_kv_prefix(mine(cache), inp.cu_cached, slots, pk[1], pv[1])
                res["mine"] = K.prefill_attention(q, k, v, inp.seq_ids, inp.cu_seqlens, inp.tile_start, pk[1], pv[1], inp.cu_cached, 128)

        pairs = chunk * prior + chunk * (chunk + 1) // 2
        line = {"case": "dequantize_kv_prefix + prefill_attention", "chunk": chunk, "prior_context": prior}
        try:
            line["triton_us"] = round(graph_us(a_ref, reps), 2)
        except Exception as e:  # noqa: BLE001
            line["triton_error"] = repr(e)[:200]
        line["ours_us"] = round(graph_us(a_mine, reps), 2)
        line["ours_tflops"] = round(4.0 * D * pairs * HQ / line["ours_us"] / 1e6, 1)
        if "ref" in res:
            d = (res["ref"].float() - res["mine"].float()).abs()
            line.update({"prefix_bits_differing_elements": int((pk[0].view(torch.int16) != pk[1].view(torch.int16)).sum().item()
                                                               + (pv[0].view(torch.int16) != pv[1].view(torch.int16)).sum().item()),
                         "max_abs_diff": float(d.max()), "mean_abs_diff": float(d.mean()),
                         "speedup_vs_triton": round(line["triton_us"] / line["ours_us"], 3)})
        line["status"] = K.check_status(dev)
        print(json.dumps(line), flush=True)


def run_linear(args):
    """--linear: the weight-streaming matmul of the decode step (kernels.skinny_matmul, tcgen05) beside cuBLAS
    (F.linear) at the five weight shapes of the Qwen3-1.7B-shaped decoder and M = 1, 8, 64 rows.  Each case is a
    CUDA graph of R calls on R distinct weight copies (R chosen so that the graph streams more than 400 MB, above the
    126 MB L2), median of `steps` replays.  GB/s = weight bytes / time; fractions are of the measured copy peak."""
    import torch
    import torch.nn.functional as F

    from inference_engine_b200 import kernels as K

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    gen = torch.Generator(device=dev).manual_seed(6)
    shapes = {"qkv": (4096, 2048), "o": (2048, 2048), "gate_up": (12288, 2048), "down": (2048, 6144), "lm_head": (151936, 2048)}
    for name, (N, Kd) in shapes.items():
        wbytes = N * Kd * 2
        R = int(min(64, max(2, -(-400_000_000 // wbytes))))
        ws = [(torch.randn(N, Kd, generator=gen, device=dev) * 0.02).to(torch.bfloat16) for _ in range(R)]
        for M in (1, 8, 64):
            x = torch.randn(M, Kd, generator=gen, device=dev).to(torch.bfloat16)

            def graph_us(fn):
                fn()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    fn()
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                ts = []
                for _ in range(args.steps):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1e3 / R)
                return statistics.median(ts)

            line = {"case": "linear", "weight": name, "N": N, "K": Kd, "M": M, "weights_in_graph": R,
                    "cublas_us": round(graph_us(lambda: [F.linear(x, w) for w in ws]), 2)}
            best = None
            for s in K.skinny_supported(M, N, Kd):
                us = graph_us(lambda: [K.skinny_matmul(x, w, s) for w in ws])
                line[f"skinny_s{s}_us"] = round(us, 2)
                if best is None or us < best[0]:
                    best = (us, s)
            line.update({"best_splits": best[1], "best_us": round(best[0], 2), "gbs": round(wbytes / best[0] / 1e3, 1),
                         "frac_of_measured": round(wbytes / best[0] / 1e3 / peak, 4),
                         "speedup_vs_cublas": round(line["cublas_us"] / best[0], 3), "status": K.check_status(dev)})
            print(json.dumps(line), flush=True)
        del ws
        torch.cuda.empty_cache()


def run_phases(args):
    """--phases: where the time of one decode_attention launch goes, from the instrumented build of the library
    (libb200kv_stamps.so: the same sources with -DB200KV_STAMPS; every warp records %globaltimer at kernel entry and
    exit, its SM id, and SM clock cycles since its entry at: metadata there, first copies issued, q loaded, first
    tile landed, last tile consumed, last piece stored, arrival counter answered, merge done, exit).  For each
    shape, planned and unplanned, six launches on six distinct caches AND six distinct page tables, each after an
    L2 flush: medians over warps in microseconds (cycles / the SM clock measured from the two timers), the slowest
    warp, how far each SM's streaming time (equal work per warp) sits from the mean, the spread of the warps inside
    an SM, and whether the slow SMs are the same ones from launch to launch.  --dump PATH also saves the raw
    per-warp words of the B=64 launches as .npy."""
    import ctypes

    import torch

    from inference_engine_b200 import _lib, build

    if not os.path.exists(build.STAMPS_LIB) or os.path.getmtime(build.STAMPS_LIB) < os.path.getmtime(build.LIB):
        build.build(force=True)
    _lib.use_library(build.STAMPS_LIB)
    from inference_engine_b200 import kernels as K

    lib = _lib.load()
    lib.b200kv_stamps_read.restype = ctypes.c_int
    lib.b200kv_stamps_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(2)
    NW = 16
    buf = np.zeros((4096, NW), np.uint64)
    reps = 6
    names = {8: "metadata_there", 2: "first_copies_issued", 9: "q_loaded", 3: "first_tile_landed", 4: "last_tile_consumed",
             10: "last_piece_stored", 13: "exit"}
    for B, n in ((64, 4096), (1, 4096), (8, 1024), (32, 2048), (1, 128)):
        pages_per_seq = (n + PAGE - 1) // PAGE
        num_pages = B * pages_per_seq + 1
        caches, tables = [], []
        for r in range(reps):
            c = K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev)
            c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device=dev, dtype=torch.int8))
            c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device=dev, dtype=torch.int8))
            c.k_scale.fill_(0.02)
            c.v_scale.fill_(0.02)
            caches.append(c)
            t = torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(100 + r)).to(torch.int32)
            tables.append(t.reshape(B, pages_per_seq).to(dev))
        q = torch.randn(B, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        cached = torch.full((B,), n - 1, dtype=torch.int32, device=dev)
        nd = torch.tensor([B], dtype=torch.int32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for planned in (False, True):
            per_sm, med, worst, in_sm, merge, raw = [], [], [], [], [], []
            for r in range(reps + 1):  # the first launch is a warm-up
                c, tab = caches[r % reps], tables[r % reps]
                plan = K.plan_decode_step(cached, tab, nd, c) if planned else None
                flush.zero_()
                torch.cuda.synchronize()
                lib.b200kv_stamps_read(buf.ctypes.data, 1)
                K.decode_attention(q, c, cached, tab, nd, D ** -0.5, out=out, plan=plan)
                torch.cuda.synchronize()
                lib.b200kv_stamps_read(buf.ctypes.data, 1)
                if r == 0:
                    continue
                live = buf[:, 0] > 0
                t = buf[live].astype(np.float64)
                raw.append(buf[live].copy())
                mhz = np.median(t[:, 13] / np.maximum(t[:, 5] - t[:, 0], 1.0)) * 1e3  # cycles per microsecond
                us = lambda col: t[:, col] / mhz
                entry = (t[:, 0] - t[:, 0].min()) / 1e3
                med.append([float(np.median(entry))] + [float(np.median(us(k))) for k in names])
                worst.append([float((entry + us(4)).max()), float((entry + us(13)).max()), float((t[:, 5].max() - t[:, 0].min()) / 1e3)])
                last = t[:, 12] > 0  # warps that merged
                if last.any():
                    merge.append([float(np.median(us(11)[last] - us(10)[last])), float(np.median(us(12)[last] - us(11)[last])),
                                  float(np.median(t[last, 7]))])
                sm = t[:, 1].astype(int)
                stream = us(4) - us(3)
                per_sm.append([float(stream[sm == i].mean()) if (sm == i).any() else float("nan") for i in range(148)])
                in_sm.append(float(np.nanmean([stream[sm == i].max() - stream[sm == i].min() for i in range(148) if (sm == i).sum() > 1] or [0.0])))
            per_sm = np.array(per_sm)
            ok = ~np.isnan(per_sm).any(axis=0)
            corr = np.corrcoef(per_sm[:, ok]) if ok.sum() > 2 else np.zeros((1, 1))
            off = corr[~np.eye(corr.shape[0], dtype=bool)] if corr.ndim == 2 else np.zeros(0)
            mean_sm = np.where(ok, np.nan_to_num(per_sm).mean(axis=0), np.nan)
            order = np.argsort(-np.nan_to_num(mean_sm))
            m, wst = np.median(np.array(med), axis=0), np.median(np.array(worst), axis=0)
            line = {"case": "decode_attn_kernel phases", "B": B, "ctx": n, "planned": planned, "launches": reps,
                    "warps_with_work": int(live.sum()), "sm_clock_mhz": round(float(mhz), 1),
                    "us_since_own_entry_median_over_warps": dict({"kernel_entry_after_first": round(m[0], 2)},
                                                                 **{nm: round(m[i + 1], 2) for i, nm in enumerate(names.values())}),
                    "us_since_first_entry_slowest_warp": {"last_tile_consumed": round(wst[0], 2), "exit": round(wst[1], 2),
                                                          "kernel_span": round(wst[2], 2)},
                    "per_sm_stream_us": {"mean": round(float(np.nanmean(mean_sm)), 2), "min": round(float(np.nanmin(mean_sm)), 2),
                                         "max": round(float(np.nanmax(mean_sm)), 2),
                                         "spread_of_warps_inside_an_sm": round(float(np.mean(in_sm)), 2),
                                         "launch_to_launch_correlation": round(float(off.mean()) if off.size else 0.0, 3),
                                         "slowest_sms": [int(i) for i in order[:40]],
                                         "by_sm": [round(float(x), 2) for x in mean_sm]}}
            if merge:
                mm = np.median(np.array(merge), axis=0)
                line["last_arriver_us"] = {"piece_stored_to_counter_answered": round(mm[0], 2), "merge": round(mm[1], 2),
                                           "pieces": mm[2]}
            print(json.dumps(line), flush=True)
            if args.dump and B == 64:
                np.save(f"{args.dump}_B{B}_ctx{n}_{'planned' if planned else 'plain'}.npy", np.stack([r[: min(len(x) for x in raw)] for r in raw]))
        del caches, tables
        torch.cuda.empty_cache()


def run_write(args):
    """--write: the fused quantize-on-write microbench (seed 1): T in {1, 64, 1024} new tokens,
    q [T,16,128], k,v [T,8,128] bf16 as strided views of one [T,4096] projection row, positions
    uniform in [0,32768), per-head QK-RMSNorm (weights 1+N(0,0.02)) + RoPE(1e6) + int8 quantize
    into a 16-token paged cache at random free slots.  Decode flavour (fused_rope_kv_decode, fp32
    all the way) for every T, prefill flavour (norm+rope -> bf16 -> calibration -> quantize) for
    T >= 64.  One JSON line per case: microseconds per call (CUDA graph of 20 calls on distinct
    caches) and algorithmic GB/s at 14,656 B per token."""
    import torch

    from inference_engine_b200 import kernels as K

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    reps = 20
    for T in (1, 64, 1024):
        qkv = torch.randn(T, (HQ + 2 * HKV) * D, generator=gen, device=dev).to(torch.bfloat16)
        q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
        q, k, v = q.view(T, HQ, D), k.view(T, HKV, D), v.view(T, HKV, D)
        qw = (1 + 0.02 * torch.randn(D, generator=gen, device=dev)).to(torch.bfloat16)
        kw = (1 + 0.02 * torch.randn(D, generator=gen, device=dev)).to(torch.bfloat16)
        pos = torch.randint(0, 32768, (T,), generator=gen, device=dev, dtype=torch.int32)
        inv_freq = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D)
        ang = pos[:, None, None] * inv_freq[None, None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        # every token is its own sequence at position pos: page 0 of its table holds the calibration row,
        # the page of its position a random free slot
        num_pages = 2 * T + 2
        perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
        table = torch.zeros(T, 32768 // PAGE, dtype=torch.int32)
        rows = torch.arange(T)
        table[rows, 0] = perm[2 * rows]
        slot = (pos.cpu() // PAGE).long()
        table[rows, slot] = torch.where(slot > 0, perm[2 * rows + 1], perm[2 * rows])
        table = table.to(dev)
        caches = [K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev) for _ in range(reps)]
        nd = torch.tensor([T], dtype=torch.int32, device=dev)

        def timed(fn):
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / reps)
            return statistics.median(ts)

        def decode_flavour():
            for c in caches:
                K.fused_rope_kv_decode(q, k, v, qw, kw, cos, sin, table, c, pos, nd, 1e-6)

        us = timed(decode_flavour)
        print(json.dumps({"case": "fused_rope_kv_decode", "T": T, "us_per_call": round(us, 2),
                          "gbs": round(T * WRITE_BYTES_PER_TOKEN / us / 1e3, 1), "kernels_per_call": 1}), flush=True)
        if T >= 64:
            # one prefill chunk of T tokens (first chunk: calibration is computed), written from position 0
            cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
            tab1 = torch.arange(1, 1 + (T + PAGE - 1) // PAGE, dtype=torch.int32, device=dev)[None, :].contiguous()
            zero = torch.zeros(1, dtype=torch.int32, device=dev)
            pcaches = [K.make_layer_cache(2 + (T + PAGE - 1) // PAGE, HKV, PAGE, D, device=dev) for _ in range(reps)]

            def prefill_flavour():
                for c in pcaches:
                    q_p, k_p = K.fused_norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
                    K.quantize_kv_prefill(k_p, v, cu, tab1, zero, zero, c)

            us = timed(prefill_flavour)
            print(json.dumps({"case": "fused_norm_rope_prefill + quantize_kv_prefill (first chunk)", "T": T,
                              "us_per_call": round(us, 2), "gbs": round(T * WRITE_BYTES_PER_TOKEN / us / 1e3, 1),
                              "kernels_per_call": 3}), flush=True)

            def fused_flavour():
                for c in pcaches:
                    K.write_prefill(q, k, v, qw, kw, cos, sin, cu, tab1, zero, zero, c, 1e-6)

            us = timed(fused_flavour)
            print(json.dumps({"case": "write_prefill (the two calls as one, first chunk)", "T": T,
                              "us_per_call": round(us, 2), "gbs": round(T * WRITE_BYTES_PER_TOKEN / us / 1e3, 1),
                              "kernels_per_call": 2}), flush=True)
            # a later chunk of the same prompt: the calibration exists, only the row kernel has work
            later = torch.tensor([T], dtype=torch.int32, device=dev)
            tab2 = torch.arange(1, 1 + (2 * T + PAGE - 1) // PAGE, dtype=torch.int32, device=dev)[None, :].contiguous()
            lcaches = [K.make_layer_cache(2 + (2 * T + PAGE - 1) // PAGE, HKV, PAGE, D, device=dev) for _ in range(reps)]

            def fused_later():
                for c in lcaches:
                    K.write_prefill(q, k, v, qw, kw, cos, sin, cu, tab2, later, zero, c, 1e-6)

            us = timed(fused_later)
            print(json.dumps({"case": "write_prefill (a later chunk: calibration loaded)", "T": T,
                              "us_per_call": round(us, 2), "gbs": round(T * WRITE_BYTES_PER_TOKEN / us / 1e3, 1),
                              "kernels_per_call": 2}), flush=True)


def run_sweep(args):
    """--sweep: decode attention alone over the 45-cell grid B in {1..256} x ctx in {128..4096}
    (the 40 cells of the sweep config plus the 5 largest it drops), one JSON line per cell.
    Every cell runs a CUDA graph of L calls on L distinct layer caches, L chosen so that the graph
    streams at least 300 MB (more than the 126 MB L2) and at least 28 layers."""
    import torch

    from inference_engine_b200 import kernels as K

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_kind = peaks()
    gen = torch.Generator(device=dev).manual_seed(2)
    dropped = {(256, 4096), (256, 2048), (128, 4096), (256, 1024), (128, 2048)}
    for B in (1, 2, 4, 8, 16, 32, 64, 128, 256):
        for n in (128, 512, 1024, 2048, 4096):
            nbytes = attn_bytes(B, n)
            L = int(min(1024, max(28, -(-300_000_000 // nbytes))))
            pages_per_seq = (n + PAGE - 1) // PAGE
            num_pages = B * pages_per_seq + 1
            caches = []
            for _ in range(L):
                c = K.make_layer_cache(num_pages, HKV, PAGE, D, device=dev)
                c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device=dev, dtype=torch.int8))
                c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device=dev, dtype=torch.int8))
                c.k_scale.fill_(0.02)
                c.v_scale.fill_(0.02)
                caches.append(c)
            table = torch.randperm(num_pages - 1, generator=torch.Generator().manual_seed(2)).to(torch.int32)
            table = table.reshape(B, pages_per_seq).to(dev)
            q = torch.randn(B, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
            out = torch.empty_like(q)
            cached = torch.full((B,), n - 1, dtype=torch.int32, device=dev)
            nd = torch.tensor([B], dtype=torch.int32, device=dev)

            plan_buf = torch.empty(K.plan_decode_bytes(dev), dtype=torch.uint8, device=dev)

            def calls():
                # the L calls stand for the layers of one decoder step: one plan kernel at its head serves them all
                plan = None if args.no_plan else K.plan_decode_step(cached, table, nd, caches[0], out=plan_buf)
                for c in caches:
                    K.decode_attention(q, c, cached, table, nd, D ** -0.5, out=out, plan=plan)

            calls()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                calls()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(args.steps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) * 1e3 / L)
            us = statistics.median(times)
            gbs = nbytes / us / 1e3
            parity = None
            if not args.no_parity:
                # the graph's last call left `out` = attention over the last cache: up to four of its sequences
                # are recomputed by the CPU oracle
                sample = sorted({0, B // 3, (2 * B) // 3, B - 1})
                res = oracle_sample_check(K, caches[-1], table.cpu().numpy(), np.full(B, n), sample,
                                          out[sample].cpu().reshape(-1, HQ, D), q_rot=q[sample].float().cpu().numpy())
                parity = {k: (round(v, 6) if isinstance(v, float) else v) for k, v in res.items() if k != "sequences"}
                if not res["within_gate"]:
                    raise SystemExit(f"sweep cell B={B} ctx={n}: output differs from the oracle: {res}")
            print(json.dumps({"B": B, "ctx": n, "layers_in_graph": L, "us_per_call": round(us, 2),
                              "us_min": round(min(times), 2), "gbs": round(gbs, 1), "pct_of_8TBs": round(gbs / 80.0, 2),
                              "frac_of_measured": round(gbs / peak, 4), "in_sweep_config": (B, n) not in dropped,
                              "planned": not args.no_plan, "bytes": nbytes, "parity": parity}), flush=True)
            del caches, graph
            torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=64, help="sequences per GPU")
    ap.add_argument("--ctx", type=int, default=4096, help="tokens attended per sequence, the new one included")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--cpu-seqs", type=int, default=64, help="sequences in the CPU baseline sample")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-early-start", action="store_true", help="launch decode attention without programmatic early start")
    ap.add_argument("--no-plan", action="store_true", help="no per-step plan: every decode_attention call derives its work split itself")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of output rows after the timed regions")
    ap.add_argument("--no-sharded", action="store_true", help="headline run: skip the sequence-sharded record that follows it")
    ap.add_argument("--sharded-layers", type=int, default=2, help="resident layer caches of the sharded record")
    ap.add_argument("--sharded", action="store_true", help="sequence-sharded decode over log-uniform contexts (torchrun for N > 1)")
    ap.add_argument("--model", action="store_true", help="--sharded: also time the whole random-init decoder on each shard")
    ap.add_argument("--seqs", type=int, default=2048, help="--sharded: concurrent sequences over all GPUs")
    ap.add_argument("--serve", action="store_true", help="offline serving run of the step loop on the random-init decoder")
    ap.add_argument("--decode-model", action="store_true", help="pure decode step of the random-init decoder (B, ctx)")
    ap.add_argument("--tune", action="store_true", help="--decode-model: let tune_linear pick the matmul per weight shape first")
    ap.add_argument("--path", action="store_true", help="each op of the mixed step's attention path timed alone")
    ap.add_argument("--prefill", action="store_true", help="chunked-prefill attention kernel alone, both kernels")
    ap.add_argument("--mixed", action="store_true", help="chunked-prefill + decode step inside the decoder scaffold")
    ap.add_argument("--write", action="store_true", help="quantize-on-write microbench (T = 1, 64, 1024)")
    ap.add_argument("--sweep", action="store_true", help="decode-attention shape sweep instead of the headline step")
    ap.add_argument("--vs-triton", action="store_true", help="the reference's Triton kernels timed beside this library's, same inputs")
    ap.add_argument("--reference", default=None, help="--vs-triton: checkout of the reference (or its qwen3-1.7b directory)")
    ap.add_argument("--all-cells", action="store_true", help="--vs-triton: also the five cells the sweep configuration drops")
    ap.add_argument("--dump", default=None, help="--phases: prefix of .npy files for the raw per-warp words")
    ap.add_argument("--linear", action="store_true", help="weight-streaming matmul for few rows beside cuBLAS")
    ap.add_argument("--phases", action="store_true", help="per-phase and per-SM times of the decode kernel (instrumented build)")
    args = ap.parse_args()
    if args.phases:
        run_phases(args)
    elif args.linear:
        run_linear(args)
    elif args.vs_triton:
        run_vs_triton(args)
    elif args.sweep:
        run_sweep(args)
    elif args.write:
        run_write(args)
    elif args.mixed:
        run_mixed(args)
    elif args.prefill:
        run_prefill(args)
    elif args.path:
        run_path(args)
    elif args.decode_model:
        run_decode_model(args)
    elif args.serve:
        run_serve(args)
    elif args.sharded:
        run_sharded(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
