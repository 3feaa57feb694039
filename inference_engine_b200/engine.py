"""Continuous-batching step loop over the paged int8 cache: scheduler, page pool and CUDA-graph replay around
the attention ops.

It plays the role of kbwal/inference-engine qwen3-1.7b/engine.py for this library's paged cache:

* the same public surface (`submit_request`, `step`, `generate`, a `Request` with prompt, output and times)
  and the same scheduling policy (engine.py:143-204): every decoding request gets its token first, then
  requests in the middle of their prompt continue, then waiting requests are admitted first come first served
  while the step's token budget lasts; a prompt's first chunk is at least `min_first_chunk` tokens (or the
  whole prompt);
* the same bookkeeping (engine.py:229-252): a request produces its first token when the last chunk of its
  prompt is in the cache, and ends on the stop token, on `max_new_tokens`, or when the cache row is full;
* the same execution scheme (engine.py:376-470): pure-decode steps replay one CUDA graph per batch-size bucket,
  steps with prefill one graph per token bucket, all inputs of a step travel in one int32 buffer at fixed
  addresses, and a step that fits no bucket runs eagerly.

What differs is the cache: the reference gives every request a cache row of `max_len` tokens (a slot); here
the cache is a pool of 16-token pages and a request holds a list of them.  `PagePool` hands pages out on
demand (append on decode, release on finish); a request is admitted only if the pages its whole lifetime can
need are still uncommitted, so a running request can never run out.  The first pages of the pool are a
scratch run no request owns: padded entries of a graph replay write there.

`Scheduler` is host-only (no torch, no GPU) so that the policy is testable on its own; `Engine` adds the
device side.  The model is the random-init decoder of scaffold.py; sampling is the library's Gumbel-max sampler
(greedy at tau = 0).
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field


@dataclass
class Request:
    id: int
    prompt_ids: list[int]
    max_new_tokens: int
    pages: list[int] = field(default_factory=list)  # physical pages, in token order
    committed: int = 0  # pages promised to this request at admission and not yet handed out
    cached_len: int = 0  # tokens currently in the cache
    output: list[int] = field(default_factory=list)
    admitted: bool = False
    t_submit: float = 0.0
    t_first_token: float | None = None
    t_finish: float | None = None

    @property
    def decoding(self) -> bool:
        return self.cached_len >= len(self.prompt_ids)


class PagePool:
    """Free list of physical pages [first, num_pages).  `commit` promises pages without choosing them,
    `take` turns one promise into a page, `release` returns pages and drops leftover promises."""

    def __init__(self, num_pages: int, first: int = 0):
        self.free = list(range(num_pages - 1, first - 1, -1))  # pop() hands out the lowest id first
        self.committed = 0
        self.capacity = num_pages - first

    def uncommitted(self) -> int:
        return len(self.free) - self.committed

    def commit(self, n: int) -> bool:
        if n > self.uncommitted():
            return False
        self.committed += n
        return True

    def take(self) -> int:
        assert self.committed > 0 and self.free
        self.committed -= 1
        return self.free.pop()

    def release(self, pages: list[int], leftover_promises: int = 0) -> None:
        assert leftover_promises <= self.committed
        self.committed -= leftover_promises
        self.free.extend(sorted(pages, reverse=True))


@dataclass
class Step:
    entries: list[tuple[Request, list[int]]]  # decoding requests first (one token each), then prefill chunks
    num_decoding: int

    @property
    def decode_only(self) -> bool:
        return self.num_decoding == len(self.entries)

    @property
    def num_tokens(self) -> int:
        return sum(len(t) for _, t in self.entries)


class Scheduler:
    def __init__(self, max_batch_size: int, max_len: int, page_size: int, pool: PagePool, max_tokens_per_step: int,
                 min_first_chunk: int, stop_token_id: int):
        assert max_tokens_per_step >= max_batch_size + min_first_chunk, \
            "the budget must fit every decoding request plus one first chunk, or prefill can stall forever"
        self.max_batch_size, self.max_len, self.page_size = max_batch_size, max_len, page_size
        self.pool, self.max_tokens_per_step, self.min_first_chunk = pool, max_tokens_per_step, min_first_chunk
        self.stop_token_id = stop_token_id
        self.running: list[Request] = []
        self.waiting: deque[Request] = deque()
        self.next_id = 0

    def submit(self, prompt_ids: list[int], max_new_tokens: int) -> Request:
        assert max_new_tokens >= 1 and len(prompt_ids) > 0
        assert len(prompt_ids) + max_new_tokens <= self.max_len, "prompt + continuation must fit max_len"
        need = math.ceil(min(len(prompt_ids) + max_new_tokens - 1, self.max_len) / self.page_size)
        if need > self.pool.capacity:  # it could never be admitted and would block the queue for ever
            raise ValueError(f"the request needs {need} pages over its lifetime, the pool holds {self.pool.capacity}")
        r = Request(self.next_id, list(prompt_ids), max_new_tokens, t_submit=time.perf_counter())
        self.next_id += 1
        self.waiting.append(r)
        return r

    def idle(self) -> bool:
        return not self.running and not self.waiting

    def lifetime_pages(self, r: Request) -> int:
        # the last generated token is never written to the cache
        return math.ceil(min(len(r.prompt_ids) + r.max_new_tokens - 1, self.max_len) / self.page_size)

    def plan(self) -> Step | None:
        budget = self.max_tokens_per_step
        entries: list[tuple[Request, list[int]]] = []
        for r in self.running:  # decoding requests are never starved and come first
            if r.decoding:
                entries.append((r, [r.output[-1]]))
                budget -= 1
        num_decoding = len(entries)
        for r in self.running:  # requests in the middle of their prompt
            if not r.decoding and budget > 0:
                n = min(len(r.prompt_ids) - r.cached_len, budget)
                entries.append((r, r.prompt_ids[r.cached_len : r.cached_len + n]))
                budget -= n
        while self.waiting and len(self.running) < self.max_batch_size and budget > 0:
            r = self.waiting[0]
            n = min(len(r.prompt_ids), budget)
            if n < min(len(r.prompt_ids), self.min_first_chunk):
                break  # first come first served: nobody overtakes it
            if not self.pool.commit(self.lifetime_pages(r)):
                break  # the pool cannot promise its whole lifetime yet
            self.waiting.popleft()
            r.committed, r.admitted = self.lifetime_pages(r), True
            self.running.append(r)
            entries.append((r, r.prompt_ids[:n]))
            budget -= n
        if not entries:
            return None
        for r, toks in entries:  # pages for the tokens this step writes
            need = math.ceil((r.cached_len + len(toks)) / self.page_size) - len(r.pages)
            for _ in range(need):
                r.pages.append(self.pool.take())
                r.committed -= 1
        return Step(entries, num_decoding)

    def commit(self, step: Step, sampled: list[int]) -> list[Request]:
        now = time.perf_counter()
        finished = []
        for (r, toks), tok in zip(step.entries, sampled):
            r.cached_len += len(toks)
            if r.decoding:
                r.output.append(int(tok))
                if len(r.output) == 1:
                    r.t_first_token = now
                if tok == self.stop_token_id or len(r.output) >= r.max_new_tokens or r.cached_len + 1 >= self.max_len:
                    self.pool.release(r.pages, r.committed)
                    r.pages, r.committed = [], 0
                    self.running.remove(r)
                    r.t_finish = now
                    finished.append(r)
        return finished


class Engine:
    """Scheduler + device execution.  `model` is a scaffold.DecoderScaffold on a CUDA device."""

    def __init__(self, model, max_batch_size: int, max_len: int, stop_token_id: int, page_size: int = 16,
                 num_pages: int | None = None, max_tokens_per_step: int = 1024, min_first_chunk: int = 64,
                 max_graph_tokens: int = 512, use_graphs: bool = True, block_m: int = 128, tau: float = 0.0, seed: int = 0):
        import numpy as np
        import torch

        from . import kernels as K
        from . import scaffold as S

        self.torch, self.K, self.S, self.np = torch, K, S, np
        self.model, self.device = model, model.device
        model.tau = float(tau)  # baked into the graphs at capture, like the reference's (engine.py:399)
        model.seed.fill_(seed)
        self.page_size, self.max_len, self.block_m = page_size, max_len, block_m
        self.max_batch_size = max_batch_size
        self.num_entries = max_batch_size + 1  # every request plus one padding entry
        self.max_pages = math.ceil(max_len / page_size)  # block-table width
        # token buckets of steps with prefill (engine.py:254-259) and batch buckets of pure-decode steps
        M = min(max_graph_tokens, max_tokens_per_step, max_len)
        self.token_buckets = sorted({b for b in (16, 32, 64) if b < M} | set(range(128, M, 128)) | {M})
        self.graph_buckets = sorted({min(1 << i, max_batch_size) for i in range(max_batch_size.bit_length() + 1)})
        # scratch run: the padding entry of the largest bucket writes that many tokens from position 0
        self.scratch_pages = math.ceil(max(self.token_buckets) / page_size)
        assert self.scratch_pages <= self.max_pages
        if num_pages is None:  # what the reference's slot rows hold: max_len tokens per request
            num_pages = self.scratch_pages + max_batch_size * self.max_pages
        self.pool = PagePool(num_pages, first=self.scratch_pages)
        self.sched = Scheduler(max_batch_size, max_len, page_size, self.pool, max_tokens_per_step, min_first_chunk,
                               stop_token_id)
        self.caches = [K.make_layer_cache(num_pages, S.HKV, page_size, S.D, device=self.device)
                       for _ in range(model.num_layers)]
        # one int32 buffer per kind of step, filled on the host and copied in one piece
        cap = sum(self.mixed_layout(max_tokens_per_step))
        self.host_mixed = torch.empty(cap, dtype=torch.int32).pin_memory()
        self.dev_mixed = torch.zeros(cap, dtype=torch.int32, device=self.device)
        capd = sum(self.decode_layout())
        self.host_decode = torch.empty(capd, dtype=torch.int32).pin_memory()
        self.dev_decode = torch.zeros(capd, dtype=torch.int32, device=self.device)
        self.np_mixed, self.np_decode = self.host_mixed.numpy(), self.host_decode.numpy()  # same memory
        self.rows: dict[int, tuple] = {}  # request id -> (pages copied so far, its block-table row as an array)
        self.scratch_row = self.np.zeros(self.max_pages, self.np.int32)
        self.scratch_row[: self.scratch_pages] = self.np.arange(self.scratch_pages)
        self.prefix_capacity = 2 * max_len
        self.prefix_k = torch.empty(S.HKV, self.prefix_capacity, S.D, device=self.device, dtype=torch.bfloat16)
        self.prefix_v = torch.empty_like(self.prefix_k)
        self.graph_pool = torch.cuda.graph_pool_handle()  # one pool for all graphs: only one runs at a time
        self.decode_graphs: dict[int, tuple] = {}
        self.mixed_graphs: dict[int, tuple] = {}
        self.steps_run = {"decode_graph": 0, "mixed_graph": 0, "eager": 0}
        self.seconds = {"plan": 0.0, "run (inputs, launch, read-back)": 0.0, "commit": 0.0, "inputs": 0.0}
        if use_graphs:
            self.capture()

    # ------------------------------------------------------------------ public surface (engine.py:120-142)
    def submit_request(self, prompt_ids: list[int], max_new_tokens: int) -> Request:
        return self.sched.submit(prompt_ids, max_new_tokens)

    def generate(self, prompts: list[list[int]], max_new_tokens: int) -> list[Request]:
        reqs = [self.submit_request(p, max_new_tokens) for p in prompts]
        while not self.sched.idle():
            self.step()
        return reqs

    def step(self) -> list[Request]:
        t0 = time.perf_counter()
        step = self.sched.plan()
        if step is None:
            return []
        t1 = time.perf_counter()
        tokens = self.run_decode(step) if step.decode_only else self.run_mixed(step)
        t2 = time.perf_counter()
        finished = self.sched.commit(step, tokens)
        for r in finished:
            self.rows.pop(r.id, None)
        self.seconds["plan"] += t1 - t0
        self.seconds["run (inputs, launch, read-back)"] += t2 - t1
        self.seconds["commit"] += time.perf_counter() - t2
        return finished

    # ------------------------------------------------------------------ input buffers
    def mixed_layout(self, n_tokens: int) -> list[int]:
        """Field lengths of a step with prefill padded to n_tokens: ids, positions, seq_ids, cu_seqlens,
        cached_lens, cu_cached, tile_start, num_decoding, block table.  The same n_tokens always gives the
        same layout, so a bucket's fields always sit at the same addresses."""
        E = self.num_entries
        return [n_tokens, n_tokens, n_tokens, E + 1, E, E + 1, math.ceil(n_tokens / self.block_m) + E, 1, E * self.max_pages]

    def decode_layout(self) -> list[int]:
        """ids, cached_lens, num_decoding, block table of a pure-decode step, sized for the largest batch; a
        bucket of b rows uses the first b of each (same start addresses for every bucket)."""
        B = self.max_batch_size
        return [B, B, 1, B * self.max_pages]

    def table_row(self, r: Request):
        """The request's block-table row as an int32 array, extended in place as pages are appended."""
        n, row = self.rows.get(r.id, (0, None))
        if row is None:
            row = self.np.zeros(self.max_pages, self.np.int32)
        if n < len(r.pages):
            row[n : len(r.pages)] = r.pages[n:]
            self.rows[r.id] = (len(r.pages), row)
        return row

    def fill_mixed(self, step: Step, n_pad: int):
        """Build the step's metadata on the host (scaffold.plan_step = the reference's fill_inputs), one copy."""
        nd = step.num_decoding
        plan = self.S.plan_step([r.cached_len for r, _ in step.entries[:nd]],
                           [(r.cached_len, len(t)) for r, t in step.entries[nd:]], n_pad, self.num_entries, self.block_m)
        sizes = self.mixed_layout(n_pad)
        buf = self.np_mixed[: sum(sizes)]
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + n)
        ids = [tok for _, toks in step.entries for tok in toks]
        buf[offs[0] : offs[0] + len(ids)] = ids
        buf[offs[0] + len(ids) : offs[1]] = 0
        for i, key in enumerate(("positions", "seq_ids", "cu_seqlens", "cached", "cu_cached", "tile_start", "num_decoding"), 1):
            assert len(plan[key]) == sizes[i]
            buf[offs[i] : offs[i + 1]] = plan[key]
        table = buf[offs[8] : offs[9]].reshape(self.num_entries, self.max_pages)
        for i, (r, _) in enumerate(step.entries):
            table[i] = self.table_row(r)
        table[len(step.entries)] = self.scratch_row  # the padding entry lives on the scratch run
        table[len(step.entries) + 1 :] = 0
        self.dev_mixed[: len(buf)].copy_(self.host_mixed[: len(buf)], non_blocking=True)
        return plan["cu_cached"][-1]

    def mixed_views(self, n_pad: int, prefix_tokens: int = 0):
        S = self.S
        v = self.dev_mixed[: sum(self.mixed_layout(n_pad))].split(self.mixed_layout(n_pad))
        inp = S.StepInputs(ids=v[0], positions=v[1], seq_ids=v[2], cu_seqlens=v[3], cached_lens=v[4], cu_cached=v[5],
                           tile_start=v[6], num_decoding=v[7], block_table=v[8].view(self.num_entries, self.max_pages),
                           prefix_tokens=prefix_tokens, block_m=self.block_m)
        pk, pv = self.prefix_k, self.prefix_v
        if prefix_tokens > self.prefix_capacity:  # a one-off buffer for this step
            pk = self.torch.empty(S.HKV, prefix_tokens, S.D, device=self.device, dtype=pk.dtype)
            pv = self.torch.empty_like(pk)
        return inp, S.PrefixScratch(pk, pv, inp.cu_cached)

    def decode_views(self, b: int):
        B = self.max_batch_size
        ids, cached, nd, table = self.dev_decode.split(self.decode_layout())
        return ids[:b], cached[:b], nd, table.view(B, self.max_pages)[:b]

    # ------------------------------------------------------------------ execution
    def forward_mixed(self, n_pad: int, prefix_tokens: int = 0):
        inp, prefix = self.mixed_views(n_pad, prefix_tokens)
        return self.model.forward(self.caches, inp, inp.ids, inp.cached_lens, inp.block_table, inp.num_decoding, prefix)

    def forward_decode(self, b: int):
        ids, cached, nd, table = self.decode_views(b)
        return self.model.forward(self.caches, None, ids, cached, table, nd)

    def capture_graph(self, run):
        """Two eager runs first (engine.py:432-449), then the recording; returns (graph, output tensor)."""
        torch = self.torch
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                run()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self.graph_pool):
            out = run()
        return g, out

    def capture(self) -> None:
        """One graph per batch bucket (rows beyond the step's requests are not decoding: num_decoding is read
        on the device) and one per token bucket (any mix of entries that fits, engine.py:412-430).  The dummy
        inputs during capture are a single padding entry on the scratch run, so what the warm-up writes is
        harmless."""
        self.dev_decode.zero_()
        for b in reversed(self.graph_buckets):
            self.decode_graphs[b] = self.capture_graph(lambda b=b: self.forward_decode(b))
        for n in reversed(self.token_buckets):
            self.fill_mixed(Step([], 0), n)
            self.mixed_graphs[n] = self.capture_graph(lambda n=n: self.forward_mixed(n))
        self.torch.cuda.synchronize()
        # the warm-up steps ran on all-idle inputs: a status bit here is a fault of the path, not of the data
        bits = self.K.check_status(self.device)
        if bits:
            raise RuntimeError(f"device status word {bits:#x} set while the step graphs were captured")

    def run_decode(self, step: Step) -> list[int]:
        torch = self.torch
        t_in = time.perf_counter()
        B = len(step.entries)
        b = next(x for x in self.graph_buckets if x >= B)
        Bm, buf = self.max_batch_size, self.np_decode
        buf[:B] = [t[0] for _, t in step.entries]
        buf[Bm : Bm + B] = [r.cached_len for r, _ in step.entries]
        buf[B:Bm] = 0
        buf[Bm + B : 2 * Bm] = 0
        buf[2 * Bm] = B
        table = buf[2 * Bm + 1 :].reshape(Bm, self.max_pages)
        for i, (r, _) in enumerate(step.entries):
            table[i] = self.table_row(r)
        table[B:] = 0
        self.dev_decode.copy_(self.host_decode, non_blocking=True)
        self.seconds["inputs"] += time.perf_counter() - t_in
        if b in self.decode_graphs:
            g, out = self.decode_graphs[b]
            g.replay()
            self.steps_run["decode_graph"] += 1
        else:
            with torch.inference_mode():
                out = self.forward_decode(b)
            self.steps_run["eager"] += 1
        return out[:B].tolist()  # the read-back ends the step

    def run_mixed(self, step: Step) -> list[int]:
        torch = self.torch
        N = step.num_tokens
        n_pad = next((x for x in self.token_buckets if x >= N), N)
        t_in = time.perf_counter()
        prefix_tokens = self.fill_mixed(step, n_pad)
        self.seconds["inputs"] += time.perf_counter() - t_in
        if n_pad in self.mixed_graphs and prefix_tokens <= self.prefix_capacity:
            g, out = self.mixed_graphs[n_pad]
            g.replay()
            self.steps_run["mixed_graph"] += 1
        else:
            with torch.inference_mode():
                out = self.forward_mixed(n_pad, prefix_tokens)
            self.steps_run["eager"] += 1
        return out[: len(step.entries)].tolist()
