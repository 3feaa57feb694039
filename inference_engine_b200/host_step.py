"""Decode step of the attention path driven from HOST buffers.

What a caller outside the GPU process boundary sees of one decode step of one layer stack:
it hands over this step's projections (the fused QKV rows of the B new tokens, per layer),
the rope rows and the batch metadata in pinned host memory, and reads the attention output
back.  The int8 KV cache itself is device-resident state that persists across steps, exactly
as in the reference engine (engine.py:472-492); it is not a per-step input.

Per step and per layer this runs the two calls `AttentionLayer.forward` makes for a pure
decode step (architecture.py:98-123): fused_rope_kv_decode, then decode_attention.

The host-buffer step is pipelined over groups of layers: while group g computes, the projections
of group g+1 are copied in on a second stream and the outputs of group g-1 are copied out on a
third, so the copies of all but the first and last group hide behind the kernels."""
from __future__ import annotations

import torch

from . import kernels as K


class HostDecodeStep:
    def __init__(self, caches: list[K.LayerKVCache], B: int, Hq: int, Hkv: int, D: int, table_shape, eps: float = 1e-6):
        dev = caches[0].k.device
        L = len(caches)
        self.caches, self.B, self.Hq, self.Hkv, self.D, self.eps = caches, B, Hq, Hkv, D, eps
        W = (Hq + 2 * Hkv) * D
        self.dev_qkv = torch.empty(L, B, W, dtype=torch.bfloat16, device=dev)
        # the step's small inputs live in one buffer, so they reach the GPU in one copy (the reference engine
        # does the same with its metadata, engine.py:72-76): rope rows, cached lengths, block table, num_decoding
        sizes = [B * (D // 2) * 2, B * (D // 2) * 2, B * 4, int(torch.tensor(table_shape).prod()) * 4, 4]
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 255) // 256 * 256
        self.dev_meta = torch.empty(total, dtype=torch.uint8, device=dev)
        self.host_meta = [torch.empty(total, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.meta_sent = [None, None]  # event after the copy that last read each staging buffer
        self.meta_turn = 0

        def views(buf):
            part = lambda i, dt, shape: buf[offs[i] : offs[i] + sizes[i]].view(dt).view(shape)
            return (part(0, torch.bfloat16, (B, 1, D // 2)), part(1, torch.bfloat16, (B, 1, D // 2)),
                    part(2, torch.int32, (B,)), part(3, torch.int32, tuple(table_shape)), part(4, torch.int32, (1,)))

        self._views = views
        self.dev_cos, self.dev_sin, self.dev_cached, self.dev_table, self.dev_nd = views(self.dev_meta)
        self.dev_out = torch.empty(L, B, Hq, D, dtype=torch.bfloat16, device=dev)
        self.q_w = [torch.ones(D, dtype=torch.bfloat16, device=dev) for _ in range(L)]
        self.k_w = [torch.ones(D, dtype=torch.bfloat16, device=dev) for _ in range(L)]
        self.plan = torch.empty(K.plan_decode_bytes(dev), dtype=torch.uint8, device=dev)  # this step's work split
        self.use_plan = True
        self.graph = None
        self.group_graphs: list[tuple[int, int, torch.cuda.CUDAGraph]] = []  # (first layer, end layer, graph)
        self.h2d_stream = torch.cuda.Stream(device=dev)
        self.d2h_stream = torch.cuda.Stream(device=dev)

    def set_norm_weights(self, q_w, k_w):
        self.q_w, self.k_w = q_w, k_w

    @property
    def h2d_bytes(self) -> int:
        ts = (self.dev_qkv, self.dev_meta)
        return sum(t.numel() * t.element_size() for t in ts)

    @property
    def d2h_bytes(self) -> int:
        return self.dev_out.numel() * self.dev_out.element_size()

    def device_step(self, first: int = 0, end: int | None = None):
        """The device part: per layer in [first, end), quantize-on-write of the new tokens then attention."""
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        end = len(self.caches) if end is None else end
        if first == 0 and self.use_plan:
            # once per step: the split depends on the step's metadata only, every layer reuses it
            K.plan_decode_step(self.dev_cached, self.dev_table, self.dev_nd, self.caches[0], out=self.plan)
        for l in range(first, end):
            cache = self.caches[l]
            q, k, v = self.dev_qkv[l].split([Hq * D, Hkv * D, Hkv * D], dim=-1)
            q = q.view(self.B, Hq, D)
            k = k.view(self.B, Hkv, D)
            v = v.view(self.B, Hkv, D)
            qr = K.fused_rope_kv_decode(q, k, v, self.q_w[l], self.k_w[l], self.dev_cos, self.dev_sin, self.dev_table,
                                        cache, self.dev_cached, self.dev_nd, self.eps)
            K.decode_attention(qr, cache, self.dev_cached, self.dev_table, self.dev_nd, D ** -0.5, out=self.dev_out[l],
                               plan=self.plan if self.use_plan else None)

    def capture(self, groups: int = 7):
        """Record device_step into a CUDA graph (two eager warm-up runs first, like engine.py:432-449), and
        once more as `groups` graphs over consecutive layer ranges for the pipelined host-buffer step."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self.device_step()
        torch.cuda.current_stream().wait_stream(s)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.device_step()
        L = len(self.caches)
        groups = max(1, min(groups, L))
        bounds = [round(i * L / groups) for i in range(groups + 1)]
        self.group_graphs = []
        for a, b in zip(bounds[:-1], bounds[1:]):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.device_step(a, b)
            self.group_graphs.append((a, b, g))

    def run_device(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.device_step()

    def run_host(self, qkv, cos, sin, cached_lens, table, num_decoding, out):
        """All arguments are pinned host tensors; `out` receives [L, B, Hq, D] bf16.  Enqueues
        H2D copies, the device step and the D2H copy on the current stream (no sync)."""
        turn = self.meta_turn
        self.meta_turn ^= 1
        if self.meta_sent[turn] is not None:
            self.meta_sent[turn].synchronize()  # the copy that read this staging buffer two steps ago is done
        for dst, src in zip(self._views(self.host_meta[turn]), (cos, sin, cached_lens, table, num_decoding)):
            dst.copy_(src)
        self.dev_meta.copy_(self.host_meta[turn], non_blocking=True)
        self.meta_sent[turn] = torch.cuda.Event()
        self.meta_sent[turn].record()
        if not self.group_graphs:
            self.dev_qkv.copy_(qkv, non_blocking=True)
            self.run_device()
            out.copy_(self.dev_out, non_blocking=True)
            return
        cur = torch.cuda.current_stream()
        self.h2d_stream.wait_stream(cur)  # after everything already enqueued (the previous step reads dev_qkv)
        self.d2h_stream.wait_stream(cur)
        for a, b, g in self.group_graphs:
            with torch.cuda.stream(self.h2d_stream):
                self.dev_qkv[a:b].copy_(qkv[a:b], non_blocking=True)
                landed = torch.cuda.Event()
                landed.record(self.h2d_stream)
            cur.wait_event(landed)
            g.replay()
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(done)
                out[a:b].copy_(self.dev_out[a:b], non_blocking=True)
        cur.wait_stream(self.d2h_stream)  # the caller's stream order covers the whole step
