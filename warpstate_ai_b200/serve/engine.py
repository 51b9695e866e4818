"""Batched prefill + decode engine.

Decoding carries, per logical depth and per sequence, only the fast and slow matrix memories
(``[H, 64, 64]`` FP32 each) plus the keys / values / memory-values of the *current* 128-token
chunk -- there is no growing KV cache (reference model: warpstate/model.py:222-274; its
training-consistent variant ops/posttrain_chat.py:94-142, whose semantics this follows: the mix
of fast/slow is applied before the read and a chunk's write is formed as ONE product
``tanh(K)^T tanh(U) / C`` when the chunk completes).

What is new relative to the reference (whose CLIs prefill token by token at batch 1):

* `prefill` pushes all complete chunks of the prompt through the training forward path (the fused
  sm_100a kernels on CUDA) and reads the memory states after the last complete chunk from the
  O(N) scan kernel; only the tokens of a trailing partial chunk are stepped one by one;
* `step` handles a whole batch in lock-step; on CUDA the step for a fixed batch size is captured
  once in a CUDA graph and replayed per token (the in-chunk position is a device scalar, the
  attention over the chunk cache is masked instead of sliced, so one graph serves all positions);
* the memory update at a chunk boundary runs outside the graph, every 128 tokens;
* on CUDA with the kernel library (BF16, head_dim 64, chunk 128, batch <= 64) the step is seven
  kernels per layer: weight-streaming tcgen05 GEMMs with swapped operand roles
  (`decode_gemm_kernel`), a fused residual + depth-modulation + RMSNorm kernel and one attention
  kernel per (sequence, head) (ops/csrc/decode.cu); the PyTorch formulation below is the
  reference for it and the fallback elsewhere.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..ops import reference as R


@dataclass
class DepthState:
    fast: torch.Tensor    # [B,H,Dh,Dh] FP32
    slow: torch.Tensor    # [B,H,Dh,Dh] FP32
    mixed: torch.Tensor   # [B,H,Dh,Dh] compute dtype: mix*fast + (1-mix)*slow, what a read uses
    k: torch.Tensor       # [B,H,C,Dh] roped keys of the current chunk
    v: torch.Tensor
    u: torch.Tensor


class DecodeEngine:
    GREEDY_CAPACITY = 1024    # tokens per sequence the history buffer of `decode_greedy` holds between read-outs

    def __init__(self, model, dtype: torch.dtype = torch.bfloat16, use_cuda_graph: bool | None = None,
                 use_kernels: bool = True, pack_weights: bool = False):
        if model.training:
            raise ValueError("Decode requires model.eval()")
        self.model = model
        self.cfg = model.cfg
        self.device = model.embed.weight.device
        self.dtype = dtype if self.device.type == "cuda" else torch.float32 if dtype == torch.float32 else dtype
        self.chunk = self.cfg.chunk_size
        self.h, self.hd = self.cfg.n_heads, self.cfg.head_dim
        self.use_graph = (self.device.type == "cuda") if use_cuda_graph is None else use_cuda_graph
        self.use_kernels = use_kernels
        self.pack_weights = pack_weights
        self._kbufs = None
        self._layer_tail = False
        self.weights = []
        with torch.no_grad():
            for depth in range(self.cfg.logical_depth):
                core = model.cores[depth % self.cfg.n_cores]
                self.weights.append(dict(
                    scale=model.depth_scale[depth].detach().float(), bias=model.depth_bias[depth].detach().float(),
                    n1=core.norm1.weight.detach().float(), n2=core.norm2.weight.detach().float(),
                    w_in=core.in_proj.weight.detach().to(self.dtype), w_out=core.out_proj.weight.detach().to(self.dtype),
                    w_ug=core.ffn.up_gate.weight.detach().to(self.dtype), w_down=core.ffn.down.weight.detach().to(self.dtype),
                    df=torch.sigmoid(core.fast_decay_logit.detach().float()).view(1, self.h, 1, 1),
                    ds=torch.sigmoid(core.slow_decay_logit.detach().float()).view(1, self.h, 1, 1),
                    mix=torch.sigmoid(core.memory_mix_logit.detach().float()).view(1, self.h, 1, 1)))
            self.embed = model.embed.weight.detach()
            self.head = model.embed.weight.detach().to(self.dtype)
            self.final_norm = model.final_norm.weight.detach().float()
        cos, sin = R.rope_tables(self.chunk, self.hd, self.device, torch.float32)
        self.cos, self.sin = cos, sin
        self.states: list[DepthState] | None = None
        self.batch = 0
        self.pos = 0            # host copy of the in-chunk position
        self._graph = None
        self._greedy_graph = None
        from .graph_stats import GraphCounters
        self.graph_counters = GraphCounters()

    # ------------------------------------------------------------------ state
    def new_state(self, batch: int) -> None:
        # Buffers made under ``torch.inference_mode()`` (as the chat entry points run) cannot be written from outside
        # it; a caller that then uses the engine directly gets fresh ones (and a fresh graph) instead of an error.
        stranded = (self.states is not None and self.states[0].fast.is_inference()
                    and not torch.is_inference_mode_enabled())
        if self.states is not None and batch == self.batch and not stranded:
            # same shapes: clear in place so that the captured graph and its buffers stay valid
            for st in self.states:
                for t in (st.fast, st.slow, st.mixed, st.k, st.v, st.u):
                    t.zero_()
            self.pos = 0
            self.pos_dev.zero_()
            return
        z = lambda *shape, dtype: torch.zeros(shape, device=self.device, dtype=dtype)
        self.states = [DepthState(z(batch, self.h, self.hd, self.hd, dtype=torch.float32),
                                  z(batch, self.h, self.hd, self.hd, dtype=torch.float32),
                                  z(batch, self.h, self.hd, self.hd, dtype=self.dtype),
                                  z(batch, self.h, self.chunk, self.hd, dtype=self.dtype),
                                  z(batch, self.h, self.chunk, self.hd, dtype=self.dtype),
                                  z(batch, self.h, self.chunk, self.hd, dtype=self.dtype))
                       for _ in range(self.cfg.logical_depth)]
        self.batch = batch
        self.pos = 0
        self.pos_dev = torch.zeros((), dtype=torch.long, device=self.device)
        self.token_buf = torch.zeros(batch, dtype=torch.long, device=self.device)
        self.logits_buf = None
        self.graph_counters.invalidations += (self._graph is not None) + (self._greedy_graph is not None)
        self._graph = self._greedy_graph = None
        self._kbufs = self._kernel_buffers(batch) if self._kernels_usable(batch) else None
        self._layer_tail = self._kbufs is not None and self._tail_kernel_usable()
        # greedy run-ahead decode: chosen tokens land in `history[:, cursor[0]]`; cursor[1] is kernel scratch
        self.history = torch.zeros(batch, self.GREEDY_CAPACITY, dtype=torch.long, device=self.device)
        self.cursor = torch.zeros(2, dtype=torch.long, device=self.device)

    # ------------------------------------------------------------------ kernel path
    def _kernels_usable(self, batch: int) -> bool:
        if self.device.type != "cuda" or self.dtype != torch.bfloat16 or self.hd != 64 or self.chunk != 128:
            return False
        if batch > 64 or self.cfg.d_model % 8 or self.cfg.ffn_hidden % 64 or not self.use_kernels:
            return False
        from ..ops import _ext
        return _ext.available()

    def _pack_weights(self) -> None:
        """With ``pack_weights=True``: tile-contiguous copies of the projection weights for the decode
        GEMM (made once; depths that share a core share the copy; the row-major weights stay for
        prefill, so the BF16 weight memory doubles).  Off by default: on B200 the 128-row TMA box over
        a row-major weight streams at the same rate as the contiguous tile (measured: 2.15 against
        2.17 ms per token at batch 64), so the default points the decode GEMM at the row-major weights."""
        if getattr(self, "_packed_done", False):
            return
        from ..ops.decode import pack_weight
        cache: dict[int, torch.Tensor] = {}

        def packed(w: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
            if not self.pack_weights:
                return w
            key = w.data_ptr()
            if key not in cache:
                cache[key] = pack_weight(w, swiglu)
            return cache[key]

        for w in self.weights:
            w["p_in"], w["p_out"] = packed(w["w_in"]), packed(w["w_out"])
            w["p_ug"], w["p_down"] = packed(w["w_ug"], True), packed(w["w_down"])
        self.head_packed = packed(self.head)
        self._packed_done = True

    def _kernel_buffers(self, batch: int) -> dict:
        ops = torch.ops.ws_b200
        d, ffn, v = self.cfg.d_model, self.cfg.ffn_hidden, self.cfg.vocab_size
        dev = self.device
        from ..ops import attention, gemm
        self._pack_weights()
        return dict(
            x=torch.zeros(batch, d, device=dev), n=torch.zeros(batch, d, device=dev, dtype=torch.bfloat16),
            qkvgu=torch.zeros(batch, 5 * d, device=dev, dtype=torch.bfloat16),
            y=torch.zeros(batch, d, device=dev, dtype=torch.bfloat16),
            act=torch.zeros(batch, ffn, device=dev, dtype=torch.bfloat16),
            p_out=torch.zeros(ops.decode_gemm_splits(d, d), batch, d, device=dev),
            p_down=torch.zeros(ops.decode_gemm_splits(d, ffn), batch, d, device=dev),
            logits=torch.zeros(batch, v, device=dev), rope=attention.rope_table(dev), flag=gemm.error_flag(dev),
            barrier=torch.zeros(2, dtype=torch.int32, device=dev))

    def _tail_kernel_usable(self) -> bool:
        """The persistent layer-tail launch (`WS_DECODE_LAYER_TAIL=1`) gives every CTA at most one work item per
        phase, one CTA per SM.  Off by default: measured at the production shape it takes 63.7 us per layer against
        52.2 us for the six launches it replaces -- its phase trace shows that what a projection costs beyond its
        bytes (first tile's round trip, accumulator drain, stores and their flush) is the same inside one launch,
        so the grid barriers buy nothing over kernel boundaries that are already dependent launches in a graph."""
        import os
        if os.environ.get("WS_DECODE_LAYER_TAIL", "0") != "1" or self.pack_weights:
            return False
        ops = torch.ops.ws_b200
        d, ffn = self.cfg.d_model, self.cfg.ffn_hidden
        if d % 128 or ffn % 64:
            return False
        slabs = (d + 127) // 128
        items = max(slabs * ops.decode_gemm_splits(d, d), slabs * ops.decode_gemm_splits(d, ffn), ffn // 64,
                    (5 * d + 127) // 128, self.batch)
        return items <= torch.cuda.get_device_properties(self.device).multi_processor_count

    def _step_kernels_tail(self, token: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """The step with one persistent launch per layer for everything after the attention (and the next layer's
        in_proj): 2 launches per layer instead of 7.  Bit-identical to `_step_kernels`."""
        ops = torch.ops.ws_b200
        k = self._kbufs
        d, eps = self.cfg.d_model, self.cfg.rms_eps
        first = self.weights[0]
        ops.decode_reduce_norm(k["x"], None, token, self.embed, first["scale"], first["bias"], first["n1"], eps, k["n"])
        ops.decode_gemm(first["w_in"], k["n"], 5 * d, 0, k["qkvgu"], k["flag"], False)
        for index, (w, st) in enumerate(zip(self.weights, self.states)):
            ops.decode_attn(k["qkvgu"], st.k, st.v, st.u, st.mixed, k["rope"], pos, self.h, k["y"])
            nxt = self.weights[index + 1] if index + 1 < len(self.weights) else None
            ops.decode_layer_tail(w["w_out"], w["w_ug"], w["w_down"], nxt["w_in"] if nxt else None, k["y"], k["x"],
                                  k["p_out"], k["p_down"], k["n"], k["act"], k["qkvgu"], w["n2"],
                                  nxt["scale"] if nxt else None, nxt["bias"] if nxt else None,
                                  nxt["n1"] if nxt else self.final_norm, eps, k["barrier"], k["flag"])
        ops.decode_gemm(self.head, k["n"], self.cfg.vocab_size, 3, k["logits"], k["flag"], False)
        return k["logits"]

    def _step_kernels(self, token: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        if self._layer_tail:
            return self._step_kernels_tail(token, pos)
        ops = torch.ops.ws_b200
        k = self._kbufs
        d, ffn, eps = self.cfg.d_model, self.cfg.ffn_hidden, self.cfg.rms_eps
        first = self.weights[0]
        ops.decode_reduce_norm(k["x"], None, token, self.embed, first["scale"], first["bias"], first["n1"], eps, k["n"])
        for index, (w, st) in enumerate(zip(self.weights, self.states)):
            ops.decode_gemm(w["p_in"], k["n"], 5 * d, 0, k["qkvgu"], k["flag"], self.pack_weights)
            ops.decode_attn(k["qkvgu"], st.k, st.v, st.u, st.mixed, k["rope"], pos, self.h, k["y"])
            ops.decode_gemm(w["p_out"], k["y"], d, 1, k["p_out"], k["flag"], self.pack_weights)
            ops.decode_reduce_norm(k["x"], k["p_out"], None, None, None, None, w["n2"], eps, k["n"])
            ops.decode_gemm(w["p_ug"], k["n"], ffn, 2, k["act"], k["flag"], self.pack_weights)
            ops.decode_gemm(w["p_down"], k["act"], d, 1, k["p_down"], k["flag"], self.pack_weights)
            if index + 1 < len(self.weights):
                nxt = self.weights[index + 1]
                ops.decode_reduce_norm(k["x"], k["p_down"], None, None, nxt["scale"], nxt["bias"], nxt["n1"], eps, k["n"])
            else:
                ops.decode_reduce_norm(k["x"], k["p_down"], None, None, None, None, self.final_norm, eps, k["n"])
        ops.decode_gemm(self.head_packed, k["n"], self.cfg.vocab_size, 3, k["logits"], k["flag"], self.pack_weights)
        return k["logits"]

    def _step_fn(self, token: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        if self._kbufs is not None:
            return self._step_kernels(token, pos)
        return self._step_math(token, pos)

    def _norm(self, x, w):
        x32 = x.float()
        return (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w).to(self.dtype)

    # ------------------------------------------------------------------ one token for the whole batch
    def _step_math(self, token: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        b = token.shape[0]
        x = self.embed[token].float()
        cos = self.cos.index_select(0, pos.view(1)).view(1, 1, self.hd)
        sin = self.sin.index_select(0, pos.view(1)).view(1, 1, self.hd)
        visible = (torch.arange(self.chunk, device=self.device) <= pos).view(1, 1, self.chunk)
        scale = 1.0 / math.sqrt(self.hd)
        for w, st in zip(self.weights, self.states):
            x = x * (1.0 + w["scale"]) + w["bias"]
            qkvgu = F.linear(self._norm(x, w["n1"]), w["w_in"])
            q, k, v, g, u = (t.view(b, self.h, self.hd) for t in qkvgu.chunk(5, dim=-1))
            q = (q.float() * cos + R.rotate_pairs(q.float()) * sin).to(self.dtype)
            k = (k.float() * cos + R.rotate_pairs(k.float()) * sin).to(self.dtype)
            index = pos.view(1)
            st.k.index_copy_(2, index, k.unsqueeze(2))
            st.v.index_copy_(2, index, v.unsqueeze(2))
            st.u.index_copy_(2, index, u.unsqueeze(2))
            scores = torch.einsum("bhd,bhcd->bhc", q.float(), st.k.float()) * scale
            p = torch.softmax(scores.masked_fill(~visible, -torch.inf), dim=-1)
            local = torch.einsum("bhc,bhcd->bhd", p, st.v.float())
            memory = torch.einsum("bhi,bhij->bhj", q.float(), st.mixed.float()) * scale
            gate = torch.sigmoid(g.float())
            y = (gate * local + (1.0 - gate) * memory).to(self.dtype).reshape(b, self.h * self.hd)
            x = x + F.linear(y, w["w_out"]).float()
            up, gt = F.linear(self._norm(x, w["n2"]), w["w_ug"]).chunk(2, dim=-1)
            x = x + F.linear(F.silu(gt) * up, w["w_down"]).float()
        return F.linear(self._norm(x, self.final_norm), self.head).float()

    def _end_of_chunk(self) -> None:
        for w, st in zip(self.weights, self.states):
            write = torch.matmul(torch.tanh(st.k).transpose(-2, -1), torch.tanh(st.u)).float() / self.chunk
            st.fast.mul_(w["df"]).add_(write * (1.0 - w["df"]))
            st.slow.mul_(w["ds"]).add_(write * (1.0 - w["ds"]))
            st.mixed.copy_((w["mix"] * st.fast + (1.0 - w["mix"]) * st.slow).to(self.dtype))

    @torch.no_grad()
    def step(self, token: torch.Tensor) -> torch.Tensor:
        """``token [B]`` (or ``[B,1]``) -> logits ``[B, V]`` FP32."""
        token = token.reshape(-1).to(self.device).contiguous()
        if self.states is None or token.shape[0] != self.batch:
            self.new_state(token.shape[0])
        self.pos_dev.fill_(self.pos)
        if self.use_graph:
            self.token_buf.copy_(token)
            if self._graph is None:
                self._capture()
            self._graph.replay()
            self.graph_counters.replay_calls += 1
            self.graph_counters.replay_calls_by_batch[self.batch] += 1
            logits = self.logits_buf
        else:
            logits = self._step_fn(token, self.pos_dev)
            self.graph_counters.eager_steps += 1
        self.pos += 1
        if self.pos == self.chunk:
            self._end_of_chunk()
            self.pos = 0
        return logits

    # ------------------------------------------------------------------ greedy decode without the host
    @torch.no_grad()
    def decode_greedy(self, token: torch.Tensor, steps: int, events: list | None = None) -> torch.Tensor:
        """Feed ``token [B]``, then ``steps`` times pick the arg-max token and feed it back: ``[B, steps]``.

        On the kernel path the pick, the hand-back of the token, the history write and the position counter are the
        last node of the step graph (`decode_pick_kernel`), so consecutive steps are queued without any host
        synchronisation; the host only counts positions to run the chunk-boundary state update in stream order.
        ``events``, when given, receives one CUDA event before the first step and one after every step.
        Elsewhere (CPU, kernels or graphs off) it is the plain loop over `step`."""
        token = token.reshape(-1).to(self.device).contiguous()
        if self.states is None or token.shape[0] != self.batch:
            self.new_state(token.shape[0])
        if self._kbufs is None or not self.use_graph:
            columns = []
            for _ in range(steps):
                token = torch.argmax(self.step(token), dim=-1)
                columns.append(token)
            return torch.stack(columns, dim=1) if columns else token.new_zeros(token.shape[0], 0)
        stream = torch.cuda.current_stream(self.device)
        self.token_buf.copy_(token)
        self.pos_dev.fill_(self.pos)
        if events is not None:
            events.append(torch.cuda.Event(enable_timing=True))
            events[-1].record(stream)
        pieces, done = [], 0
        while done < steps:
            run = min(steps - done, self.GREEDY_CAPACITY)
            self.cursor.zero_()
            for _ in range(run):
                if self._greedy_graph is None:
                    self._capture_greedy()
                self._greedy_graph.replay()
                self.graph_counters.replay_calls += 1
                self.graph_counters.replay_calls_by_batch[self.batch] += 1
                self.pos += 1
                if self.pos == self.chunk:      # the graph left pos_dev at `chunk`: fold the chunk, start the next
                    self._end_of_chunk()
                    self.pos = 0
                    self.pos_dev.zero_()
                if events is not None:
                    events.append(torch.cuda.Event(enable_timing=True))
                    events[-1].record(stream)
            pieces.append(self.history[:, :run].clone())
            done += run
        return torch.cat(pieces, dim=1) if len(pieces) != 1 else pieces[0]

    def _capture_greedy(self) -> None:
        if self._graph is None:
            self._capture()                     # warms the step's kernels up on a side stream
        from ..ops import _ext
        self._greedy_graph = torch.cuda.CUDAGraph()
        launched = _ext.launch_count()
        with torch.cuda.graph(self._greedy_graph):
            logits = self._step_fn(self.token_buf, self.pos_dev)
            torch.ops.ws_b200.decode_pick(logits, self.token_buf, self.history, self.cursor, self.pos_dev)
        self.graph_counters.capture_calls += 1
        self.graph_counters.kernels_per_replay = _ext.launch_count() - launched

    def _capture(self) -> None:
        # warm up on a side stream (allocator + lazy initialisations), then capture once;
        # the cache writes of the warm-up land at the current position and are overwritten by the
        # identical values of the captured replay
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):
                self._step_fn(self.token_buf, self.pos_dev)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        from ..ops import _ext
        self._graph = torch.cuda.CUDAGraph()
        launched = _ext.launch_count()
        with torch.cuda.graph(self._graph):
            self.logits_buf = self._step_fn(self.token_buf, self.pos_dev)
        self.graph_counters.capture_calls += 1
        self.graph_counters.kernels_per_replay = _ext.launch_count() - launched

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """``ids [B, T]``: fills the state with the whole prompt; returns the logits after its
        last token ``[B, V]``."""
        ids = ids.to(self.device)
        b, t = ids.shape
        self.new_state(b)
        full = (t // self.chunk) * self.chunk
        logits = None
        if full:
            hidden = self._prefill_chunks(ids[:, :full])
            if full == t:
                logits = F.linear(self._norm(hidden[:, -1], self.final_norm), self.head).float()
        for i in range(full, t):
            logits = self.step(ids[:, i])
        return logits

    def _prefill_chunks(self, ids: torch.Tensor) -> torch.Tensor:
        model = self.model
        use_fused = False
        if self.device.type == "cuda" and self.dtype == torch.bfloat16:
            from ..ops import fused
            with torch.autocast("cuda", dtype=torch.bfloat16):
                use_fused = fused.active(self.embed)
        x = self.embed[ids].float()
        for depth, (w, st) in enumerate(zip(self.weights, self.states)):
            core = model.cores[depth % self.cfg.n_cores]
            if use_fused:
                from ..ops import fused
                x, fast, slow = fused.core_prefill(core, x, model.depth_scale[depth], model.depth_bias[depth])
            else:
                x = x * (1.0 + w["scale"]) + w["bias"]
                x, (fast, slow) = core.forward_with_state(x)
            st.fast.copy_(fast.float())
            st.slow.copy_(slow.float())
            st.mixed.copy_((w["mix"] * st.fast + (1.0 - w["mix"]) * st.slow).to(self.dtype))
        return x
