"""Layer object for the fused MXFP4 MoE: weights resident in HBM, every buffer of a step carved
out of ONE device allocation made when the layer is built, the serving call sequence of the
reference binding (src/python/vkernels/vllm_experts.py:813-1092).

Scratch policy. The reference keeps persistent scratch tensors that are sized at a token budget
and refuses to grow them while a CUDA graph is being captured
(src/python/vkernels/vllm_experts.py:142-246). Here the question of growth does not arise: the
layer takes its token budget as a constructor argument, lays all per-step buffers out in a single
arena at that budget, and a batch beyond the budget is rejected whether or not a capture is
active. Addresses therefore never change after construction, which is what graph replay needs.
"""
from __future__ import annotations

import contextlib
import os

import torch

from . import native_runtime as nr
from . import torch_ops as ops

DEFAULT_TOKEN_BUDGET = 8192


class StepArena:
    """A single uint8 device allocation divided into named, 256-byte aligned regions.

    ``plan`` maps a region name to ``(dtype, element count at the token budget)``. ``take(name, n)``
    returns the first ``n`` elements of the region as a typed 1-D tensor; asking for more than was
    planned raises ``ValueError`` (the budget was too small), never reallocates."""

    def __init__(self, plan: dict, device):
        self.device = torch.device(device)
        self._regions = {}
        offset = 0
        for name, (dtype, count) in plan.items():
            nbytes = count * torch.empty((), dtype=dtype).element_size()
            self._regions[name] = (offset, dtype, count)
            offset += (nbytes + 255) // 256 * 256
        self.nbytes = offset
        self._store = torch.empty(max(offset, 256), dtype=torch.uint8, device=self.device)

    def take(self, name: str, count: int) -> torch.Tensor:
        offset, dtype, cap = self._regions[name]
        if count < 0 or count > cap:
            raise ValueError(f"[vkernels_b200] region {name!r} holds {cap} elements, {count} requested: "
                             f"the layer was built for a smaller token budget (max_tokens)")
        size = torch.empty((), dtype=dtype).element_size()
        return self._store[offset: offset + count * size].view(dtype)


@contextlib.contextmanager
def _region(name: str):
    """Profiler range around one phase of a layer call, named like the reference binding's
    regions (``moe:apply.gpu_align``, ``moe:apply.launch``; vllm_experts.py:897,1063) so its
    per-call profile tooling reads both. Off unless VK_MOE_NVTX=1: a range costs a microsecond
    of host time per phase, which a decode step does not have to spare."""
    if not _NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NVTX = os.environ.get("VK_MOE_NVTX", "0") == "1"


def set_profile_ranges(on: bool) -> None:
    global _NVTX
    _NVTX = bool(on)


class FusedMoEMxfp4:
    """Router + alignment + fused experts for one MoE layer on one GPU.

    Weights hold ``n_local`` routed experts followed by ``n_shared`` always-on experts.
    ``forward`` takes device activations; ``forward_host`` takes pinned host buffers and
    includes the copies (the end-to-end path of the benchmark).
    """

    def __init__(self, w13, w13_scale, w2, w2_scale, *, top_k: int, router_weight=None,
                 router_bias=None, routing: str = "softmax", renorm: bool = True,
                 scaling: float = 1.0, n_group: int = 1, topk_group: int = 1, n_shared: int = 0,
                 swiglu_limit: float = 0.0, activation: int = ops.moe_fused_mxfp4.SWIGLU,
                 beta: float = 4.0, linear_beta: float = 25.0, b13=None, b2=None,
                 max_tokens: int = DEFAULT_TOKEN_BUDGET, block_size: int = 16, prepack: bool = False):
        """``prepack``: also keep the weights in the prepacked form (``ops.prepack_weights``; about as
        large as the checkpoint form again) and run decode-size batches from it - their kernels
        then expand nothing and run at the memory rate. Off by default because of the memory; a
        weight set with codes the form cannot express (inf / NaN) silently stays on the
        checkpoint layout (``self.prepacked`` is None then)."""
        ops.same_gpu_contiguous(w13, w13_scale, w2, w2_scale)
        self.w13, self.w13_scale, self.w2, self.w2_scale = w13, w13_scale, w2, w2_scale
        self.b13, self.b2 = b13, b2
        self.device = w13.device
        self.n_experts_total = w13.shape[0]
        self.n_shared = n_shared
        self.n_routed = self.n_experts_total - n_shared
        self.ispp = w13.shape[1] // 2
        self.hidden = w13.shape[2] * 2
        self.top_k = top_k
        self.slots = top_k + n_shared
        self.routing, self.renorm, self.scaling = routing, renorm, scaling
        self.n_group, self.topk_group = n_group, topk_group
        self.swiglu_limit, self.activation, self.beta, self.linear_beta = (swiglu_limit, activation,
                                                                          beta, linear_beta)
        self.router_weight, self.router_bias = router_weight, router_bias
        # the router scores every routed expert of the model; under expert parallelism this
        # layer holds only a slice of them
        self.n_router = self.n_routed if router_weight is None else router_weight.shape[0]
        self.block_size = block_size
        self.max_tokens = int(max_tokens or DEFAULT_TOKEN_BUDGET)
        self.capture_stream = None
        self.prepacked = None
        if prepack:
            packed = ops.prepack_weights(w13, w13_scale, w2, w2_scale)
            self.prepacked = packed if packed.usable else None
        self._reserve()

    # -- sizing ------------------------------------------------------------------------------
    def _em_bound(self, T: int) -> int:
        return ops.align_em_bound(T, self.slots, self.n_experts_total, self.block_size)

    # Batches up to this many tokens take the bf16-output form of the layer: ordered combine, no
    # fp32 output buffer to zero and convert (two launches less per step, bit-reproducible).
    ORDERED_COMBINE_TOKENS = 256
    TINY_SLOTS = 12

    def _workspace_bytes(self) -> int:
        T = self.max_tokens
        lib = nr.load_library()
        plain = lib.vk_cuda_moe_workspace_bytes(self._em_bound(T), self.hidden, self.ispp, self.n_experts_total,
                                                T * self.slots)
        Ts = min(T, self.ORDERED_COMBINE_TOKENS)
        small = lib.vk_cuda_moe_workspace_bytes_bf16(self._em_bound(Ts), self.hidden, self.ispp, self.n_experts_total,
                                                     Ts * self.slots)
        return max(plain, small)

    def _reserve(self) -> None:
        """Everything a step needs, allocated once: the library scratch of the current stream and
        the layer's own arena, both at the token budget."""
        T = self.max_tokens
        cap_em = self._em_bound(T)
        ops.reserve_workspace(self._workspace_bytes(), self.device)
        self.arena = StepArena({
            "logits": (torch.float32, T * self.n_router),
            "ids": (torch.int32, T * self.slots),
            "w": (torch.float32, T * self.slots),
            "sids": (torch.int32, cap_em),
            "eids": (torch.int32, cap_em // self.block_size),
            "out_em": (torch.int32, 1),
            "act": (torch.bfloat16, cap_em * self.ispp),
            "out": (torch.float32, T * self.hidden),
            "x": (torch.bfloat16, T * self.hidden),
            "y": (torch.bfloat16, T * self.hidden),
        }, self.device)

    def _buffers(self, T: int):
        em = self._em_bound(T)
        a = self.arena
        return {"logits": a.take("logits", T * self.n_router), "ids": a.take("ids", T * self.slots),
                "w": a.take("w", T * self.slots), "sids": a.take("sids", em),
                "eids": a.take("eids", em // self.block_size), "out_em": a.take("out_em", 1),
                "act": a.take("act", em * self.ispp), "out": a.take("out", T * self.hidden),
                "x": a.take("x", T * self.hidden), "y": a.take("y", T * self.hidden)}

    # -- stages ------------------------------------------------------------------------------
    def route(self, x: torch.Tensor, bufs=None, logits: torch.Tensor | None = None):
        """(ids [T, slots] int32, weights [T, slots] fp32) for activations x, or for given logits."""
        T = x.shape[0] if logits is None else logits.shape[0]
        bufs = bufs or self._buffers(T)
        if logits is None:
            if self.router_weight is None:
                raise TypeError("this layer has no router weight; pass logits or topk ids")
            logits = ops.router_logits(x, self.router_weight,
                                       out=bufs["logits"].view(T, self.n_router))
        ids = bufs["ids"].view(T, self.slots)
        w = bufs["w"].view(T, self.slots)
        ops.route_topk(logits, self.top_k, bias=self.router_bias,
                       sigmoid=self.routing == "sigmoid_group", n_group=self.n_group,
                       topk_group=self.topk_group, renorm=self.renorm, scaling=self.scaling,
                       n_shared=self.n_shared, out=(ids, w))
        return ids, w

    def experts_fp32(self, x, topk_ids, topk_w):
        """Like :meth:`experts` but returns the fp32 accumulator [T, hidden] (a view of the
        persistent buffer: consume it before the next call)."""
        return self.experts(x, topk_ids, topk_w, return_fp32=True)

    def experts(self, x, topk_ids, topk_w, bufs=None, out_bf16=None, return_fp32=False, aligned=None):
        """Alignment + the two grouped GEMMs for given routing; returns bf16 [T, hidden].
        ``aligned`` = (sorted_ids, expert_ids) skips the alignment (the fused small-batch router
        has already produced it)."""
        T = x.shape[0]
        bufs = bufs or self._buffers(T)
        em = self._em_bound(T)
        if aligned is not None:
            sids, eids = aligned
        else:
            with _region("moe:apply.gpu_align"):
                sids, eids, _ = ops.moe_align_block_size(
                    topk_ids, self.n_experts_total, self.block_size, max_EM=em,
                    out=(bufs["sids"], bufs["eids"], bufs["out_em"]))
        if not return_fp32 and T <= self.ORDERED_COMBINE_TOKENS:
            y = bufs["y"].view(T, self.hidden) if out_bf16 is None else out_bf16
            kw = dict(top_k=topk_ids.shape[1], block_size=self.block_size, swiglu_limit=self.swiglu_limit,
                      activation=self.activation, beta=self.beta, linear_beta=self.linear_beta, b13=self.b13, b2=self.b2)
            with _region("moe:apply.launch"):
                # (up to twelve routed slots the library runs two flat kernels on the checkpoint layout)
                if self.prepacked is not None and T * topk_ids.shape[1] > self.TINY_SLOTS:
                    ops.fused_moe_mxfp4_bf16_prepacked_into(y, bufs["act"], x, self.prepacked, topk_w.reshape(-1), sids,
                                                            eids, **kw)
                else:
                    ops.fused_moe_mxfp4_bf16_into(y, bufs["act"], x, self.w13, self.w13_scale, self.w2, self.w2_scale,
                                                  topk_w.reshape(-1), sids, eids, **kw)
            return y
        out = bufs["out"].view(T, self.hidden)
        with _region("moe:apply.launch"):
            out.zero_()
            ops.fused_moe_mxfp4_into(out, bufs["act"], x, self.w13, self.w13_scale, self.w2,
                                     self.w2_scale, topk_w.reshape(-1), sids, eids,
                                     top_k=topk_ids.shape[1], block_size=self.block_size,
                                     swiglu_limit=self.swiglu_limit, activation=self.activation,
                                     beta=self.beta, linear_beta=self.linear_beta, b13=self.b13,
                                     b2=self.b2)
        if return_fp32:
            return out
        y = bufs["y"].view(T, self.hidden) if out_bf16 is None else out_bf16
        with _region("moe:apply.convert"):
            y.copy_(out)
        return y

    def experts_rows(self, a_rows, out_rows, topk_ids, topk_w, store_slots: bool = False):
        """Alignment + the two grouped GEMMs on rows given by ADDRESS (int64 [R] each): reads
        every activation row where it lives and adds every result row where it belongs (see
        ``ops.fused_moe_mxfp4_rows_into``). The output rows must be zeroed by their owner."""
        R = a_rows.shape[0]
        bufs = self._buffers(R)
        em = self._em_bound(R)
        sids, eids, _ = ops.moe_align_block_size(
            topk_ids, self.n_experts_total, self.block_size, max_EM=em,
            out=(bufs["sids"], bufs["eids"], bufs["out_em"]))
        ops.fused_moe_mxfp4_rows_into(bufs["act"], a_rows, out_rows, self.w13, self.w13_scale, self.w2,
                                      self.w2_scale, topk_w.reshape(-1), sids, eids,
                                      top_k=topk_ids.shape[1], block_size=self.block_size,
                                      swiglu_limit=self.swiglu_limit, activation=self.activation,
                                      beta=self.beta, linear_beta=self.linear_beta, b13=self.b13, b2=self.b2,
                                      store_slots=store_slots)

    def forward(self, x: torch.Tensor, *, logits: torch.Tensor | None = None, out_bf16=None):
        """route -> align -> gate/up -> down+combine, all on the current stream."""
        ops.require(x.dim() == 2 and x.shape[1] == self.hidden, "x must be [T, hidden]")
        bufs = self._buffers(x.shape[0])
        T = x.shape[0]
        if T * self.slots <= 1024 and (logits is not None or self.router_weight is not None):
            # decode-size batch: router top-k and alignment in one kernel
            with _region("moe:apply.route"):
                if logits is None:
                    logits = ops.router_logits(x, self.router_weight, out=bufs["logits"].view(T, self.n_router))
                ids, w, sids, eids, _ = ops.route_align_small(
                    logits, self.top_k, block_size=self.block_size, bias=self.router_bias,
                    sigmoid=self.routing == "sigmoid_group", n_group=self.n_group, topk_group=self.topk_group,
                    renorm=self.renorm, scaling=self.scaling, n_shared=self.n_shared, max_EM=self._em_bound(T),
                    out=(bufs["ids"].view(T, self.slots), bufs["w"].view(T, self.slots), bufs["sids"], bufs["eids"],
                         bufs["out_em"]))
            return self.experts(x, ids, w, bufs, out_bf16=out_bf16, aligned=(sids, eids))
        with _region("moe:apply.route"):
            ids, w = self.route(x, bufs, logits=logits)
        return self.experts(x, ids, w, bufs, out_bf16=out_bf16)

    __call__ = forward

    def capture(self, x: torch.Tensor):
        """Captures ``forward(x)`` into a CUDA graph. Returns ``(graph, y)``: ``graph.replay()`` reruns the
        whole step (router, alignment, both GEMMs, conversion) on whatever ``x``'s storage holds
        then and leaves the result in ``y``. A decode step is a dozen short kernels; replaying
        them as one graph removes the launch gaps between them. Everything the step needs is
        allocated before the capture (two eager warm-up calls)."""
        side = self.capture_stream or torch.cuda.Stream(device=self.device)
        self.capture_stream = side
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            # the library scratch belongs to a stream: this one needs its block before the capture
            ops.reserve_workspace(self._workspace_bytes(), self.device)
            for _ in range(2):
                self.forward(x)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y = self.forward(x)
        return graph, y

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """Host activations in, host bf16 result out (both pinned), copies included; returns after
        the result has landed."""
        T = x_host.shape[0]
        bufs = self._buffers(T)
        x = bufs["x"].view(T, self.hidden)
        x.copy_(x_host, non_blocking=True)
        y = self.forward(x)
        out_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host


class HostPipeline:
    """End-to-end serving loop over pinned host batches: the host-to-device copy of step i + 1,
    the layer on step i and the device-to-host copy of step i - 1 run at the same time on three
    streams (two device input buffers, two device output buffers; the layer itself runs one
    step at a time on its stream). ``submit(x_host, y_host)`` enqueues a step and returns at once;
    ``drain()`` waits for everything submitted. Every step still pays its own two copies - they
    are merely off the critical path, as in a server that receives the next batch while it
    computes the current one."""

    def __init__(self, layer: "FusedMoEMxfp4", max_tokens: int | None = None, step=None):
        self.layer = layer
        dev = layer.device
        T = max_tokens or layer.max_tokens
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.x = [torch.empty((T, layer.hidden), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.y = [torch.empty((T, layer.hidden), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.x_free = [torch.cuda.Event() for _ in range(2)]     # the layer has consumed x[i]
        self.y_free = [torch.cuda.Event() for _ in range(2)]     # y[i] has reached the host
        self.n = 0
        self._step = step or (lambda x, y: layer.forward(x, out_bf16=y))
        with torch.cuda.device(dev), torch.cuda.stream(self.compute):
            ops.reserve_workspace(layer._workspace_bytes(), dev)   # the compute stream's scratch block

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        i = self.n & 1
        T = x_host.shape[0]
        x, y = self.x[i][:T], self.y[i][:T]
        with torch.cuda.stream(self.h2d):
            if self.n >= 2:
                self.h2d.wait_event(self.x_free[i])
            x.copy_(x_host, non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(loaded)
            if self.n >= 2:
                self.compute.wait_event(self.y_free[i])
            self._step(x, y)
            self.x_free[i].record(self.compute)
            done = torch.cuda.Event()
            done.record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(done)
            y_host.copy_(y, non_blocking=True)
            self.y_free[i].record(self.d2h)
        self.n += 1

    def drain(self) -> None:
        self.d2h.synchronize()


def layer_from_config(cfg, weights: dict, router: dict | None, *, max_tokens: int | None = None, prepack: bool = False):
    """Build the layer for a ``synthetic.MoEConfig`` from generated tensors."""
    return FusedMoEMxfp4(
        weights["w13"], weights["w13_scale"], weights["w2"], weights["w2_scale"], top_k=cfg.top_k,
        router_weight=None if router is None else router["wr"],
        router_bias=None if router is None else router["bias"], routing=cfg.routing,
        renorm=cfg.renorm, scaling=cfg.scaling, n_group=cfg.n_group, topk_group=cfg.topk_group,
        n_shared=cfg.shared_experts, swiglu_limit=cfg.swiglu_limit, max_tokens=max_tokens, prepack=prepack)
