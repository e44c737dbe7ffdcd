"""Layer object for the fused MXFP4 MoE: weights resident in HBM, persistent
scratch sized once, the serving call sequence of the reference binding.

``CaptureSafeScratch`` restates the reference's persistent-scratch manager
(src/python/vkernels/vllm_experts.py:142-246): buffers are sized once at the
token budget, later calls slice them, and growing is refused while a CUDA graph
is being captured because the captured graph still points at the old storage.
"""
from __future__ import annotations

import os

import torch

from . import native_runtime as nr
from . import torch_ops as ops


def _default_capture_probe() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class CaptureSafeScratch:
    """Persistent device buffers keyed by (device index, key)."""

    def __init__(self, capture_probe=None):
        self._buffers: dict = {}
        self._capture_probe = capture_probe or _default_capture_probe

    def keys(self):
        return list(self._buffers.keys())

    def get(self, key, count: int, *, dtype, device, capacity: int | None = None,
            name: str = "scratch") -> torch.Tensor:
        if count < 0:
            raise ValueError(f"{name}: count must be non-negative, got {count}")
        k = (device.index, key)
        store = self._buffers.get(k)
        if store is not None and store.numel() >= count:
            return store[:count]
        if self._capture_probe():
            cap = 0 if store is None else store.numel()
            raise RuntimeError(
                f"[vkernels_b200] persistent {name} (dev={device.index}, key={key!r}, cap={cap}) "
                f"is too small for {count} elements and a CUDA-graph capture is active - refusing "
                f"to grow (the captured graph references the old storage). Size it before capture.")
        cap = max(count, capacity) if capacity is not None else count
        store = torch.empty(cap, dtype=dtype, device=device)
        self._buffers[k] = store
        return store[:count]

    def reset(self) -> None:
        self._buffers.clear()


def max_num_tokens_hint() -> int:
    """Token budget used to size persistent scratch (reference vllm_experts.py:254-271)."""
    for k in ("MAX_NUM_BATCHED_TOKENS", "VLLM_MAX_NUM_BATCHED_TOKENS"):
        v = os.environ.get(k)
        if v:
            try:
                n = int(v)
                if n > 0:
                    return n
            except ValueError:
                pass
    return 8192


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
                 max_tokens: int | None = None, block_size: int = 16):
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
        self.max_tokens = max_tokens or max_num_tokens_hint()
        self.scratch = CaptureSafeScratch()
        self._reserve()

    # -- sizing ------------------------------------------------------------------------------
    def _em_bound(self, T: int) -> int:
        return ops.align_em_bound(T, self.slots, self.n_experts_total, self.block_size)

    def _reserve(self) -> None:
        T = self.max_tokens
        em = self._em_bound(T)
        lib = nr.load_library()
        with torch.cuda.device(self.device):
            need = lib.vk_cuda_moe_workspace_bytes(em, self.hidden, self.ispp, self.n_experts_total,
                                                   T * self.slots)
            nr.check(lib.vk_cuda_moe_reserve_workspace(need), "reserve_workspace")
        self._buffers(T)  # pins every persistent buffer at the budget

    def _buffers(self, T: int):
        d, s, cap_t = self.device, self.scratch, self.max_tokens
        cap_em = self._em_bound(cap_t)
        em = self._em_bound(T)
        g = lambda key, n, dt, cap: s.get(key, n, dtype=dt, device=d, capacity=cap, name=str(key))
        return {
            "logits": g("logits", T * self.n_router, torch.float32, cap_t * self.n_router),
            "ids": g("ids", T * self.slots, torch.int32, cap_t * self.slots),
            "w": g("w", T * self.slots, torch.float32, cap_t * self.slots),
            "sids": g("sids", em, torch.int32, cap_em),
            "eids": g("eids", em // self.block_size, torch.int32, cap_em // self.block_size),
            "out_em": g("out_em", 1, torch.int32, 1),
            "act": g("act", em * self.ispp, torch.bfloat16, cap_em * self.ispp),
            "out": g("out", T * self.hidden, torch.float32, cap_t * self.hidden),
            "x": g("x", T * self.hidden, torch.bfloat16, cap_t * self.hidden),
            "y": g("y", T * self.hidden, torch.bfloat16, cap_t * self.hidden),
        }

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

    def experts(self, x, topk_ids, topk_w, bufs=None, out_bf16=None, return_fp32=False):
        """Alignment + the two grouped GEMMs for given routing; returns bf16 [T, hidden]."""
        T = x.shape[0]
        bufs = bufs or self._buffers(T)
        em = self._em_bound(T)
        sids, eids, _ = ops.moe_align_block_size(
            topk_ids, self.n_experts_total, self.block_size, max_EM=em,
            out=(bufs["sids"], bufs["eids"], bufs["out_em"]))
        out = bufs["out"].view(T, self.hidden)
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
        y.copy_(out)
        return y

    def experts_rows(self, a_rows, out_rows, topk_ids, topk_w):
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
                                      beta=self.beta, linear_beta=self.linear_beta, b13=self.b13, b2=self.b2)

    def forward(self, x: torch.Tensor, *, logits: torch.Tensor | None = None, out_bf16=None):
        """route -> align -> gate/up -> down+combine, all on the current stream."""
        ops.require(x.dim() == 2 and x.shape[1] == self.hidden, "x must be [T, hidden]")
        bufs = self._buffers(x.shape[0])
        ids, w = self.route(x, bufs, logits=logits)
        return self.experts(x, ids, w, bufs, out_bf16=out_bf16)

    __call__ = forward

    def capture(self, x: torch.Tensor):
        """Captures ``forward(x)`` into a CUDA graph. Returns ``(graph, y)``: ``graph.replay()`` reruns the
        whole step (router, alignment, both GEMMs, conversion) on whatever ``x``'s storage holds
        then and leaves the result in ``y``. A decode step is a dozen short kernels; replaying
        them as one graph removes the launch gaps between them. Everything the step needs is
        allocated before the capture (two eager warm-up calls)."""
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
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


def layer_from_config(cfg, weights: dict, router: dict | None, *, max_tokens: int | None = None):
    """Build the layer for a ``synthetic.MoEConfig`` from generated tensors."""
    return FusedMoEMxfp4(
        weights["w13"], weights["w13_scale"], weights["w2"], weights["w2_scale"], top_k=cfg.top_k,
        router_weight=None if router is None else router["wr"],
        router_bias=None if router is None else router["bias"], routing=cfg.routing,
        renorm=cfg.renorm, scaling=cfg.scaling, n_group=cfg.n_group, topk_group=cfg.topk_group,
        n_shared=cfg.shared_experts, swiglu_limit=cfg.swiglu_limit, max_tokens=max_tokens)
