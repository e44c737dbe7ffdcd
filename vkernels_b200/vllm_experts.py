"""Serving-side glue for a fused-MoE caller of the vLLM kind: the weight-format pass-through and an
experts object with the reference binding's ``apply`` call sequence.

What the reference does (src/python/vkernels/vllm_experts.py): ``convert_weights_for_vkernel``
(:531-582) hands the checkpoint's ``create_weights()`` layout through untouched - separated gate/up
halves, N-major ue8m0 scales - and only casts the bf16 biases to fp32, because the C ABI declares
``const float* b13 / b2``; ``VkernelFusedExperts.apply`` (:813-1092) aligns on the device with a
host-side bound on EM, launches the fused layer on the current stream into persistent buffers and
writes ``output`` as bf16. This module keeps both behaviours for the B200 library. vLLM itself is
not imported: ``B200FusedExperts`` is duck-typed (``workspace_shapes`` / ``apply`` with the
argument lists of vLLM's modular-kernel experts interface), so a vLLM integration subclasses its
own base class and forwards to it.
"""
from __future__ import annotations

import torch

from . import torch_ops as ops
from .torch_ops._dispatch import OpNotEligible, require

ACT_SWIGLU, ACT_SITU = 0, 1
# activation names a caller may pass (vLLM's MoEActivation members by name) -> the layer's epilogue
_ACTIVATIONS = {"silu": ACT_SWIGLU, "swigluoai": ACT_SWIGLU, "swigluoai_uninterleave": ACT_SWIGLU,
                "swiglustep": ACT_SWIGLU, "situ": ACT_SITU}


def convert_weights_for_b200(w13_weight, w2_weight, w13_weight_scale, w2_weight_scale, *rest, w13_bias=None,
                             w2_bias=None, **_ignored):
    """Pass raw ``create_weights()``-layout MXFP4 MoE weights through to the kernels and check that
    they really are in that layout (a silently different layout is the failure this shim exists
    to prevent: the kernels would compute on shuffled weights without any error).

    Accepts both call shapes of the reference shim: ``(w13, w2, w13_scale, w2_scale, w13_bias,
    w2_bias)`` and the variant that carries further positional entries after the biases (input
    scales, permute indices), which are ignored - the layer takes no activation scales.
    Returns ``(w13, w2, w13_scale, w2_scale, w13_bias_fp32, w2_bias_fp32)``.

    Layout: w13 ``[E, 2*ispp, hidden/2]`` uint8 (gate rows, then up rows; low nibble = even k),
    w2 ``[E, hidden, ispp/2]`` uint8, scales ``[E, rows, K/32]`` uint8 (ue8m0, one per 32 K).
    """
    if len(rest) >= 1 and rest[0] is not None:
        w13_bias = rest[0]
    if len(rest) >= 2 and rest[1] is not None:
        w2_bias = rest[1]
    w13, w2 = getattr(w13_weight, "data", w13_weight), getattr(w2_weight, "data", w2_weight)
    s13, s2 = getattr(w13_weight_scale, "data", w13_weight_scale), getattr(w2_weight_scale, "data", w2_weight_scale)
    for name, t in (("w13", w13), ("w2", w2), ("w13_scale", s13), ("w2_scale", s2)):
        require(t.dtype == torch.uint8 and t.dim() == 3, f"{name} must be uint8 [E, rows, cols]")
        require(t.is_contiguous(), f"{name} must be contiguous (the kernels read rows by pointer arithmetic)")
    E, two_i, half_h = w13.shape
    require(two_i % 2 == 0, "w13 must hold gate rows followed by up rows: an even row count")
    ispp, hidden = two_i // 2, half_h * 2
    require(hidden % 64 == 0 and ispp % 64 == 0, "hidden and ispp must be multiples of 64")
    require(w2.shape == (E, hidden, ispp // 2), f"w2 must be [E, hidden, ispp/2] = {(E, hidden, ispp // 2)}, got {tuple(w2.shape)}")
    require(s13.shape == (E, two_i, hidden // 32), f"w13_scale must be [E, 2*ispp, hidden/32], got {tuple(s13.shape)} "
                                                    "(a pre-shuffled or K-major scale layout is not what the kernels read)")
    require(s2.shape == (E, hidden, ispp // 32), f"w2_scale must be [E, hidden, ispp/32], got {tuple(s2.shape)}")

    def bias(b, cols, name):
        if b is None:
            return None
        b = getattr(b, "data", b)
        require(tuple(b.shape) == (E, cols), f"{name} must be [E, {cols}]")
        return b.to(torch.float32).contiguous()

    return w13, w2, s13, s2, bias(w13_bias, two_i, "w13_bias"), bias(w2_bias, hidden, "w2_bias")


class B200FusedExperts:
    """Experts object with the reference's ``VkernelFusedExperts`` call sequence (vllm_experts.py
    :734-1092) on the B200 library: device alignment bounded on the host, the fused layer on the
    current stream, bf16 written into ``output``. Scratch lives in ``workspace13`` when the caller's
    is large enough (it belongs to the caller's graph pool, so its address is stable), else in a
    buffer of this object sized at ``max_num_tokens`` and never reallocated afterwards."""

    def __init__(self, *, w13_scale, w2_scale, w13_bias=None, w2_bias=None, swiglu_limit: float = 0.0,
                 beta: float = 4.0, linear_beta: float = 25.0, max_num_tokens: int = 8192, prepack: bool = False):
        """``prepack``: on the first decode-size call (M <= 256) rewrite the weights once into the
        form the decode kernels read without expanding anything (``ops.prepack_weights``; costs a
        second copy of the weights) and serve such calls from it. Weights that hold the layer's
        inf / NaN codes stay on the checkpoint layout."""
        self.prepack, self._packed, self._packed_key = prepack, None, None
        self.w13_scale, self.w2_scale, self.b13, self.b2 = w13_scale, w2_scale, w13_bias, w2_bias
        self.swiglu_limit, self.beta, self.linear_beta = swiglu_limit, beta, linear_beta
        self.max_num_tokens = max_num_tokens
        self._act = None          # own act scratch, allocated once

    @staticmethod
    def supports_activation(name: str) -> bool:
        return str(name).lower() in _ACTIVATIONS

    @staticmethod
    def block_size(M: int) -> int:
        return 16     # tokens are the MMA's N dimension here: 16-row alignment packs best at every M

    def workspace_shapes(self, M, N, K, topk, global_num_experts, local_num_experts, expert_tokens_meta=None,
                         activation=None):
        """(workspace13, workspace2, output) shapes: ``workspace13`` = act_scratch [EM_max, ispp]
        bf16 (reference :784-811); the fp32 accumulator is not the caller's concern."""
        bs = self.block_size(M)
        em = ops.align_em_bound(M, topk, local_num_experts, bs)
        return (em, N // 2), (0,), (M, K)

    def apply(self, output, hidden_states, w1, w2, topk_weights, topk_ids, activation="silu", global_num_experts=-1,
              expert_map=None, a1q_scale=None, a2_scale=None, workspace13=None, workspace2=None,
              expert_tokens_meta=None, apply_router_weight_on_input: bool = False) -> None:
        if apply_router_weight_on_input:
            raise OpNotEligible("routing weights are applied in the down-GEMM epilogue, not on the input")
        act_kind = _ACTIVATIONS.get(str(getattr(activation, "name", activation)).lower())
        if act_kind is None:
            raise OpNotEligible(f"activation {activation!r} is not one of {sorted(_ACTIVATIONS)}")
        M, hidden = hidden_states.shape
        E_local, two_i, _ = w1.shape
        ispp = two_i // 2
        top_k = topk_ids.shape[1]
        n_global = E_local if global_num_experts in (None, -1) else global_num_experts
        bs = self.block_size(M)
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        sids, eids, _ = ops.moe_align_block_size(ids.contiguous(), n_global, bs, expert_map=expert_map, local_n=E_local,
                                                 max_EM=ops.align_em_bound(M, top_k, E_local, bs))
        em = sids.numel()
        if workspace13 is not None and workspace13.dtype == torch.bfloat16 and workspace13.numel() >= em * ispp:
            act = workspace13.view(-1)[: em * ispp]
        else:
            if self._act is None:
                cap = ops.align_em_bound(self.max_num_tokens, top_k, E_local, bs) * ispp
                self._act = torch.empty(cap, dtype=torch.bfloat16, device=hidden_states.device)
            require(self._act.numel() >= em * ispp, "batch exceeds max_num_tokens of this experts object")
            act = self._act[: em * ispp]
        y = output if output.dtype == torch.bfloat16 and output.is_contiguous() else \
            torch.empty((M, hidden), dtype=torch.bfloat16, device=hidden_states.device)
        kw = dict(top_k=top_k, block_size=bs, swiglu_limit=self.swiglu_limit, activation=act_kind, beta=self.beta,
                  linear_beta=self.linear_beta, b13=self.b13, b2=self.b2)
        tw = topk_weights.to(torch.float32).reshape(-1).contiguous()
        packed = None
        if self.prepack and M <= 256:
            key = (w1.data_ptr(), w2.data_ptr())
            if self._packed_key != key:      # first decode-size call (or the weights moved): rewrite once
                self._packed, self._packed_key = ops.prepack_weights(w1, self.w13_scale, w2, self.w2_scale), key
            packed = self._packed if self._packed.usable else None
        if packed is not None:
            ops.fused_moe_mxfp4_bf16_prepacked_into(y, act, hidden_states, packed, tw, sids, eids, **kw)
        else:
            ops.fused_moe_mxfp4_bf16_into(y, act, hidden_states, w1, self.w13_scale, w2, self.w2_scale, tw, sids, eids, **kw)
        if y is not output:
            output.copy_(y)
