"""Torch-tensor ops over the C ABI: alignment, routing, the fused layer.

Call sequence and buffer ownership follow the reference's serving binding
(src/python/vkernels/vllm_experts.py:813-1092): the caller's current stream, a
device-side alignment with a host-computed bound on EM (no host round trip), an
fp32 output zeroed before every launch, one fp32 -> bf16 conversion at the end.
"""
from __future__ import annotations

import torch

from .. import native_runtime as nr
from ._dispatch import require, same_gpu_contiguous

SWIGLU, SITU = 0, 1


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def set_impl(name: str) -> None:
    """"tcgen05" (default) or "simt" (CUDA-core cross-check kernels)."""
    impl = {"tcgen05": 0, "simt": 1}.get(name)
    if impl is None:
        raise TypeError(f"unknown implementation {name!r}")
    nr.check(nr.load_library().vk_cuda_moe_set_impl(impl), "set_impl")


def kernel_status() -> None:
    """Synchronise and raise if a tensor-core kernel gave up on a bounded wait."""
    nr.check(nr.load_library().vk_cuda_moe_kernel_status(), "kernel_status")


def align_em_bound(M: int, top_k: int, local_n: int, block_size: int) -> int:
    """Tight host-side upper bound on EM, a constant of the batch shape
    (reference vllm_experts.py:481-500): min(N, local_n) experts with one
    token each, the rest of the tokens in one more expert."""
    N = M * top_k
    if N <= 0:
        return block_size
    head = min(N, local_n) * block_size
    if N <= local_n:
        return head
    return head + ((N - local_n) + block_size - 1) // block_size * block_size


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int = 16, *,
                         expert_map: torch.Tensor | None = None, local_n: int | None = None,
                         max_EM: int | None = None, out=None):
    """Device alignment. Returns (sorted_ids[max_EM], expert_ids[max_EM/bs], out_em[1]), all
    int32 device tensors; nothing is read back. ``out`` may pass preallocated tensors."""
    require(topk_ids.dim() == 2, "topk_ids must be [M, top_k]")
    require(topk_ids.dtype == torch.int32, "topk_ids must be int32")
    same_gpu_contiguous(topk_ids, *([expert_map] if expert_map is not None else []))
    M, top_k = topk_ids.shape
    local_n = num_experts if local_n is None else local_n
    if max_EM is None:
        max_EM = align_em_bound(M, top_k, local_n, block_size)
    dev = topk_ids.device
    if out is None:
        sorted_ids = torch.empty(max_EM, dtype=torch.int32, device=dev)
        expert_ids = torch.empty(max_EM // block_size, dtype=torch.int32, device=dev)
        out_em = torch.empty(1, dtype=torch.int32, device=dev)
    else:
        sorted_ids, expert_ids, out_em = out
        require(sorted_ids.numel() >= max_EM and expert_ids.numel() >= max_EM // block_size,
                "preallocated alignment buffers are too small")
    with torch.cuda.device(dev):
        rc = nr.load_library().vk_hip_moe_align_block_size(
            _ptr(topk_ids), _ptr(expert_map), M, top_k, block_size, num_experts, local_n, max_EM,
            _ptr(sorted_ids), _ptr(expert_ids), _ptr(out_em), _stream(topk_ids))
    nr.check(rc, "moe_align_block_size")
    return sorted_ids[:max_EM], expert_ids[: max_EM // block_size], out_em


def router_logits(x: torch.Tensor, wr: torch.Tensor, out: torch.Tensor | None = None):
    """logits [T, E] fp32 = x [T, H] bf16 @ wr [E, H] fp32 ^T."""
    require(x.dtype == torch.bfloat16 and wr.dtype == torch.float32, "x bf16, wr fp32 expected")
    require(x.dim() == 2 and wr.dim() == 2 and x.shape[1] == wr.shape[1], "x [T,H], wr [E,H]")
    same_gpu_contiguous(x, wr)
    T, H = x.shape
    E = wr.shape[0]
    if out is None:
        out = torch.empty((T, E), dtype=torch.float32, device=x.device)
    require(out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous(), "out must be fp32 [T, E]")
    with torch.cuda.device(x.device):
        nr.check(nr.load_library().vk_cuda_moe_router_logits(_ptr(x), _ptr(wr), _ptr(out), T, H, E,
                                                            _stream(x)), "router_logits")
    return out


def route_topk(logits: torch.Tensor, top_k: int, *, bias: torch.Tensor | None = None,
               sigmoid: bool = False, n_group: int = 1, topk_group: int = 1, renorm: bool = True,
               scaling: float = 1.0, n_shared: int = 0, out=None):
    """Returns (ids int32 [T, top_k + n_shared], weights fp32 [T, top_k + n_shared])."""
    require(logits.dtype == torch.float32 and logits.dim() == 2, "logits must be fp32 [T, E]")
    same_gpu_contiguous(logits, *([bias] if bias is not None else []))
    require(bias is None or (bias.dtype == torch.float32 and bias.shape == (logits.shape[1],)),
            "bias must be fp32 [E]")
    T, E = logits.shape
    kk = top_k + n_shared
    if out is None:
        ids = torch.empty((T, kk), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, kk), dtype=torch.float32, device=logits.device)
    else:
        ids, w = out
    with torch.cuda.device(logits.device):
        rc = nr.load_library().vk_cuda_moe_route_topk(
            _ptr(logits), _ptr(bias), T, E, top_k, int(sigmoid), n_group, topk_group, int(renorm),
            float(scaling), n_shared, _ptr(ids), _ptr(w), _stream(logits))
    nr.check(rc, "route_topk")
    return ids, w


def route_align_small(logits: torch.Tensor, top_k: int, *, block_size: int = 16, bias: torch.Tensor | None = None,
                      sigmoid: bool = False, n_group: int = 1, topk_group: int = 1, renorm: bool = True,
                      scaling: float = 1.0, n_shared: int = 0, max_EM: int | None = None, out=None):
    """``route_topk`` and ``moe_align_block_size`` as ONE kernel for at most 1024 routed slots
    (``T * (top_k + n_shared)``). Returns ``(ids, weights, sorted_ids, expert_ids, out_em)``;
    ``out`` may pass these five tensors preallocated."""
    require(logits.dtype == torch.float32 and logits.dim() == 2, "logits must be fp32 [T, E]")
    same_gpu_contiguous(logits, *([bias] if bias is not None else []))
    T, E = logits.shape
    kk = top_k + n_shared
    require(0 < T * kk <= 1024, "route_align_small takes 1..1024 routed slots")
    if max_EM is None:
        max_EM = align_em_bound(T, kk, E + n_shared, block_size)
    dev = logits.device
    if out is None:
        ids = torch.empty((T, kk), dtype=torch.int32, device=dev)
        w = torch.empty((T, kk), dtype=torch.float32, device=dev)
        sorted_ids = torch.empty(max_EM, dtype=torch.int32, device=dev)
        expert_ids = torch.empty(max_EM // block_size, dtype=torch.int32, device=dev)
        out_em = torch.empty(1, dtype=torch.int32, device=dev)
    else:
        ids, w, sorted_ids, expert_ids, out_em = out
        require(sorted_ids.numel() >= max_EM and expert_ids.numel() >= max_EM // block_size,
                "preallocated alignment buffers are too small")
    with torch.cuda.device(dev):
        rc = nr.load_library().vk_cuda_moe_route_align_small(
            _ptr(logits), _ptr(bias), T, E, top_k, int(sigmoid), n_group, topk_group, int(renorm), float(scaling),
            n_shared, block_size, max_EM, _ptr(ids), _ptr(w), _ptr(sorted_ids), _ptr(expert_ids), _ptr(out_em),
            _stream(logits))
    nr.check(rc, "route_align_small")
    return ids, w, sorted_ids[:max_EM], expert_ids[: max_EM // block_size], out_em


def reset_kernel_status() -> None:
    """Synchronise and clear the status word of the current device."""
    nr.check(nr.load_library().vk_cuda_moe_reset_kernel_status(), "reset_kernel_status")


def reserve_workspace(nbytes: int, device) -> None:
    """Allocate the library scratch of the CURRENT stream of `device` ahead of time (the layer
    launchers then allocate nothing; mandatory before capturing that stream)."""
    device = torch.device(device)
    with torch.cuda.device(device):
        nr.check(nr.load_library().vk_cuda_moe_reserve_workspace_on(
            int(nbytes), torch.cuda.current_stream(device).cuda_stream), "reserve_workspace")


def mxfp4_dequant_rows(packed: torch.Tensor, scale: torch.Tensor, path: str = "permute") -> torch.Tensor:
    """[rows, K/2] uint8 + [rows, K/32] uint8 -> [rows, K] bf16 through one of the kernels' own
    decoders: "permute" (CTA-pair form) or "table" (lone-CTA form)."""
    require(packed.dtype == torch.uint8 and scale.dtype == torch.uint8, "uint8 inputs expected")
    same_gpu_contiguous(packed, scale)
    rows, kb = packed.shape
    K = kb * 2
    require(scale.shape == (rows, K // 32), "scale must be [rows, K/32]")
    out = torch.empty((rows, K), dtype=torch.bfloat16, device=packed.device)
    with torch.cuda.device(packed.device):
        sel = {"permute": 0, "table": 1}[path]
        nr.check(nr.load_library().vk_cuda_mxfp4_dequant_rows_path(_ptr(packed), _ptr(scale), _ptr(out),
                                                                  rows, K, sel, _stream(packed)),
                 "mxfp4_dequant_rows")
    return out


def _check_layer_shapes(hidden_states, w13, w13_scale, w2, w2_scale, b13, b2):
    require(hidden_states.dtype == torch.bfloat16 and hidden_states.dim() == 2,
            "hidden_states must be bf16 [M, hidden]")
    for t in (w13, w13_scale, w2, w2_scale):
        require(t.dtype == torch.uint8 and t.dim() == 3, "weights and scales must be uint8 [E, rows, cols]")
    M, hidden = hidden_states.shape
    E, two_i, hk = w13.shape
    ispp = two_i // 2
    require(two_i % 2 == 0 and hk * 2 == hidden, "w13 must be [E, 2*ispp, hidden/2]")
    require(hidden % 64 == 0 and ispp % 64 == 0, "hidden and ispp must be multiples of 64")
    require(w13_scale.shape == (E, two_i, hidden // 32), "w13_scale must be [E, 2*ispp, hidden/32]")
    require(w2.shape == (E, hidden, ispp // 2), "w2 must be [E, hidden, ispp/2]")
    require(w2_scale.shape == (E, hidden, ispp // 32), "w2_scale must be [E, hidden, ispp/32]")
    require(b13 is None or (b13.dtype == torch.float32 and b13.shape == (E, two_i)),
            "b13 must be fp32 [E, 2*ispp]")
    require(b2 is None or (b2.dtype == torch.float32 and b2.shape == (E, hidden)),
            "b2 must be fp32 [E, hidden]")
    return M, hidden, ispp, E


def fused_moe_mxfp4_into(out_fp32, act_scratch, hidden_states, w13, w13_scale, w2, w2_scale,
                         topk_weights, sorted_ids, expert_ids, *, top_k: int, block_size: int = 16,
                         swiglu_limit: float = 0.0, activation: int = SWIGLU, beta: float = 4.0,
                         linear_beta: float = 25.0, b13=None, b2=None, weights_sorted: bool = False):
    """Raw launch: accumulates into ``out_fp32`` [M, hidden] (zero it first), writes
    ``act_scratch`` [EM, ispp] bf16. Everything is caller-owned; nothing is allocated."""
    M, hidden, ispp, _ = _check_layer_shapes(hidden_states, w13, w13_scale, w2, w2_scale, b13, b2)
    same_gpu_contiguous(hidden_states, w13, w13_scale, w2, w2_scale, topk_weights, sorted_ids,
                        expert_ids, out_fp32, act_scratch, *[t for t in (b13, b2) if t is not None])
    EM = sorted_ids.numel()
    require(EM % block_size == 0 and expert_ids.numel() * block_size >= EM,
            "sorted_ids / expert_ids do not match block_size")
    require(out_fp32.dtype == torch.float32 and out_fp32.numel() >= M * hidden, "out must be fp32 [M, hidden]")
    require(act_scratch.dtype == torch.bfloat16 and act_scratch.numel() >= EM * ispp,
            "act_scratch must be bf16 [EM, ispp]")
    require(topk_weights.dtype == torch.float32, "topk_weights must be fp32")
    require(topk_weights.numel() >= (EM if weights_sorted else M * top_k), "topk_weights too small")
    lib = nr.load_library()
    with torch.cuda.device(hidden_states.device):
        if weights_sorted:
            rc = lib.vk_cuda_fused_moe_mxfp4_sorted_w(
                _ptr(hidden_states), _ptr(w13), _ptr(w13_scale), _ptr(w2), _ptr(w2_scale),
                _ptr(topk_weights), _ptr(act_scratch), _ptr(out_fp32), M, hidden, ispp, top_k,
                _ptr(sorted_ids), _ptr(expert_ids), EM, float(swiglu_limit), int(activation),
                float(beta), float(linear_beta), _ptr(b13), _ptr(b2), block_size,
                _stream(hidden_states))
            nr.check(rc, "fused_moe_mxfp4")
        else:
            lib.vk_set_last_error(0, b"")
            lib.vk_hip_fused_moe_mxfp4(
                _ptr(hidden_states), _ptr(w13), _ptr(w13_scale), _ptr(w2), _ptr(w2_scale), None,
                _ptr(topk_weights), _ptr(act_scratch), _ptr(out_fp32), M, hidden, ispp, top_k,
                _ptr(sorted_ids), _ptr(expert_ids), EM, float(swiglu_limit), int(activation),
                float(beta), float(linear_beta), _ptr(b13), _ptr(b2), block_size,
                _stream(hidden_states))
            nr.check(lib.vk_last_error_code(), "fused_moe_mxfp4")
    return out_fp32


def fused_moe_mxfp4_bf16_into(y_bf16, act_scratch, hidden_states, w13, w13_scale, w2, w2_scale, topk_weights,
                              sorted_ids, expert_ids, *, top_k: int, block_size: int = 16, swiglu_limit: float = 0.0,
                              activation: int = SWIGLU, beta: float = 4.0, linear_beta: float = 25.0, b13=None, b2=None):
    """The layer with a bf16 result written by an ordered, atomic-free combine (each token's expert
    contributions added in ascending expert order): ``y_bf16`` [M, hidden] is overwritten, nothing
    needs zeroing or converting. Everything is caller-owned; the library scratch of the current
    stream must have been reserved at ``vk_cuda_moe_workspace_bytes_bf16`` (the layer object does)."""
    M, hidden, ispp, _ = _check_layer_shapes(hidden_states, w13, w13_scale, w2, w2_scale, b13, b2)
    same_gpu_contiguous(hidden_states, w13, w13_scale, w2, w2_scale, topk_weights, sorted_ids, expert_ids, y_bf16,
                        act_scratch, *[t for t in (b13, b2) if t is not None])
    EM = sorted_ids.numel()
    require(EM % block_size == 0 and expert_ids.numel() * block_size >= EM, "sorted_ids / expert_ids do not match block_size")
    require(y_bf16.dtype == torch.bfloat16 and y_bf16.numel() >= M * hidden, "y must be bf16 [M, hidden]")
    require(act_scratch.dtype == torch.bfloat16 and act_scratch.numel() >= EM * ispp, "act_scratch must be bf16 [EM, ispp]")
    require(topk_weights.dtype == torch.float32 and topk_weights.numel() >= M * top_k, "topk_weights too small")
    with torch.cuda.device(hidden_states.device):
        rc = nr.load_library().vk_cuda_fused_moe_mxfp4_bf16(
            _ptr(hidden_states), _ptr(w13), _ptr(w13_scale), _ptr(w2), _ptr(w2_scale), _ptr(topk_weights),
            _ptr(act_scratch), _ptr(y_bf16), M, hidden, ispp, top_k, _ptr(sorted_ids), _ptr(expert_ids), EM,
            float(swiglu_limit), int(activation), float(beta), float(linear_beta), _ptr(b13), _ptr(b2), block_size,
            _stream(hidden_states))
    nr.check(rc, "fused_moe_mxfp4_bf16")
    return y_bf16


class PrepackedWeights:
    """Both weight sets of a layer in the prepacked form of ``vk_cuda_moe_prepack_weights`` plus
    the shapes they were made from. ``nonfinite`` is the number of 32-element groups that hold a
    code this form cannot express (inf / NaN in the layer's table); when it is not zero the
    object must not be used (``usable`` is False) and the checkpoint-layout weights stay in charge."""

    def __init__(self, w13_codes, w13_sf, w2_codes, w2_sf, E, hidden, ispp, nonfinite):
        self.w13_codes, self.w13_sf, self.w2_codes, self.w2_sf = w13_codes, w13_sf, w2_codes, w2_sf
        self.E, self.hidden, self.ispp, self.nonfinite = E, hidden, ispp, nonfinite

    @property
    def usable(self) -> bool:
        return self.nonfinite == 0


def prepack_weights(w13, w13_scale, w2, w2_scale) -> PrepackedWeights:
    """One-time rewrite of checkpoint-layout MXFP4 weights into the form the decode kernels read
    without expanding anything (see ``vk_cuda_moe_prepack_weights``). Allocates the two code
    buffers (checkpoint size + padding) and the regrouped scales; reads back one int."""
    import ctypes

    require(w13.dtype == torch.uint8 and w13.dim() == 3 and w2.dtype == torch.uint8 and w2.dim() == 3,
            "w13 / w2 must be uint8 [E, rows, K/2]")
    same_gpu_contiguous(w13, w13_scale, w2, w2_scale)
    E, two_i, half_h = w13.shape
    ispp, hidden = two_i // 2, half_h * 2
    require(tuple(w2.shape) == (E, hidden, ispp // 2), "w2 must be [E, hidden, ispp/2]")
    require(tuple(w13_scale.shape) == (E, two_i, hidden // 32) and tuple(w2_scale.shape) == (E, hidden, ispp // 32),
            "scales must be [E, rows, K/32]")
    lib = nr.load_library()
    out, bad = [], torch.zeros(2, dtype=torch.int32, device=w13.device)
    with torch.cuda.device(w13.device):
        for which, (w, sc) in enumerate(((w13, w13_scale), (w2, w2_scale))):
            wb, sb = ctypes.c_size_t(0), ctypes.c_size_t(0)
            nr.check(lib.vk_cuda_moe_prepack_sizes(which, E, hidden, ispp, ctypes.addressof(wb), ctypes.addressof(sb)),
                     "moe_prepack_sizes")
            codes = torch.empty(wb.value, dtype=torch.uint8, device=w13.device)
            sf = torch.empty(sb.value, dtype=torch.uint8, device=w13.device)
            nr.check(lib.vk_cuda_moe_prepack_weights(which, _ptr(w), _ptr(sc), E, hidden, ispp, _ptr(codes), _ptr(sf),
                                                     bad.data_ptr() + 4 * which, _stream(w13)), "moe_prepack_weights")
            out += [codes, sf]
    return PrepackedWeights(out[0], out[1], out[2], out[3], E, hidden, ispp, int(bad.sum().item()))


def fused_moe_mxfp4_bf16_prepacked_into(y_bf16, act_scratch, hidden_states, packed: PrepackedWeights, topk_weights,
                                        sorted_ids, expert_ids, *, top_k: int, block_size: int = 16,
                                        swiglu_limit: float = 0.0, activation: int = SWIGLU, beta: float = 4.0,
                                        linear_beta: float = 25.0, b13=None, b2=None):
    """``fused_moe_mxfp4_bf16_into`` on prepacked weights: decode-size batches only (the library
    refuses a batch whose token tiles would exceed 64 rows; M <= 256 never does)."""
    require(packed.usable, "these weights hold codes the prepacked form cannot express; use the checkpoint layout")
    M, hidden = hidden_states.shape
    ispp = packed.ispp
    require(hidden == packed.hidden and hidden_states.dtype == torch.bfloat16, "hidden_states must be bf16 [M, hidden]")
    same_gpu_contiguous(hidden_states, packed.w13_codes, packed.w13_sf, packed.w2_codes, packed.w2_sf, topk_weights,
                        sorted_ids, expert_ids, y_bf16, act_scratch, *[t for t in (b13, b2) if t is not None])
    for b, cols, name in ((b13, 2 * ispp, "b13"), (b2, hidden, "b2")):
        require(b is None or (b.dtype == torch.float32 and tuple(b.shape) == (packed.E, cols)), f"{name} must be fp32 [E, {cols}]")
    EM = sorted_ids.numel()
    require(EM % block_size == 0 and expert_ids.numel() * block_size >= EM, "sorted_ids / expert_ids do not match block_size")
    require(y_bf16.dtype == torch.bfloat16 and y_bf16.numel() >= M * hidden, "y must be bf16 [M, hidden]")
    require(act_scratch.dtype == torch.bfloat16 and act_scratch.numel() >= EM * ispp, "act_scratch must be bf16 [EM, ispp]")
    require(topk_weights.dtype == torch.float32 and topk_weights.numel() >= M * top_k, "topk_weights too small")
    with torch.cuda.device(hidden_states.device):
        rc = nr.load_library().vk_cuda_fused_moe_mxfp4_bf16_prepacked(
            _ptr(hidden_states), _ptr(packed.w13_codes), _ptr(packed.w13_sf), _ptr(packed.w2_codes), _ptr(packed.w2_sf),
            _ptr(topk_weights), _ptr(act_scratch), _ptr(y_bf16), M, hidden, ispp, top_k, _ptr(sorted_ids),
            _ptr(expert_ids), EM, float(swiglu_limit), int(activation), float(beta), float(linear_beta), _ptr(b13),
            _ptr(b2), block_size, _stream(hidden_states))
    nr.check(rc, "fused_moe_mxfp4_bf16_prepacked")
    return y_bf16


def fused_moe_mxfp4_rows_into(act_scratch, a_rows, out_rows, w13, w13_scale, w2, w2_scale, topk_weights,
                              sorted_ids, expert_ids, *, top_k: int, block_size: int = 16,
                              swiglu_limit: float = 0.0, activation: int = SWIGLU, beta: float = 4.0,
                              linear_beta: float = 25.0, b13=None, b2=None, store_slots: bool = False):
    """The layer with row ADDRESSES in place of the activation and output tensors: ``a_rows`` /
    ``out_rows`` are int64 [M] device tensors holding, per token, the address of its bf16
    activation row and of its fp32 output row (which may be in another GPU's memory mapped into
    this process). Results are added to the output rows; everything is caller-owned. With
    ``store_slots`` an output address names a [top_k, hidden] fp32 block instead and slot j's
    unweighted row is stored at its row j (no atomics; see ``vk_cuda_fused_moe_mxfp4_rows_store``)."""
    require(a_rows.dtype == torch.int64 and out_rows.dtype == torch.int64 and a_rows.dim() == 1 and
            a_rows.shape == out_rows.shape, "a_rows / out_rows must be int64 [M]")
    same_gpu_contiguous(a_rows, out_rows, w13, w13_scale, w2, w2_scale, topk_weights, sorted_ids, expert_ids,
                        act_scratch, *[t for t in (b13, b2) if t is not None])
    M = a_rows.shape[0]
    ispp, hidden = w13.shape[1] // 2, w13.shape[2] * 2
    EM = sorted_ids.numel()
    require(EM % block_size == 0 and expert_ids.numel() * block_size >= EM,
            "sorted_ids / expert_ids do not match block_size")
    require(act_scratch.dtype == torch.bfloat16 and act_scratch.numel() >= EM * ispp,
            "act_scratch must be bf16 [EM, ispp]")
    require(topk_weights.dtype == torch.float32 and topk_weights.numel() >= M * top_k, "topk_weights too small")
    with torch.cuda.device(a_rows.device):
        lib = nr.load_library()
        fn = lib.vk_cuda_fused_moe_mxfp4_rows_store if store_slots else lib.vk_cuda_fused_moe_mxfp4_rows
        rc = fn(
            _ptr(a_rows), _ptr(w13), _ptr(w13_scale), _ptr(w2), _ptr(w2_scale), _ptr(topk_weights),
            _ptr(act_scratch), _ptr(out_rows), M, hidden, ispp, top_k, _ptr(sorted_ids), _ptr(expert_ids), EM,
            float(swiglu_limit), int(activation), float(beta), float(linear_beta), _ptr(b13), _ptr(b2),
            block_size, _stream(a_rows))
    nr.check(rc, "fused_moe_mxfp4_rows")


# ---- the layer in four stages (tensor parallelism): see include/vkernels_b200.h -------------------

def moe_gateup_preact(A, w13_shard, w13_scale_shard, sorted_ids, expert_ids, gate_up, *, top_k: int, k_base: int = 0):
    """gate_up [EM, 2*ispp] fp32 = gather(A)[:, k_base : k_base + hidden_k] @ w13_shard^T (no bias, no
    activation); ``w13_shard`` is [E, 2*ispp, hidden_k/2]. The caller adds the ranks' results."""
    same_gpu_contiguous(A, w13_shard, w13_scale_shard, sorted_ids, expert_ids, gate_up)
    M, hidden = A.shape
    ispp, hidden_k = w13_shard.shape[1] // 2, w13_shard.shape[2] * 2
    EM = sorted_ids.numel()
    require(gate_up.dtype == torch.float32 and gate_up.shape == (EM, 2 * ispp), "gate_up must be fp32 [EM, 2*ispp]")
    with torch.cuda.device(A.device):
        nr.check(nr.load_library().vk_cuda_moe_gateup_preact(
            _ptr(A), _ptr(w13_shard), _ptr(w13_scale_shard), _ptr(sorted_ids), _ptr(expert_ids), _ptr(gate_up), M,
            hidden, ispp, top_k, EM, k_base, hidden_k, _stream(A)), "moe_gateup_preact")
    return gate_up


def moe_act_epilogue(gate_up, act, sorted_ids, expert_ids, *, M: int, top_k: int, b13=None, swiglu_limit: float = 0.0,
                     activation: int = SWIGLU, beta: float = 4.0, linear_beta: float = 25.0):
    """act [EM, ispp] bf16 = activation(gate_up + b13), one rounding; padding rows are not written."""
    same_gpu_contiguous(gate_up, act, sorted_ids, expert_ids, *([b13] if b13 is not None else []))
    EM, ispp = act.shape
    require(gate_up.shape == (EM, 2 * ispp) and act.dtype == torch.bfloat16, "gate_up fp32 [EM, 2*ispp], act bf16 [EM, ispp]")
    with torch.cuda.device(act.device):
        nr.check(nr.load_library().vk_cuda_moe_act_epilogue(
            _ptr(gate_up), _ptr(b13), _ptr(act), _ptr(sorted_ids), _ptr(expert_ids), M, top_k, EM, ispp,
            float(swiglu_limit), int(activation), float(beta), float(linear_beta), _stream(act)), "moe_act_epilogue")
    return act


def moe_down_preact(act, w2_shard, w2_scale_shard, sorted_ids, expert_ids, partial, *, M: int, top_k: int,
                    k_base: int = 0):
    """partial [EM, hidden] fp32 = act[:, k_base : k_base + ispp_k] @ w2_shard^T; ``w2_shard`` is
    [E, hidden, ispp_k/2]. The caller adds the ranks' results."""
    same_gpu_contiguous(act, w2_shard, w2_scale_shard, sorted_ids, expert_ids, partial)
    EM, ispp = act.shape
    hidden, ispp_k = w2_shard.shape[1], w2_shard.shape[2] * 2
    require(partial.dtype == torch.float32 and partial.shape == (EM, hidden), "partial must be fp32 [EM, hidden]")
    with torch.cuda.device(act.device):
        nr.check(nr.load_library().vk_cuda_moe_down_preact(
            _ptr(act), _ptr(w2_shard), _ptr(w2_scale_shard), _ptr(sorted_ids), _ptr(expert_ids), _ptr(partial), M,
            ispp, hidden, top_k, EM, k_base, ispp_k, _stream(act)), "moe_down_preact")
    return partial


def moe_combine(partial, topk_w_sorted, sorted_ids, expert_ids, out, *, top_k: int, b2=None):
    """out [M, hidden] fp32 += (partial + b2) * topk_w_sorted per real row (zero ``out`` first)."""
    same_gpu_contiguous(partial, topk_w_sorted, sorted_ids, expert_ids, out, *([b2] if b2 is not None else []))
    EM, hidden = partial.shape
    M = out.shape[0]
    require(out.dtype == torch.float32 and out.shape[1] == hidden and topk_w_sorted.numel() >= EM,
            "out fp32 [M, hidden], topk_w_sorted [EM]")
    with torch.cuda.device(out.device):
        nr.check(nr.load_library().vk_cuda_moe_combine(
            _ptr(partial), _ptr(b2), _ptr(topk_w_sorted), _ptr(sorted_ids), _ptr(expert_ids), _ptr(out), M, hidden,
            top_k, EM, _stream(out)), "moe_combine")
    return out


def fused_moe_mxfp4(hidden_states, w13, w13_scale, w2, w2_scale, topk_ids, topk_weights, *,
                    swiglu_limit: float = 0.0, activation: int = SWIGLU, beta: float = 4.0,
                    linear_beta: float = 25.0, b13=None, b2=None, expert_map=None,
                    global_num_experts: int | None = None, block_size: int = 16,
                    return_fp32: bool = False):
    """Align on the device, run the layer, return bf16 [M, hidden] (or the fp32 accumulator).

    ``w13``/``w2`` hold the LOCAL experts; with ``expert_map`` (global -> local, -1 = not on
    this rank) ``topk_ids`` carry global ids, as in the reference binding."""
    M, hidden, ispp, E_local = _check_layer_shapes(hidden_states, w13, w13_scale, w2, w2_scale, b13, b2)
    require(topk_ids.shape == topk_weights.shape and topk_ids.dim() == 2 and topk_ids.shape[0] == M,
            "topk_ids / topk_weights must be [M, top_k]")
    top_k = topk_ids.shape[1]
    n_global = E_local if global_num_experts in (None, -1) else global_num_experts
    dev = hidden_states.device
    out = torch.zeros((M, hidden), dtype=torch.float32, device=dev)
    if M == 0:
        return out if return_fp32 else out.to(torch.bfloat16)
    sorted_ids, expert_ids, _ = moe_align_block_size(topk_ids.contiguous(), n_global, block_size,
                                                     expert_map=expert_map, local_n=E_local)
    act = torch.empty((sorted_ids.numel(), ispp), dtype=torch.bfloat16, device=dev)
    fused_moe_mxfp4_into(out, act, hidden_states, w13, w13_scale, w2, w2_scale,
                         topk_weights.contiguous().view(-1), sorted_ids, expert_ids, top_k=top_k,
                         block_size=block_size, swiglu_limit=swiglu_limit, activation=activation,
                         beta=beta, linear_beta=linear_beta, b13=b13, b2=b2)
    return out if return_fp32 else out.to(torch.bfloat16)
