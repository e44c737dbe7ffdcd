"""PyTorch-tensor front end of the fused MXFP4 MoE layer (tensors only at the
boundary; the work happens behind the C ABI of ``libvkernels_b200.so``)."""
from ._dispatch import OpNotEligible, require, same_gpu_contiguous
from .moe_fused_mxfp4 import (align_em_bound, fused_moe_mxfp4, fused_moe_mxfp4_bf16_into, fused_moe_mxfp4_into,
                              fused_moe_mxfp4_rows_into, PrepackedWeights, prepack_weights,
                              fused_moe_mxfp4_bf16_prepacked_into,
                              kernel_status, moe_act_epilogue, moe_align_block_size, moe_combine,
                              moe_down_preact, moe_gateup_preact, mxfp4_dequant_rows, reserve_workspace,
                              reset_kernel_status, route_align_small, route_topk, router_logits, set_impl)

__all__ = ["OpNotEligible", "require", "same_gpu_contiguous", "align_em_bound", "fused_moe_mxfp4",
           "fused_moe_mxfp4_bf16_into", "fused_moe_mxfp4_into", "fused_moe_mxfp4_rows_into", "PrepackedWeights", "prepack_weights",
           "fused_moe_mxfp4_bf16_prepacked_into", "kernel_status", "moe_act_epilogue",
           "moe_align_block_size", "moe_combine", "moe_down_preact", "moe_gateup_preact",
           "mxfp4_dequant_rows", "reserve_workspace", "reset_kernel_status", "route_align_small", "route_topk", "router_logits",
           "set_impl"]
