"""Helpers for the -m gpu parity tests: run the CUDA path through the C ABI and the CPU
oracle on the same seeded inputs."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from helpers import bf16_to_u16, expand_expert_ids
from vkernels_b200 import synthetic as syn
from vkernels_b200 import torch_ops as ops

DEV = "cuda:0"


def to_np(t):
    return t.detach().cpu().numpy()


def gpu_layer(A, w, ids, tw, *, impl="tcgen05", block_size=16, return_parts=False, **kw):
    """A bf16 [T,H] cuda, w dict of cuda uint8, ids int32 [T,k], tw fp32 [T,k] -> out fp32."""
    ops.set_impl(impl)
    try:
        T, H = A.shape
        E = w["w13"].shape[0]
        ispp = w["w13"].shape[1] // 2
        sids, eids, out_em = ops.moe_align_block_size(ids, E, block_size)
        out = torch.zeros((T, H), dtype=torch.float32, device=A.device)
        act = torch.zeros((sids.numel(), ispp), dtype=torch.bfloat16, device=A.device)
        ops.fused_moe_mxfp4_into(out, act, A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"],
                                 tw.reshape(-1).contiguous(), sids, eids, top_k=ids.shape[1],
                                 block_size=block_size, **kw)
        torch.cuda.synchronize()
        ops.kernel_status()
    finally:
        ops.set_impl("tcgen05")
    if return_parts:
        return out, act, sids, eids, out_em
    return out


def oracle_layer(A, w, ids, tw, *, tokens=None, **kw):
    wn = {k: to_np(v) for k, v in w.items()}
    return oracle.moe_layer(bf16_to_u16(A), wn["w13"], wn["w13_scale"], wn["w2"], wn["w2_scale"],
                            to_np(ids), to_np(tw), num_experts=wn["w13"].shape[0], tokens=tokens, **kw)


def make_case(cfg, T, *, codes="finite", seed=None, backend="numpy", routed=True):
    """Weights, activations, router and oracle routing for a configuration, on the GPU."""
    w = syn.make_expert_weights(cfg, codes=codes, seed=seed, backend=backend, device=DEV)
    A = syn.make_activations(cfg, T, seed=seed, backend=backend, device=DEV)
    r = syn.make_router(cfg, seed=seed, device=DEV)
    return w, A, r


def oracle_route(cfg, A, r, logits=None):
    """(ids, weights, margin) from the CPU routing restatement, with shared slots appended."""
    if logits is None:
        logits = oracle.router_logits(bf16_to_u16(A), to_np(r["wr"]))
    if cfg.routing == "sigmoid_group":
        ids, w, m = oracle.route_sigmoid_group_topk(logits, to_np(r["bias"]), cfg.top_k, n_group=cfg.n_group,
                                                    topk_group=cfg.topk_group, renorm=cfg.renorm,
                                                    scaling=cfg.scaling)
    else:
        ids, w, m = oracle.route_softmax_topk(logits, cfg.top_k, renorm=cfg.renorm, scaling=cfg.scaling)
    if cfg.shared_experts:
        T = ids.shape[0]
        ids = np.concatenate([ids, np.full((T, 1), cfg.E, np.int32)], 1)
        w = np.concatenate([w, np.ones((T, 1), np.float32)], 1)
    return ids, w, m
