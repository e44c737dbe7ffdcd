"""The layer split into its four stages (tensor parallelism), against the oracle's stage functions
(the reference's moe_gateup_cpu / moe_act_epilogue_cpu / moe_down_cpu / moe_combine_cpu,
moe_fused.cpp:235-564): stage by stage on the full reduction, and as two K-shards whose partial
results are added before the next stage - the call sequence of one tensor-parallel rank with the
all-reduce replaced by a sum on one GPU (reference tests/kernels/moe/test_dist_moe.cpp:277-291)."""
import numpy as np
import pytest
import torch

from gpu_common import DEV, make_case, to_np
from helpers import assert_close_bf16, bf16_to_u16

pytestmark = pytest.mark.gpu


def _setup(T, E=8, top_k=2, H=512, I=256, seed=3):
    import oracle
    from vkernels_b200 import synthetic as syn
    from vkernels_b200 import torch_ops as ops

    cfg = syn.scaled(syn.CONFIGS["c0"], H=H, I=I, E=E, top_k=top_k)
    w, A, _ = make_case(cfg, T)
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.int32)
    tw = rng.random((T, top_k), dtype=np.float32)
    b13 = (rng.standard_normal((E, 2 * I)) * 0.1).astype(np.float32)
    b2 = (rng.standard_normal((E, H)) * 0.1).astype(np.float32)
    sids, eids, _ = ops.moe_align_block_size(torch.from_numpy(ids).to(DEV), E, 16)
    tws = oracle.gather_sorted_weights(tw, to_np(sids))
    wn = {k: to_np(v) for k, v in w.items()}
    ref = oracle.moe_stages(bf16_to_u16(A), wn["w13"], wn["w13_scale"], wn["w2"], wn["w2_scale"], to_np(sids), tws,
                            to_np(eids), top_k=top_k, b13=b13, b2=b2, swiglu_limit=7.0)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    return cfg, w, A, sids, eids, dev(tws), dev(b13), dev(b2), ref


def _run_stages(cfg, w, A, sids, eids, tws, b13, b2, tp):
    from vkernels_b200 import torch_ops as ops

    T, H = A.shape
    I = cfg.I
    EM = sids.numel()
    gate_up = torch.zeros((EM, 2 * I), dtype=torch.float32, device=DEV)
    for r in range(tp):   # this rank's K-shard of w13; the sum over r stands for the all-reduce
        hk = H // tp
        part = torch.zeros_like(gate_up)
        ops.moe_gateup_preact(A, w["w13"][:, :, r * hk // 2:(r + 1) * hk // 2].contiguous(),
                              w["w13_scale"][:, :, r * hk // 32:(r + 1) * hk // 32].contiguous(), sids, eids, part,
                              top_k=cfg.top_k, k_base=r * hk)
        gate_up += part
    act = torch.zeros((EM, I), dtype=torch.bfloat16, device=DEV)
    ops.moe_act_epilogue(gate_up, act, sids, eids, M=T, top_k=cfg.top_k, b13=b13, swiglu_limit=7.0)
    partial = torch.zeros((EM, H), dtype=torch.float32, device=DEV)
    for r in range(tp):
        ik = I // tp
        part = torch.zeros_like(partial)
        ops.moe_down_preact(act, w["w2"][:, :, r * ik // 2:(r + 1) * ik // 2].contiguous(),
                            w["w2_scale"][:, :, r * ik // 32:(r + 1) * ik // 32].contiguous(), sids, eids, part, M=T,
                            top_k=cfg.top_k, k_base=r * ik)
        partial += part
    out = torch.zeros((T, H), dtype=torch.float32, device=DEV)
    ops.moe_combine(partial, tws, sids, eids, out, top_k=cfg.top_k, b2=b2)
    torch.cuda.synchronize()
    ops.kernel_status()
    return gate_up, act, partial, out


@pytest.mark.parametrize("T,tp", [(48, 1), (48, 2), (700, 1), (700, 2)])
def test_stage_split_matches_the_oracle_stages(T, tp):
    cfg, w, A, sids, eids, tws, b13, b2, ref = _setup(T)
    gate_up, act, partial, out = _run_stages(cfg, w, A, sids, eids, tws, b13, b2, tp)
    used = np.repeat(to_np(eids) >= 0, 16)   # rows of blocks that hold an expert
    assert_close_bf16(to_np(gate_up)[used], ref["gate_up"][used], f"gate_up T={T} tp={tp}")
    real = to_np(sids) < T * cfg.top_k
    got_act = to_np(act.view(torch.int16)).view(np.uint16)
    f32 = lambda u: (u.astype(np.uint32) << 16).view(np.float32)
    assert_close_bf16(f32(got_act[real]), f32(ref["act"][real]), f"act T={T} tp={tp}", got_is_bf16=True)
    assert np.all(got_act[~real] == 0), "padding rows of act must stay untouched"
    assert_close_bf16(to_np(partial)[used], ref["partial"][used], f"partial T={T} tp={tp}")
    assert_close_bf16(to_np(out), ref["out"], f"out T={T} tp={tp}")


def test_stage_split_rejects_bad_shards():
    from vkernels_b200 import torch_ops as ops

    cfg, w, A, sids, eids, tws, b13, b2, _ = _setup(16)
    gate_up = torch.zeros((sids.numel(), 2 * cfg.I), dtype=torch.float32, device=DEV)
    with pytest.raises((ValueError, RuntimeError)):   # shard reaches past the full reduction length
        ops.moe_gateup_preact(A, w["w13"], w["w13_scale"], sids, eids, gate_up, top_k=cfg.top_k, k_base=64)
