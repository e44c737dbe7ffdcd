"""Pins the C restatement (oracle/moe_oracle.c) to the reference's own sources
compiled in place (oracle/_ref/libvkref.so): bit-for-bit equality of every stage
on seeded random problems, of the alignment, and of the expert-parallel plan,
dispatch and forward (reference tests/kernels/moe/test_dist_moe.cpp:451-555)."""
import numpy as np
import pytest

from helpers import bf16_to_u16, numpy_align
from vkernels_b200 import synthetic as syn


@pytest.fixture(scope="module")
def ref(oracle_mod):
    if not oracle_mod.have_reference():
        pytest.skip("oracle/_ref/libvkref.so not built")
    return oracle_mod


def small_problem(seed, T=24, H=192, I=128, E=6, k=3, codes="finite", scale_exp=(-8, -4)):
    cfg = syn.scaled(syn.CONFIGS["c0"], H=H, I=I, E=E, top_k=k, scale_exp=scale_exp)
    w = {n: t.numpy() for n, t in syn.make_expert_weights(cfg, seed=seed, codes=codes).items()}
    A = bf16_to_u16(syn.make_activations(cfg, T, seed=seed))
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    tw = rng.random((T, k), dtype=np.float32)
    return cfg, w, A, ids, tw


@pytest.mark.parametrize("seed,codes,limit,act,bias", [(1, "finite", 0.0, 0, False),
                                                       (2, "finite", 0.5, 0, True),
                                                       (3, "finite", 0.0, 1, True),
                                                       (4, "all", 0.0, 0, False)])
def test_all_stages_bit_exact(ref, seed, codes, limit, act, bias):
    cfg, w, A, ids, tw = small_problem(seed, codes=codes)
    s, e, EM = ref.moe_align_block_size(ids, cfg.E, 16)
    ws = ref.gather_sorted_weights(tw, s)
    rng = np.random.default_rng(seed + 100)
    b13 = rng.standard_normal((cfg.E, 2 * cfg.I)).astype(np.float32) if bias else None
    b2 = rng.standard_normal((cfg.E, cfg.H)).astype(np.float32) if bias else None
    kw = dict(top_k=cfg.top_k, swiglu_limit=limit, activation=act, b13=b13, b2=b2)
    a = ref.moe_stages(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, impl="port", **kw)
    b = ref.moe_stages(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, impl="reference", **kw)
    for name in ("gate_up", "act", "partial", "out"):
        x, y = a[name], b[name]
        xv = x.view(np.uint32) if x.dtype == np.float32 else x
        yv = y.view(np.uint32) if y.dtype == np.float32 else y
        same = (xv == yv) | (np.isnan(x.astype(np.float32) if x.dtype != np.uint16 else ref.bf16_to_f32(x))
                             & np.isnan(y.astype(np.float32) if y.dtype != np.uint16 else ref.bf16_to_f32(y)))
        assert same.all(), f"stage {name} differs at {np.argwhere(~same)[:3]}"
    # composed call, single-thread reference, threaded reference driver and restatement agree
    o_port, _ = ref.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, impl="port", **kw)
    o_ref, _ = ref.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, impl="reference", **kw)
    o_mt, _ = ref.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, impl="reference",
                                  threads=3, **kw)
    eq = lambda p, q: bool(((p.view(np.uint32) == q.view(np.uint32)) | (np.isnan(p) & np.isnan(q))).all())
    assert eq(o_port, o_ref) and eq(o_mt, o_ref)


@pytest.mark.parametrize("M,k,E,bs", [(8, 4, 4, 16), (64, 2, 8, 16), (200, 8, 256, 64), (33, 3, 40, 32), (1, 16, 256, 16)])
def test_align_matches_reference_and_numpy(ref, M, k, E, bs):
    rng = np.random.default_rng(M * 131 + k)
    ids = rng.integers(0, E, (M, k), dtype=np.int32)
    ids[rng.random((M, k)) < 0.05] = -3       # garbage ids are skipped
    ids[rng.random((M, k)) < 0.05] = E + 5
    a = ref.moe_align_block_size(ids, E, bs, impl="port")
    b = ref.moe_align_block_size(ids, E, bs, impl="reference")
    c = numpy_align(ids, E, bs)
    for x, y, z in zip(a, b, c):
        assert np.array_equal(x, y) and np.array_equal(x, z)


def test_align_empty(ref):
    ids = np.zeros((0, 4), np.int32)
    for impl in ("port", "reference"):
        s, e, EM = ref.moe_align_block_size(ids, 8, 16, impl=impl)
        assert EM == 0 and s.size == 0


@pytest.mark.parametrize("E,ep", [(8, 1), (8, 2), (8, 4), (7, 3), (256, 8), (129, 8)])
def test_ep_plan_and_dispatch(ref, E, ep):
    rng = np.random.default_rng(E * 7 + ep)
    ids = rng.integers(0, E, (40, 4), dtype=np.int32)
    covered = []
    for r in range(ep):
        assert ref.moe_ep_plan(E, ep, r, "port") == ref.moe_ep_plan(E, ep, r, "reference")
        b, e = ref.moe_ep_plan(E, ep, r)
        covered += list(range(b, e))
        pa = ref.moe_ep_dispatch(ids, E, 16, ep, r, "port")
        pb = ref.moe_ep_dispatch(ids, E, 16, ep, r, "reference")
        for x, y in zip(pa, pb):
            assert np.array_equal(x, y)
    assert covered == list(range(E))
    with pytest.raises(ValueError):
        ref.moe_ep_plan(4, 8, 0, "port")
    with pytest.raises(ValueError):
        ref.moe_ep_plan(4, 8, 0, "reference")


@pytest.mark.parametrize("ep", [1, 2, 4, 3])
def test_ep_forward_sums_to_single_rank(ref, ep):
    """Sum of the reference's per-rank outputs == single-rank oracle within 1e-3
    (test_dist_moe.cpp:516-555), and the restatement reproduces each rank bit for bit."""
    cfg, w, A, ids, tw = small_problem(11, E=7 if ep == 3 else 8)
    full = ref.moe_layer(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw, num_experts=cfg.E)
    outs = ref.fused_moe_mxfp4_ep_reference(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw,
                                            num_experts=cfg.E, ep=ep)
    assert np.max(np.abs(outs.sum(0) - full)) < 1e-3 * max(1.0, float(np.abs(full).max()))
    for r in range(ep):
        b, e = ref.moe_ep_plan(cfg.E, ep, r)
        s, x, EM = ref.moe_ep_dispatch(ids, cfg.E, 16, ep, r, "port")
        ws = ref.gather_sorted_weights(tw, s)
        o, _ = ref.fused_moe_mxfp4(A, w["w13"][b:e], w["w13_scale"][b:e], w["w2"][b:e], w["w2_scale"][b:e],
                                   s, ws, x, top_k=cfg.top_k, impl="port")
        assert np.array_equal(o.view(np.uint32), outs[r].view(np.uint32))


def test_token_subset_equals_full_run(ref):
    """A token's output depends only on its own row and experts: evaluating a subset of the
    tokens reproduces the full run's rows bit for bit (the basis of the sub-sampled parity
    checks at the large configurations)."""
    cfg, w, A, ids, tw = small_problem(21, T=48)
    full = ref.moe_layer(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw, num_experts=cfg.E)
    sub = np.array([3, 17, 18, 40])
    part = ref.moe_layer(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw, num_experts=cfg.E,
                         tokens=sub)
    assert np.array_equal(full[sub].view(np.uint32), part.view(np.uint32))


def test_round_bf16(ref):
    x = np.array([1.0, 1.00390625, -2.5, 3.1415927, 1e-40, np.inf], np.float32)
    assert np.array_equal(ref.round_bf16(x, "port"), ref.round_bf16(x, "reference"))
