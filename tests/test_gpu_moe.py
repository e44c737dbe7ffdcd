"""-m gpu: the fused layer through the C ABI against the CPU oracle.

Gate (the layer's stated tolerance): outputs rounded to bf16, max-abs <= 2e-2 and relative L2
<= 1e-2 against the oracle; NaN / inf masks must be equal. The CUDA-core cross-check path
("simt") adds in the oracle's order and is held to a much tighter bound."""
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from gpu_common import DEV, gpu_layer, make_case, oracle_layer, oracle_route, to_np  # noqa: E402
from helpers import (assert_close_bf16, bf2f, bf16_to_u16, expand_expert_ids, pack_pair, u16_to_bf16,  # noqa: E402
                     uniform_problem)
from vkernels_b200 import native_runtime as nr  # noqa: E402
from vkernels_b200 import synthetic as syn  # noqa: E402
from vkernels_b200 import torch_ops as ops  # noqa: E402
from vkernels_b200.experts import layer_from_config  # noqa: E402

IMPLS = ["simt", "tcgen05"]


def run_uniform(impl, prob, sorted_ids, ws, eids, top_k=1, out_init=0.0, **kw):
    """Known-answer problems take explicit sorted_ids / sorted weights: use the sorted-weight
    entry point, as the CPU entry point does."""
    A, w13, w13s, w2, w2s = prob
    M, H = A.shape
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    out = torch.full((M, H), out_init, dtype=torch.float32, device=DEV)
    act = torch.zeros((len(sorted_ids), w13.shape[1] // 2), dtype=torch.bfloat16, device=DEV)
    b13, b2 = kw.pop("b13", None), kw.pop("b2", None)
    ops.set_impl(impl)
    try:
        ops.fused_moe_mxfp4_into(out, act, u16_to_bf16(A, DEV), t(w13), t(w13s), t(w2), t(w2s),
                                 t(np.asarray(ws, np.float32)), t(np.asarray(sorted_ids, np.int32)),
                                 t(np.asarray(eids, np.int32)), top_k=top_k, weights_sorted=True,
                                 b13=None if b13 is None else t(b13), b2=None if b2 is None else t(b2), **kw)
        torch.cuda.synchronize()
        ops.kernel_status()
    finally:
        ops.set_impl("tcgen05")
    return to_np(out), bf16_to_u16(act)


IDENT = (np.arange(16), np.ones(16), np.zeros(1))


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_tiny_bias_clamp_situ(impl):
    """reference tests/kernels/moe/test_moe_fused.cpp:71-282."""
    out, act = run_uniform(impl, uniform_problem(), *IDENT)
    exp_act = 128.0 / (1.0 + math.exp(-128.0)) * 128.0
    assert np.max(np.abs(out - exp_act * 64) / (exp_act * 64)) < 1e-2 and np.max(np.abs(bf2f(act) - exp_act)) < 0.5
    b13 = np.concatenate([np.full(64, 1.0), np.full(64, 2.0)]).astype(np.float32)[None]
    out, act = run_uniform(impl, uniform_problem(a=0.0, w13_byte=0, w2_byte=0), *IDENT, b13=b13,
                           b2=np.ones((1, 128), np.float32))
    assert np.max(np.abs(bf2f(act) - 2.0 / (1.0 + math.exp(-1.0)))) < 1e-2 and np.max(np.abs(out - 1.0)) < 1e-4
    out, act = run_uniform(impl, uniform_problem(), *IDENT, swiglu_limit=10.0)
    e10 = 10.0 / (1.0 + math.exp(-10.0)) * 10.0
    assert np.max(np.abs(bf2f(act) - e10)) < 0.2 and np.max(np.abs(out - e10 * 64) / (e10 * 64)) < 1e-2
    out, act = run_uniform(impl, uniform_problem(), *IDENT, swiglu_limit=1.0, activation=1, beta=4.0, linear_beta=25.0)
    sig = 1.0 / (1.0 + math.exp(-128.0))
    es = (4.0 * math.tanh(32.0) * sig) * (25.0 * math.tanh(128.0 / 25.0))
    assert np.max(np.abs(bf2f(act) - es)) < 0.5 and np.max(np.abs(out - es * 64) / (es * 64)) < 1e-2
    _, act = run_uniform(impl, uniform_problem(), *IDENT, swiglu_limit=1.0, activation=1, beta=4.0, linear_beta=0.0)
    assert np.max(np.abs(bf2f(act) - 4.0 * math.tanh(32.0) * sig * 128.0)) < 0.5


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_decode_edges(impl):
    """+-0.25 codes, inf/NaN codes, the 2^-127 scale, padding rows, dead blocks
    (test_moe_fused.cpp:291-533)."""
    out, act = run_uniform(impl, uniform_problem(w13_byte=0x11, w2_byte=0x11), *IDENT)
    assert np.max(np.abs(bf2f(act) - 32.0 / (1.0 + math.exp(-32.0)) * 32.0)) < 0.5 and np.all(out > 0)
    out, act = run_uniform(impl, uniform_problem(w13_byte=0x76, w2_byte=0x22), *IDENT)
    assert np.all(np.isnan(bf2f(act))) and np.all(np.isnan(out))
    out, act = run_uniform(impl, uniform_problem(w13_byte=0x22, w2_byte=0x22, scale=0), *IDENT)
    assert np.max(np.abs(bf2f(act))) < 1e-30 and np.max(np.abs(out)) < 1e-30
    sid = np.full(16, 8)
    sid[:8] = np.arange(8)
    out, act = run_uniform(impl, uniform_problem(M=8), sid, np.ones(16), np.zeros(1))
    exp = 128.0 / (1.0 + math.exp(-128.0)) * 128.0 * 64
    assert np.max(np.abs(out - exp) / exp) < 1e-2 and np.all(act[8:] == 0)
    out, _ = run_uniform(impl, uniform_problem(), np.arange(16), np.ones(16), np.array([-1]), out_init=99.0)
    assert np.all(out == 99.0)


@pytest.mark.parametrize("impl", IMPLS)
def test_kat_k3_routing_top16(impl):
    """E = 256, top-16, one token: every 16-row block holds one real row (test_moe_fused.cpp:669-736)."""
    E, top_k, hidden, ispp = 256, 16, 128, 64
    prob = uniform_problem(M=1, hidden=hidden, ispp=ispp, E=E)
    s, e, EM = oracle.moe_align_block_size(np.arange(top_k, dtype=np.int32)[None], E, 16)
    out, act = run_uniform(impl, prob, s, oracle.gather_sorted_weights(np.ones(top_k, np.float32), s), e, top_k=top_k)
    exp_act = hidden / (1.0 + math.exp(-hidden)) * hidden
    real = s < top_k
    assert np.max(np.abs(bf2f(act[real]) - exp_act)) < 0.5 and np.all(act[~real] == 0)
    assert np.max(np.abs(out - top_k * exp_act * ispp) / (top_k * exp_act * ispp)) < 1e-2


def _parity(cfg, T, *, impl, codes="finite", block_size=16, tokens=None, seed=None, logits=None, backend="numpy"):
    w, A, r = make_case(cfg, T, codes=codes, seed=seed, backend=backend)
    ids_np, tw_np, _ = oracle_route(cfg, A, r, logits=None if logits is None else to_np(logits))
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    got = to_np(gpu_layer(A, w, ids, tw, impl=impl, block_size=block_size, swiglu_limit=cfg.swiglu_limit))
    ref = oracle_layer(A, w, ids, tw, tokens=tokens, swiglu_limit=cfg.swiglu_limit)
    if tokens is not None:
        got = got[tokens]
    return assert_close_bf16(got, ref, f"{cfg.name} T={T} {impl}")


@pytest.mark.parametrize("impl", IMPLS)
def test_c0_smoke_matches_oracle_and_golden(impl):
    cfg = syn.CONFIGS["c0"]
    _parity(cfg, 64, impl=impl)
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "c0_smoke.npz"))
    w, A, _ = make_case(cfg, 64)
    got = to_np(gpu_layer(A, w, torch.from_numpy(g["topk_ids"]).to(DEV), torch.from_numpy(g["topk_w"]).to(DEV), impl=impl))
    assert_close_bf16(got, g["out"], "c0 vs golden (reference output)")


@pytest.mark.parametrize("impl", IMPLS)
def test_c0_all_sixteen_codes_nan_mask(impl):
    """With all 16 nibble codes a quarter of the weights are +-inf / NaN: the NaN mask of the
    output must equal the oracle's (here: everything)."""
    _parity(syn.CONFIGS["c0"], 64, impl=impl, codes="all")


@pytest.mark.parametrize("T", [1, 8, 32, 64, 128])
def test_c1_decode_sweep(T):
    _parity(syn.CONFIGS["c1"], T, impl="tcgen05")


def test_c1_golden_shape():
    cfg = syn.scaled(syn.CONFIGS["c1"], E=4, top_k=2)
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "c1_shape_T8_E4.npz"))
    w, A, _ = make_case(cfg, 8)
    for impl in IMPLS:
        got = to_np(gpu_layer(A, w, torch.from_numpy(g["topk_ids"]).to(DEV), torch.from_numpy(g["topk_w"]).to(DEV),
                              impl=impl, swiglu_limit=cfg.swiglu_limit))
        assert_close_bf16(got, g["out"], f"c1-shape golden {impl}")


@pytest.mark.parametrize("block_size", [16, 64, 128])
def test_block_sizes_and_bias(block_size):
    cfg = syn.scaled(syn.CONFIGS["c0"], H=384, I=192, E=6, top_k=3)
    w, A, r = make_case(cfg, 100)
    ids_np, tw_np, _ = oracle_route(cfg, A, r)
    rng = np.random.default_rng(1)
    b13 = rng.standard_normal((cfg.E, 2 * cfg.I)).astype(np.float32)
    b2 = rng.standard_normal((cfg.E, cfg.H)).astype(np.float32)
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    for impl in IMPLS:
        for act_kw in (dict(swiglu_limit=0.7), dict(activation=1, beta=4.0, linear_beta=25.0)):
            got = to_np(gpu_layer(A, w, ids, tw, impl=impl, block_size=block_size, b13=torch.from_numpy(b13).to(DEV),
                                  b2=torch.from_numpy(b2).to(DEV), **act_kw))
            ref = oracle_layer(A, w, ids, tw, b13=b13, b2=b2, **act_kw)
            assert_close_bf16(got, ref, f"block {block_size} {impl} {act_kw}")


def test_simt_accumulators_follow_the_oracle_order():
    """The cross-check kernels add in the oracle's order: their act differs from the oracle's
    only through the device expf, a few bf16 ulps on a handful of elements."""
    cfg = syn.CONFIGS["c0"]
    w, A, r = make_case(cfg, 64)
    ids_np, tw_np, _ = oracle_route(cfg, A, r)
    out, act, sids, eids, _ = gpu_layer(A, w, torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV),
                                        impl="simt", return_parts=True)
    s, e, EM = oracle.moe_align_block_size(ids_np, cfg.E, 16)
    wn = {k: to_np(v) for k, v in w.items()}
    st = oracle.moe_stages(bf16_to_u16(A), wn["w13"], wn["w13_scale"], wn["w2"], wn["w2_scale"], s,
                           oracle.gather_sorted_weights(tw_np, s), e, top_k=cfg.top_k)
    real = s < ids_np.size
    ga, ra = bf16_to_u16(act)[:EM][real].astype(np.int32), st["act"][real].astype(np.int32)
    assert (ga != ra).mean() < 0.01 and np.abs(ga - ra).max() <= 2
    assert np.max(np.abs(to_np(out) - st["out"])) < 1e-4 * max(1.0, np.abs(st["out"]).max())


@pytest.mark.parametrize("name,T,n_sub", [("c2", 8192, 192), ("c4", 4096, 128)])
def test_prefill_shapes_on_a_token_subsample(name, T, n_sub):
    """Full-size GPU run; the oracle evaluates a seeded subsample of the tokens, which equals
    the full oracle run on those tokens (every row is independent)."""
    cfg = syn.CONFIGS[name]
    rng = np.random.default_rng(T)
    tokens = np.sort(rng.choice(T, n_sub, replace=False))
    logits = syn.make_zipf_logits(cfg, T, device=DEV) if cfg.zipf_alpha else None
    _parity(cfg, T, impl="tcgen05", tokens=tokens, logits=logits, backend="torch")


@pytest.mark.parametrize("n_hot", [129, 256, 257, 272, 300, 320, 321, 400, 641])
def test_token_tile_edges_of_the_cta_pair_form(n_hot):
    """One expert receives exactly n_hot tokens: the sizes around the 256-token main accumulator,
    the 64-token extension (257..320), the split into two items (321+), and a tile just over the
    lone-CTA limit (129). Every token also visits a second, lightly loaded expert."""
    cfg = syn.scaled(syn.CONFIGS["c0"], H=512, I=256, E=8, top_k=2)
    T = max(n_hot + 37, 330)   # more than 256 tokens, so the CTA-pair form is selected
    w, A, _ = make_case(cfg, T)
    rng = np.random.default_rng(n_hot)
    ids = np.empty((T, 2), np.int32)
    hot = np.zeros(T, bool)
    hot[rng.choice(T, n_hot, replace=False)] = True
    ids[:, 0] = np.where(hot, 3, rng.integers(4, 8, T))
    ids[:, 1] = rng.integers(0, 3, T)
    tw = rng.random((T, 2), dtype=np.float32)
    idt, twt = torch.from_numpy(ids).to(DEV), torch.from_numpy(tw).to(DEV)
    got = to_np(gpu_layer(A, w, idt, twt, impl="tcgen05"))
    ref = oracle_layer(A, w, idt, twt)
    assert_close_bf16(got, ref, f"{n_hot} tokens on one expert")


def test_status_word_survives_the_alignment_scratch():
    """The chunked alignment (more than 1024 routed slots) keeps its histograms in the library
    workspace, whose first 4 KB also hold the GEMM kernels' status word. With 16 local experts
    the second chunk's first counter used to land exactly on that word and made a healthy run
    look like a timed-out one."""
    cfg = syn.scaled(syn.CONFIGS["c0"], H=512, I=256, E=16, top_k=4)
    T = 1536
    w, A, _ = make_case(cfg, T)
    rng = np.random.default_rng(16)
    ids = np.stack([rng.permutation(cfg.E)[: cfg.top_k] for _ in range(T)]).astype(np.int32)
    tw = rng.random((T, cfg.top_k), dtype=np.float32)
    tokens = np.sort(rng.choice(T, 48, replace=False))
    idt, twt = torch.from_numpy(ids).to(DEV), torch.from_numpy(tw).to(DEV)
    got = to_np(gpu_layer(A, w, idt, twt, impl="tcgen05"))   # gpu_layer checks the status word
    ref = oracle_layer(A, w, idt, twt, tokens=tokens)
    assert_close_bf16(got[tokens], ref, "16 experts, 6144 routed slots")


def test_c3_shape_with_shared_expert_on_a_token_subsample():
    """The DeepSeek-V3-shaped configuration at its stated batch (T = 16384, 256 routed experts
    plus the always-on shared one, full-size weights); the oracle evaluates 64 seeded tokens."""
    cfg = syn.CONFIGS["c3"]
    T = 16384
    rng = np.random.default_rng(3)
    tokens = np.sort(rng.choice(T, 64, replace=False))
    _parity(cfg, T, impl="tcgen05", tokens=tokens, backend="torch")


@pytest.mark.parametrize("T", [1, 16, 256])
def test_c4_zipf_small_batches(T):
    """The load-imbalance configuration at its small batch sizes (Zipf 1.2 expert popularity):
    a few hot experts collect most tokens while the launch is still in the small-tile regime,
    the sizes at which the tile cap and the form choice flip."""
    cfg = syn.CONFIGS["c4"]
    logits = syn.make_zipf_logits(cfg, T, device=DEV)
    tokens = None if T <= 64 else np.sort(np.random.default_rng(T).choice(T, 64, replace=False))
    _parity(cfg, T, impl="tcgen05", tokens=tokens, logits=logits, backend="torch")


def test_full_size_properties_c2():
    """Size-independent checks at the full prefill size: (1) doubling every routing weight doubles
    the output (the combine is linear in the weights), (2) the tensor-core path and the
    oracle-ordered CUDA-core path agree on every token, (3) permuting the tokens permutes the
    output rows."""
    cfg = syn.CONFIGS["c2"]
    T = 8192
    w, A, r = make_case(cfg, T, backend="torch")
    lg = ops.router_logits(A, r["wr"])
    ids, tw = ops.route_topk(lg, cfg.top_k)
    ids, tw = ids.clone(), tw.clone()
    base = gpu_layer(A, w, ids, tw, impl="tcgen05")
    twice = gpu_layer(A, w, ids, tw * 2.0, impl="tcgen05")
    assert_close_bf16(to_np(twice), 2.0 * to_np(base), "linearity in the routing weights")
    simt = gpu_layer(A, w, ids, tw, impl="simt")
    assert_close_bf16(to_np(base), to_np(simt), "tcgen05 vs oracle-ordered CUDA cores, all 8192 tokens")
    perm = torch.randperm(T, device=DEV)
    moved = gpu_layer(A[perm].contiguous(), w, ids[perm].contiguous(), tw[perm].contiguous(), impl="tcgen05")
    assert_close_bf16(to_np(moved), to_np(base[perm]), "token permutation")


@pytest.mark.parametrize("name,T", [("c0", 64), ("c1", 8), ("c1", 128), ("c4", 256), ("c2", 1024)])
def test_bf16_form_with_ordered_combine(name, T):
    """vk_cuda_fused_moe_mxfp4_bf16: result within the layer's tolerance of the oracle, equal
    (to bf16 rounding) to the atomic form, bit-identical from run to run, and with biases."""
    cfg = syn.CONFIGS[name]
    w, A, r = make_case(cfg, T, backend="torch")
    logits = syn.make_zipf_logits(cfg, T, device=DEV) if cfg.zipf_alpha else None
    ids_np, tw_np, _ = oracle_route(cfg, A, r, logits=None if logits is None else to_np(logits))
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    E = w["w13"].shape[0]
    rng = np.random.default_rng(T)
    b13 = torch.from_numpy(rng.standard_normal((E, 2 * cfg.I)).astype(np.float32) * 0.1).to(DEV)
    b2 = torch.from_numpy(rng.standard_normal((E, cfg.H)).astype(np.float32) * 0.1).to(DEV)
    sids, eids, _ = ops.moe_align_block_size(ids, E, 16)
    act = torch.zeros((sids.numel(), cfg.I), dtype=torch.bfloat16, device=DEV)
    ys = []
    for _ in range(2):
        y = torch.full((T, cfg.H), 7.0, dtype=torch.bfloat16, device=DEV)    # must be overwritten, not added to
        ops.fused_moe_mxfp4_bf16_into(y, act, A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], tw.reshape(-1).contiguous(),
                                      sids, eids, top_k=ids.shape[1], swiglu_limit=cfg.swiglu_limit, b13=b13, b2=b2)
        torch.cuda.synchronize()
        ops.kernel_status()
        ys.append(y.clone())
    assert torch.equal(ys[0], ys[1]), "the ordered combine must be bit-reproducible"
    tokens = None if T <= 64 else np.sort(rng.choice(T, 48, replace=False))
    ref = oracle_layer(A, w, ids, tw, tokens=tokens, swiglu_limit=cfg.swiglu_limit, b13=to_np(b13), b2=to_np(b2))
    got = to_np(ys[0].float())
    assert_close_bf16(got if tokens is None else got[tokens], ref, f"bf16 form {name} T={T}", got_is_bf16=True)


@pytest.mark.parametrize("name,T", [("c0", 1), ("c0", 6), ("c1", 1), ("c1", 2), ("c1", 3), ("c3_small", 1), ("c4", 2)])
def test_flat_form_for_a_handful_of_slots(name, T):
    """Up to twelve routed slots the bf16 entry point runs two flat kernels (moe_gemv.cu) instead
    of the grouped GEMMs: against the oracle, against the fp32 form, bit-reproducible, with
    biases, with a slot whose expert is not local (id -1) and with a 0xFF scale group."""
    # c3_small: the sigmoid / group-limited router with its always-on shared expert (8 + 1 slots), at a size the oracle likes
    cfg = syn.scaled(syn.CONFIGS["c3"], H=1024, I=512, E=32) if name == "c3_small" else syn.CONFIGS[name]
    w, A, r = make_case(cfg, T, backend="torch")
    w["w13_scale"][0, 3, 1] = 0xFF
    logits = syn.make_zipf_logits(cfg, T, device=DEV) if cfg.zipf_alpha else None
    ids_np, tw_np, _ = oracle_route(cfg, A, r, logits=None if logits is None else to_np(logits))
    assert ids_np.size <= 12
    if name == "c1" and T == 3:
        ids_np = ids_np.copy()
        ids_np[1, 2] = -1                       # a slot some other rank owns
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    E = w["w13"].shape[0]
    rng = np.random.default_rng(T + 11)
    b13 = torch.from_numpy(rng.standard_normal((E, 2 * cfg.I)).astype(np.float32) * 0.1).to(DEV)
    b2 = torch.from_numpy(rng.standard_normal((E, cfg.H)).astype(np.float32) * 0.1).to(DEV)
    sids, eids, _ = ops.moe_align_block_size(ids, E, 16)
    act = torch.zeros((sids.numel(), cfg.I), dtype=torch.bfloat16, device=DEV)
    kw = dict(top_k=ids.shape[1], swiglu_limit=cfg.swiglu_limit, b13=b13, b2=b2)
    ys = []
    for _ in range(2):
        y = torch.full((T, cfg.H), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.fused_moe_mxfp4_bf16_into(y, act, A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], tw.reshape(-1).contiguous(),
                                      sids, eids, **kw)
        torch.cuda.synchronize()
        ys.append(y.clone())
    assert torch.equal(ys[0], ys[1])
    ref = oracle_layer(A, w, ids, tw, swiglu_limit=cfg.swiglu_limit, b13=to_np(b13), b2=to_np(b2))
    assert_close_bf16(to_np(ys[0].float()), ref, f"flat form {name} T={T}", got_is_bf16=True)
    base = gpu_layer(A, w, ids, tw, impl="tcgen05", swiglu_limit=cfg.swiglu_limit, b13=b13, b2=b2)
    assert_close_bf16(to_np(ys[0].float()), to_np(base), f"flat form vs fp32 form {name} T={T}", got_is_bf16=True)


def _ocp_decode(codes_u8, K):
    """Prepacked code bytes [rows, K/2] -> values as the tensor core reads e2m1, halved."""
    ocp = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    lo, hi = codes_u8 & 15, codes_u8 >> 4
    nib = np.stack([lo, hi], axis=-1).reshape(codes_u8.shape[0], K)
    return np.where(nib & 8, -1.0, 1.0).astype(np.float32) * ocp[nib & 7] * 0.5


def test_prepack_rewrites_codes_and_scales_exactly():
    """The prepacked codes, read with the e2m1 table and halved, are the layer's table values;
    0xFF groups become zeros with scale 1; the regrouped scales sit where the kernel reads
    them; inf / NaN codes are counted."""
    cfg = syn.scaled(syn.CONFIGS["c1"], H=320, I=192, E=3)      # K = 320: one and a quarter stages; down tiles 128 + 128 + 64 rows
    w = syn.make_expert_weights(cfg, device=DEV)
    w13s = w["w13_scale"].clone()
    w13s[1, 5, 3] = 0xFF
    w13s[2, 100, 0] = 0xFF
    pk = ops.prepack_weights(w["w13"], w13s, w["w2"], w["w2_scale"])
    assert pk.usable and pk.nonfinite == 0
    table = np.array([0, .25, 1, 1.5, 2, 3], np.float32)
    for which, (wt, sc, codes, sf, K, n_feat) in enumerate([
            (w["w13"], w13s, pk.w13_codes, pk.w13_sf, cfg.H, cfg.I), (w["w2"], w["w2_scale"], pk.w2_codes, pk.w2_sf, cfg.I, cfg.H)]):
        raw = to_np(wt).reshape(-1, K // 2)
        scn = to_np(sc).reshape(-1, K // 32)
        rows = raw.shape[0]
        got = _ocp_decode(to_np(codes)[: rows * (K // 2)].reshape(rows, K // 2), K)
        nib = np.stack([raw & 15, raw >> 4], axis=-1).reshape(rows, K)
        want = np.where(nib & 8, -1.0, 1.0).astype(np.float32) * table[nib & 7]
        want = want * (np.repeat(scn, 32, axis=1) != 0xFF)
        assert np.array_equal(got, want), which
        assert not to_np(codes)[rows * (K // 2):].any(), "padding must be zero"
        # scales: [E][tile][stage][128 accumulator rows][8 groups]
        n_ft = n_feat // 64 if which == 0 else (n_feat + 127) // 128
        n_kw = (K + 255) // 256
        sft = to_np(sf).reshape(cfg.E, n_ft, n_kw, 128, 8)
        rows_e = rows // cfg.E
        for e, f, L in [(0, 0, 0), (1, 0, 13), (2, n_ft - 1, 127), (1, 1, 72), (2, 1, 36)]:
            if which == 0:
                sr = ((L >> 3) & 1) * 64 + (L >> 4) * 8 + (L & 7)
                row = f * 64 + sr if sr < 64 else n_feat + f * 64 + sr - 64
            else:
                row = f * 128 + L if f * 128 + L < n_feat else -1
            for kw in range(n_kw):
                for b in range(8):
                    kb = kw * 8 + b
                    want_b = 0x7F
                    if row >= 0 and kb < K // 32:
                        want_b = int(scn[e * rows_e + row, kb])
                        want_b = 0x7F if want_b == 0xFF else want_b
                    assert int(sft[e, f, kw, L, b]) == want_b, (which, e, f, L, kw, b)
    bad = syn.make_expert_weights(cfg, codes="all", device=DEV)
    assert not ops.prepack_weights(bad["w13"], bad["w13_scale"], bad["w2"], bad["w2_scale"]).usable


@pytest.mark.parametrize("name,T", [("c0", 64), ("c1", 1), ("c1", 8), ("c1", 64), ("c1", 128), ("c4", 16), ("c4", 256)])
def test_prepacked_decode_form(name, T):
    """vk_cuda_fused_moe_mxfp4_bf16_prepacked: within the layer's tolerance of the oracle, within
    bf16 rounding of the checkpoint-layout form, bit-identical from run to run, with biases and
    with a 0xFF (zero) scale group in the weights."""
    cfg = syn.CONFIGS[name]
    w, A, r = make_case(cfg, T, backend="torch")
    w["w13_scale"][0, 3, 1] = 0xFF
    w["w2_scale"][1 % w["w2"].shape[0], 7, 0] = 0xFF
    logits = syn.make_zipf_logits(cfg, T, device=DEV) if cfg.zipf_alpha else None
    ids_np, tw_np, _ = oracle_route(cfg, A, r, logits=None if logits is None else to_np(logits))
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    E = w["w13"].shape[0]
    rng = np.random.default_rng(T + 5)
    b13 = torch.from_numpy(rng.standard_normal((E, 2 * cfg.I)).astype(np.float32) * 0.1).to(DEV)
    b2 = torch.from_numpy(rng.standard_normal((E, cfg.H)).astype(np.float32) * 0.1).to(DEV)
    pk = ops.prepack_weights(w["w13"], w["w13_scale"], w["w2"], w["w2_scale"])
    assert pk.usable
    sids, eids, _ = ops.moe_align_block_size(ids, E, 16)
    act = torch.zeros((sids.numel(), cfg.I), dtype=torch.bfloat16, device=DEV)
    kw = dict(top_k=ids.shape[1], swiglu_limit=cfg.swiglu_limit, b13=b13, b2=b2)
    ys = []
    for _ in range(2):
        y = torch.full((T, cfg.H), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.fused_moe_mxfp4_bf16_prepacked_into(y, act, A, pk, tw.reshape(-1).contiguous(), sids, eids, **kw)
        torch.cuda.synchronize()
        ops.kernel_status()
        ys.append(y.clone())
    assert torch.equal(ys[0], ys[1]), "the prepacked form must be bit-reproducible"
    base = torch.empty((T, cfg.H), dtype=torch.bfloat16, device=DEV)
    ops.fused_moe_mxfp4_bf16_into(base, act, A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], tw.reshape(-1).contiguous(),
                                  sids, eids, **kw)
    assert_close_bf16(to_np(ys[0].float()), to_np(base.float()), f"prepacked vs checkpoint layout {name} T={T}", got_is_bf16=True)
    tokens = None if T <= 64 else np.sort(rng.choice(T, 48, replace=False))
    ref = oracle_layer(A, w, ids, tw, tokens=tokens, swiglu_limit=cfg.swiglu_limit, b13=to_np(b13), b2=to_np(b2))
    got = to_np(ys[0].float())
    assert_close_bf16(got if tokens is None else got[tokens], ref, f"prepacked form {name} T={T}", got_is_bf16=True)


def test_prepacked_form_refuses_prefill_batches():
    cfg = syn.scaled(syn.CONFIGS["c1"], H=256, I=128, E=2, top_k=1)
    T = 2048                                       # 1024 rows per expert: far beyond a 64-row tile
    w, A, r = make_case(cfg, T, backend="torch")
    ids_np, tw_np, _ = oracle_route(cfg, A, r)
    ids, tw = torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)
    pk = ops.prepack_weights(w["w13"], w["w13_scale"], w["w2"], w["w2_scale"])
    sids, eids, _ = ops.moe_align_block_size(ids, cfg.E, 16)
    act = torch.zeros((sids.numel(), cfg.I), dtype=torch.bfloat16, device=DEV)
    y = torch.zeros((T, cfg.H), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="decode-size"):
        ops.fused_moe_mxfp4_bf16_prepacked_into(y, act, A, pk, tw.reshape(-1).contiguous(), sids, eids, top_k=1)


def test_host_pointer_abi():
    """vk_fused_moe_mxfp4 with HOST buffers (the CPU entry point's signature): copies in,
    kernels, copies out; accumulates into `out` like the reference."""
    cfg = syn.scaled(syn.CONFIGS["c0"], H=256, I=128, E=4, top_k=2)
    w = {k: v.numpy() for k, v in syn.make_expert_weights(cfg).items()}
    A = bf16_to_u16(syn.make_activations(cfg, 20))
    r = syn.make_router(cfg)
    ids, tw, _ = oracle.route_softmax_topk(oracle.router_logits(A, r["wr"].numpy()), cfg.top_k)
    s, e, EM = oracle.moe_align_block_size(ids, cfg.E, 16)
    ws = oracle.gather_sorted_weights(tw, s)
    ref, _ = oracle.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e, top_k=cfg.top_k)
    out = np.full((20, cfg.H), 1.0, np.float32)
    act = np.zeros((EM, cfg.I), np.uint16)
    p = lambda a: a.ctypes.data
    rc = nr.load_library().vk_fused_moe_mxfp4(p(A), p(w["w13"]), p(w["w13_scale"]), p(w["w2"]), p(w["w2_scale"]), p(s),
                                              p(ws), p(e), p(act), p(out), 20, cfg.H, cfg.I, cfg.top_k, EM, 32, 0.0, 0,
                                              4.0, 25.0, None, None)
    assert rc == 0, nr.last_error()
    assert_close_bf16(out - 1.0, ref, "host-pointer ABI")


def test_layer_object_end_to_end():
    """route -> align -> experts through the layer object, device and pinned-host entry."""
    cfg = syn.CONFIGS["c0"]
    w, A, r = make_case(cfg, 64)
    layer = layer_from_config(cfg, w, r, max_tokens=128)
    y = layer(A)
    ids_np, tw_np, margin = oracle_route(cfg, A, r)
    ref = oracle_layer(A, w, torch.from_numpy(ids_np), torch.from_numpy(tw_np))
    ok = margin > 2e-5
    assert_close_bf16(to_np(y.float())[ok], ref[ok], "layer object", got_is_bf16=True)
    xh = A.cpu().pin_memory()
    yh = torch.empty((64, cfg.H), dtype=torch.bfloat16).pin_memory()
    layer.forward_host(xh, yh)
    assert_close_bf16(yh.float().numpy()[ok], ref[ok], "layer object, pinned host entry", got_is_bf16=True)
