"""-m gpu: dequantisation, alignment and routing kernels against the CPU oracle, bit-exact
(integer / index work) through the C ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from gpu_common import DEV, to_np  # noqa: E402
from helpers import bf16_to_u16, numpy_align  # noqa: E402
from vkernels_b200 import native_runtime as nr  # noqa: E402
from vkernels_b200 import synthetic as syn  # noqa: E402
from vkernels_b200 import torch_ops as ops  # noqa: E402


@pytest.mark.parametrize("path", ["permute", "table"])
def test_dequant_all_bytes_all_scales_bit_exact(path):
    """Every (packed byte, scale byte) pair, through both decoders the GEMM kernels use (byte
    permutes in the CTA-pair form, the shared-memory table in the lone-CTA form): equal to the CPU
    definition bit for bit on finite values, same NaN positions
    (reference tests/kernels/moe/test_moe_fused.cpp:591-621)."""
    rows, K = 256, 512
    packed = (torch.arange(rows * K // 2, device=DEV) & 0xFF).to(torch.uint8).view(rows, K // 2)
    # row r uses scale byte r; every row contains every byte value
    scale = torch.arange(256, device=DEV, dtype=torch.uint8).view(rows, 1).expand(rows, K // 32).contiguous()
    got = bf16_to_u16(ops.mxfp4_dequant_rows(packed, scale, path=path))
    ref = np.empty((rows, K), np.uint16)
    pk, sc = to_np(packed), to_np(scale)
    for r in range(rows):
        ref[r] = oracle.dequant_weight_tile(pk[r:r + 1], sc[r:r + 1], 1, K)[:, 0]
    nan_g, nan_r = np.isnan(oracle.bf16_to_f32(got)), np.isnan(oracle.bf16_to_f32(ref))
    assert np.array_equal(nan_g, nan_r)
    assert np.array_equal(got[~nan_r], ref[~nan_r])


@pytest.mark.parametrize("path", ["permute", "table"])
def test_dequant_random_rows(path):
    g = torch.Generator(device=DEV).manual_seed(3)
    packed = torch.randint(0, 256, (64, 1440), generator=g, device=DEV, dtype=torch.uint8)
    scale = torch.randint(0, 256, (64, 90), generator=g, device=DEV, dtype=torch.uint8)
    got = bf16_to_u16(ops.mxfp4_dequant_rows(packed, scale, path=path))
    ref = oracle.dequant_weight_tile(to_np(packed), to_np(scale), 64, 2880).T
    nan_r = np.isnan(oracle.bf16_to_f32(ref))
    assert np.array_equal(np.isnan(oracle.bf16_to_f32(got)), nan_r)
    assert np.array_equal(got[~nan_r], ref[~nan_r])


ALIGN_CASES = [
    # M, k, E, block, kind
    (1, 4, 32, 16, "random"), (8, 4, 4, 16, "random"), (128, 4, 32, 16, "random"),
    (256, 4, 128, 64, "random"), (200, 8, 256, 128, "random"), (1024, 1, 8, 16, "random"),
    (257, 4, 128, 16, "random"),                      # first size past one chunk
    (8192, 4, 128, 16, "random"), (8192, 4, 128, 64, "zipf"),
    (16384, 9, 257, 16, "random"),                    # the largest configuration, shared slot included
    (4096, 4, 128, 16, "one_expert"), (64, 4, 256, 16, "distinct"), (300, 2, 16, 16, "garbage"),
]


@pytest.mark.parametrize("M,k,E,bs,kind", ALIGN_CASES)
def test_align_bit_exact(M, k, E, bs, kind):
    rng = np.random.default_rng(M * 7 + k + E)
    if kind == "zipf":
        p = 1.0 / (1 + np.arange(E)) ** 1.2
        ids = rng.choice(E, (M, k), p=p / p.sum())
    elif kind == "one_expert":
        ids = np.full((M, k), 5)
    elif kind == "distinct":
        ids = np.arange(M * k).reshape(M, k) % E
    else:
        ids = rng.integers(0, E, (M, k))
    ids = ids.astype(np.int32)
    if kind == "garbage":
        ids[rng.random((M, k)) < 0.2] = -1
        ids[rng.random((M, k)) < 0.1] = E + 3
    max_EM = ops.align_em_bound(M, k, E, bs)
    s, e, em = ops.moe_align_block_size(torch.from_numpy(ids).to(DEV), E, bs)
    torch.cuda.synchronize()
    rs, re, rEM = oracle.moe_align_block_size_map(ids, None, E, E, bs, max_EM)
    assert int(em.item()) == rEM
    assert np.array_equal(to_np(s), rs) and np.array_equal(to_np(e), re)
    # and the host contract of the reference's own align on the real part
    hs, he, hEM = oracle.moe_align_block_size(ids, E, bs)
    assert hEM == rEM and np.array_equal(rs[:hEM], hs) and np.array_equal(re[: hEM // bs], he)


def test_align_expert_map_and_empty():
    """No map, 1:1 map, a shard map with skipped experts, nothing routed, M = 0
    (the matrix of reference meta/benchmarks/test_capi_moe_align.hip:251-309)."""
    rng = np.random.default_rng(9)
    E, bs = 32, 16
    ids = rng.integers(0, E, (50, 4)).astype(np.int32)
    t = torch.from_numpy(ids).to(DEV)
    for emap, local_n in [(np.arange(E), E), (np.where(np.arange(E) // 8 == 2, np.arange(E) - 16, -1), 8),
                          (np.full(E, -1), 8)]:
        emap = emap.astype(np.int32)
        max_EM = ops.align_em_bound(50, 4, local_n, bs)
        s, e, em = ops.moe_align_block_size(t, E, bs, expert_map=torch.from_numpy(emap).to(DEV),
                                            local_n=local_n, max_EM=max_EM)
        rs, re, rEM = oracle.moe_align_block_size_map(ids, emap, E, local_n, bs, max_EM)
        assert int(em.item()) == rEM and np.array_equal(to_np(s), rs) and np.array_equal(to_np(e), re)
    empty = torch.zeros((0, 4), dtype=torch.int32, device=DEV)
    s, e, em = ops.moe_align_block_size(empty, E, bs)
    assert int(em.item()) == bs and s.numel() == bs and int(e[0].item()) == -1


def test_align_host_abi():
    """vk_moe_align_block_size with HOST buffers: GPU execution, host contract."""
    lib = nr.load_library()
    ids = np.array([[0] * 4, [0, 1, 1, 1], [1] * 4, [1] * 4, [2] * 4, [2] * 4, [2] * 4, [2] * 4], np.int32)
    cap = lib.vk_moe_align_block_size_max_em(8, 4, 16, 4)
    s = np.full(cap, -9, np.int32)
    e = np.full(cap // 16, -9, np.int32)
    em = np.zeros(1, np.int32)
    assert lib.vk_moe_align_block_size(ids.ctypes.data, 8, 4, 16, 4, s.ctypes.data, e.ctypes.data, em.ctypes.data) == 0
    rs, re, rEM = oracle.moe_align_block_size(ids, 4, 16)
    assert em[0] == rEM == 48 and np.array_equal(s[:48], rs) and np.array_equal(e[:3], re)
    bad = np.full((4, 2), -1, np.int32)
    assert lib.vk_moe_align_block_size(bad.ctypes.data, 4, 2, 16, 4, s.ctypes.data, e.ctypes.data, em.ctypes.data) == 0
    assert em[0] == 0


def _check_route(cfg, T, logits=None, seed=None):
    from gpu_common import make_case, oracle_route
    r = syn.make_router(cfg, seed=seed, device=DEV)
    A = syn.make_activations(cfg, T, seed=seed, device=DEV)
    if logits is None:
        lg = ops.router_logits(A, r["wr"])
        ref_logits = oracle.router_logits(bf16_to_u16(A), to_np(r["wr"]))
        # Both sides round an fp32 sum of H exact products, in different orders (the oracle adds
        # sequentially, the device adds tensor-core partial sums of 64 products). The yardstick is
        # the oracle's own rounding noise against the float64 dot: the device must be at least
        # as close to the exact value, and the two may differ by no more than twice that noise.
        exact = A.float().cpu().numpy().astype(np.float64) @ to_np(r["wr"]).astype(np.float64).T
        noise = float(np.abs(ref_logits - exact).max())
        assert float(np.abs(to_np(lg) - exact).max()) <= noise + 2e-6
        assert float(np.abs(to_np(lg) - ref_logits).max()) <= 2 * noise + 2e-6
    else:
        lg = logits
        ref_logits = to_np(logits)
        noise = 0.0
    ids, w = ops.route_topk(lg, cfg.top_k, bias=r["bias"], sigmoid=cfg.routing == "sigmoid_group",
                            n_group=cfg.n_group, topk_group=cfg.topk_group, renorm=cfg.renorm,
                            scaling=cfg.scaling, n_shared=cfg.shared_experts)
    rid, rw, margin = oracle_route(cfg, A, r, logits=ref_logits)
    # tokens whose every pick is decided by more than fp32 reassociation noise (the device sums
    # the logits and the softmax denominator in another order; observed differences are ~1e-6)
    # scores move by at most a quarter of a logit change (softmax and sigmoid slopes), the two
    # logit sets differ by at most 2 * noise, so a margin above `noise` cannot flip a pick
    ok = margin > max(2e-5, noise)
    assert ok.mean() > 0.9, f"only {ok.mean():.3f} of the tokens are well separated"
    assert np.array_equal(to_np(ids)[ok], rid[ok]), "routing indices differ"
    assert np.allclose(to_np(w)[ok], rw[ok], rtol=1e-4, atol=1e-6)
    return int((~ok).sum())


@pytest.mark.parametrize("name,T", [("c0", 64), ("c1", 128), ("c2", 1024), ("c3", 1024)])
def test_routing_indices_bit_exact(name, T):
    _check_route(syn.CONFIGS[name], T)


@pytest.mark.parametrize("T,E,H", [(513, 128, 2880), (1000, 48, 512), (640, 256, 1024), (8192, 128, 2880), (700, 16, 64)])
def test_router_logits_tensor_core_kernel(T, E, H):
    """Prefill-size router logits (tcgen05; token counts that are no multiple of its 128-token
    tile, expert counts from one MMA-N granule to the largest tile, one to eight K slices): at
    least as close to the float64 dot products as the oracle's sequential fp32 sums, and equal
    from run to run."""
    cfg = syn.scaled(syn.CONFIGS["c2"], H=H, E=E)
    r = syn.make_router(cfg, device=DEV)
    A = syn.make_activations(cfg, T, device=DEV)
    lg = ops.router_logits(A, r["wr"])
    lg2 = ops.router_logits(A, r["wr"])
    torch.cuda.synchronize()
    ops.kernel_status()
    assert torch.equal(lg, lg2)
    exact = A.float().cpu().numpy().astype(np.float64) @ to_np(r["wr"]).astype(np.float64).T
    ref = oracle.router_logits(bf16_to_u16(A), to_np(r["wr"]))
    noise = float(np.abs(ref - exact).max())
    assert float(np.abs(to_np(lg) - exact).max()) <= noise + 2e-6


def test_routing_zipf_logits():
    cfg = syn.CONFIGS["c4"]
    _check_route(cfg, 4096, logits=syn.make_zipf_logits(cfg, 4096, device=DEV))


@pytest.mark.parametrize("name,T", [("c0", 64), ("c1", 1), ("c1", 128), ("c3", 100), ("c4", 16)])
def test_fused_route_align_equals_the_two_kernels(name, T):
    """The single-CTA small-batch kernel (router top-k + alignment) produces, bit for bit, what
    route_topk followed by moe_align_block_size produce."""
    cfg = syn.CONFIGS[name]
    r = syn.make_router(cfg, device=DEV)
    A = syn.make_activations(cfg, T, device=DEV)
    lg = syn.make_zipf_logits(cfg, T, device=DEV) if cfg.zipf_alpha else ops.router_logits(A, r["wr"])
    kw = dict(bias=r["bias"], sigmoid=cfg.routing == "sigmoid_group", n_group=cfg.n_group, topk_group=cfg.topk_group,
              renorm=cfg.renorm, scaling=cfg.scaling, n_shared=cfg.shared_experts)
    ids, w = ops.route_topk(lg, cfg.top_k, **kw)
    s, e, em = ops.moe_align_block_size(ids, cfg.n_weight_experts, 16)
    ids2, w2, s2, e2, em2 = ops.route_align_small(lg, cfg.top_k, block_size=16, **kw)
    assert torch.equal(ids, ids2) and torch.equal(w, w2)
    assert torch.equal(s, s2) and torch.equal(e, e2) and int(em.item()) == int(em2.item())


def test_routing_golden():
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "routing.npz"))
    ids, w = ops.route_topk(torch.from_numpy(g["softmax_logits"]).to(DEV), 4)
    assert (to_np(ids) == g["softmax_ids"]).all(1).mean() > 0.95
    ids, w = ops.route_topk(torch.from_numpy(g["sig_logits"]).to(DEV), 8, bias=torch.from_numpy(g["sig_bias"]).to(DEV),
                            sigmoid=True, n_group=8, topk_group=4, scaling=2.5)
    same = (to_np(ids) == g["sig_ids"]).all(1)
    assert same.mean() > 0.9 and np.allclose(to_np(w)[same], g["sig_w"][same], rtol=1e-4, atol=1e-6)
