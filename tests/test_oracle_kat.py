"""Known-answer cases of the reference's own tests for this path, restated
against both CPU checkers (tests/kernels/moe/test_moe_fused.cpp:71-736): every
expectation below is the analytic value that file derives."""
import math

import numpy as np
import pytest

from helpers import bf2f, f2bf, pack_pair, uniform_problem


def run(oracle, impl, A, w13, w13s, w2, w2s, sorted_ids, ws, eids, top_k=1, **kw):
    return oracle.fused_moe_mxfp4(A, w13, w13s, w2, w2s, sorted_ids, ws, eids, top_k=top_k, impl=impl, **kw)


def identity_routing(EM=16):
    return np.arange(EM, dtype=np.int32), np.ones(EM, np.float32), np.zeros(EM // 16, np.int32)


def test_tiny_sanity(oracle_mod, impl):
    out, act = run(oracle_mod, impl, *uniform_problem(), *identity_routing())
    silu = 128.0 / (1.0 + math.exp(-128.0))
    exp_act = silu * 128.0
    assert np.max(np.abs(out - exp_act * 64) / (exp_act * 64)) < 1e-2
    assert np.max(np.abs(bf2f(act) - exp_act)) < 0.5


def test_bias_only(oracle_mod, impl):
    A, w13, w13s, w2, w2s = uniform_problem(a=0.0, w13_byte=0, w2_byte=0)
    b13 = np.concatenate([np.full(64, 1.0), np.full(64, 2.0)]).astype(np.float32)[None]
    b2 = np.ones((1, 128), np.float32)
    out, act = run(oracle_mod, impl, A, w13, w13s, w2, w2s, *identity_routing(), b13=b13, b2=b2)
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    assert np.max(np.abs(bf2f(act) - silu1 * 2.0)) < 1e-2
    assert np.max(np.abs(out - 1.0)) < 1e-4


def test_swiglu_clamp(oracle_mod, impl):
    out, act = run(oracle_mod, impl, *uniform_problem(), *identity_routing(), swiglu_limit=10.0)
    exp_act = 10.0 / (1.0 + math.exp(-10.0)) * 10.0
    assert np.max(np.abs(bf2f(act) - exp_act)) < 0.2
    assert np.max(np.abs(out - exp_act * 64) / (exp_act * 64)) < 1e-2


def test_situ(oracle_mod, impl):
    beta, lb = 4.0, 25.0
    out, act = run(oracle_mod, impl, *uniform_problem(), *identity_routing(), swiglu_limit=1.0,
                   activation=1, beta=beta, linear_beta=lb)
    sig = 1.0 / (1.0 + math.exp(-128.0))
    exp_act = (beta * math.tanh(128.0 / beta) * sig) * (lb * math.tanh(128.0 / lb))
    assert np.max(np.abs(bf2f(act) - exp_act)) < 0.5
    assert np.max(np.abs(out - exp_act * 64) / (exp_act * 64)) < 1e-2
    # linear_beta <= 0 passes `up` through
    _, act2 = run(oracle_mod, impl, *uniform_problem(), *identity_routing(), swiglu_limit=1.0,
                  activation=1, beta=beta, linear_beta=0.0)
    assert np.max(np.abs(bf2f(act2) - beta * math.tanh(128.0 / beta) * sig * 128.0)) < 0.5


def test_e2m1_quarter(oracle_mod, impl):
    out, act = run(oracle_mod, impl, *uniform_problem(w13_byte=0x11, w2_byte=0x11), *identity_routing())
    exp_act = 32.0 / (1.0 + math.exp(-32.0)) * 32.0
    assert np.max(np.abs(bf2f(act) - exp_act)) < 0.5
    assert np.all(np.isfinite(out)) and np.all(out > 0)


def test_inf_nan_propagate(oracle_mod, impl):
    out, act = run(oracle_mod, impl, *uniform_problem(w13_byte=0x76, w2_byte=0x22), *identity_routing())
    assert np.all(np.isnan(bf2f(act))) and np.all(np.isnan(out))


def test_ue8m0_zero_byte_is_subnormal(oracle_mod, impl):
    out, act = run(oracle_mod, impl, *uniform_problem(w13_byte=0x22, w2_byte=0x22, scale=0), *identity_routing())
    assert np.max(np.abs(bf2f(act))) < 1e-30 and np.max(np.abs(out)) < 1e-30
    assert oracle_mod.ue8m0_value(0) == 2.0 ** -127 and oracle_mod.ue8m0_value(255) == 0.0
    assert oracle_mod.ue8m0_value(127) == 1.0


def test_padding_rows_never_written(oracle_mod, impl):
    A, w13, w13s, w2, w2s = uniform_problem(M=8)
    sorted_ids = np.full(16, 8, np.int32)
    sorted_ids[:8] = np.arange(8)
    out, act = run(oracle_mod, impl, A, w13, w13s, w2, w2s, sorted_ids, np.ones(16, np.float32),
                   np.zeros(1, np.int32))
    exp = 128.0 / (1.0 + math.exp(-128.0)) * 128.0 * 64
    assert np.max(np.abs(out - exp) / exp) < 1e-2
    assert np.all(act[8:] == 0)


def test_multi_expert(oracle_mod, impl):
    M, E = 8, 4
    A, w13, w13s, w2, w2s = uniform_problem(M=M, E=E)
    for e in range(E):
        w13[e] = pack_pair(1.0 + e, 1.0 + e)
        w2[e] = pack_pair(1.0 + e, 1.0 + e)
    sorted_ids = (np.arange(16) % M).astype(np.int32)
    out, _ = run(oracle_mod, impl, A, w13, w13s, w2, w2s, sorted_ids, np.ones(16, np.float32),
                 np.array([0], np.int32))
    assert np.all(np.isfinite(out)) and np.all(out > 0)


def test_expert_filter_leaves_out_untouched(oracle_mod, impl):
    A, w13, w13s, w2, w2s = uniform_problem()
    out = np.full((16, 128), 99.0, np.float32)
    s, w, _ = identity_routing()
    run(oracle_mod, impl, A, w13, w13s, w2, w2s, s, w, np.array([-1], np.int32), out=out)
    assert np.all(out == 99.0)


def test_align_basic_8x4(oracle_mod, impl):
    ids = np.array([[0] * 4, [0, 1, 1, 1], [1] * 4, [1] * 4, [2] * 4, [2] * 4, [2] * 4, [2] * 4], np.int32)
    s, e, EM = oracle_mod.moe_align_block_size(ids, 4, 16, impl=impl)
    assert EM == 48 and list(e) == [0, 1, 2]
    assert list(s[:5]) == [0, 1, 2, 3, 4] and np.all(s[5:16] == 32)
    assert sorted(s[32:48]) == list(range(16, 32))


def test_k3_routing_top16(oracle_mod, impl):
    E, top_k, hidden, ispp = 256, 16, 128, 64
    A, w13, w13s, w2, w2s = uniform_problem(M=1, hidden=hidden, ispp=ispp, E=E)
    ids = np.arange(top_k, dtype=np.int32)[None]
    s, e, EM = oracle_mod.moe_align_block_size(ids, E, 16, impl=impl)
    ws = oracle_mod.gather_sorted_weights(np.ones(top_k, np.float32), s)
    assert int((ws > 0).sum()) == top_k
    out, act = run(oracle_mod, impl, A, w13, w13s, w2, w2s, s, ws, e, top_k=top_k)
    exp_act = hidden / (1.0 + math.exp(-hidden)) * hidden
    real = s < top_k
    assert np.max(np.abs(bf2f(act[real]) - exp_act)) < 0.5 and np.all(act[~real] == 0)
    assert np.max(np.abs(out - top_k * exp_act * ispp) / (top_k * exp_act * ispp)) < 1e-2


def test_dequant_every_byte_times_every_scale(oracle_mod):
    """Both reference dequant variants and the restatement agree bit for bit on all 256 x 256
    (byte, scale) pairs (test_moe_fused.cpp:591-621)."""
    N = K = 64
    packed = (np.arange(N * K // 2) & 0xFF).astype(np.uint8).reshape(N, K // 2)
    for s in range(256):
        scale = np.full((N, 2), s, np.uint8)
        port = oracle_mod.dequant_weight_tile(packed, scale, N, K)
        if oracle_mod.have_reference():
            a = oracle_mod.dequant_weight_tile(packed, scale, N, K, impl="reference")
            b = oracle_mod.dequant_weight_tile(packed, scale, N, K, impl="reference", variant="_ref")
            assert np.array_equal(a, b) and np.array_equal(a, port), f"scale byte {s}"
        # spot values of the table itself
        if s == 127:
            assert bf2f(port[0, 0]) == 0.0  # byte 0x00, low nibble
    assert [oracle_mod.e2m1_value(c) for c in range(6)] == [0.0, 0.25, 1.0, 1.5, 2.0, 3.0]
    assert math.isinf(oracle_mod.e2m1_value(6)) and math.isnan(oracle_mod.e2m1_value(7))
    assert oracle_mod.e2m1_value(9) == -0.25 and oracle_mod.e2m1_value(14) == -math.inf


def test_dequant_varying_scale_random_tiles(oracle_mod):
    if not oracle_mod.have_reference():
        pytest.skip("needs the reference build")
    rng = np.random.default_rng(7)
    for _ in range(50):
        packed = rng.integers(0, 256, (64, 32), dtype=np.uint8)
        scale = rng.integers(0, 256, (64, 2), dtype=np.uint8)
        a = oracle_mod.dequant_weight_tile(packed, scale, 64, 64)
        b = oracle_mod.dequant_weight_tile(packed, scale, 64, 64, impl="reference")
        assert np.array_equal(a, b)
