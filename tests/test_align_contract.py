"""Alignment contract cases of the reference's oracle tests
(tests/kernels/moe/test_moe_align_oracle.cpp:87-244) on the CPU checkers, plus the
device-style contract (expert_map, max_EM, EM = block_size when empty) and the host-side
bound on EM used to size launches without a device read-back."""
import numpy as np
import pytest

from helpers import numpy_align
from vkernels_b200.torch_ops import align_em_bound


def test_padding_sentinels(oracle_mod, impl):
    ids = np.array([[2, 0], [2, 1], [0, 2]], np.int32)
    s, e, EM = oracle_mod.moe_align_block_size(ids, 3, 4, impl=impl)
    assert EM == 12 and list(e) == [0, 1, 2]
    assert list(s) == [1, 4, 6, 6, 3, 6, 6, 6, 0, 2, 5, 6]


def test_garbage_ids_are_skipped(oracle_mod, impl):
    ids = np.array([[-1, 7], [100, 1], [1, -5]], np.int32)
    s, e, EM = oracle_mod.moe_align_block_size(ids, 4, 16, impl=impl)
    assert EM == 16 and list(e) == [1] and list(s[:2]) == [3, 4] and np.all(s[2:] == 6)


@pytest.mark.parametrize("bs", [16, 32, 64])
def test_e256_against_independent_statement(oracle_mod, impl, bs):
    rng = np.random.default_rng(bs)
    ids = rng.integers(0, 256, (128, 8), dtype=np.int32)
    got = oracle_mod.moe_align_block_size(ids, 256, bs, impl=impl)
    for x, y in zip(got, numpy_align(ids, 256, bs)):
        assert np.array_equal(x, y)


def test_device_contract_with_map(oracle_mod):
    rng = np.random.default_rng(5)
    E, local_n, bs = 16, 4, 16
    ids = rng.integers(0, E, (20, 2), dtype=np.int32)
    emap = np.full(E, -1, np.int32)
    emap[8:12] = np.arange(4)
    max_EM = align_em_bound(20, 2, local_n, bs)
    s, e, EM = oracle_mod.moe_align_block_size_map(ids, emap, E, local_n, bs, max_EM)
    rs, re, rEM = numpy_align(ids, E, bs, emap)
    assert EM == rEM and np.array_equal(s[:EM], rs) and np.array_equal(e[: EM // bs], re)
    assert np.all(s[EM:] == 40) and np.all(e[EM // bs:] == -1)
    # nothing routes -> one padding block
    s, e, EM = oracle_mod.moe_align_block_size_map(ids, np.full(E, -1, np.int32), E, local_n, bs, max_EM)
    assert EM == bs and np.all(s == 40) and np.all(e == -1)


@pytest.mark.parametrize("routing", ["uniform", "hot", "powerlaw", "distinct"])
@pytest.mark.parametrize("bs", [16, 64])
def test_em_bound_covers_oracle(oracle_mod, routing, bs):
    """align_em_bound >= the real EM for every routing (test_moe_align_oracle.cpp:180-232)."""
    rng = np.random.default_rng(3)
    for M, k, E in [(1, 4, 32), (7, 4, 32), (128, 4, 32), (300, 8, 256), (5, 16, 256)]:
        if routing == "uniform":
            ids = rng.integers(0, E, (M, k))
        elif routing == "hot":
            ids = np.zeros((M, k), np.int64)
        elif routing == "powerlaw":
            ids = np.minimum((rng.pareto(1.2, (M, k))).astype(np.int64), E - 1)
        else:
            ids = (np.arange(M * k).reshape(M, k)) % E
        _, _, EM = oracle_mod.moe_align_block_size(ids.astype(np.int32), E, bs)
        assert align_em_bound(M, k, E, bs) >= EM
    assert align_em_bound(0, 4, 32, bs) == bs
