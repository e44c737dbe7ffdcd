"""The routing restatement (oracle/moe_oracle.c) against a torch-eager statement of the same
formulas - the form the reference's own router tests use (tests/python/test_tokenspeed_amd.py:
516-540: softmax -> topk -> renormalise -> scale; tests/python/test_glm_router.py:76-106 and
torch_ops/glm_router.py:184-201: stable descending argsort for the lowest-index tie-break)."""
import numpy as np
import pytest
import torch


def eager_softmax(logits, k, scaling=1.0, renorm=True):
    scores = torch.softmax(torch.from_numpy(logits), dim=-1)
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)[:, :k]
    w = scores.gather(1, order)
    if renorm:
        den = w.sum(-1, keepdim=True)
        w = w / torch.where(den != 0, den, torch.ones_like(den))
    return order.numpy().astype(np.int32), (w * scaling).numpy()


def eager_sigmoid_group(logits, bias, k, n_group, topk_group, scaling, renorm=True):
    l = torch.from_numpy(logits)
    scores = torch.sigmoid(l)
    choice = scores + torch.from_numpy(bias)
    T, E = l.shape
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        gscore = g.topk(2, dim=-1).values.sum(-1)
        gorder = torch.argsort(gscore, dim=-1, descending=True, stable=True)[:, :topk_group]
        mask = torch.zeros(T, n_group, dtype=torch.bool).scatter_(1, gorder, True)
        choice = torch.where(mask[:, :, None].expand_as(g).reshape(T, E), choice,
                             torch.full_like(choice, float("-inf")))
    order = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, :k]
    w = scores.gather(1, order)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return order.numpy().astype(np.int32), (w * scaling).numpy()


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (33, 32, 4), (50, 128, 4), (9, 256, 8)])
def test_softmax_topk(oracle_mod, T, E, k):
    rng = np.random.default_rng(T + E)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    ids, w, margin = oracle_mod.route_softmax_topk(logits, k)
    rid, rw = eager_softmax(logits, k)
    ok = margin > 1e-5
    assert ok.mean() > 0.9
    assert np.array_equal(ids[ok], rid[ok])
    assert np.allclose(w[ok], rw[ok], rtol=1e-5, atol=1e-7)
    assert np.allclose(w.sum(-1), 1.0, atol=1e-5)


def test_softmax_ties_take_lowest_index(oracle_mod):
    logits = np.zeros((3, 16), np.float32)
    logits[1, [5, 9]] = 1.0
    ids, w, _ = oracle_mod.route_softmax_topk(logits, 4)
    assert list(ids[0]) == [0, 1, 2, 3] and list(ids[1]) == [5, 9, 0, 1]
    assert np.allclose(w[0], 0.25)


@pytest.mark.parametrize("T,E,k,ng,tg", [(40, 256, 8, 8, 4), (17, 64, 6, 4, 2), (25, 32, 4, 1, 1)])
def test_sigmoid_group_topk(oracle_mod, T, E, k, ng, tg):
    rng = np.random.default_rng(E + k)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    bias = (0.01 * rng.standard_normal(E)).astype(np.float32)
    ids, w, margin = oracle_mod.route_sigmoid_group_topk(logits, bias, k, n_group=ng, topk_group=tg,
                                                         scaling=2.5)
    rid, rw = eager_sigmoid_group(logits, bias, k, ng, tg, 2.5)
    ok = margin > 1e-5
    assert ok.mean() > 0.8
    assert np.array_equal(ids[ok], rid[ok])
    assert np.allclose(w[ok], rw[ok], rtol=1e-5, atol=1e-7)
    if ng > 1:  # every pick lies in a kept group: at most tg distinct groups per token
        groups = ids // (E // ng)
        assert max(len(set(r)) for r in groups) <= tg


def test_sigmoid_weights_are_unbiased_scores(oracle_mod):
    logits = np.array([[0.0, 2.0, -1.0, 0.5]], np.float32)
    bias = np.array([10.0, 0.0, 0.0, 0.0], np.float32)  # the bias decides the pick, not the weight
    ids, w, _ = oracle_mod.route_sigmoid_group_topk(logits, bias, 2, renorm=False, scaling=1.0)
    assert list(ids[0]) == [0, 1]
    assert np.allclose(w[0], [0.5, 1 / (1 + np.exp(-2.0))], rtol=1e-6)


def test_router_logits_fp32(oracle_mod):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 96)).astype(np.float32)
    from helpers import round_to_bf16_f32
    xb = round_to_bf16_f32(x)
    xu = (xb.view(np.uint32) >> 16).astype(np.uint16)
    wr = (0.02 * rng.standard_normal((7, 96))).astype(np.float32)
    got = oracle_mod.router_logits(xu, wr)
    assert np.allclose(got, xb.astype(np.float64) @ wr.astype(np.float64).T, rtol=1e-5, atol=1e-6)
