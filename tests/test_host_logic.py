"""Host-side pieces that need no GPU: the C ABI library loads and exports what the header
declares, argument errors surface as status codes, the layer's step arena never reallocates,
the workload generator is reproducible."""
import os
import re

import numpy as np
import pytest
import torch

from vkernels_b200 import native_runtime as nr
from vkernels_b200 import synthetic as syn
from vkernels_b200.experts import StepArena
from vkernels_b200.torch_ops import OpNotEligible, fused_moe_mxfp4, moe_align_block_size

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "vkernels_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = nr.load_library()
    names = header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/vkernels_b200.h but not exported"
    assert set(names) == set(nr.EXPORTED), "loader signature table and header disagree"
    assert lib.vk_has_cuda() == 1 and lib.vk_version().startswith(b"0.")


def test_max_em_matches_reference_formula():
    lib = nr.load_library()
    assert lib.vk_moe_align_block_size_max_em(8, 4, 16, 4) == (2 + 4) * 16
    assert lib.vk_moe_align_block_size_max_em(8, 4, 0, 4) == 0


def test_argument_errors_become_status_codes():
    """Host validation runs before any CUDA call, so these work without a GPU
    (reference hip_capi.cpp:71-90, capi_moe.cpp:119-130)."""
    lib = nr.load_library()
    one = np.zeros(4, np.int32).ctypes.data
    assert lib.vk_hip_moe_align_block_size(one, None, 1, 1, 0, 4, 4, 16, one, one, one, None) == 1
    assert b"block_size" in lib.vk_last_error()
    assert lib.vk_hip_moe_align_block_size(one, None, 1, 1, 16, 4, 4, 24, one, one, one, None) == 1
    assert lib.vk_hip_moe_align_block_size(one, None, 1, 1, 16, 4, 8, 16, one, one, one, None) == 1
    assert lib.vk_hip_moe_align_block_size(one, None, 1, 1, 16, 4, 4, 16, one, one, None, None) == 1
    assert lib.vk_moe_align_block_size(one, -1, 1, 16, 4, one, one, one) == 1
    assert lib.vk_moe_align_block_size(None, 0, 4, 16, 4, None, None, one) == 0  # M = 0 is a no-op
    assert lib.vk_fused_moe_mxfp4(*([one] * 10), 1, 64, 64, 1, 16, 16, 0.0, 0, 4.0, 25.0, None, None) == 1
    assert b"group_size" in lib.vk_last_error()
    assert lib.vk_cuda_moe_set_impl(7) == 1
    lib.vk_set_last_error(3, b"hello")
    assert lib.vk_last_error_code() == 3 and lib.vk_last_error() == b"hello"
    # the void device entry point records its contract violation instead of launching
    lib.vk_set_last_error(0, b"")
    lib.vk_hip_fused_moe_mxfp4(*([one] * 9), 4, 100, 64, 1, one, one, 16, 0.0, 0, 4.0, 25.0, None, None, 16, None)
    assert lib.vk_last_error_code() == 1 and b"hidden" in lib.vk_last_error()


def test_ops_reject_cpu_tensors_instead_of_falling_back():
    ids = torch.zeros((4, 2), dtype=torch.int32)
    with pytest.raises(OpNotEligible):
        moe_align_block_size(ids, 8)
    x = torch.zeros((4, 64), dtype=torch.bfloat16)
    w13 = torch.zeros((1, 128, 32), dtype=torch.uint8)
    w13s = torch.zeros((1, 128, 2), dtype=torch.uint8)
    w2 = torch.zeros((1, 64, 32), dtype=torch.uint8)
    w2s = torch.zeros((1, 64, 2), dtype=torch.uint8)
    with pytest.raises(OpNotEligible):
        fused_moe_mxfp4(x, w13, w13s, w2, w2s, ids[:, :1], torch.ones((4, 1)))


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setenv("VKERNELS_LIB", "/nonexistent/libvkernels_b200.so")
    monkeypatch.setattr(nr, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        nr.load_library()


def test_step_arena_is_carved_once_and_never_grows():
    """The layer's buffers are regions of one allocation laid out at the token budget: a smaller
    request is a slice at the same address, a larger one is refused (what the reference's
    capture-safe scratch guarantees during graph capture, tests/python/test_vllm_experts.py:346-376,
    holds here at all times)."""
    arena = StepArena({"out": (torch.float32, 100), "ids": (torch.int32, 7), "act": (torch.bfloat16, 33)}, "cpu")
    a = arena.take("out", 10)
    b = arena.take("out", 100)
    assert a.numel() == 10 and a.dtype == torch.float32 and b.data_ptr() == a.data_ptr()
    assert arena.take("ids", 7).data_ptr() % 256 == arena.take("out", 1).data_ptr() % 256   # 256-byte pitch
    assert arena.take("act", 33).data_ptr() >= arena.take("ids", 7).data_ptr() + 7 * 4
    a.fill_(3.0)
    arena.take("ids", 7).fill_(-1)
    assert float(arena.take("out", 10).sum()) == 30.0                  # regions do not overlap
    with pytest.raises(ValueError, match="token budget"):
        arena.take("out", 101)
    with pytest.raises(ValueError):
        arena.take("out", -1)
    with pytest.raises(KeyError):
        arena.take("nope", 1)


def test_generator_is_reproducible_and_in_range():
    cfg = syn.CONFIGS["c0"]
    a = syn.make_expert_weights(cfg)
    b = syn.make_expert_weights(cfg)
    for k in a:
        assert torch.equal(a[k], b[k])
    assert a["w13"].shape == (8, 512, 256) and a["w2_scale"].shape == (8, 512, 8)
    lo, hi = a["w13"] & 15, a["w13"] >> 4
    assert int(((lo & 7) >= 6).sum()) == 0 and int(((hi & 7) >= 6).sum()) == 0  # finite codes only
    s = a["w13_scale"].to(torch.int32) - 127
    assert int(s.min()) == -8 and int(s.max()) == -4
    allc = syn.make_expert_weights(cfg, codes="all")["w13"]
    assert int((((allc & 15) & 7) >= 6).sum()) > 0
    x = syn.make_activations(cfg, 64)
    assert x.dtype == torch.bfloat16 and abs(float(x.float().std()) - 1.0) < 0.05
    assert cfg.expert_weight_bytes() == int(1.59375 * cfg.I * cfg.H)
    c1 = syn.CONFIGS["c1"]
    assert c1.expert_weight_bytes() == 13_219_200 and c1.flops(1) == 6 * 4 * 2880 * 2880


def test_zipf_logits_make_a_hot_expert():
    cfg = syn.CONFIGS["c4"]
    logits = syn.make_zipf_logits(cfg, 4096).numpy()
    top = np.argsort(-logits, axis=1)[:, :4]
    share = np.bincount(top.ravel(), minlength=cfg.E).max() / 4096
    assert share > 0.20   # the hottest expert receives more than 20 % of the tokens


def test_balanced_expert_order_evens_out_a_zipf_load():
    """balanced_expert_order: a permutation that keeps every rank's share of experts and brings
    the heaviest rank's load under the contiguous plan's, down to the floor a single dominant
    expert sets."""
    from vkernels_b200.dist import balanced_expert_order, ep_plan

    rng = np.random.default_rng(5)
    E = 128
    load = (20000.0 / np.arange(1, E + 1) ** 1.2)[rng.permutation(E)]
    for world in (2, 4, 8, 3):
        order = balanced_expert_order(load.tolist(), world)
        assert sorted(order) == list(range(E))
        def rank_loads(numbering):
            return [sum(load[numbering[i]] for i in range(*ep_plan(E, world, r))) for r in range(world)]
        before, after = rank_loads(list(range(E))), rank_loads(order)
        assert max(after) <= max(before) + 1e-9
        floor = max(load.max(), load.sum() / world)
        assert max(after) <= 1.15 * floor, (world, max(after), floor)
        for r in range(world):     # inside a rank the experts stay in ascending order
            b, e = ep_plan(E, world, r)
            assert order[b:e] == sorted(order[b:e])
