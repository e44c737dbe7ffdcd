"""-m gpu: the launcher's runtime contract - bounded waits and the status word, scratch per
(device, stream), refusal to allocate during stream capture, two layers in flight on two
streams. No test here faults, traps or hangs the GPU: the give-up path is exercised by a
one-warp probe whose wait is limited to a fraction of a millisecond."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_common import DEV, make_case, oracle_layer, oracle_route, to_np  # noqa: E402
from helpers import assert_close_bf16  # noqa: E402
from vkernels_b200 import native_runtime as nr  # noqa: E402
from vkernels_b200 import synthetic as syn  # noqa: E402
from vkernels_b200 import torch_ops as ops  # noqa: E402
from vkernels_b200.experts import layer_from_config  # noqa: E402


def test_bounded_wait_gives_up_and_reports():
    """A wait nobody satisfies returns after its limit, the status word reports it as
    VK_ERROR_INTERNAL until it is reset, and a healthy layer call afterwards passes."""
    lib = nr.load_library()
    ops.kernel_status()                       # clean to begin with
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.vk_cuda_moe_test_wait_timeout(200000, stream) == 0     # ~0.1 ms of SM clock
    torch.cuda.synchronize()
    assert lib.vk_cuda_moe_kernel_status() == 4                      # VK_ERROR_INTERNAL
    assert "bounded wait" in nr.last_error()
    assert lib.vk_cuda_moe_kernel_status() == 4                      # sticky until reset
    ops.reset_kernel_status()
    ops.kernel_status()
    assert lib.vk_cuda_moe_test_wait_timeout(0, stream) == 1         # limit out of range
    cfg = syn.CONFIGS["c0"]
    w, A, r = make_case(cfg, 32)
    layer = layer_from_config(cfg, w, r, max_tokens=32)
    layer(A)
    torch.cuda.synchronize()
    ops.kernel_status()


def _routed(cfg, T, seed):
    w, A, r = make_case(cfg, T, seed=seed)
    ids_np, tw_np, _ = oracle_route(cfg, A, r)
    return w, A, torch.from_numpy(ids_np).to(DEV), torch.from_numpy(tw_np).to(DEV)


def test_two_layers_on_two_streams():
    """Two different layers run concurrently on two streams, several calls each, with the
    chunked alignment (more than 1024 routed slots) in play: each stream has its own scratch
    block, so both results match the oracle."""
    cfg_a = syn.scaled(syn.CONFIGS["c0"], H=512, I=256, E=16, top_k=4)
    cfg_b = syn.scaled(syn.CONFIGS["c0"], H=384, I=192, E=6, top_k=3)
    Ta, Tb = 1536, 700
    wa, Aa, ia, ta = _routed(cfg_a, Ta, 11)
    wb, Ab, ib, tb = _routed(cfg_b, Tb, 12)
    la = layer_from_config(cfg_a, wa, None, max_tokens=Ta)
    lb = layer_from_config(cfg_b, wb, None, max_tokens=Tb)
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs_a, outs_b = [], []
    for _ in range(4):
        with torch.cuda.stream(sa):
            outs_a.append(la.experts(Aa, ia, ta).float().clone())
        with torch.cuda.stream(sb):
            outs_b.append(lb.experts(Ab, ib, tb).float().clone())
    torch.cuda.synchronize()
    ops.kernel_status()
    rng = np.random.default_rng(5)
    tok_a, tok_b = np.sort(rng.choice(Ta, 48, replace=False)), np.sort(rng.choice(Tb, 48, replace=False))
    ref_a = oracle_layer(Aa, wa, ia, ta, tokens=tok_a)
    ref_b = oracle_layer(Ab, wb, ib, tb, tokens=tok_b)
    for o in outs_a:
        assert_close_bf16(to_np(o)[tok_a], ref_a, "stream A", got_is_bf16=True)
    for o in outs_b:
        assert_close_bf16(to_np(o)[tok_b], ref_b, "stream B", got_is_bf16=True)


def test_capture_refuses_to_allocate_and_replay_survives_growth():
    """(1) A layer call on a stream that is being captured and has no scratch block yet is
    refused with a clear message instead of allocating. (2) A captured step keeps replaying
    correctly after a LARGER layer has been built and run on the same stream (the outgrown block
    stays alive for the graph)."""
    cfg = syn.scaled(syn.CONFIGS["c0"], H=512, I=256, E=8, top_k=2)
    T = 48
    w, A, r = make_case(cfg, T)
    layer = layer_from_config(cfg, w, r, max_tokens=T)
    # (1) fresh stream, no block: capture must fail cleanly
    fresh = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with pytest.raises((ValueError, RuntimeError), match="capture"):
        with torch.cuda.graph(g, stream=fresh):
            ids = torch.zeros((T, cfg.top_k), dtype=torch.int32, device=DEV)
            tw = torch.ones((T, cfg.top_k), dtype=torch.float32, device=DEV)
            ops.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw)
    torch.cuda.synchronize()
    # (2) capture, then outgrow, then replay
    graph, y = layer.capture(A)
    graph.replay()
    torch.cuda.synchronize()
    first = y.float().clone()
    live0 = nr.load_library().vk_cuda_moe_workspace_live_bytes()
    big_cfg = syn.scaled(syn.CONFIGS["c0"], H=512, I=256, E=8, top_k=2)
    wb, Ab, rb = make_case(big_cfg, 4096, seed=9)
    big = layer_from_config(big_cfg, wb, rb, max_tokens=4096)
    with torch.cuda.stream(layer.capture_stream):
        big(Ab)
    torch.cuda.synchronize()
    assert nr.load_library().vk_cuda_moe_workspace_live_bytes() >= live0
    graph.replay()
    torch.cuda.synchronize()
    ops.kernel_status()
    assert torch.equal(y.float(), first) or torch.allclose(y.float(), first, atol=2e-2)
    ids_np, tw_np, margin = oracle_route(cfg, A, r)
    ref = oracle_layer(A, w, torch.from_numpy(ids_np), torch.from_numpy(tw_np))
    ok = margin > 2e-5
    assert_close_bf16(to_np(y.float())[ok], ref[ok], "replay after growth", got_is_bf16=True)
