"""-m gpu: the allocation-free alignment entry point against the regular one.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has
already executed every other test. It must pass on its own in a fresh process and after the rest
of the suite, so it relies on no state left by other tests.

Who needs it: callers that cannot allocate device memory inside a call - a server that gave all
free memory to its own pool after warm-up, or a step that cannot afford cudaMalloc's device-wide
stall. The entry point keeps its scratch in a fixed array inside the library; here we check that
it produces the regular entry point's output bit for bit on two calls in a row (the array keeps
the first call's contents when the second starts) and that it refuses sizes beyond its limits.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from vkernels_b200 import native_runtime as nr  # noqa: E402
from vkernels_b200 import torch_ops as ops  # noqa: E402

DEV = "cuda:0"


def _call(fn_name, ids, expert_map, E, local_n, bs, max_EM):
    lib = nr.load_library()
    M, k = ids.shape
    s = torch.full((max_EM,), -5, dtype=torch.int32, device=DEV)
    e = torch.full((max_EM // bs,), -5, dtype=torch.int32, device=DEV)
    em = torch.full((1,), -5, dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        rc = getattr(lib, fn_name)(ids.data_ptr(), None if expert_map is None else expert_map.data_ptr(), M, k, bs,
                                   E, local_n, max_EM, s.data_ptr(), e.data_ptr(), em.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, s.cpu().numpy(), e.cpu().numpy(), int(em.item())


def test_noalloc_align_matches_regular_entry_point_twice():
    rng = np.random.default_rng(11)
    cases = [
        # M, top_k, E, local_n, block, with_map  - the second call is smaller than the first, so it
        # runs over scratch still holding the first call's histograms
        (8192, 4, 128, 128, 16, False),
        (3000, 8, 256, 64, 64, True),
        (1, 4, 32, 32, 16, False),
        (0, 4, 32, 32, 16, False),
    ]
    for M, k, E, local_n, bs, with_map in cases:
        ids = torch.from_numpy(rng.integers(-1, E, (M, k)).astype(np.int32)).to(DEV)
        emap = None
        if with_map:
            m = np.full(E, -1, np.int32)
            m[64:64 + local_n] = np.arange(local_n)
            emap = torch.from_numpy(m).to(DEV)
        max_EM = ops.align_em_bound(M, k, local_n, bs)
        rc0, s0, e0, em0 = _call("vk_hip_moe_align_block_size", ids, emap, E, local_n, bs, max_EM)
        rc1, s1, e1, em1 = _call("vk_cuda_moe_align_block_size_noalloc", ids, emap, E, local_n, bs, max_EM)
        assert rc0 == 0 and rc1 == 0, nr.last_error()
        assert em0 == em1 and np.array_equal(s0, s1) and np.array_equal(e0, e1), (M, k, E, bs)


def test_noalloc_align_at_its_limits_matches_the_oracle():
    """The largest problem the fixed array holds - 262144 routed slots over 512 local experts, which
    also takes the kernels' large shared-memory configuration - plus the same size through an
    expert map and a call with no local expert at all, against the CPU oracle's alignment and the
    regular entry point."""
    import oracle

    oracle.build()
    rng = np.random.default_rng(12)
    E, bs = 512, 16
    M, k = 32768, 8                                   # M * k = 262144
    ids_np = rng.integers(0, E, (M, k)).astype(np.int32)
    ids = torch.from_numpy(ids_np).to(DEV)
    for emap_np, local_n in [(None, 512), (np.where(np.arange(E) % 2 == 0, np.arange(E) // 2, -1).astype(np.int32), 256),
                             (np.full(E, -1, np.int32), 0)]:
        emap = None if emap_np is None else torch.from_numpy(emap_np).to(DEV)
        max_EM = ops.align_em_bound(M, k, max(local_n, 1), bs)
        rc1, s1, e1, em1 = _call("vk_cuda_moe_align_block_size_noalloc", ids, emap, E, local_n, bs, max_EM)
        assert rc1 == 0, nr.last_error()
        rc0, s0, e0, em0 = _call("vk_hip_moe_align_block_size", ids, emap, E, local_n, bs, max_EM)
        assert rc0 == 0 and em0 == em1 and np.array_equal(s0, s1) and np.array_equal(e0, e1)
        full_map = np.arange(E, dtype=np.int32) if emap_np is None else emap_np
        rs, re, rEM = oracle.moe_align_block_size_map(ids_np, full_map, E, local_n, bs, max_EM)
        assert em1 == rEM and np.array_equal(s1, rs) and np.array_equal(e1, re), local_n


def test_noalloc_align_rejects_sizes_beyond_its_fixed_scratch():
    lib = nr.load_library()
    one = torch.zeros(16, dtype=torch.int32, device=DEV)
    p = one.data_ptr()
    # 262145 routed slots: one more than the array was sized for
    assert lib.vk_cuda_moe_align_block_size_noalloc(p, None, 262145, 1, 16, 8, 8, 16, p, p, p, None) == 1
    assert b"262144" in lib.vk_last_error()
    # 513 local experts
    assert lib.vk_cuda_moe_align_block_size_noalloc(p, None, 4, 1, 16, 1024, 513, 16, p, p, p, None) == 1
    assert b"512" in lib.vk_last_error()
