"""Shared test utilities: dtype plumbing, tolerances, small problem builders."""
from __future__ import annotations

import numpy as np
import torch

# Output gate of the layer (bf16 outputs of O(1) magnitude): max-abs 2e-2 and
# relative L2 1e-2 against the CPU oracle; fp32 accumulation order differs.
MAX_ABS_TOL = 2e-2
REL_L2_TOL = 1e-2


def bf16_to_u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u16_to_bf16(a: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(device)


def f2bf(x: float) -> int:
    b = int(np.float32(x).view(np.uint32))
    b += 0x7FFF + ((b >> 16) & 1)
    return (b >> 16) & 0xFFFF


def bf2f(u16) -> np.ndarray:
    return (np.asarray(u16, np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16_f32(x: np.ndarray) -> np.ndarray:
    """RNE to bf16, returned as fp32; NaN stays NaN whatever its payload."""
    x = np.ascontiguousarray(x, np.float32)
    b = x.view(np.uint32).astype(np.uint64)
    b = b + 0x7FFF + ((b >> 16) & 1)
    r = ((b >> 16).astype(np.uint32) << 16).view(np.float32)
    return np.where(np.isnan(x), np.float32(np.nan), r)


def e2m1_nibble(v: float) -> int:
    """Nearest finite code of the layer's table {0, .25, 1, 1.5, 2, 3} with sign."""
    neg = v < 0
    av = abs(v)
    if av == 0:
        return 0x8 if neg else 0x0
    vals = [0.25, 1.0, 1.5, 2.0, 3.0]
    best = min(range(5), key=lambda i: abs(av - vals[i])) + 1
    return best | (0x8 if neg else 0)


def pack_pair(v0: float, v1: float) -> int:
    return e2m1_nibble(v0) | (e2m1_nibble(v1) << 4)


def uniform_problem(M=16, hidden=128, ispp=64, E=1, a=1.0, w13_byte=None, w2_byte=None, scale=127):
    """All-constant problem used by the analytic known-answer cases."""
    one = pack_pair(1.0, 1.0)
    A = np.full((M, hidden), f2bf(a), np.uint16)
    w13 = np.full((E, 2 * ispp, hidden // 2), one if w13_byte is None else w13_byte, np.uint8)
    w13s = np.full((E, 2 * ispp, hidden // 32), scale, np.uint8)
    w2 = np.full((E, hidden, ispp // 2), one if w2_byte is None else w2_byte, np.uint8)
    w2s = np.full((E, hidden, ispp // 32), scale, np.uint8)
    return A, w13, w13s, w2, w2s


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of bf16 (8 significant bits) at |x|."""
    ax = np.maximum(np.abs(x.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(ax)) - 7)


def assert_close_bf16(got_f32: np.ndarray, ref_f32: np.ndarray, what="", got_is_bf16=False):
    """The layer's output gate against the CPU oracle (fp32 accumulation order differs):

    * NaN and inf masks equal;
    * fp32 accumulators: max-abs <= 2e-2 (skipped when `got` was already rounded to bf16);
    * bf16 outputs: every element within max(2e-2, one bf16 ulp of the reference) - two fp32
      values a hair apart can round to neighbouring bf16 values, and above |x| = 4 one bf16 ulp
      already exceeds 2e-2;
    * relative L2 of the bf16 outputs <= 1e-2.
    """
    got_f32 = np.asarray(got_f32, np.float32)
    ref_f32 = np.asarray(ref_f32, np.float32)
    assert np.array_equal(np.isnan(got_f32), np.isnan(ref_f32)), f"{what}: NaN masks differ"
    assert np.array_equal(np.isinf(got_f32), np.isinf(ref_f32)), f"{what}: inf masks differ"
    fin = np.isfinite(ref_f32)
    if not fin.any():
        return 0.0, 0.0
    if not got_is_bf16:
        acc_err = float(np.max(np.abs(got_f32[fin].astype(np.float64) - ref_f32[fin])))
        assert acc_err <= MAX_ABS_TOL, f"{what}: fp32 max-abs {acc_err:.3e} > {MAX_ABS_TOL}"
    g = round_to_bf16_f32(got_f32)[fin].astype(np.float64)
    r = round_to_bf16_f32(ref_f32)[fin].astype(np.float64)
    d = np.abs(g - r)
    allowed = np.maximum(MAX_ABS_TOL, bf16_ulp(r))
    worst = int(np.argmax(d - allowed))
    assert (d <= allowed).all(), f"{what}: bf16 diff {d[worst]:.3e} at |ref|={abs(r[worst]):.3f} exceeds {allowed[worst]:.3e}"
    rel_l2 = float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))
    assert rel_l2 <= REL_L2_TOL, f"{what}: rel-L2 {rel_l2:.3e} > {REL_L2_TOL}"
    return float(d.max()), rel_l2


def expand_expert_ids(expert_ids: np.ndarray, block_size: int) -> np.ndarray:
    """expert id per `block_size` rows -> per 16 rows (what the CPU oracle consumes)."""
    return np.repeat(np.asarray(expert_ids, np.int32), block_size // 16)


def numpy_align(topk_ids, num_experts, block_size, expert_map=None):
    """Independent statement of the alignment contract used to cross-check both oracles."""
    ids = np.asarray(topk_ids, np.int32).ravel()
    N = ids.size
    groups = {}
    for i, e in enumerate(ids):
        if e < 0 or e >= num_experts:
            continue
        le = int(e) if expert_map is None else int(expert_map[e])
        if le < 0:
            continue
        groups.setdefault(le, []).append(i)
    sorted_ids, expert_ids = [], []
    for le in sorted(groups):
        rows = groups[le]
        nb = -(-len(rows) // block_size)
        sorted_ids += rows + [N] * (nb * block_size - len(rows))
        expert_ids += [le] * nb
    return np.array(sorted_ids, np.int32), np.array(expert_ids, np.int32), len(sorted_ids)
