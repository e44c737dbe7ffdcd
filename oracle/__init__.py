"""CPU checkers for the fused MXFP4 MoE path. TEST INFRASTRUCTURE ONLY.

Two shared libraries, both built by ``oracle/Makefile``:

* ``libvkoracle.so`` - this repository's C restatement (``moe_oracle.c``),
  functions prefixed ``vko_``;
* ``_ref/libvkref.so`` - the reference's own ``moe_fused.cpp`` /
  ``dist_moe.cpp`` compiled in place behind ``ref_shim.cpp``, prefix ``vkr_``.
  Present only where the reference tree was available at build time.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg
may import this package. The library under ``vkernels_b200/`` never does.

All functions take and return numpy arrays (bf16 travels as ``uint16``).
``impl`` selects the backend: ``"port"`` (the restatement) or ``"reference"``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint8, c_uint16, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_PATH = os.path.join(_HERE, "libvkoracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libvkref.so")

_libs: dict[str, ctypes.CDLL | None] = {}


def build(quiet: bool = True) -> None:
    """Run the Makefile (restatement always; reference only if its tree exists)."""
    subprocess.run(
        ["make", "-C", _HERE],
        check=True,
        stdout=subprocess.DEVNULL if quiet else None,
        stderr=subprocess.STDOUT if quiet else None,
    )
    _libs.clear()


def _load(kind: str) -> ctypes.CDLL | None:
    if kind not in _libs:
        path = _PORT_PATH if kind == "port" else _REF_PATH
        if kind == "port" and not os.path.exists(path):
            build()
        _libs[kind] = ctypes.CDLL(path) if os.path.exists(path) else None
    return _libs[kind]


def have_reference() -> bool:
    return _load("reference") is not None


def _sym(impl: str, name: str):
    lib = _load(impl)
    if lib is None:
        raise RuntimeError(f"oracle backend {impl!r} is not built")
    return getattr(lib, ("vko_" if impl == "port" else "vkr_") + name)


def _p(a: np.ndarray | None, ctype=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arguments must be contiguous"
    return a.ctypes.data_as(c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(_load("port").vko_num_threads())


def set_num_threads(n: int) -> None:
    _load("port").vko_set_num_threads(c_int(int(n)))


# ---------------------------------------------------------------------------
# scalars
# ---------------------------------------------------------------------------


def e2m1_value(nibble: int) -> float:
    f = _load("port").vko_e2m1_value
    f.restype = c_float
    return float(f(c_int(nibble)))


def ue8m0_value(s: int) -> float:
    f = _load("port").vko_ue8m0_value
    f.restype = c_float
    return float(f(c_int(s)))


def round_bf16(x: np.ndarray, impl: str = "port") -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    n = c_int64(x.size) if impl == "port" else c_int(x.size)
    _sym(impl, "round_bf16")(_p(x), _p(out), n)
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------
# dequant / align
# ---------------------------------------------------------------------------


def dequant_weight_tile(packed, scale, N, K, group_size=32, stride_packed=None, stride_scale_n=None,
                        stride_scale_k=1, impl="port", variant=""):
    """Returns the [K, N] uint16 (bf16) transposed tile."""
    packed = _c(packed, np.uint8)
    scale = _c(scale, np.uint8)
    stride_packed = K // 2 if stride_packed is None else stride_packed
    stride_scale_n = K // group_size if stride_scale_n is None else stride_scale_n
    out = np.zeros((K, N), np.uint16)
    name = "dequant_weight_tile" + (variant if impl == "reference" else "")
    _sym(impl, name)(_p(packed), _p(scale), _p(out), c_int(N), c_int(K), c_int(group_size),
                     c_int(stride_packed), c_int(stride_scale_n), c_int(stride_scale_k))
    return out


def max_em(M, top_k, block_size, num_experts):
    """capi_moe.cpp:110-117."""
    return ((M * top_k + block_size - 1) // block_size + num_experts) * block_size


def moe_align_block_size(topk_ids, num_experts, block_size, impl="port"):
    """Host contract (moe_fused.cpp:609-661). Returns (sorted_ids[EM], expert_ids[EM/bs], EM)."""
    ids = _c(topk_ids, np.int32)
    M, top_k = (ids.shape if ids.ndim == 2 else (ids.size, 1))
    cap = max_em(M, top_k, block_size, num_experts)
    s = np.full(cap, -7, np.int32)
    e = np.full(cap // block_size, -7, np.int32)
    f = _sym(impl, "moe_align_block_size")
    f.restype = c_int
    EM = int(f(_p(ids), c_int(M), c_int(top_k), c_int(block_size), c_int(num_experts), _p(s), _p(e)))
    return s[:EM].copy(), e[: EM // block_size].copy(), EM


def moe_align_block_size_map(topk_ids, expert_map, num_experts, local_n, block_size, max_EM):
    """Device contract (restatement only): all of sorted_ids[max_EM] is written."""
    ids = _c(topk_ids, np.int32)
    M, top_k = (ids.shape if ids.ndim == 2 else (ids.size, 1))
    emap = _c(expert_map, np.int32)
    s = np.full(max_EM, -7, np.int32)
    e = np.full(max_EM // block_size, -7, np.int32)
    f = _load("port").vko_moe_align_block_size_map
    f.restype = c_int
    EM = int(f(_p(ids), _p(emap), c_int(M), c_int(top_k), c_int(block_size), c_int(num_experts),
               c_int(local_n), c_int(max_EM), _p(s), _p(e)))
    return s, e, EM


# ---------------------------------------------------------------------------
# the four stages and their composition
# ---------------------------------------------------------------------------


def _moe_args(A, w13, w13_scale, w2, w2_scale):
    return (_c(A, np.uint16), _c(w13, np.uint8), _c(w13_scale, np.uint8), _c(w2, np.uint8),
            _c(w2_scale, np.uint8))


def fused_moe_mxfp4(A, w13, w13_scale, w2, w2_scale, sorted_ids, topk_w_sorted, expert_ids, *,
                    top_k, swiglu_limit=0.0, activation=0, beta=4.0, linear_beta=25.0, b13=None,
                    b2=None, group_size=32, out=None, act=None, impl="port", threads=0):
    """fused_moe_mxfp4_cpu (moe_fused.cpp:569-603). Returns (out fp32 [M,H], act u16 [EM,I]).

    ``out`` accumulates in place when given (the caller-zeroes contract);
    ``threads`` > 0 with impl="reference" uses the 16-row-sliced driver.
    """
    A, w13, w13_scale, w2, w2_scale = _moe_args(A, w13, w13_scale, w2, w2_scale)
    M, hidden = A.shape
    ispp = w13.shape[-2] // 2
    sorted_ids = _c(sorted_ids, np.int32)
    expert_ids = _c(expert_ids, np.int32)
    topk_w_sorted = _c(topk_w_sorted, np.float32)
    EM = sorted_ids.size
    if out is None:
        out = np.zeros((M, hidden), np.float32)
    if act is None:
        act = np.zeros((max(EM, 1), ispp), np.uint16)
    b13 = _c(b13, np.float32)
    b2 = _c(b2, np.float32)
    args = [_p(A), _p(w13), _p(w13_scale), _p(w2), _p(w2_scale), _p(sorted_ids), _p(topk_w_sorted),
            _p(expert_ids), _p(act), _p(out), c_int(M), c_int(hidden), c_int(ispp), c_int(top_k),
            c_int(EM), c_int(group_size), c_float(swiglu_limit), c_int(activation), c_float(beta),
            c_float(linear_beta), _p(b13), _p(b2)]
    if impl == "reference" and threads > 0:
        f = _sym(impl, "fused_moe_mxfp4_mt")
        args.append(c_int(threads))
    else:
        f = _sym(impl, "fused_moe_mxfp4")
    f.restype = c_int
    rc = f(*args)
    if rc != 0:
        raise RuntimeError(f"oracle fused_moe_mxfp4 failed ({rc})")
    return out, act[:EM]


def moe_stages(A, w13, w13_scale, w2, w2_scale, sorted_ids, topk_w_sorted, expert_ids, *, top_k,
               swiglu_limit=0.0, activation=0, beta=4.0, linear_beta=25.0, b13=None, b2=None,
               group_size=32, impl="port"):
    """The four stage functions called one by one. Returns dict with the
    intermediates gate_up fp32 [EM,2I], act u16 [EM,I], partial fp32 [EM,H], out fp32 [M,H]."""
    A, w13, w13_scale, w2, w2_scale = _moe_args(A, w13, w13_scale, w2, w2_scale)
    M, hidden = A.shape
    ispp = w13.shape[-2] // 2
    sorted_ids = _c(sorted_ids, np.int32)
    expert_ids = _c(expert_ids, np.int32)
    topk_w_sorted = _c(topk_w_sorted, np.float32)
    b13 = _c(b13, np.float32)
    b2 = _c(b2, np.float32)
    EM = sorted_ids.size
    gate_up = np.zeros((EM, 2 * ispp), np.float32)
    act = np.zeros((EM, ispp), np.uint16)
    partial = np.zeros((EM, hidden), np.float32)
    out = np.zeros((M, hidden), np.float32)
    _sym(impl, "moe_gateup")(_p(A), _p(w13), _p(w13_scale), _p(sorted_ids), _p(expert_ids),
                             _p(gate_up), c_int(M), c_int(hidden), c_int(0), c_int(hidden),
                             c_int(ispp), c_int(top_k), c_int(EM), c_int(group_size))
    _sym(impl, "moe_act_epilogue")(_p(gate_up), _p(b13), _p(act), _p(sorted_ids), _p(expert_ids),
                                   c_int(M), c_int(top_k), c_int(EM), c_int(ispp),
                                   c_float(swiglu_limit), c_int(activation), c_float(beta),
                                   c_float(linear_beta))
    _sym(impl, "moe_down")(_p(act), _p(w2), _p(w2_scale), _p(sorted_ids), _p(expert_ids),
                           _p(partial), c_int(M), c_int(ispp), c_int(0), c_int(ispp), c_int(hidden),
                           c_int(top_k), c_int(EM), c_int(group_size))
    _sym(impl, "moe_combine")(_p(partial), _p(b2), _p(topk_w_sorted), _p(sorted_ids),
                              _p(expert_ids), _p(out), c_int(M), c_int(hidden), c_int(top_k),
                              c_int(EM))
    return {"gate_up": gate_up, "act": act, "partial": partial, "out": out}


def gather_sorted_weights(topk_w, sorted_ids):
    """topk_w_sorted[r] = topk_w[flat] for real rows, 0 for padding
    (dist_moe.cpp:311-318; tests/kernels/moe/test_moe_fused.cpp:698-704)."""
    w = np.ascontiguousarray(topk_w, np.float32).ravel()
    s = np.asarray(sorted_ids)
    real = (s >= 0) & (s < w.size)
    out = np.zeros(s.size, np.float32)
    out[real] = w[s[real]]
    return out


def moe_layer(A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, *, num_experts, swiglu_limit=0.0,
              activation=0, beta=4.0, linear_beta=25.0, b13=None, b2=None, impl="port", threads=0,
              tokens=None):
    """align (block 16) -> gather weights -> fused call. Returns out fp32 [M,H].

    ``tokens`` restricts the evaluation to a subset of token rows: every row of
    the layer is independent of the others and a token's combine order depends
    only on its own experts, so the result equals the full run on those rows.
    """
    ids = np.ascontiguousarray(topk_ids, np.int32)
    tw = np.ascontiguousarray(topk_w, np.float32)
    A = np.ascontiguousarray(A, np.uint16)
    if tokens is not None:
        tokens = np.asarray(tokens)
        ids, tw, A = ids[tokens].copy(), tw[tokens].copy(), A[tokens].copy()
    s, e, EM = moe_align_block_size(ids, num_experts, 16, impl="port")
    ws = gather_sorted_weights(tw, s)
    out, _ = fused_moe_mxfp4(A, w13, w13_scale, w2, w2_scale, s, ws, e, top_k=ids.shape[1],
                             swiglu_limit=swiglu_limit, activation=activation, beta=beta,
                             linear_beta=linear_beta, b13=b13, b2=b2, impl=impl, threads=threads)
    return out


# ---------------------------------------------------------------------------
# expert parallelism
# ---------------------------------------------------------------------------


def moe_ep_plan(num_experts, ep, rank, impl="port"):
    b, e = c_int(0), c_int(0)
    f = _sym(impl, "moe_ep_plan")
    f.restype = c_int
    if f(c_int(num_experts), c_int(ep), c_int(rank), ctypes.byref(b), ctypes.byref(e)) != 0:
        raise ValueError("moe_ep_plan: invalid argument")
    return b.value, e.value


def moe_ep_dispatch(topk_ids, num_experts, block_size, ep, rank, impl="port"):
    ids = _c(topk_ids, np.int32)
    M, top_k = ids.shape
    b, e = moe_ep_plan(num_experts, ep, rank, impl)
    cap = M * top_k + (e - b) * block_size + block_size
    s = np.full(cap, -7, np.int32)
    x = np.full(cap // block_size + 1, -7, np.int32)
    f = _sym(impl, "moe_ep_dispatch")
    f.restype = c_int
    if impl == "port":
        EM = f(_p(ids), c_int(M), c_int(top_k), c_int(num_experts), c_int(block_size), c_int(b),
               c_int(e), _p(s), _p(x))
    else:
        EM = f(_p(ids), c_int(M), c_int(top_k), c_int(num_experts), c_int(block_size), c_int(ep),
               c_int(rank), _p(s), _p(x))
    return s[:EM].copy(), x[: EM // block_size].copy(), int(EM)


def fused_moe_mxfp4_ep_reference(A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, *, num_experts,
                                 ep, swiglu_limit=0.0, activation=0, beta=4.0, linear_beta=25.0,
                                 b13=None, b2=None, block_size=16):
    """The reference's in-process EP forward (dist_moe.cpp:276-328): [ep, M, H] partial outs."""
    A, w13, w13_scale, w2, w2_scale = _moe_args(A, w13, w13_scale, w2, w2_scale)
    ids = _c(topk_ids, np.int32)
    tw = _c(topk_w, np.float32)
    M, hidden = A.shape
    ispp = w13.shape[-2] // 2
    outs = np.zeros((ep, M, hidden), np.float32)
    f = _sym("reference", "fused_moe_mxfp4_ep")
    f.restype = c_int
    rc = f(_p(A), _p(w13), _p(w13_scale), _p(w2), _p(w2_scale), _p(ids), _p(tw),
           _p(_c(b13, np.float32)), _p(_c(b2, np.float32)), c_int(M), c_int(hidden), c_int(ispp),
           c_int(ids.shape[1]), c_int(num_experts), c_int(32), c_float(swiglu_limit),
           c_int(activation), c_float(beta), c_float(linear_beta), c_int(block_size), c_int(ep),
           _p(outs))
    if rc != 0:
        raise RuntimeError("reference EP forward failed")
    return outs


# ---------------------------------------------------------------------------
# routing (restatement only; the reference has no CPU router)
# ---------------------------------------------------------------------------


def router_logits(x_bf16, wr):
    x = _c(x_bf16, np.uint16)
    wr = _c(wr, np.float32)
    T, H = x.shape
    E = wr.shape[0]
    out = np.empty((T, E), np.float32)
    _load("port").vko_router_logits(_p(x), _p(wr), _p(out), c_int(T), c_int(H), c_int(E))
    return out


def route_softmax_topk(logits, k, *, bias=None, renorm=True, scaling=1.0):
    """Returns (ids int32 [T,k], weights fp32 [T,k], margin fp32 [T])."""
    l = _c(logits, np.float32)
    T, E = l.shape
    ids = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    margin = np.empty(T, np.float32)
    _load("port").vko_route_softmax_topk(_p(l), _p(_c(bias, np.float32)), c_int(T), c_int(E), c_int(k),
                                         c_int(int(renorm)), c_float(scaling), _p(ids), _p(w),
                                         _p(margin))
    return ids, w, margin


def route_sigmoid_group_topk(logits, bias, k, *, n_group=1, topk_group=1, renorm=True, scaling=1.0):
    l = _c(logits, np.float32)
    T, E = l.shape
    ids = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    margin = np.empty(T, np.float32)
    _load("port").vko_route_sigmoid_group_topk(_p(l), _p(_c(bias, np.float32)), c_int(T), c_int(E),
                                               c_int(k), c_int(n_group), c_int(topk_group),
                                               c_int(int(renorm)), c_float(scaling), _p(ids), _p(w),
                                               _p(margin))
    return ids, w, margin
