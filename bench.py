#!/usr/bin/env python
"""Benchmark of the fused MXFP4 MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|c4] [--impl reference]

One step = one pass of the hot path (route -> align -> gate/up GEMM + activation -> down GEMM with
fused weighted combine) over one batch of seeded synthetic tokens. Default workload: the
gpt-oss-120b-shaped prefill layer (H = I = 2880, E = 128, top-4, T = 8192), the configuration the
headline metric is quoted on at 1, 2, 4 and 8 GPUs; with --gpus N > 1 (launched under torchrun)
the experts are partitioned over the ranks; token rows are read and results added across NVLink
by the expert kernels themselves (peer memory; VK_EP_FORM=collective selects the NCCL all-to-all
form). Strong scaling: the global batch is fixed. The same JSON line also carries the single-GPU decode sweep of the
gpt-oss-20b-shaped layer (T in 1..128) with its HBM roofline.

Prints ONE JSON line on rank 0. `--impl reference` times the reference's own CPU implementation
of the path (oracle/_ref, else the C restatement) on the host cores over a bounded token sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from vkernels_b200 import synthetic as syn  # noqa: E402

METRIC = "MXFP4 MoE layer tokens/s"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.stop = threading.Event()
        self.t = None

    # NVML (read-only queries) every 5 ms when the module is there, else nvidia-smi every 100 ms:
    # the timed region of a default run is a few tens of milliseconds long.
    def _poll_nvml(self, nv, h):
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        sm_max = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        while not self.stop.is_set():
            try:
                mask = int(get_reasons(h))
                row = [str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(sm_max),
                       str(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)]
                row += ["Active" if mask & bit else "Not Active" for bit in names.values()]
                self.rows.append(row)
            except Exception:  # noqa: BLE001 - a failed sample is skipped
                pass
            self.stop.wait(0.005)

    def __enter__(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            uuid = None
            try:
                uuid = torch.cuda.get_device_properties(self.index).uuid
            except Exception:  # noqa: BLE001
                pass
            h = nv.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}") if uuid is not None else nv.nvmlDeviceGetHandleByIndex(self.index)
            self.t = threading.Thread(target=self._poll_nvml, args=(nv, h), daemon=True)
            self.t.start()
            return self
        except Exception:  # noqa: BLE001 - fall back to the command-line tool
            self.t = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.t is not None:
            self.t.join(timeout=1)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = []
        for i, name in enumerate(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]):
            if any(r[3 + i] == "Active" for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][1]),
                "power_w_max": max(float(r[2]) for r in self.rows), "samples": len(self.rows), "reasons": reasons}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own implementation of the path on a bounded token sample
# ------------------------------------------------------------------------------------------------

def cpu_sample_rate(cfg, n_tokens, n_experts_gen, repeats=1, prefer_reference=True):
    """tokens/s of the CPU path (route restatement + reference layer) on `n_tokens` seeded tokens.
    Weights of `n_experts_gen` experts are generated; routing is over those experts."""
    import oracle

    oracle.build()
    small = syn.scaled(cfg, E=n_experts_gen, n_group=1, topk_group=1) if n_experts_gen != cfg.E else cfg
    w = {k: v.numpy() for k, v in syn.make_expert_weights(small, n_experts=small.n_weight_experts).items()}
    A = syn.make_activations(small, n_tokens)
    Au = A.view(torch.int16).numpy().view(np.uint16)
    r = syn.make_router(small)
    cores = os.cpu_count() or 1
    kind = "reference" if (prefer_reference and oracle.have_reference()) else "port"
    oracle.set_num_threads(cores)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        logits = oracle.router_logits(Au, r["wr"].numpy())
        if small.routing == "sigmoid_group":
            ids, tw, _ = oracle.route_sigmoid_group_topk(logits, r["bias"].numpy(), small.top_k, scaling=small.scaling)
        else:
            ids, tw, _ = oracle.route_softmax_topk(logits, small.top_k)
        if small.shared_experts:
            ids = np.concatenate([ids, np.full((n_tokens, 1), small.E, np.int32)], 1)
            tw = np.concatenate([tw, np.ones((n_tokens, 1), np.float32)], 1)
        oracle.moe_layer(Au, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw,
                         num_experts=small.n_weight_experts, swiglu_limit=small.swiglu_limit, impl=kind,
                         threads=cores if kind == "reference" else 0)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": n_tokens / best, "unit": UNIT, "cores": cores, "kind": kind, "seconds": best,
            "sample": f"{n_tokens} seeded tokens of the workload routed over {n_experts_gen} of its experts "
                      f"(same H, I, top_k); one pass of router + layer on all {cores} host threads"}


def run_reference_arm(args, cfg, T):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_tok = min(T, args.cpu_tokens)
    n_exp = min(cfg.E, 16)
    for _ in range(args.warmup and 1):
        cpu_sample_rate(cfg, min(n_tok, 16), n_exp)
    vals = [cpu_sample_rate(cfg, n_tok, n_exp) for _ in range(max(1, min(args.steps, 3)))]
    best = max(vals, key=lambda v: v["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(vals), "warmup": 1, "ms_per_step": best["seconds"] * 1e3 * T / n_tok,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x mxfp4 -> fp32",
            "data": "synthetic", "config": workload_config(cfg, T, args.gpus),
            "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(cfg, T, n_gpus):
    return {"workload": f"{cfg.name}: T={T} H={cfg.H} I={cfg.I} E={cfg.E}+{cfg.shared_experts} top{cfg.top_k} "
                        f"{cfg.routing}", "tokens": T, "hidden": cfg.H, "ispp": cfg.I, "experts": cfg.E,
            "top_k": cfg.top_k, "parallelism": "single GPU" if n_gpus == 1 else
            f"ep{n_gpus} (experts split; token rows and results cross NVLink inside the kernels, NCCL all-to-all as fallback)",
            "weights": "MXFP4, 12 finite E2M1 codes uniform, ue8m0 exponent uniform in "
                       f"[{cfg.scale_exp[0]},{cfg.scale_exp[1]}]",
            "l2": "expert weights touched per step exceed the 126 MB L2"}


# ------------------------------------------------------------------------------------------------
# checks outside the timed region: the layer's output and routing against the CPU oracle
# ------------------------------------------------------------------------------------------------

def oracle_parity(cfg, A, y, ids, tw, weights, n_tokens, seed, logits=None, router=None, threads=None):
    """Compares `n_tokens` seeded rows of one rank's result with the CPU oracle run on the SAME
    routing (ids / weights as the GPU produced them), and the routing itself with the CPU routing
    restatement on tokens whose decisive score gap exceeds fp32 reassociation noise.

    A [T, H] bf16 (device), y [T, H] bf16 (device), ids / tw [T, k (+ shared)] (device), weights:
    dict of device tensors holding ALL experts (routed + shared). Only the experts the sampled
    tokens touch are copied to the host. Returns a dict for the JSON line."""
    import oracle

    oracle.build()
    T = A.shape[0]
    rng = np.random.default_rng(seed)
    tokens = np.sort(rng.choice(T, min(n_tokens, T), replace=False))
    tok_t = torch.from_numpy(tokens).to(A.device)
    ids_s = ids.index_select(0, tok_t).cpu().numpy().astype(np.int32)
    tw_s = tw.index_select(0, tok_t).cpu().numpy().astype(np.float32)
    touched = np.unique(ids_s)
    remap = np.full(int(weights["w13"].shape[0]), -1, np.int32)
    remap[touched] = np.arange(touched.size, dtype=np.int32)
    sel = torch.from_numpy(touched.astype(np.int64)).to(A.device)
    wn = {k: v.index_select(0, sel).cpu().numpy() for k, v in weights.items()}
    Au = A.index_select(0, tok_t).cpu().view(torch.int16).numpy().view(np.uint16)
    oracle.set_num_threads(threads or os.cpu_count() or 1)
    ref = oracle.moe_layer(Au, wn["w13"], wn["w13_scale"], wn["w2"], wn["w2_scale"], remap[ids_s], tw_s,
                           num_experts=int(touched.size), swiglu_limit=cfg.swiglu_limit)
    got = y.index_select(0, tok_t).float().cpu().numpy()
    ref_bf = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    fin = np.isfinite(ref_bf)
    d = np.abs(got - ref_bf)[fin]
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref_bf[fin]), 2.0 ** -126))) - 7)
    max_abs = float(d.max()) if d.size else 0.0
    rel_l2 = float(np.linalg.norm((got - ref_bf)[fin]) / max(np.linalg.norm(ref_bf[fin]), 1e-30))
    ok = bool(np.array_equal(np.isfinite(got), fin) and (d <= np.maximum(2e-2, ulp)).all() and rel_l2 <= 1e-2)
    res = {"tokens": int(tokens.size), "max_abs": max_abs, "rel_l2": rel_l2, "ok": ok,
           "tolerance": "bf16 |diff| <= max(2e-2, 1 bf16 ulp of the reference), rel-L2 <= 1e-2"}
    # routing against the restatement
    if router is not None or logits is not None:
        if logits is None:
            lg = oracle.router_logits(Au, router["wr"].cpu().numpy())
        else:
            lg = logits.index_select(0, tok_t).cpu().numpy()
        if cfg.routing == "sigmoid_group":
            rid, _, margin = oracle.route_sigmoid_group_topk(lg, router["bias"].cpu().numpy(), cfg.top_k, n_group=cfg.n_group,
                                                             topk_group=cfg.topk_group, renorm=cfg.renorm, scaling=cfg.scaling)
        else:
            rid, _, margin = oracle.route_softmax_topk(lg, cfg.top_k, renorm=cfg.renorm, scaling=cfg.scaling)
        well = margin > 2e-5
        equal = bool(np.array_equal(ids_s[:, : cfg.top_k][well], rid[well]))
        res.update({"routing_equal": equal, "routing_margin_filtered": int((~well).sum())})
        res["ok"] = res["ok"] and equal
    return res


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

def time_steps(fn, steps, warmup, barrier=None):
    """CUDA-event time of `steps` calls of fn after `warmup` untimed ones; returns per-step ms list."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]


def kernel_times(fn, calls):
    """Average device time (ms) of the gate/up and the down kernel over `calls` layer calls."""
    import ctypes

    from vkernels_b200 import native_runtime as nr

    lib = nr.load_library()
    nr.check(lib.vk_cuda_moe_timing_begin(calls), "timing_begin")
    for _ in range(calls):
        fn()
    g, d, n = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
    nr.check(lib.vk_cuda_moe_timing_end(ctypes.byref(g), ctypes.byref(d), ctypes.byref(n)), "timing_end")
    return g.value / max(n.value, 1), d.value / max(n.value, 1), n.value


# DRAM bytes (read + write) of one launch of the gate/up GEMM, from the ncu capture summarised in
# profiles/moe_gemm_sm100_c2_prefill_T8192_sections.txt (1.467 TB/s x 1.0246 ms, cold caches).
# The kernel is tensor-bound; its algorithmic bytes are 1.51 GB (packed weights, scales, token
# rows in, activation rows out), so every byte crosses HBM once.
GATEUP_DRAM_BYTES = {("c2_gptoss120b_prefill", 8192): 1.503e9}


def launches_per_step(T, slots, H=2880, E=128):
    """Kernels of this library per layer call: router logits (prefill sizes: weight split, tcgen05
    GEMM, and the sum of its K-slice planes when the batch is cut into slices) + top-k, alignment
    (1 kernel up to 1024 routed slots, else 3), row gather (which also builds the tile list), gate/up
    GEMM, down GEMM; small token tiles: row split (+ tile list), gate/up, activation split, down."""
    router = 1
    if T > 512:
        tiles = (T + 127) // 128
        z = max(1, min(8, (H // 64) // 4, torch.cuda.get_device_properties(0).multi_processor_count // tiles))
        router = 2 + (1 if z > 1 else 0)
    small_tiles = T <= 256 or T * slots <= 48 * E
    return router + 1 + (1 if T * slots <= 1024 else 3) + (4 if small_tiles else 3)


def decode_sweep(peaks, steps, warmup, prepack=True, parity_tokens=8):
    """gpt-oss-20b-shaped layer, T in {1, 8, 32, 64, 128}: tokens/s and HBM roofline fraction on the
    weight bytes of the experts the batch touches (+ activations, output, router weight).
    `prepack`: the layer objects keep the one-time prepacked form of their weights and run these
    batches from it (a serving stack does this at model load); the checkpoint-layout time of
    every batch size is printed beside it. The T = 8 result of the first weight copy is checked
    against the CPU oracle."""
    from vkernels_b200.experts import layer_from_config

    cfg = syn.CONFIGS["c1"]
    dev = "cuda:0"
    # several weight copies so that a small batch cannot live in L2 between steps
    n_copies = 4     # T = 1 touches 53 MB per copy: four copies exceed the 126 MB L2
    layers = []
    r = syn.make_router(cfg, device=dev)
    for c in range(n_copies):
        w = syn.make_expert_weights(cfg, seed=cfg.seed + 17 * c, backend="torch", device=dev)
        layers.append(layer_from_config(cfg, w, r, max_tokens=128, prepack=prepack))
        if c == 0:
            w0 = w
    prepacked = all(layer.prepacked is not None for layer in layers)
    out = []
    for T in cfg.T:
        A = syn.make_activations(cfg, T, backend="torch", device=dev)
        ids, tw = layers[0].route(A)
        touched = int(torch.unique(ids).numel())

        def timed():
            state = {"i": 0}
            graphs = [layer.capture(A)[0] for layer in layers]   # one CUDA graph per weight copy

            def step():
                graphs[state["i"] % n_copies].replay()
                state["i"] += 1

            ms = time_steps(step, max(steps, 20), max(warmup, 5))
            return statistics.median(ms), min(ms)

        med, lo = timed()
        bytes_alg = syn.decode_algorithmic_bytes(cfg, T, touched)
        gbs = bytes_alg / (med * 1e-3) / 1e9
        row = {"T": T, "experts_touched": touched, "launch": "CUDA graph replay", "ms_per_step": med, "ms_min": lo,
               "weights": "prepacked at load" if prepacked else "checkpoint layout",
               "tokens_per_s": T / (med * 1e-3), "algorithmic_bytes": bytes_alg, "achieved_gbs": gbs,
               "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8tbs": gbs / 8000.0}
        if prepacked:
            if T == 8 and parity_tokens:
                y = layers[0](A)
                par = oracle_parity(cfg, A, y, ids, tw, w0, parity_tokens, cfg.seed, router=r)
                row["parity"] = {k: par[k] for k in ("tokens", "max_abs", "rel_l2", "ok") if k in par}
                if par["ok"] is False:
                    print(json.dumps({"error": "decode parity check against the CPU oracle failed", "parity": par}), flush=True)
                    sys.exit(3)
            keep = [layer.prepacked for layer in layers]
            for layer in layers:
                layer.prepacked = None
            row["checkpoint_layout_ms_per_step"], _ = timed()
            for layer, pk in zip(layers, keep):
                layer.prepacked = pk
        out.append(row)
    return out


def run_single_gpu(args, cfg, T):
    from vkernels_b200 import torch_ops as ops
    from vkernels_b200.experts import layer_from_config

    dev = "cuda:0"
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    w = syn.make_expert_weights(cfg, backend="torch", device=dev)
    r = syn.make_router(cfg, device=dev)
    A = syn.make_activations(cfg, T, backend="torch", device=dev)
    logits = syn.make_zipf_logits(cfg, T, device=dev) if cfg.zipf_alpha else None
    layer = layer_from_config(cfg, w, r, max_tokens=T, prepack=args.prepack)
    step = (lambda: layer(A, logits=logits))

    # outside the timed region: this very layer object against the CPU oracle on a token sample
    y0 = layer(A, logits=logits)
    ids0, tw0 = layer.route(A, logits=logits)
    parity = {"skipped": True, "ok": None} if args.skip_parity else \
        oracle_parity(cfg, A, y0, ids0, tw0, w, args.parity_tokens, cfg.seed, logits=logits, router=r)
    if parity["ok"] is False:
        print(json.dumps({"error": "parity check against the CPU oracle failed", "parity": parity}), flush=True)
        sys.exit(3)

    with ClockSampler(0) as clk:
        ms = time_steps(step, args.steps, args.warmup)
    clocks = clk.summary()
    ops.kernel_status()
    total_ms = sum(ms)
    ms_per_step = total_ms / args.steps
    value = T / (ms_per_step * 1e-3)

    g_ms, d_ms, n_calls = kernel_times(step, max(3, min(args.steps, 10)))
    flops_gateup = 4 * T * cfg.slots * cfg.I * cfg.H
    flops_down = 2 * T * cfg.slots * cfg.I * cfg.H
    # The timed region is a few tens of milliseconds at full clock: the burst figure is the
    # denominator that applies (the sustained one was taken in a seconds-long loop under the
    # power cap, at a lower clock); both fractions are printed.
    tensor_peak, sustained = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
    achieved = flops_gateup / (g_ms * 1e-3) / 1e12
    down_ach = flops_down / (d_ms * 1e-3) / 1e12
    layer_ach = cfg.flops(T) / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "moe_gemm_sm100_kernel<gate/up>", "achieved": achieved,
                "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "frac_of_sustained": achieved / sustained,
                "peak_source": f"{peaks['source']} burst cuBLAS bf16 (sustained {sustained})",
                "traffic": GATEUP_DRAM_BYTES.get((cfg.name, T)), "traffic_unit": "bytes",
                "algorithmic_flops_per_launch": flops_gateup, "ms_per_launch": g_ms,
                "down_kernel": {"achieved": down_ach, "ms_per_launch": d_ms, "frac": down_ach / tensor_peak,
                                "frac_of_sustained": down_ach / sustained},
                "layer": {"achieved": layer_ach, "frac": layer_ach / tensor_peak,
                          "frac_of_sustained": layer_ach / sustained}}

    # end to end: pinned host activations in, pinned host bf16 result out, copies inside the region
    xh = A.cpu().pin_memory()
    yh = torch.empty((T, cfg.H), dtype=torch.bfloat16).pin_memory()
    if logits is None and not args.skip_parity:
        # serial: copy in, layer, copy out, wait - one step at a time
        e2e_step = lambda: layer.forward_host(xh, yh)
        for _ in range(args.warmup):
            e2e_step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        serial_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        # pipelined: the same three things per step, with the copies of neighbouring steps
        # overlapping the layer (two pinned input and two pinned output batches in rotation)
        from vkernels_b200.experts import HostPipeline

        pipe = HostPipeline(layer, T)
        xhs = [xh, xh.clone().pin_memory()]
        yhs = [yh, torch.empty_like(yh).pin_memory()]
        for i in range(args.warmup):
            pipe.submit(xhs[i & 1], yhs[i & 1])
        pipe.drain()
        t0 = time.perf_counter()
        for i in range(args.steps):
            pipe.submit(xhs[i & 1], yhs[i & 1])
        pipe.drain()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        # the same loop in steady state: from the arrival of the last warm-up step's result on the host to the
        # arrival of the K-th timed one (no drain in between, so no pipeline fill and drain inside the K steps)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(max(args.warmup, 2)):
            pipe.submit(xhs[i & 1], yhs[i & 1])
        ev0.record(pipe.d2h)
        for i in range(args.steps):
            pipe.submit(xhs[i & 1], yhs[i & 1])
        ev1.record(pipe.d2h)
        pipe.drain()
        steady_ms = ev0.elapsed_time(ev1) / args.steps
        yh = yhs[(args.steps - 1) & 1]
        e2e_dev = yh.to(dev)
        e2e_par = oracle_parity(cfg, A, e2e_dev, ids0, tw0, w, min(args.parity_tokens, 32), cfg.seed + 1)
        e2e = {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T * cfg.H * 2,
               "d2h_bytes_per_step": T * cfg.H * 2, "ms_per_step": e2e_ms, "ms_per_step_serial": serial_ms,
               "ms_per_step_steady_state": steady_ms,
               "how": "HostPipeline: every step copies its batch in from pinned memory and its result out; the copies "
                      "of neighbouring steps overlap the layer on separate streams; value / ms_per_step: K steps from an idle "
                      "pipeline to the last result on the host (fill and drain included); ms_per_step_steady_state: "
                      "result-to-result time of K steps inside a running pipeline",
               "parity": {k: e2e_par[k] for k in ("tokens", "max_abs", "rel_l2", "ok")}}
        if not e2e_par["ok"]:
            print(json.dumps({"error": "end-to-end output differs from the CPU oracle", "parity": e2e_par}), flush=True)
            sys.exit(3)
    else:
        e2e = None

    cpu = cpu_sample_rate(cfg, min(T, args.cpu_tokens), min(cfg.E, 16))
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "ms_per_step_min": min(ms), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 x mxfp4 -> fp32", "data": "synthetic",
            "config": workload_config(cfg, T, 1), "roofline": roofline, "parity": parity,
            "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}, "e2e": e2e,
            "gpu_launches": launches_per_step(T, cfg.slots, cfg.H, cfg.E) * args.steps, "clocks": clocks}
    if args.decode_sweep:
        del layer, w
        torch.cuda.empty_cache()
        line["decode_sweep"] = {"workload": syn.describe(syn.CONFIGS["c1"]), "bound": "hbm",
                                "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                                "points": decode_sweep(peaks, args.steps, args.warmup)}
    print(json.dumps(line), flush=True)


def run_multi_gpu(args, cfg, T):
    import torch.distributed as dist

    from vkernels_b200 import torch_ops as ops
    from vkernels_b200.dist import ExpertParallelMoE

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    T_global = T * world if args.weak else T
    T_local = T_global // world
    sl = slice(rank * T_local, (rank + 1) * T_local)
    A_full = syn.make_activations(cfg, T_global, backend="torch", device=dev, seed=cfg.seed)
    lg_full = syn.make_zipf_logits(cfg, T_global, device=dev) if cfg.zipf_alpha else None
    order = None
    if args.placement == "balanced":
        # experts renumbered so that the contiguous plan's ranks carry even loads: the load is measured on this
        # very batch (every rank computes the same global routing, so all arrive at the same numbering)
        from vkernels_b200.dist import balanced_expert_order

        scores = lg_full if lg_full is not None else A_full.float() @ syn.make_router(cfg, device=dev)["wr"].t()
        load = torch.bincount(scores.topk(cfg.top_k, dim=1).indices.flatten(), minlength=cfg.E)
        order = balanced_expert_order(load.cpu().tolist(), world)
        if lg_full is not None:
            lg_full = lg_full[:, torch.tensor(order, device=dev)].contiguous()
    layer = ExpertParallelMoE.from_config(cfg, rank=rank, world=world, device=dev, max_tokens=T_local, expert_order=order)
    if os.environ.get("VK_EP_FORM", "peer") == "peer":
        layer.enable_peer_memory(T_local)   # falls back to the collective form when unavailable
    A = A_full[sl].contiguous()
    logits = lg_full[sl].contiguous() if lg_full is not None else None
    del A_full, lg_full
    if layer._peer is not None:
        # inputs resident in HBM means: resident in the rank's registered activation buffer, which the
        # owners of the experts read in place
        A_in = layer.input_buffer(T_local)
        A_in.copy_(A)
        A = A_in
    eager_step = lambda: layer(A, logits=logits)
    step = eager_step
    barrier = lambda: dist.barrier()

    # Outside the timed region: every rank checks a seeded sample of ITS rows against the CPU
    # oracle (on the routing the GPU produced) and its routing against the restatement; the run
    # stops when any rank misses the tolerance. The full weight set is drawn again for this (the
    # layer keeps only its own experts) and freed before timing.
    y0 = layer(A, logits=logits)
    ids0, tw0 = layer._last_routing
    if cfg.shared_experts:
        ids0 = torch.cat([ids0, torch.full((T_local, 1), cfg.E, dtype=torch.int32, device=dev)], 1)
        tw0 = torch.cat([tw0, torch.ones((T_local, 1), dtype=torch.float32, device=dev)], 1)
    full_w = syn.make_expert_weights(cfg, backend="torch", device=dev)
    router_full = syn.make_router(cfg, device=dev)
    if order is not None:      # the checker sees the same renumbering as the layer
        oi = torch.tensor(order + list(range(cfg.E, cfg.n_weight_experts)), device=dev)
        full_w = {k: v.index_select(0, oi) for k, v in full_w.items()}
        ro = torch.tensor(order, device=dev)
        router_full = {k: (None if v is None else v.index_select(0, ro).contiguous()) for k, v in router_full.items()}
    # (the ranks share the host's cores: each takes its share of the threads and a smaller sample)
    par = oracle_parity(cfg, A, y0, ids0.contiguous(), tw0.contiguous(), full_w, min(args.parity_tokens, max(8, 64 // world)),
                        cfg.seed + rank, logits=logits, router=router_full,
                        threads=max(1, (os.cpu_count() or 1) // world))
    del full_w
    torch.cuda.empty_cache()
    agg = torch.tensor([par["max_abs"], par["rel_l2"], 0.0 if par["ok"] else 1.0,
                        float(par.get("routing_margin_filtered", 0)), 0.0 if par.get("routing_equal", True) else 1.0],
                       device=dev, dtype=torch.float64)
    worst = agg.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    total = agg.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    ep_parity = {"tokens_per_rank": par["tokens"], "ranks": world, "max_abs": float(worst[0]), "rel_l2": float(worst[1]),
                 "routing_equal": float(worst[4]) == 0.0, "routing_margin_filtered": int(total[3]),
                 "ok": float(worst[2]) == 0.0, "tolerance": par["tolerance"], "form": layer.last_stats().get("form")}
    if not ep_parity["ok"]:
        if rank == 0:
            print(json.dumps({"error": "expert-parallel output differs from the CPU oracle", "ep_parity": ep_parity}), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(3)

    # The peer-memory step has no host reads and no collective calls, so it replays as one CUDA
    # graph: at 8 ranks a step is ~20 kernels in a few hundred microseconds, which launched one by
    # one from Python is bound by the host. VK_EP_GRAPH=0 times the eager step instead.
    y_graph = None
    if layer._peer is not None and os.environ.get("VK_EP_GRAPH", "1") == "1":
        graph, y_graph = layer.capture(A, logits=logits)
        step = graph.replay
    with ClockSampler(local) as clk:
        ms = time_steps(step, args.steps, args.warmup, barrier=barrier)
    t = torch.tensor([sum(ms)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    ops.kernel_status()

    # this rank's two GEMM kernels (every rank times its own; rank 0 reports its pair)
    layer.count_local_slots = True
    g_ms, d_ms, _ = kernel_times(eager_step, max(3, min(args.steps, 10)))
    layer.time_phases = True
    eager_step()
    stats = layer.last_stats()
    stats["launch"] = "CUDA graph replay" if y_graph is not None else "eager"
    stats["placement"] = "experts renumbered by measured load (balanced_expert_order)" if order is not None else "contiguous"
    layer.count_local_slots = False
    layer.time_phases = False
    # load per rank: expert slots each rank computed in that step, slowest rank's phases
    slots_t = torch.tensor([float(stats["local_slots"] or 0)], device=dev)
    all_slots = [torch.zeros_like(slots_t) for _ in range(world)]
    dist.all_gather(all_slots, slots_t)
    per_rank = [int(v.item()) for v in all_slots]
    stats["slots_per_rank"] = per_rank
    stats["imbalance_max_over_mean"] = max(per_rank) / max(1e-9, sum(per_rank) / world)
    peaks = measured_peaks()
    tensor_peak, sustained = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
    flops_gateup = 4 * stats["local_slots"] * cfg.I * cfg.H
    achieved = flops_gateup / (g_ms * 1e-3) / 1e12
    down_ach = flops_gateup / 2 / (d_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "moe_gemm_sm100_kernel<gate/up> (rank 0)", "achieved": achieved,
                "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "frac_of_sustained": achieved / sustained,
                "peak_source": f"{peaks['source']} burst cuBLAS bf16 (sustained {sustained})",
                "traffic": None, "algorithmic_flops_per_launch": flops_gateup, "ms_per_launch": g_ms,
                "down_kernel": {"achieved": down_ach, "ms_per_launch": d_ms, "frac": down_ach / tensor_peak,
                                "frac_of_sustained": down_ach / sustained}}

    # end to end: every rank copies its token slice from pinned host memory, runs the sharded
    # layer and reads its output rows back; wall clock between barriers, max over ranks
    xh = A.cpu().pin_memory()
    yh = torch.empty((T_local, cfg.H), dtype=torch.bfloat16).pin_memory()
    xd = layer.input_buffer(T_local) if layer._peer is not None else torch.empty_like(A)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        if y_graph is not None:     # xd is the buffer the captured step reads
            step()
            yh.copy_(y_graph, non_blocking=True)
        else:
            yh.copy_(layer(xd, logits=logits), non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        e2e_step()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    te = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps], device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())
    e2e = {"value": T_global / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": T_global * cfg.H * 2,
           "d2h_bytes_per_step": T_global * cfg.H * 2, "ms_per_step": e2e_ms}
    ops.kernel_status()
    if rank == 0:
        stats["parity"] = ep_parity
        line = {"metric": METRIC, "value": T_global / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak" if args.weak else "strong",
                "vs_baseline": None, "dtype": "bf16 x mxfp4 -> fp32", "data": "synthetic",
                "config": workload_config(cfg, T_global, world), "roofline": roofline, "cpu_baseline": None,
                "e2e": e2e, "gpu_launches": stats["launches_per_step"] * args.steps, "clocks": clk.summary(),
                "ep": stats}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=list(syn.CONFIGS))
    ap.add_argument("--tokens", type=int, default=0, help="override the batch size of the workload")
    ap.add_argument("--cpu-tokens", type=int, default=256, help="token sample of the CPU baseline")
    ap.add_argument("--parity-tokens", type=int, default=48, help="tokens per rank checked against the CPU oracle")
    ap.add_argument("--skip-parity", action="store_true",
                    help="profiling runs only: no oracle check and no end-to-end leg (single GPU)")
    ap.add_argument("--prepack", action="store_true",
                    help="single GPU, batches up to 256 tokens: run from weights prepacked at load (the decode sweep always does)")
    ap.add_argument("--placement", default="contiguous", choices=["contiguous", "balanced"],
                    help="multi-GPU: contiguous expert ranges in the checkpoint's numbering (the reference plan), or experts "
                         "renumbered by measured load first")
    ap.add_argument("--weak", action="store_true", help="multi-GPU: keep the batch PER RANK fixed (weak scaling)")
    ap.add_argument("--no-decode-sweep", dest="decode_sweep", action="store_false")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    cfg = syn.CONFIGS[args.workload]
    T = args.tokens or max(cfg.T)
    if args.impl == "reference":
        run_reference_arm(args, cfg, T)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        run_multi_gpu(args, cfg, T)
    else:
        run_single_gpu(args, cfg, T)


if __name__ == "__main__":
    main()
