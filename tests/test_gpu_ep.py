"""Expert parallelism on real GPUs: two NCCL ranks, each holding a contiguous slice of the experts,
exchange token rows with all_to_all_single and must reproduce the single-rank layer (and the CPU
oracle) on every rank's own tokens. The counterpart of the reference's two-rank EP check
(tests/c/test_dist_moe.cpp), with its in-process ranks replaced by one process per GPU.

Needs two visible GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev))
    try:
        import oracle
        from helpers import bf16_to_u16
        from vkernels_b200 import synthetic as syn
        from vkernels_b200.dist import ExpertParallelMoE
        from vkernels_b200.experts import layer_from_config

        cfg = syn.scaled(syn.CONFIGS["c0"], E=max(6, world + 1), top_k=3)   # uneven split of the experts
        T_local = 48
        T = T_local * world
        ep = ExpertParallelMoE.from_config(cfg, rank=rank, world=world, device=dev, max_tokens=T_local)
        A = syn.make_activations(cfg, T, backend="torch", device=dev, seed=cfg.seed)
        lo, hi = rank * T_local, (rank + 1) * T_local

        # routed by this rank's router on its own tokens
        y = ep(A[lo:hi].contiguous())
        torch.cuda.synchronize()
        stats = ep.last_stats()

        # single-rank layer with all experts on this GPU, same seeded weights and router
        wt = syn.make_expert_weights(cfg, backend="torch", device=dev)
        full = layer_from_config(cfg, wt, syn.make_router(cfg, device=dev), max_tokens=T)
        ids, w = full.route(A)
        y_full = full.experts(A, ids, w)
        torch.cuda.synchronize()
        got = y.float().cpu().numpy()
        want = y_full[lo:hi].float().cpu().numpy()
        scale = max(float(np.abs(want).max()), 1.0)
        # fp32 partial sums are rounded to bf16 once on both paths; the ranks add their partial
        # rows in rank order, the single-rank layer in expert order: one bf16 ulp of slack
        err_single = float(np.max(np.abs(got - want)))
        ok = err_single <= 2 ** -7 * scale

        # the CPU oracle on the same routing
        wts = {k: v.cpu().numpy() for k, v in wt.items()}
        ref = oracle.moe_layer(bf16_to_u16(A.cpu()), wts["w13"], wts["w13_scale"], wts["w2"], wts["w2_scale"],
                               ids[:, : cfg.top_k].cpu().numpy(), w[:, : cfg.top_k].cpu().numpy(), num_experts=cfg.E)
        err_oracle = float(np.max(np.abs(got - ref[lo:hi])))
        ok = ok and err_oracle <= 2 ** -6 * scale
        ok = ok and T_local <= stats["rows_sent"] <= T_local * world

        # peer-memory form: same routing, rows read and results added in the home rank's memory
        peer = ep.enable_peer_memory(T_local)
        err_peer = -1.0
        if peer:
            for _ in range(2):   # twice: the buffers are reused from step to step
                y2 = ep(A[lo:hi].contiguous())
            torch.cuda.synchronize()
            err_peer = float(np.max(np.abs(y2.float().cpu().numpy() - want)))
            ok = ok and err_peer <= 2 ** -7 * scale and ep.last_stats()["form"] == "peer memory"
        open(os.path.join(tmp, f"rank{rank}.txt"), "w").write(
            f"{int(ok)} err_single={err_single} err_oracle={err_oracle} peer={peer} err_peer={err_peer} "
            f"scale={scale} {stats} {ep.last_stats()}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_ranks_match_single_rank(world, tmp_path, oracle_mod):
    import torch.multiprocessing as mp
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        txt = (tmp_path / f"rank{r}.txt").read_text()
        assert txt.startswith("1"), f"rank {r}: {txt}"


def _tp_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev))
    try:
        from vkernels_b200 import synthetic as syn
        from vkernels_b200.dist import TensorParallelMoE, tp_plan, tp_shard_weights
        from vkernels_b200.experts import layer_from_config

        cfg = syn.scaled(syn.CONFIGS["c0"], E=6, top_k=3)   # H = 512, I = 256: shards of 256 and 128
        T = 96
        w = syn.make_expert_weights(cfg, backend="torch", device=dev)
        A = syn.make_activations(cfg, T, backend="torch", device=dev, seed=cfg.seed)
        full = layer_from_config(cfg, w, syn.make_router(cfg, device=dev), max_tokens=T)
        ids, tw = full.route(A)
        ids, tw = ids.clone(), tw.clone()
        want = full.experts(A, ids, tw, return_fp32=True).clone()
        shards = tp_shard_weights(w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], tp_plan(cfg.H, cfg.I, world), rank)
        tp = TensorParallelMoE(shards, hidden=cfg.H, ispp=cfg.I, num_experts=cfg.E, top_k=cfg.top_k, rank=rank,
                               world=world, swiglu_limit=cfg.swiglu_limit)
        got = tp(A, ids, tw)
        torch.cuda.synchronize()
        err = float((got - want).abs().max())
        scale = max(float(want.abs().max()), 1.0)
        ok = err <= 2 ** -7 * scale   # the sum over K is split in two and the bf16 activation rounds once on both paths
        open(os.path.join(tmp, f"rank{rank}.txt"), "w").write(f"{int(ok)} err={err} scale={scale}")
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_two_ranks_match_single_rank(tmp_path, oracle_mod):
    """The stage split under a real all-reduce: two NCCL ranks with K-sharded weights reproduce the
    single-rank layer (reference tests/kernels/moe/test_dist_moe.cpp:277-330)."""
    import torch.multiprocessing as mp
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        txt = (tmp_path / f"rank{r}.txt").read_text()
        assert txt.startswith("1"), f"rank {r}: {txt}"
