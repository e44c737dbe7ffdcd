"""The expert-parallel exchange logic on CPU ranks (gloo, world size 2 and 3): counts, variable
all-to-all splits, row bookkeeping and the rank-ordered combine, with the device steps replaced
by a numpy stand-in and the CPU oracle as the local experts. The sum over ranks must equal the
single-rank oracle, and the reference's own EP forward (dist_moe.cpp:276-328)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class NumpyBackend:
    """CPU stand-in for vkernels_b200.dist.CudaBackend (same contract, no GPU)."""

    def __init__(self, weights, num_experts, rank, world):
        from vkernels_b200.dist import ep_plan
        self.w = weights
        self.b, self.e = ep_plan(num_experts, world, rank)

    def pack(self, x, ids, w, n_shared, world, rank, begins, cursor, row_of, send_x, send_ids, send_w, phase):
        T, k = ids.shape
        bg = begins.tolist()
        for t in range(T):
            need = {rank} if n_shared else set()
            for j in range(k):
                e = int(ids[t, j])
                if 0 <= e < bg[-1]:
                    need.add(max(r for r in range(world) if bg[r] <= e))
            for d in range(world):
                if d not in need:
                    if phase == 1:
                        row_of[t, d] = -1
                    continue
                row = int(cursor[d])
                cursor[d] += 1
                if phase == 0:
                    continue
                row_of[t, d] = row
                send_x[row] = x[t]
                for j in range(k + n_shared):
                    if j < k:
                        e = int(ids[t, j])
                        own = bg[d] <= e < bg[d + 1]
                        send_ids[row, j] = e - bg[d] if own else -1
                        send_w[row, j] = float(w[t, j]) if own else 0.0
                    else:
                        send_ids[row, j] = (bg[d + 1] - bg[d]) + (j - k) if d == rank else -1
                        send_w[row, j] = 1.0 if d == rank else 0.0

    def experts(self, rows, ids, w):
        import oracle
        A = rows.view(torch.int16).numpy().view(np.uint16)
        sl = slice(self.b, self.e)
        out = oracle.moe_layer(A, self.w["w13"][sl], self.w["w13_scale"][sl], self.w["w2"][sl], self.w["w2_scale"][sl],
                               ids.numpy(), w.numpy(), num_experts=self.e - self.b)
        return torch.from_numpy(out)

    def combine(self, back_rows, row_of, T, H, world, out):
        acc = torch.zeros((T, H), dtype=torch.float32)
        for d in range(world):
            r = row_of[:, d].long()
            m = r >= 0
            acc[m] += back_rows[r[m]]
        out.copy_(acc.to(out.dtype))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from helpers import bf16_to_u16
        from vkernels_b200 import synthetic as syn
        from vkernels_b200.dist import ExpertParallelMoE

        cfg = syn.scaled(syn.CONFIGS["c0"], H=128, I=64, E=7, top_k=3)
        w = {k: v.numpy() for k, v in syn.make_expert_weights(cfg).items()}
        T = 12 * world
        A = syn.make_activations(cfg, T)
        rng = np.random.default_rng(5)
        ids = np.stack([rng.permutation(cfg.E)[: cfg.top_k] for _ in range(T)]).astype(np.int32)
        tw = rng.random((T, cfg.top_k), dtype=np.float32)
        lo, hi = rank * 12, (rank + 1) * 12
        layer = ExpertParallelMoE(NumpyBackend(w, cfg.E, rank, world), num_experts=cfg.E, top_k=cfg.top_k,
                                  hidden=cfg.H, rank=rank, world=world)
        y = layer(A[lo:hi].contiguous(), topk=(torch.from_numpy(ids[lo:hi]), torch.from_numpy(tw[lo:hi])))
        full = oracle.moe_layer(bf16_to_u16(A), w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], ids, tw,
                                num_experts=cfg.E)
        err = float(np.max(np.abs(y.float().numpy() - full[lo:hi])))
        scale = float(np.abs(full).max())
        stats = layer.last_stats()
        ok = err <= 2 ** -7 * max(scale, 1.0) and stats["rows_sent"] >= 12 and stats["rows_sent"] <= 12 * world
        if oracle.have_reference() and rank == 0:
            outs = oracle.fused_moe_mxfp4_ep_reference(bf16_to_u16(A), w["w13"], w["w13_scale"], w["w2"],
                                                       w["w2_scale"], ids, tw, num_experts=cfg.E, ep=world)
            ok = ok and float(np.max(np.abs(outs.sum(0)[lo:hi] - y.float().numpy()))) <= 2 ** -7 * max(scale, 1.0)
        open(os.path.join(tmp, f"rank{rank}.txt"), "w").write(f"{int(ok)} err={err} scale={scale} {stats}")
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 3])
def test_ep_exchange_on_gloo_ranks(world, tmp_path, oracle_mod):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        txt = (tmp_path / f"rank{r}.txt").read_text()
        assert txt.startswith("1"), f"rank {r}: {txt}"


def _leaving_worker(rank, world, port, tmp):
    """Rank `world - 1` runs one healthy step and then leaves between steps (no collective in
    flight); the others start a second step and must get an error out of their exchange within
    the process group's timeout instead of waiting forever."""
    import datetime
    import time

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from vkernels_b200 import synthetic as syn
    from vkernels_b200.dist import ExpertParallelMoE

    cfg = syn.scaled(syn.CONFIGS["c0"], H=128, I=64, E=6, top_k=2)
    w = {k: v.numpy() for k, v in syn.make_expert_weights(cfg).items()}
    A = syn.make_activations(cfg, 8 * world)
    rng = np.random.default_rng(rank)
    ids = torch.from_numpy(np.stack([rng.permutation(cfg.E)[: cfg.top_k] for _ in range(8)]).astype(np.int32))
    tw = torch.from_numpy(rng.random((8, cfg.top_k), dtype=np.float32))
    layer = ExpertParallelMoE(NumpyBackend(w, cfg.E, rank, world), num_experts=cfg.E, top_k=cfg.top_k,
                              hidden=cfg.H, rank=rank, world=world)
    x = A[rank * 8:(rank + 1) * 8].contiguous()
    layer(x, topk=(ids, tw))                       # step 1: everybody is there
    verdict = "left"
    if rank != world - 1:
        t0 = time.time()
        try:
            layer(x, topk=(ids, tw))               # step 2: one rank is gone
            verdict = "no error"
        except Exception as e:  # noqa: BLE001 - any error out of the exchange is the expected outcome
            verdict = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    open(os.path.join(tmp, f"rank{rank}.txt"), "w").write(verdict)
    # no destroy_process_group: the group is broken on purpose; the process simply exits
    os._exit(0)


def test_a_rank_that_leaves_between_steps_surfaces_as_an_error(tmp_path, oracle_mod):
    world = 3
    ctx = mp.spawn(_leaving_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    deadline = 90
    import time
    t0 = time.time()
    while not ctx.join(timeout=1.0):
        assert time.time() - t0 < deadline, "ranks are still waiting for the one that left"
    assert (tmp_path / f"rank{world - 1}.txt").read_text() == "left"
    for r in range(world - 1):
        txt = (tmp_path / f"rank{r}.txt").read_text()
        assert txt.startswith("error after"), f"rank {r}: {txt}"


def test_ep_plan_matches_oracle(oracle_mod):
    from vkernels_b200.dist import ep_plan, expert_begins
    for E, ep in [(8, 2), (7, 3), (128, 8), (257, 8), (5, 5)]:
        for r in range(ep):
            assert ep_plan(E, ep, r) == oracle_mod.moe_ep_plan(E, ep, r)
        assert expert_begins(E, ep)[-1] == E
    with pytest.raises(ValueError):
        ep_plan(4, 8, 0)


def test_tp_plan_geometry_and_rejections():
    """Shard geometry of the tensor-parallel split (reference moe_tp_plan, dist_moe.hpp:61-81; its
    own example: hidden 7168 and ispp 3072 at tp = 8 give 896 and 384)."""
    from vkernels_b200.dist import tp_plan
    p = tp_plan(7168, 3072, 8)
    assert (p["hidden_shard"], p["ispp_shard"]) == (896, 384)
    assert p["w13_shard_bytes"] == 2 * 3072 * 448 and p["w13s_shard_bytes"] == 2 * 3072 * 28
    assert p["w2_shard_bytes"] == 7168 * 192 and p["w2s_shard_bytes"] == 7168 * 12
    assert tp_plan(512, 256, 1)["hidden_shard"] == 512
    for bad in [(512, 256, 0), (512, 256, 3), (2880, 2880, 2), (512, 256, 8)]:   # 1440, 64/32: not multiples of 64
        with pytest.raises(ValueError):
            tp_plan(*bad)


def test_tp_shards_are_column_slices():
    from vkernels_b200.dist import tp_plan, tp_shard_weights
    E, H, I = 3, 256, 128
    g = torch.Generator().manual_seed(1)
    w13 = torch.randint(0, 256, (E, 2 * I, H // 2), dtype=torch.uint8, generator=g)
    s13 = torch.randint(0, 256, (E, 2 * I, H // 32), dtype=torch.uint8, generator=g)
    w2 = torch.randint(0, 256, (E, H, I // 2), dtype=torch.uint8, generator=g)
    s2 = torch.randint(0, 256, (E, H, I // 32), dtype=torch.uint8, generator=g)
    plan = tp_plan(H, I, 2)
    parts = [tp_shard_weights(w13, s13, w2, s2, plan, r) for r in range(2)]
    assert torch.equal(torch.cat([p["w13"] for p in parts], 2), w13)
    assert torch.equal(torch.cat([p["w13_scale"] for p in parts], 2), s13)
    assert torch.equal(torch.cat([p["w2"] for p in parts], 2), w2)
    assert torch.equal(torch.cat([p["w2_scale"] for p in parts], 2), s2)
    assert all(p["w13"].is_contiguous() and p["w2_scale"].is_contiguous() for p in parts)
