"""Expert-parallel fused MXFP4 MoE over torch.distributed (NCCL on NVLink / NVSwitch).

Partition: rank r owns a contiguous expert range, ``E // world`` each with the first
``E % world`` ranks taking one more (reference src/c/vkernels/dist/dist_moe.cpp:225-240).
Each rank owns ``T / world`` tokens and routes them locally. One layer call is

  1. route the local tokens                                   (router kernels)
  2. count the tokens that must visit each rank, exchange the counts (one small all-to-all; the
     only host read of the step, needed for the split sizes of the variable-size exchanges)
  3. pack one activation row per (token, destination rank) with its slots rewritten to the
     destination's LOCAL expert ids, -1 for slots owned elsewhere - the masking rule of
     dist_moe.cpp:242-274                                      (pack kernel)
  4. all-to-all: activation rows (bf16) and slot metadata
  5. the single-GPU alignment + fused layer on the received rows -> fp32 partial rows
  6. all-to-all back: partial rows (fp32 on the wire)
  7. per token, add the at most ``world`` returned rows in ascending rank order -> bf16
                                                                 (combine kernel)

The reference's own EP forward keeps the activations replicated and sums dense per-rank
outputs (dist_moe.cpp:276-328); the sum over ranks computed here is the same quantity, and
tests check it against that function. Always-on shared experts are replicated: each rank applies
them to its own tokens as extra local experts after its routed ones.

Peer-memory form (``ExpertParallelMoE.enable_peer_memory``, CUDA only): steps 3-7 shrink to an
exchange of routing records. Every rank keeps its activations and an fp32 output buffer in
symmetric memory (``torch.distributed._symmetric_memory``: each rank's buffer is mapped into every
other rank's address space); the row gather of the expert kernels reads a token's row where it
lives (peer loads over NVLink) and the down-GEMM epilogue adds its result into the home rank's
output row (``red.global.add.v4.f32`` over NVLink). Dispatch and combine are thereby fused into
the two kernels that needed the data anyway; two cross-rank barriers bracket the expert kernels
(inputs written and outputs zeroed before; all additions done after). If symmetric memory cannot
be set up the layer stays on the collective form above.

The device-side steps are reached through a small ``backend`` object so the exchange logic can be
exercised on CPU ranks (gloo) with a stand-in backend; the default backend calls the CUDA library
and has no CPU path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import native_runtime as nr


def balanced_expert_order(load, world: int):
    """Expert numbering that evens out the ranks' load under the contiguous plan of ``ep_plan``:
    experts are dealt to the ranks heaviest first, each to the rank with the least load so far that
    still has room (every rank keeps exactly its ``ep_plan`` share), and the result lists rank 0's
    experts (ascending), then rank 1's, and so on. ``load``: slots per expert measured on a
    representative batch. Returns a list ``order`` with ``order[new_id] = old_id``. The reference
    plan (src/c/vkernels/dist/dist_moe.cpp:225-260) is contiguous in the checkpoint's numbering;
    renumbering the experts (weights and router rows together) keeps that plan and its dispatch
    unchanged. One expert heavier than a rank's fair share still sets the floor: replication is
    not built."""
    E = len(load)
    sizes = [ep_plan(E, world, r)[1] - ep_plan(E, world, r)[0] for r in range(world)]
    members = [[] for _ in range(world)]
    total = [0.0] * world
    for e in sorted(range(E), key=lambda i: (-float(load[i]), i)):
        r = min((r for r in range(world) if len(members[r]) < sizes[r]), key=lambda r: (total[r], r))
        members[r].append(e)
        total[r] += float(load[e])
    return [e for r in range(world) for e in sorted(members[r])]


def ep_plan(num_experts: int, ep: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the experts owned by `rank` (dist_moe.cpp:225-240)."""
    if ep <= 0 or not (0 <= rank < ep) or num_experts < ep:
        raise ValueError("ep_plan: need ep > 0, 0 <= rank < ep, num_experts >= ep")
    base, rem = divmod(num_experts, ep)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def expert_begins(num_experts: int, ep: int) -> list[int]:
    return [ep_plan(num_experts, ep, r)[0] for r in range(ep)] + [num_experts]


# ---------------------------------------------------------------------------------------------
# tensor parallelism (weights sharded along the reduction dimensions)
# ---------------------------------------------------------------------------------------------

def tp_plan(hidden: int, ispp: int, tp: int) -> dict:
    """Shard geometry of one tensor-parallel rank (reference dist_moe.hpp:61-81, ``moe_tp_plan``):
    w13 is cut along hidden, w2 along ispp; both shards must stay multiples of 64."""
    if tp <= 0 or hidden % tp or ispp % tp:
        raise ValueError("tp_plan: tp must be positive and divide hidden and ispp")
    hs, ish = hidden // tp, ispp // tp
    if hs % 64 or ish % 64:
        raise ValueError("tp_plan: hidden / tp and ispp / tp must be multiples of 64")
    return {"tp": tp, "hidden": hidden, "ispp": ispp, "hidden_shard": hs, "ispp_shard": ish,
            "w13_shard_bytes": 2 * ispp * (hs // 2), "w13s_shard_bytes": 2 * ispp * (hs // 32),
            "w2_shard_bytes": hidden * (ish // 2), "w2s_shard_bytes": hidden * (ish // 32)}


def tp_shard_weights(w13, w13_scale, w2, w2_scale, plan: dict, rank: int) -> dict:
    """Rank ``rank``'s contiguous column slices of the packed weights and scales (reference
    ``moe_tp_shard_w13`` / ``moe_tp_shard_w2``, dist_moe.hpp:83-98); biases stay whole."""
    hs, ish = plan["hidden_shard"], plan["ispp_shard"]
    return {"w13": w13[:, :, rank * hs // 2:(rank + 1) * hs // 2].contiguous(),
            "w13_scale": w13_scale[:, :, rank * hs // 32:(rank + 1) * hs // 32].contiguous(),
            "w2": w2[:, :, rank * ish // 2:(rank + 1) * ish // 2].contiguous(),
            "w2_scale": w2_scale[:, :, rank * ish // 32:(rank + 1) * ish // 32].contiguous()}


class TensorParallelMoE:
    """One rank of the tensor-parallel layer (reference ``fused_moe_mxfp4_tp_rank``,
    dist_moe.hpp:100-131): activations and routing are replicated, the rank holds K-shards of
    the weights, and the two partial results are all-reduced over the group between the stages:

        gate/up partial sums -> all-reduce -> bias + activation -> down partial sums
        -> all-reduce -> bias, routing weight, combine

    CUDA only (NCCL all-reduce on the current stream)."""

    def __init__(self, shards: dict, *, hidden: int, ispp: int, num_experts: int, top_k: int, rank: int, world: int,
                 group=None, b13=None, b2=None, swiglu_limit: float = 0.0, activation: int = 0, beta: float = 4.0,
                 linear_beta: float = 25.0):
        self.plan = tp_plan(hidden, ispp, world)
        self.w = shards
        self.hidden, self.ispp, self.num_experts, self.top_k = hidden, ispp, num_experts, top_k
        self.rank, self.world, self.group = rank, world, group
        self.b13, self.b2 = b13, b2
        self.swiglu_limit, self.activation, self.beta, self.linear_beta = swiglu_limit, activation, beta, linear_beta

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        """x [T, hidden] bf16 (the same on every rank), routing [T, k] -> fp32 [T, hidden] (the same
        on every rank)."""
        from . import torch_ops as ops

        T = x.shape[0]
        dev = x.device
        sids, eids, _ = ops.moe_align_block_size(topk_ids, self.num_experts, 16)
        EM = sids.numel()
        flat = sids.long().clamp(max=T * self.top_k - 1)
        tws = torch.where(sids < T * self.top_k, topk_w.reshape(-1)[flat], torch.zeros((), device=dev))
        hs, ish = self.plan["hidden_shard"], self.plan["ispp_shard"]
        gate_up = torch.zeros((EM, 2 * self.ispp), dtype=torch.float32, device=dev)
        ops.moe_gateup_preact(x, self.w["w13"], self.w["w13_scale"], sids, eids, gate_up, top_k=self.top_k,
                              k_base=self.rank * hs)
        dist.all_reduce(gate_up, group=self.group)
        act = torch.zeros((EM, self.ispp), dtype=torch.bfloat16, device=dev)
        ops.moe_act_epilogue(gate_up, act, sids, eids, M=T, top_k=self.top_k, b13=self.b13,
                             swiglu_limit=self.swiglu_limit, activation=self.activation, beta=self.beta,
                             linear_beta=self.linear_beta)
        partial = torch.zeros((EM, self.hidden), dtype=torch.float32, device=dev)
        ops.moe_down_preact(act, self.w["w2"], self.w["w2_scale"], sids, eids, partial, M=T, top_k=self.top_k,
                            k_base=self.rank * ish)
        dist.all_reduce(partial, group=self.group)
        out = torch.zeros((T, self.hidden), dtype=torch.float32, device=dev)
        ops.moe_combine(partial, tws.contiguous(), sids, eids, out, top_k=self.top_k, b2=self.b2)
        return out

    __call__ = forward


class CudaBackend:
    """Device steps of the EP layer on the CUDA library."""

    def __init__(self, layer, device):
        self.layer = layer          # vkernels_b200.experts.FusedMoEMxfp4 holding the LOCAL experts
        self.device = torch.device(device)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def route(self, x, logits=None):
        return self.layer.route(x, logits=logits)

    def pack(self, x, ids, w, n_shared, world, rank, begins, cursor, row_of, send_x, send_ids, send_w, phase):
        T, H = x.shape
        p = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_pack(
                p(x), p(ids), p(w), T, H, ids.shape[1], n_shared, world, rank, p(begins), p(cursor),
                p(row_of), p(send_x), p(send_ids), p(send_w), phase, self._stream())
        nr.check(rc, "ep_pack")

    def experts(self, rows, ids, w):
        """fp32 [R, H]: the local experts applied to received rows."""
        return self.layer.experts_fp32(rows, ids, w)

    def pack_meta(self, ids, w, n_shared, world, rank, begins, cursor, meta):
        T = ids.shape[0]
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_pack_meta(
                ids.data_ptr(), w.data_ptr(), T, ids.shape[1], n_shared, world, rank, begins.data_ptr(),
                cursor.data_ptr(), meta.data_ptr(), self._stream())
        nr.check(rc, "ep_pack_meta")

    def unpack_meta(self, meta, R, slots, recv_counts, world, x_bases, out_bases, H, ids, w, a_rows, out_rows):
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_unpack_meta(
                meta.data_ptr(), R, slots, recv_counts.data_ptr(), world, x_bases.data_ptr(),
                out_bases.data_ptr(), H, ids.data_ptr(), w.data_ptr(), a_rows.data_ptr(),
                out_rows.data_ptr(), self._stream())
        nr.check(rc, "ep_unpack_meta")

    def pack_meta_peer(self, ids, w, n_shared, world, rank, begins, cursor, meta_bases, count_bases, cap):
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_pack_meta_peer(
                ids.data_ptr(), w.data_ptr(), ids.shape[0], ids.shape[1], n_shared, world, rank,
                begins.data_ptr(), cursor.data_ptr(), meta_bases.data_ptr(), count_bases.data_ptr(), cap,
                self._stream())
        nr.check(rc, "ep_pack_meta_peer")

    def flag_barrier(self, flag_bases, world, rank, slot, epoch_counter, limit_clocks):
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_flag_barrier(flag_bases.data_ptr(), world, rank, slot, 0,
                                                               limit_clocks, epoch_counter.data_ptr(), self._stream())
        nr.check(rc, "ep_flag_barrier")

    def unpack_meta_peer(self, meta, recv_counts, world, cap, slots, x_bases, out_bases, H, out_rows_per_token, ids, w,
                         a_rows, out_rows):
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_unpack_meta_peer(
                meta.data_ptr(), recv_counts.data_ptr(), world, cap, slots, x_bases.data_ptr(),
                out_bases.data_ptr(), H, out_rows_per_token, ids.data_ptr(), w.data_ptr(), a_rows.data_ptr(),
                out_rows.data_ptr(), self._stream())
        nr.check(rc, "ep_unpack_meta_peer")

    def experts_rows(self, a_rows, out_rows, ids, w, store_slots=False):
        self.layer.experts_rows(a_rows, out_rows, ids, w, store_slots=store_slots)

    def combine_slots(self, part, ids, w, n_experts, y):
        T, k = ids.shape
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_combine_slots(part.data_ptr(), ids.data_ptr(), w.data_ptr(), T, k,
                                                                n_experts, y.shape[1], y.data_ptr(), None, self._stream())
        nr.check(rc, "ep_combine_slots")

    def combine(self, back_rows, row_of, T, H, world, out):
        with torch.cuda.device(self.device):
            rc = nr.load_library().vk_cuda_moe_ep_combine(back_rows.data_ptr(), row_of.data_ptr(), T, H, world,
                                                          out.data_ptr(), None, self._stream())
        nr.check(rc, "ep_combine")


class ExpertParallelMoE:
    """One MoE layer sharded over the ranks of a process group."""

    def __init__(self, backend, *, num_experts: int, top_k: int, hidden: int, n_shared: int = 0,
                 rank: int | None = None, world: int | None = None, group=None, device="cpu"):
        self.backend = backend
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.num_experts, self.top_k, self.hidden, self.n_shared = num_experts, top_k, hidden, n_shared
        self.slots = top_k + n_shared
        self.device = torch.device(device)
        self.begins_host = expert_begins(num_experts, self.world)
        self.begins = torch.tensor(self.begins_host, dtype=torch.int32, device=self.device)
        self._stats = {}
        self.count_local_slots = False   # last_stats()["local_slots"]: one extra host read per step
        self.time_phases = False         # last_stats()["phase_ms"]: CUDA events between the phases
        self._peer = None                # symmetric buffers of the peer-memory form
        self._last_routing = None        # (ids, w) of the most recent call (views of layer buffers)

    @classmethod
    def from_config(cls, cfg, *, rank, world, device, max_tokens, group=None, seed=None, expert_order=None):
        """Generates this rank's slice of the seeded weights of a benchmark configuration.
        ``expert_order`` (see ``balanced_expert_order``): position p of the layer's expert numbering
        holds expert ``expert_order[p]`` of the configuration - weights and router rows alike, so
        the layer is the same function with its experts renumbered, and the contiguous ranges of
        the plan become whatever sets the order groups together."""
        from . import synthetic as syn
        from .experts import FusedMoEMxfp4

        b, e = ep_plan(cfg.E, world, rank)
        # every rank draws the same stream and keeps its slice (+ the shared experts)
        full = syn.make_expert_weights(cfg, seed=seed, backend="torch", device=device)
        order = list(range(cfg.E)) if expert_order is None else [int(v) for v in expert_order]
        if sorted(order) != list(range(cfg.E)):
            raise ValueError("expert_order must be a permutation of the routed experts")
        if expert_order is not None and cfg.n_group != 1:
            raise ValueError("group-limited routing depends on the experts' numbering: no renumbering for it")
        keep = order[b:e] + list(range(cfg.E, cfg.n_weight_experts))
        idx = torch.tensor(keep, device=device)
        w = {k: v.index_select(0, idx).contiguous() for k, v in full.items()}
        del full
        torch.cuda.empty_cache()
        r = syn.make_router(cfg, seed=seed, device=device)
        if expert_order is not None:
            oi = torch.tensor(order, device=device)
            r = {k: (None if v is None else v.index_select(0, oi).contiguous()) for k, v in r.items()}
        local = FusedMoEMxfp4(w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], top_k=cfg.top_k,
                              router_weight=r["wr"], router_bias=r["bias"], routing=cfg.routing,
                              renorm=cfg.renorm, scaling=cfg.scaling, n_group=cfg.n_group,
                              topk_group=cfg.topk_group, n_shared=cfg.shared_experts,
                              swiglu_limit=cfg.swiglu_limit, max_tokens=max_tokens * world)
        return cls(CudaBackend(local, device), num_experts=cfg.E, top_k=cfg.top_k, hidden=cfg.H,
                   n_shared=cfg.shared_experts, rank=rank, world=world, group=group, device=device)

    def last_stats(self) -> dict:
        return dict(self._stats)

    def enable_peer_memory(self, max_tokens: int) -> bool:
        """Sets up the peer-memory form for up to ``max_tokens`` local tokens per call. Collective:
        every rank of the group must call it. Returns False (and leaves the layer on the collective
        form) when symmetric memory is unavailable on any rank."""
        ok, err = 1, ""
        peer = None
        try:
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else dist.group.WORLD
            H = self.hidden
            x_sym = symm.empty((max_tokens, H), dtype=torch.bfloat16, device=self.device)
            # one fp32 row per (token, slot): the owners of the experts store their results here
            out_sym = symm.empty((max_tokens, self.slots, H), dtype=torch.float32, device=self.device)
            stride = 1 + 2 * self.slots
            meta_sym = symm.empty((self.world * max_tokens, stride), dtype=torch.int32, device=self.device)
            cnt_sym = symm.empty((32,), dtype=torch.int32, device=self.device)
            flag_sym = symm.empty((8 * 32,), dtype=torch.int32, device=self.device)
            flag_sym.zero_()
            hx = symm.rendezvous(x_sym, group)
            ho = symm.rendezvous(out_sym, group)
            hm = symm.rendezvous(meta_sym, group)
            hc = symm.rendezvous(cnt_sym, group)
            hf = symm.rendezvous(flag_sym, group)
            dev_ptrs = lambda h: torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=self.device)
            n_rows = self.world * max_tokens
            peer = {"x": x_sym, "out": out_sym, "meta": meta_sym, "cnt": cnt_sym, "hx": hx, "ho": ho,
                    "x_bases": dev_ptrs(hx), "out_bases": dev_ptrs(ho), "meta_bases": dev_ptrs(hm),
                    "cnt_bases": dev_ptrs(hc), "flags": flag_sym, "flag_bases": dev_ptrs(hf),
                    # barrier epochs live on the device (one counter per barrier slot), so a captured
                    # step replays them; every rank runs the same number of barriers
                    "epochs": torch.zeros(8, dtype=torch.int32, device=self.device),
                    "max_tokens": max_tokens,
                    # routing arrays and row addresses of the expert call, one per record slot
                    "ids": torch.empty((n_rows, self.slots), dtype=torch.int32, device=self.device),
                    "w": torch.empty((n_rows, self.slots), dtype=torch.float32, device=self.device),
                    "a_rows": torch.empty(n_rows, dtype=torch.int64, device=self.device),
                    "out_rows": torch.empty(n_rows, dtype=torch.int64, device=self.device),
                    "cursor": torch.zeros(self.world, dtype=torch.int32, device=self.device)}
        except Exception as e:  # noqa: BLE001 - any failure means "not available here"
            ok, err = 0, f"{type(e).__name__}: {e}"
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        # also orders every rank's zeroed flag array before anyone's first flag barrier
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            self._peer = peer
            return True
        self._peer = None
        self._stats["peer_memory_error"] = err
        return False

    # A cross-rank wait must end by itself when a rank has left: about four seconds of SM clock,
    # after which the status word reports the missing rank (``torch_ops.kernel_status``).
    BARRIER_LIMIT_CLOCKS = 8_000_000_000

    def _barrier(self, slot: int) -> None:
        """Flag barrier over the ranks of the peer-memory form, as a kernel on the current stream
        (bounded wait; see ``vk_cuda_moe_ep_flag_barrier``). Both slots advance once per step."""
        peer = self._peer
        self.backend.flag_barrier(peer["flag_bases"], self.world, self.rank, slot, peer["epochs"],
                                  self.BARRIER_LIMIT_CLOCKS)

    def capture(self, x: torch.Tensor, logits=None):
        """Captures one step of the peer-memory form on ``x`` (use ``input_buffer``) into a CUDA
        graph; returns ``(graph, y)``. The step has no host reads and no collective calls - router,
        record exchange, both flag barriers, the expert kernels and the combine are kernels on one
        stream - so a replay costs one launch of host time instead of twenty, which is what a
        sub-millisecond step at 8 ranks is otherwise bound by. Collective: every rank captures, and
        afterwards every rank replays the same number of times."""
        if self._peer is None:
            raise RuntimeError("capture needs the peer-memory form (enable_peer_memory)")
        from . import torch_ops as ops

        self.time_phases = self.count_local_slots = False
        layer = self.backend.layer
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            ops.reserve_workspace(layer._workspace_bytes(), self.device)   # this stream's scratch block
            for _ in range(2):
                self.forward(x, logits=logits)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y = self.forward(x, logits=logits)
        self._capture_stream = side
        return graph, y

    def input_buffer(self, T: int) -> torch.Tensor:
        """The first T rows of this rank's activation buffer in peer-visible memory ([T, H] bf16).
        Activations written (or copied from the host) straight into it are read by the owners of
        the experts where they lie: ``forward`` then skips its own copy."""
        if self._peer is None:
            raise RuntimeError("input_buffer needs the peer-memory form (enable_peer_memory)")
        return self._peer["x"][:T]

    def _forward_peer(self, x: torch.Tensor, topk=None, logits=None) -> torch.Tensor:
        """One step of the peer-memory form: route -> routing records to the owners (peer stores)
        -> barrier -> local experts over all record slots, reading token rows where they live and
        STORING every slot's result row into the home rank's [T, slots, H] buffer -> barrier ->
        ordered sum of each token's slots on the home rank (bf16 out). No atomics and no
        zeroing: every slot row is written exactly once per step."""
        T, H = x.shape
        world, rank, slots = self.world, self.rank, self.slots
        dev = x.device
        peer = self._peer
        marks = []

        def mark(name):
            if self.time_phases:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        if topk is None:
            ids_full, w_full = self.backend.route(x, logits=logits) if logits is not None else self.backend.route(x)
        else:
            ids_full, w_full = topk
            if self.n_shared and ids_full.shape[1] == self.top_k:   # append the always-on slots
                sh = torch.arange(self.num_experts, self.num_experts + self.n_shared, dtype=torch.int32, device=dev)
                ids_full = torch.cat([ids_full, sh.expand(T, -1)], 1).contiguous()
                w_full = torch.cat([w_full, torch.ones((T, self.n_shared), dtype=torch.float32, device=dev)], 1).contiguous()
        ids, w = ids_full[:, : self.top_k].contiguous(), w_full[:, : self.top_k].contiguous()
        self._last_routing = (ids, w)
        mark("route")
        # this rank's tokens where every rank can reach them (no copy when the caller wrote them there)
        x_sym, part = peer["x"][:T], peer["out"][:T]
        if x.data_ptr() != x_sym.data_ptr():
            x_sym.copy_(x)
        # routing records straight into the destination ranks' receive areas, then the counts
        cap = peer["max_tokens"]
        self.backend.pack_meta_peer(ids, w, self.n_shared, world, rank, self.begins, peer["cursor"], peer["meta_bases"],
                                    peer["cnt_bases"], cap)
        mark("records")
        # every rank's tokens, records and counts are in place
        self._barrier(0)
        mark("barrier_in")
        r_ids, r_w, a_rows, out_rows = peer["ids"], peer["w"], peer["a_rows"], peer["out_rows"]
        self.backend.unpack_meta_peer(peer["meta"], peer["cnt"], world, cap, slots, peer["x_bases"],
                                      peer["out_bases"], H, slots, r_ids, r_w, a_rows, out_rows)
        self.backend.experts_rows(a_rows, out_rows, r_ids, r_w, store_slots=True)
        mark("experts")
        R_send = R_recv = local_slots = None
        if self.count_local_slots:   # host reads, for reporting only
            R_recv = int(peer["cnt"][:world].sum())
            local_slots = int((r_ids >= 0).sum())
        # every rank's stores into this rank's slot rows are done
        self._barrier(1)
        mark("barrier_out")
        out = torch.empty((T, H), dtype=x.dtype, device=dev)
        self.backend.combine_slots(part, ids_full, w_full, self.num_experts + self.n_shared, out)
        mark("combine")
        phase_ms = None
        if self.time_phases:
            torch.cuda.synchronize(dev)
            phase_ms = {marks[i + 1][0]: round(marks[i][1].elapsed_time(marks[i + 1][1]), 4) for i in range(len(marks) - 1)}
        stride = 1 + 2 * slots
        known = R_recv is not None
        self._stats = {"rows_sent": R_send, "rows_received": R_recv, "tokens_local": T, "form": "peer memory",
                       # router (weight split + GEMM + plane sum at prefill sizes) + top-k, records + counts, barrier,
                       # unpack, alignment, gather (+ tile list) + two GEMMs, barrier, combine
                       "launches_per_step": (4 if T > 512 else 2) + 2 + 1 + 1 + (1 if world * cap * slots <= 1024 else 3) + 3 + 1 + 1,
                       "dispatch_bytes": R_recv * stride * 4 if known else None, "combine_bytes": 0,
                       "peer_read_bytes": R_recv * H * 2 if known else None,
                       "peer_store_bytes": local_slots * H * 4 if local_slots is not None else None,
                       "local_slots": local_slots, "phase_ms": phase_ms}
        return out

    def forward(self, x: torch.Tensor, topk=None, logits=None) -> torch.Tensor:
        """x [T_local, H] bf16 -> bf16 [T_local, H]. `topk` = (ids [T, k] int32 GLOBAL expert ids,
        weights [T, k] fp32) skips the router; `logits` [T_local, E] fp32 replaces the router GEMM."""
        if self._peer is not None:
            # Every rank must take the same form (one waits at flags, the other inside a NCCL
            # all-to-all otherwise), so a batch beyond the registered buffers is an error here
            # rather than a silent switch of form on this rank alone.
            if x.shape[0] > self._peer["max_tokens"]:
                raise ValueError(f"peer-memory form was set up for {self._peer['max_tokens']} tokens per rank, "
                                 f"got {x.shape[0]}; call enable_peer_memory with a larger budget on every rank")
            return self._forward_peer(x, topk, logits)
        T, H = x.shape
        world, rank, slots = self.world, self.rank, self.slots
        dev = x.device
        marks = []

        def mark(name):
            if self.time_phases:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        if topk is None:
            ids, w = self.backend.route(x, logits=logits) if logits is not None else self.backend.route(x)
            ids, w = ids[:, : self.top_k].contiguous(), w[:, : self.top_k].contiguous()
        else:
            ids, w = topk
        self._last_routing = (ids, w)
        mark("route")
        # 2. counts
        counts = torch.zeros(world, dtype=torch.int32, device=dev)
        self.backend.pack(x, ids, w, self.n_shared, world, rank, self.begins, counts, None, None, None, None, 0)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)
        both = torch.stack([counts, recv_counts]).cpu()          # the step's one host read
        send_n, recv_n = both[0].tolist(), both[1].tolist()
        R_send, R_recv = sum(send_n), sum(recv_n)
        mark("counts")
        # 3. pack
        cursor = (torch.cumsum(counts, 0) - counts).to(torch.int32)
        row_of = torch.empty((T, world), dtype=torch.int32, device=dev)
        send_x = torch.empty((max(R_send, 1), H), dtype=x.dtype, device=dev)
        send_ids = torch.empty((max(R_send, 1), slots), dtype=torch.int32, device=dev)
        send_w = torch.empty((max(R_send, 1), slots), dtype=torch.float32, device=dev)
        self.backend.pack(x, ids, w, self.n_shared, world, rank, self.begins, cursor, row_of, send_x,
                          send_ids, send_w, 1)
        mark("pack")
        # 4. dispatch
        recv_x = torch.empty((max(R_recv, 1), H), dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv_x[:R_recv], send_x[:R_send], recv_n, send_n, group=self.group)
        recv_ids = torch.empty((max(R_recv, 1), slots), dtype=torch.int32, device=dev)
        recv_w = torch.empty((max(R_recv, 1), slots), dtype=torch.float32, device=dev)
        dist.all_to_all_single(recv_ids[:R_recv], send_ids[:R_send], recv_n, send_n, group=self.group)
        dist.all_to_all_single(recv_w[:R_recv], send_w[:R_send], recv_n, send_n, group=self.group)
        mark("dispatch")
        # 5. local experts
        if R_recv > 0:
            part = self.backend.experts(recv_x[:R_recv], recv_ids[:R_recv], recv_w[:R_recv])
        else:
            part = torch.zeros((0, H), dtype=torch.float32, device=dev)
        mark("experts")
        local_slots = int((recv_ids[:R_recv] >= 0).sum()) if self.count_local_slots else None
        # 6. return
        back = torch.empty((max(R_send, 1), H), dtype=torch.float32, device=dev)
        dist.all_to_all_single(back[:R_send], part, send_n, recv_n, group=self.group)
        mark("return")
        # 7. combine
        out = torch.empty((T, H), dtype=x.dtype, device=dev)
        self.backend.combine(back, row_of, T, H, world, out)
        mark("combine")
        phase_ms = None
        if self.time_phases:
            torch.cuda.synchronize(dev)
            phase_ms = {marks[i + 1][0]: round(marks[i][1].elapsed_time(marks[i + 1][1]), 4) for i in range(len(marks) - 1)}
        self._stats = {"rows_sent": R_send, "rows_received": R_recv, "tokens_local": T,
                       "launches_per_step": 2 + 2 + 1 + (1 if R_recv * slots <= 1024 else 3) + 4,
                       "dispatch_bytes": R_send * (H * 2 + slots * 8), "combine_bytes": R_recv * H * 4,
                       "form": "collective", "local_slots": local_slots, "phase_ms": phase_ms}
        return out

    __call__ = forward
