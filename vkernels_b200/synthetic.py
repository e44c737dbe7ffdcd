"""Seeded synthetic workloads with the shapes and value distributions of the
five benchmark configurations of the fused MXFP4 MoE layer.

No dataset is involved: every tensor is drawn from a seeded generator.

* activations ``A [T, H]``: bf16 = RNE(N(0, 1))
* router weight ``Wr [E, H]`` fp32 ~ N(0, 0.02); sigmoid-router bias ``[E]`` ~ N(0, 0.01)
* expert weights: E2M1 nibble codes drawn uniformly, low nibble = even k, and one
  ue8m0 scale byte per 32 K-elements = 127 + uniform integer exponent.
  ``codes="finite"`` draws from the 12 codes whose value is finite under the
  layer's table (0..5 and 8..13; codes 6/7/14/15 decode to +-inf/NaN and turn
  every output into NaN); ``codes="all"`` draws from all 16 and is used only to
  check that inf/NaN propagate the same way as in the CPU oracle.

``backend="numpy"`` (PCG64) is bit-reproducible on any machine and is what the
committed golden vectors use; ``backend="torch"`` draws on the target device
and is meant for the multi-gigabyte configurations.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

BASE_SEED = 0xB200
FINITE_CODES = np.array([0, 1, 2, 3, 4, 5, 8, 9, 10, 11, 12, 13], dtype=np.uint8)


@dataclasses.dataclass(frozen=True)
class MoEConfig:
    name: str
    config_id: int
    H: int
    I: int
    E: int
    top_k: int
    T: tuple  # the batch sizes the configuration names
    routing: str = "softmax"  # "softmax" | "sigmoid_group"
    renorm: bool = True
    scaling: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    swiglu_limit: float = 0.0
    scale_exp: tuple = (-9, -5)
    shared_experts: int = 0
    zipf_alpha: float | None = None

    @property
    def seed(self) -> int:
        return BASE_SEED + self.config_id

    @property
    def n_weight_experts(self) -> int:
        return self.E + self.shared_experts

    @property
    def slots(self) -> int:
        return self.top_k + self.shared_experts

    def expert_weight_bytes(self) -> int:
        """Packed codes + scales of one expert: 1.59375 * I * H."""
        ih = self.I * self.H
        return ih + ih // 16 + ih // 2 + ih // 32

    def flops(self, T: int) -> int:
        """Useful flops: 6*T*slots*I*H (gate, up, down; padding rows not counted)."""
        return 6 * T * self.slots * self.I * self.H


CONFIGS = {
    "c0": MoEConfig("c0_smoke", 0, H=512, I=256, E=8, top_k=2, T=(64,), scale_exp=(-8, -4)),
    "c1": MoEConfig("c1_gptoss20b_decode", 1, H=2880, I=2880, E=32, top_k=4, T=(1, 8, 32, 64, 128),
                    swiglu_limit=7.0),
    "c2": MoEConfig("c2_gptoss120b_prefill", 2, H=2880, I=2880, E=128, top_k=4, T=(8192,)),
    "c3": MoEConfig("c3_deepseekv3", 3, H=7168, I=2048, E=256, top_k=8, T=(16384,),
                    routing="sigmoid_group", scaling=2.5, n_group=8, topk_group=4,
                    shared_experts=1),
    "c4": MoEConfig("c4_zipf", 4, H=2880, I=2880, E=128, top_k=4, T=(1, 16, 256, 4096),
                    zipf_alpha=1.2),
}


def scaled(cfg: MoEConfig, **kw) -> MoEConfig:
    """A smaller/larger variant of a configuration (used by tests)."""
    return dataclasses.replace(cfg, **kw)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    b = b + 0x7FFF + ((b >> 16) & 1)
    return (b >> 16).astype(np.uint16)


def _np_rng(cfg: MoEConfig, stream: int, seed: int | None):
    return np.random.Generator(np.random.PCG64([cfg.seed if seed is None else seed, stream]))


def make_expert_weights(cfg: MoEConfig, *, codes: str = "finite", seed: int | None = None,
                        backend: str = "numpy", device="cpu", n_experts: int | None = None) -> dict:
    """Returns torch uint8 tensors w13 [E', 2I, H/2], w13_scale [E', 2I, H/32],
    w2 [E', H, I/2], w2_scale [E', H, I/32] with E' = routed + shared experts."""
    En = cfg.n_weight_experts if n_experts is None else n_experts
    shapes = {
        "w13": (En, 2 * cfg.I, cfg.H // 2),
        "w13_scale": (En, 2 * cfg.I, cfg.H // 32),
        "w2": (En, cfg.H, cfg.I // 2),
        "w2_scale": (En, cfg.H, cfg.I // 32),
    }
    lo, hi = cfg.scale_exp
    out = {}
    if backend == "numpy":
        rng = _np_rng(cfg, 1, seed)
        n_codes = 12 if codes == "finite" else 16
        for name, shp in shapes.items():
            if name.endswith("_scale"):
                arr = (127 + rng.integers(lo, hi + 1, size=shp, dtype=np.int16)).astype(np.uint8)
            else:
                arr = np.empty(shp, np.uint8)
                for e in range(En):  # per expert, to bound temporary memory
                    c = rng.integers(0, n_codes, size=(2,) + shp[1:], dtype=np.uint8)
                    if codes == "finite":
                        c = FINITE_CODES[c]
                    arr[e] = c[0] | (c[1] << 4)
            out[name] = torch.from_numpy(arr).to(device)
        return out
    if backend != "torch":
        raise ValueError(f"unknown backend {backend!r}")
    g = torch.Generator(device=device)
    g.manual_seed((cfg.seed if seed is None else seed) * 7919 + 1)
    for name, shp in shapes.items():
        if name.endswith("_scale"):
            out[name] = (127 + torch.randint(lo, hi + 1, shp, generator=g, device=device,
                                             dtype=torch.int16)).to(torch.uint8)
        else:
            # a few large launches per tensor (in slabs of at most ~1 GB of temporaries)
            t = torch.empty(shp, dtype=torch.uint8, device=device)
            per = max(1, (1 << 29) // (shp[1] * shp[2]))
            for e0 in range(0, En, per):
                e1 = min(En, e0 + per)
                n_codes = 12 if codes == "finite" else 16
                c = torch.randint(0, n_codes, (2, e1 - e0) + shp[1:], generator=g, device=device,
                                  dtype=torch.uint8)
                if codes == "finite":
                    c += (c >= 6).to(torch.uint8) * 2     # 0..11 -> {0..5, 8..13}
                t[e0:e1] = c[0] | (c[1] << 4)
                del c
            out[name] = t
    return out


def make_activations(cfg: MoEConfig, T: int, *, seed: int | None = None, stream: int = 2,
                     backend: str = "numpy", device="cpu") -> torch.Tensor:
    """A [T, H] bf16 = RNE(N(0,1))."""
    if backend == "numpy":
        x = _np_rng(cfg, stream, seed).standard_normal((T, cfg.H), dtype=np.float32)
        bits = f32_to_bf16_bits(x)
        return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(device)
    g = torch.Generator(device=device)
    g.manual_seed((cfg.seed if seed is None else seed) * 7919 + stream)
    return torch.randn((T, cfg.H), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def make_router(cfg: MoEConfig, *, seed: int | None = None, device="cpu") -> dict:
    """Router weight Wr [E, H] fp32 ~ N(0, 0.02) and, for the sigmoid router, bias [E] ~ N(0, 0.01)."""
    rng = _np_rng(cfg, 3, seed)
    wr = (0.02 * rng.standard_normal((cfg.E, cfg.H), dtype=np.float32)).astype(np.float32)
    out = {"wr": torch.from_numpy(wr).to(device), "bias": None}
    if cfg.routing == "sigmoid_group":
        out["bias"] = torch.from_numpy(
            (0.01 * rng.standard_normal(cfg.E, dtype=np.float32)).astype(np.float32)).to(device)
    return out


def zipf_log_popularity(cfg: MoEConfig, *, seed: int | None = None) -> np.ndarray:
    """log p(e) with p ~ rank^-alpha over a seeded permutation of the experts."""
    rng = _np_rng(cfg, 4, seed)
    perm = rng.permutation(cfg.E)
    p = (1.0 + np.arange(cfg.E, dtype=np.float64)) ** (-float(cfg.zipf_alpha))
    p /= p.sum()
    logp = np.empty(cfg.E, np.float64)
    logp[perm] = np.log(p)
    return logp.astype(np.float32)


def make_zipf_logits(cfg: MoEConfig, T: int, *, seed: int | None = None, device="cpu") -> torch.Tensor:
    """Router logits [T, E] fp32 = Gumbel(0,1) noise + log p_zipf(e): the top-1 pick of a row
    is an exact draw from p, further picks are draws without replacement."""
    rng = _np_rng(cfg, 5, seed)
    u = rng.random((T, cfg.E), dtype=np.float64)
    gumbel = -np.log(-np.log(np.clip(u, 1e-12, 1.0 - 1e-12)))
    logits = (gumbel + zipf_log_popularity(cfg, seed=seed)[None, :]).astype(np.float32)
    return torch.from_numpy(logits).to(device)


def weight_bytes_touched(cfg: MoEConfig, n_touched: int) -> int:
    return n_touched * cfg.expert_weight_bytes()


def decode_algorithmic_bytes(cfg: MoEConfig, T: int, n_touched: int) -> int:
    """Weight bytes of the experts the batch touches + A in + bf16 out + router weight."""
    return weight_bytes_touched(cfg, n_touched) + 2 * T * cfg.H * 2 + cfg.E * cfg.H * 4


def describe(cfg: MoEConfig) -> str:
    r = cfg.routing + (f"(g{cfg.n_group}/{cfg.topk_group})" if cfg.n_group > 1 else "")
    return (f"{cfg.name}: H={cfg.H} I={cfg.I} E={cfg.E}+{cfg.shared_experts} top{cfg.top_k} {r} "
            f"scale_exp={cfg.scale_exp} limit={cfg.swiglu_limit}")


__all__ = [n for n in dir() if not n.startswith("_") and n not in ("np", "torch", "math", "dataclasses")]
