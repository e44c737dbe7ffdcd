"""Generates tests/golden/*.npz from the REFERENCE's own code (oracle/_ref/libvkref.so, built
from the reference sources in place) on seeded inputs of the benchmark shapes.

    python tests/golden/make_golden.py

Run where the reference tree is mounted. Inputs are not stored: they are regenerated from the
seeds by vkernels_b200.synthetic (numpy PCG64) and their SHA-256 digests are stored to prove
the regeneration is identical. Routing goldens come from the torch-eager statement in
tests/test_routing_oracle.py (the reference has no CPU router).
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from helpers import bf16_to_u16  # noqa: E402
from test_routing_oracle import eager_sigmoid_group, eager_softmax  # noqa: E402
from vkernels_b200 import synthetic as syn  # noqa: E402


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def layer_case(name, cfg, T, codes="finite"):
    w = {k: v.numpy() for k, v in syn.make_expert_weights(cfg, codes=codes).items()}
    A = bf16_to_u16(syn.make_activations(cfg, T))
    r = syn.make_router(cfg)
    logits = oracle.router_logits(A, r["wr"].numpy())
    ids, tw, margin = oracle.route_softmax_topk(logits, cfg.top_k)
    s, e, EM = oracle.moe_align_block_size(ids, cfg.E, 16, impl="reference")
    ws = oracle.gather_sorted_weights(tw, s)
    out, act = oracle.fused_moe_mxfp4(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"], s, ws, e,
                                      top_k=cfg.top_k, swiglu_limit=cfg.swiglu_limit, impl="reference")
    np.savez_compressed(os.path.join(HERE, name + ".npz"), topk_ids=ids, topk_w=tw, sorted_ids=s,
                        expert_ids=e, out=out, act=act, margin=margin,
                        input_digest=np.array(digest(A, w["w13"], w["w13_scale"], w["w2"], w["w2_scale"])),
                        meta=np.array([T, cfg.H, cfg.I, cfg.E, cfg.top_k], np.int64))
    print(name, "EM", EM, "out max", float(np.nanmax(np.abs(out))) if np.isfinite(out).any() else "nan")


def main():
    if not oracle.have_reference():
        raise SystemExit("oracle/_ref/libvkref.so is missing: run `make -C oracle` with the reference mounted")
    layer_case("c0_smoke", syn.CONFIGS["c0"], 64)
    layer_case("c0_smoke_all_codes", syn.CONFIGS["c0"], 64, codes="all")
    # the decode shape (H = I = 2880) with 4 experts so the weights regenerate quickly
    layer_case("c1_shape_T8_E4", syn.scaled(syn.CONFIGS["c1"], E=4, top_k=2), 8)
    # routing: softmax top-4 of 128 and group-limited sigmoid top-8 of 256
    rng = np.random.default_rng(0xB200)
    l1 = rng.standard_normal((64, 128)).astype(np.float32)
    i1, w1 = eager_softmax(l1, 4)
    l3 = rng.standard_normal((64, 256)).astype(np.float32)
    b3 = (0.01 * rng.standard_normal(256)).astype(np.float32)
    i3, w3 = eager_sigmoid_group(l3, b3, 8, 8, 4, 2.5)
    np.savez_compressed(os.path.join(HERE, "routing.npz"), softmax_logits=l1, softmax_ids=i1, softmax_w=w1,
                        sig_logits=l3, sig_bias=b3, sig_ids=i3, sig_w=w3)
    print("routing goldens written")


if __name__ == "__main__":
    main()
