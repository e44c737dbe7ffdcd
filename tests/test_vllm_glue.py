"""The serving glue: the weight-format pass-through refuses layouts the kernels would misread
(CPU), and the experts object's ``apply`` reproduces the oracle through the reference binding's
call sequence (GPU)."""
import numpy as np
import pytest
import torch

from vkernels_b200 import synthetic as syn
from vkernels_b200.torch_ops import OpNotEligible
from vkernels_b200.vllm_experts import B200FusedExperts, convert_weights_for_b200


def _weights(E=3, H=128, I=64):
    g = torch.Generator().manual_seed(4)
    u8 = lambda *s: torch.randint(0, 256, s, dtype=torch.uint8, generator=g)
    return u8(E, 2 * I, H // 2), u8(E, H, I // 2), u8(E, 2 * I, H // 32), u8(E, H, I // 32)


def test_shim_passes_the_checkpoint_layout_through_and_casts_biases():
    """reference convert_weights_for_vkernel (vllm_experts.py:531-582): no weight or scale
    transform, bf16 biases become fp32, both call shapes are accepted."""
    w13, w2, s13, s2 = _weights()
    b13 = torch.randn(3, 128).to(torch.bfloat16)
    b2 = torch.randn(3, 128).to(torch.bfloat16)
    out = convert_weights_for_b200(w13, w2, s13, s2, w13_bias=b13, w2_bias=b2)
    assert out[0].data_ptr() == w13.data_ptr() and out[1].data_ptr() == w2.data_ptr()
    assert out[2].data_ptr() == s13.data_ptr() and out[3].data_ptr() == s2.data_ptr()
    assert out[4].dtype == torch.float32 and torch.equal(out[4], b13.float()) and out[5].dtype == torch.float32
    # positional biases followed by entries the layer has no use for (input scales, permute indices)
    out2 = convert_weights_for_b200(w13, w2, s13, s2, b13, b2, None, None, "perm", unknown_kw=1)
    assert torch.equal(out2[4], b13.float()) and torch.equal(out2[5], b2.float())
    assert convert_weights_for_b200(w13, w2, s13, s2)[4] is None
    # torch.nn.Parameter-like holders are unwrapped
    assert convert_weights_for_b200(torch.nn.Parameter(w13.float(), requires_grad=False).to(torch.uint8), w2, s13, s2)[0].dtype == torch.uint8


@pytest.mark.parametrize("bad", ["w2_shape", "scale_kmajor", "scale_shuffled_shape", "dtype", "noncontig", "bias_shape", "odd_rows"])
def test_shim_refuses_layouts_the_kernels_would_misread(bad):
    w13, w2, s13, s2 = _weights()
    kw = {}
    if bad == "w2_shape":
        w2 = w2.transpose(1, 2).contiguous()
    elif bad == "scale_kmajor":
        s13 = s13.transpose(1, 2).contiguous()
    elif bad == "scale_shuffled_shape":
        s2 = s2.reshape(3, 64, 4)
    elif bad == "dtype":
        w13 = w13.to(torch.int8)
    elif bad == "noncontig":
        w13 = torch.cat([w13, w13], 2)[:, :, ::2]
    elif bad == "bias_shape":
        kw["w13_bias"] = torch.zeros(3, 64)
    elif bad == "odd_rows":
        w13, s13 = w13[:, :127].contiguous(), s13[:, :127].contiguous()
    with pytest.raises(OpNotEligible):
        convert_weights_for_b200(w13, w2, s13, s2, **kw)


def test_experts_object_shapes_and_eligibility():
    ex = B200FusedExperts(w13_scale=None, w2_scale=None)
    ws13, ws2, out = ex.workspace_shapes(100, 512, 384, 4, 32, 32)
    assert ws13 == (32 * 16 + ((400 - 32 + 15) // 16) * 16, 256) and ws2 == (0,) and out == (100, 384)
    assert ex.supports_activation("SILU") and ex.supports_activation("situ") and not ex.supports_activation("gelu")


@pytest.mark.gpu
def test_experts_apply_matches_the_oracle():
    from gpu_common import DEV, make_case, oracle_layer, oracle_route, to_np
    from helpers import assert_close_bf16

    cfg = syn.scaled(syn.CONFIGS["c0"], H=384, I=192, E=6, top_k=3)
    w, A, r = make_case(cfg, 70)
    ids_np, tw_np, _ = oracle_route(cfg, A, r)
    rng = np.random.default_rng(2)
    b13 = torch.from_numpy(rng.standard_normal((cfg.E, 2 * cfg.I)).astype(np.float32)).to(DEV)
    b2 = torch.from_numpy(rng.standard_normal((cfg.E, cfg.H)).astype(np.float32)).to(DEV)
    w13, w2, s13, s2, b13c, b2c = convert_weights_for_b200(w["w13"], w["w2"], w["w13_scale"], w["w2_scale"],
                                                           b13.to(torch.bfloat16), b2.to(torch.bfloat16))
    ex = B200FusedExperts(w13_scale=s13, w2_scale=s2, w13_bias=b13c, w2_bias=b2c, swiglu_limit=0.7, max_num_tokens=128)
    out = torch.zeros((70, cfg.H), dtype=torch.bfloat16, device=DEV)
    ids = torch.from_numpy(ids_np).to(DEV).to(torch.int64)       # vLLM hands int64 ids over
    tw = torch.from_numpy(tw_np).to(DEV)
    ws13 = torch.empty(ex.workspace_shapes(70, 2 * cfg.I, cfg.H, cfg.top_k, cfg.E, cfg.E)[0], dtype=torch.bfloat16, device=DEV)
    for ws in (ws13, None):                                      # the caller's workspace, then the object's own
        out.zero_()
        ex.apply(out, A, w13, w2, tw, ids, activation="swigluoai", global_num_experts=cfg.E, workspace13=ws)
        torch.cuda.synchronize()
        ref = oracle_layer(A, w, torch.from_numpy(ids_np), tw, swiglu_limit=0.7, b13=to_np(b13c), b2=to_np(b2c))
        assert_close_bf16(to_np(out.float()), ref, "experts.apply", got_is_bf16=True)
    # the same call served from weights prepacked on first use
    exp = B200FusedExperts(w13_scale=s13, w2_scale=s2, w13_bias=b13c, w2_bias=b2c, swiglu_limit=0.7, max_num_tokens=128,
                           prepack=True)
    for _ in range(2):
        out.zero_()
        exp.apply(out, A, w13, w2, tw, ids, activation="swigluoai", global_num_experts=cfg.E, workspace13=ws13)
        torch.cuda.synchronize()
        assert exp._packed is not None and exp._packed.usable
        assert_close_bf16(to_np(out.float()), ref, "experts.apply, prepacked", got_is_bf16=True)
    with pytest.raises(OpNotEligible):
        ex.apply(out, A, w13, w2, tw, ids, activation="gelu", global_num_experts=cfg.E)
