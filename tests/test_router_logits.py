"""Router logits from hidden states (b200moe_load_router / router_logits / forward_hidden)
against the reference's matvec (src/ref.cpp:68-77) as restated by the oracle."""
import os

import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
import oracle
from gfx1151_engine_b200 import synth

from test_gpu_parity import (assert_output_close, bf16_out_to_f32, bf16_tensor, bits, dev_bytes, make_op)


def test_oracle_logits_are_the_layer_oracles():
    """orc_router_logits + logits-given forward == the forward that derives its own logits."""
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=64, router=True)
    layer = synth.make_layer(spec, seed=5)
    x = synth.bf16_bits_to_f32(synth.make_x(synth.rng_for(5, 9), 6, spec.d))
    lg = oracle.router_logits(layer["router_w"], x)
    y0, ids0, w0 = oracle.moe_forward(spec, layer, x)
    y1, ids1, w1 = oracle.moe_forward(spec, layer, x, logits=lg)
    assert np.array_equal(bits(y0), bits(y1)) and np.array_equal(ids0, ids1) and np.array_equal(bits(w0), bits(w1))


def _logits(torch, op, spec, xb):
    T = xb.shape[0]
    x = bf16_tensor(torch, xb, (T, spec.d))
    lg = torch.full((T, spec.experts), float("nan"), dtype=torch.float32, device="cuda")
    op.router_logits(0, x, lg)
    op.synchronize()
    return lg.cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("T", [1, 5, 16])
def test_router_logits_few_tokens(cuda, T):
    """T <= 16: double sums of the exact products -- the reference's float except on a rounding
    boundary -- and the reference's own arithmetic for the experts that decide the top-k."""
    torch = cuda
    spec = synth.LayerSpec(experts=64, topk=8, d=2048, mid=512, router=True)
    layer = synth.make_layer(spec, seed=11)
    xb = synth.make_x(synth.rng_for(11, 9), T, spec.d)
    op = make_op(torch, spec, 16, layer=layer)
    op.load_router(0, dev_bytes(torch, layer["router_w"]))
    lg = _logits(torch, op, spec, xb)
    lg_o = oracle.router_logits(layer["router_w"], synth.bf16_bits_to_f32(xb))
    assert np.abs(lg - lg_o).max() <= 1.2e-7 * max(1.0, np.abs(lg_o).max())   # at most the last bit
    assert (bits(lg) != bits(lg_o)).mean() < 0.01
    ids, w = oracle.router_topk(lg, spec.topk)
    ids_o, w_o = oracle.router_topk(lg_o, spec.topk)
    assert np.array_equal(ids, ids_o)
    np.testing.assert_allclose(w, w_o, rtol=1e-6, atol=0)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(300, 64, 512), (700, 512, 1024), (257, 200, 256)])
def test_router_logits_gemm_and_exact_routing(cuda, shape):
    """Tensor-core logits are within 2e-5 of the reference's; after the exact recomputation of
    near-tied tokens the top-k ids (and their order) are the reference's for every token."""
    torch = cuda
    T, E, d = shape
    spec = synth.LayerSpec(experts=E, topk=min(8, E // 4), d=d, mid=128, router=True)
    layer = synth.make_layer(spec, seed=12)
    xb = synth.make_x(synth.rng_for(12, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    op.load_router(0, dev_bytes(torch, layer["router_w"]))
    lg = _logits(torch, op, spec, xb)
    lg_o = oracle.router_logits(layer["router_w"], synth.bf16_bits_to_f32(xb))
    assert np.isfinite(lg).all()
    assert np.abs(lg - lg_o).max() <= 2e-5 * max(1.0, np.abs(lg_o).max())
    ids, _ = oracle.router_topk(lg, spec.topk)
    ids_o, _ = oracle.router_topk(lg_o, spec.topk)
    assert np.array_equal(ids[:, :spec.topk], ids_o[:, :spec.topk])


@pytest.mark.gpu
def test_forward_hidden_against_reference_golden(cuda, golden_dir):
    """Configuration 1 from hidden states: the golden output is the reference's Model::moe, which
    derives its logits from the router weight."""
    torch = cuda
    g = np.load(os.path.join(golden_dir, "moe_config1.npz"))
    spec = synth.CONFIG1
    layer = synth.make_layer(spec, seed=0)
    xb = synth.make_x(synth.rng_for(0, 9), 16, spec.d)
    x = synth.bf16_bits_to_f32(xb)
    _, ids_o, w_o = oracle.moe_forward(spec, layer, x)
    op = make_op(torch, spec, 16, layer=layer)
    op.load_router(0, dev_bytes(torch, layer["router_w"]))
    out = torch.full((16, spec.d), float("nan"), dtype=torch.bfloat16, device="cuda")
    op.moe_hidden(0, bf16_tensor(torch, xb, (16, spec.d)), out)
    op.synchronize()
    ids, w = op.get_routing(16)[:2]
    assert np.array_equal(ids[:, :spec.topk], ids_o[:, :spec.topk])
    np.testing.assert_allclose(w[:, :spec.topk], w_o[:, :spec.topk], rtol=1e-6, atol=0)
    assert_output_close(bf16_out_to_f32(torch, out), g["y"], "config 1 from hidden states")


@pytest.mark.gpu
def test_forward_hidden_prefill_matches_logits_entry(cuda):
    """T > 16: forward_hidden = router_logits + forward, byte for byte."""
    torch = cuda
    spec = synth.LayerSpec(experts=64, topk=8, d=512, mid=128, router=True)
    layer = synth.make_layer(spec, seed=13)
    T = 300
    xb = synth.make_x(synth.rng_for(13, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    op.load_router(0, dev_bytes(torch, layer["router_w"]))
    x = bf16_tensor(torch, xb, (T, spec.d))
    lg = torch.empty((T, spec.experts), dtype=torch.float32, device="cuda")
    op.router_logits(0, x, lg)
    a = torch.zeros((T, spec.d), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    op.moe_b(0, x, lg, a)
    op.moe_hidden(0, x, b)
    op.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    y_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb))
    assert_output_close(bf16_out_to_f32(torch, b), y_o, "forward from hidden states")
