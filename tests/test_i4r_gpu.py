"""GPU: hgn v2 i4r routed experts (dtype 23, Hadamard-rotated 4-bit, scale per 128 columns)
through the C ABI against the CPU restatement oracle/i4r.py, which is pinned on the reference
converter's decode and un-rotation (tests/golden/i4r_layer.npz).

Rows of the repacked images decode bit-exactly; the layer output is held to the suite's usual
bound (max-abs 2e-2, mean-rel 1e-3 after rounding both sides to bf16; the reference's own
check of its tensor-core i4r kernels allows relative L2 1e-2, tools/moe_lut_test.cu:33)."""
import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
import oracle
from gfx1151_engine_b200 import synth
from helpers import assert_output_close, bf16_out_to_f32, bf16_tensor, dev_bytes
from oracle import i4r

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def make_i4r_op(torch, E, k, d, mid, max_tokens, layer, **kw):
    op = pkg.MoeOperator(E, k, d, mid, max_tokens, **kw)
    op.load_i4r(0, dev_bytes(torch, layer["gate_up"]), dev_bytes(torch, layer["down"]),
                dev_bytes(torch, layer["gu_suh"]), dev_bytes(torch, layer["gu_svh"]),
                dev_bytes(torch, layer["dn_suh"]), dev_bytes(torch, layer["dn_svh"]))
    return op


def run(torch, op, d, xb, logits):
    T = xb.shape[0]
    x = bf16_tensor(torch, xb, (T, d))
    lg = torch.from_numpy(np.ascontiguousarray(logits, np.float32)).cuda()
    out = torch.full((T, d), float("nan"), dtype=torch.bfloat16, device="cuda")   # NaN-prefilled: must be fully written
    op.moe_b(0, x, lg, out)
    op.synchronize()
    return bf16_out_to_f32(torch, out)


def test_i4r_rows_bit_exact(cuda):
    torch = cuda
    E, k, d, mid = 4, 2, 256, 128
    L = synth.make_i4r_layer(E, d, mid, seed=13)
    op = make_i4r_op(torch, E, k, d, mid, 8, L)
    for which, rows_per, cols, key in ((0, 2 * mid, d, "gate_up"), (1, d, mid, "down")):
        for e in (0, 3):
            out = torch.empty((rows_per, cols), dtype=torch.float32, device="cuda")
            op.dequant_rows(0, which, e, 0, rows_per, out)
            op.synchronize()
            want = i4r.dequant_rot(L[key], E * rows_per, cols, e * rows_per, rows_per)
            assert np.array_equal(bits(out.cpu().numpy()), bits(want)), (key, e)
    op.close()


@pytest.mark.parametrize("T", [1, 5, 40, 300])
def test_i4r_layer_matches_oracle(cuda, T):
    """Decode, verify and prefill sizes (all on the tensor-core kernels), host AND device pointers
    for the weights, every output element written."""
    torch = cuda
    E, k, d, mid = 16, 4, 512, 256
    L = synth.make_i4r_layer(E, d, mid, seed=17)
    logits = synth.make_logits(synth.rng_for(17, T), T, E, zipf=T > 16)
    xb = synth.make_x(synth.rng_for(17, 9), T, d)
    op = make_i4r_op(torch, E, k, d, mid, T, L)
    y = run(torch, op, d, xb, logits)
    ids, w, *_ = op.get_routing(T)
    ids_o, w_o = oracle.router_topk(logits, k)
    assert np.array_equal(ids[:, :k], ids_o[:, :k])
    y_o = i4r.moe_forward(E, d, mid, L, synth.bf16_bits_to_f32(xb), ids_o, w_o, k)
    max_abs, mean_rel = assert_output_close(y, y_o, "i4r T=%d" % T)
    print("i4r T=%d max-abs %.2e mean-rel %.2e" % (T, max_abs, mean_rel))
    if T == 5:   # the same from host pointers
        op2 = pkg.MoeOperator(E, k, d, mid, T)
        op2.load_i4r(0, L["gate_up"], L["down"], L["gu_suh"], L["gu_svh"], L["dn_suh"], L["dn_svh"])
        assert np.array_equal(bits(run(torch, op2, d, xb, logits)), bits(y))
        op2.close()
    op.close()


def test_i4r_engine_shape_and_row_invariance(cuda):
    """The engine's layer shape (d=2560, mid=640: 20 and 5 blocks of 128, odd numbers of K blocks
    in neither GEMM) against the oracle on a few tokens, and a token's bytes inside a 40-token
    call equal its bytes inside a 300-token call."""
    torch = cuda
    E, k, d, mid = 8, 2, 2560, 640
    L = synth.make_i4r_layer(E, d, mid, seed=19)
    T = 300
    logits = synth.make_logits(synth.rng_for(19, 1), T, E, zipf=True)
    xb = synth.make_x(synth.rng_for(19, 9), T, d)
    op = make_i4r_op(torch, E, k, d, mid, T, L)
    y300 = run(torch, op, d, xb, logits)
    y40 = run(torch, op, d, xb[:40], logits[:40])
    assert np.array_equal(bits(y40), bits(y300[:40]))
    sel = np.arange(0, 300, 50)
    ids_o, w_o = oracle.router_topk(logits[sel], k)
    y_o = i4r.moe_forward(E, d, mid, L, synth.bf16_bits_to_f32(xb[sel]), ids_o, w_o, k)
    assert_output_close(y300[sel], y_o, "i4r d=2560 mid=640")
    op.close()


def test_i4r_hc_write_back_and_refusals(cuda):
    """forward_hc adds the rotated-back result into the residual state as for the other formats;
    a handle with a shared expert or the fp32 kernels refuses the format."""
    torch = cuda
    E, k, d, mid, T = 8, 2, 256, 128, 24
    L = synth.make_i4r_layer(E, d, mid, seed=23)
    logits = synth.make_logits(synth.rng_for(23, 1), T, E)
    xb = synth.make_x(synth.rng_for(23, 9), T, d)
    op = make_i4r_op(torch, E, k, d, mid, T, L)
    y = run(torch, op, d, xb, logits)
    y_o = i4r.moe_forward(E, d, mid, L, synth.bf16_bits_to_f32(xb), *oracle.router_topk(logits, k), k)
    assert_output_close(y, y_o, "i4r T=24")
    rng = synth.rng_for(23, 5)
    r0_bits = synth.f32_to_bf16_bits(rng.normal(0.0, 1.0, size=(T, 4, d)).astype(np.float32))
    w4 = rng.normal(0.0, 2.0, size=(T, 4)).astype(np.float32)
    inj = (np.float32(2.0) / (np.float32(1.0) + np.exp(-w4 * np.float32(0.25)))).astype(np.float32)
    want = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(r0_bits) + inj[:, :, None] * y_o[:, None, :]))
    state = bf16_tensor(torch, r0_bits, (T, 4, d))
    op.moe_b_hc(0, bf16_tensor(torch, xb, (T, d)), torch.from_numpy(logits).cuda(), torch.from_numpy(w4).cuda(), state)
    op.synchronize()
    got = bf16_out_to_f32(torch, state.reshape(T * 4, d)).reshape(T, 4, d)
    assert np.isfinite(got).all()
    assert np.all(np.abs(got - want) <= 2 * 2e-2 + np.abs(want) * 2.0 ** -7)
    assert float(np.mean(got == want)) > 0.95
    op.close()
    for kw in ({"has_shared": True}, {"gemm_impl": pkg.GEMM_SIMT}):
        bad = pkg.MoeOperator(E, k, d, mid, T, **kw)
        with pytest.raises(pkg.B200MoeError) as ei:
            bad.load_i4r(0, L["gate_up"], L["down"], L["gu_suh"], L["gu_svh"], L["dn_suh"], L["dn_svh"])
        assert ei.value.status == 2   # B200MOE_ERR_UNSUPPORTED
        bad.close()
