"""GPU: parity at the shapes the benchmark runs, not only at small ones.

Configurations of the benchmark (E=512, top-10, d=4096, mid=1024): the decode / verify
calls with the shared expert (T=1, T=5), a full 16384-token Zipf-routed prefill chunk, the
GGUF variant (Q4_K gate/up, Q5_1 down) at 8192 tokens, the engine's production layer shape
d=2560 / mid=640 (whose q4cp scale records are padded from 40 to 48 bytes, src/hgn.h:230 of
the reference) from memory and from an .hgn file, and intermediate sizes with an odd number
of 64-wide K blocks in the down GEMM. Integer results (top-k ids, permutation) are compared
bit for bit on every token; the layer output against the CPU oracle on a sample of tokens
(the oracle costs ~0.3 core-seconds per token at these shapes) chosen so that tokens of the
most loaded expert and tokens of single-row experts are both in it: max-abs 2e-2, mean-rel
1e-3 after rounding both sides to bf16.
"""
import dataclasses

import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
import oracle
from gfx1151_engine_b200 import synth
from helpers import assert_output_close, bf16_out_to_f32, bf16_tensor, dev_bytes
from test_gpu_parity import bits, make_op, run_layer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big_layer():
    """Routed + shared expert tensors of the benchmark layer (3.6 GB + 21 MB), made once."""
    return synth.make_layer(synth.CONFIG2, seed=0)


def stratified_sample(ids, k, E, n, rng):
    """Token indices: a third with a pair on the most loaded expert, a third with a pair on a
    single-row expert (as far as there are such tokens), the rest drawn at random."""
    T = ids.shape[0]
    hist = np.bincount(ids[:, :k].reshape(-1), minlength=E)
    hot = int(np.argmax(hist))
    on_hot = np.flatnonzero((ids[:, :k] == hot).any(axis=1))
    single = np.flatnonzero(hist == 1)
    on_single = np.flatnonzero(np.isin(ids[:, :k], single).any(axis=1))
    pick = list(rng.permutation(on_hot)[: n // 3]) + list(rng.permutation(on_single)[: n // 3])
    rest = np.setdiff1d(np.arange(T), np.array(pick, dtype=np.int64))
    pick += list(rng.permutation(rest)[: n - len(pick)])
    return np.array(sorted(set(int(t) for t in pick)), dtype=np.int64), hist


def check_integer_routing(op, logits, k, E):
    T = logits.shape[0]
    ids, w, tok, pw, eoff, pid = op.get_routing(T)
    ids_o, w_o, probs = oracle.router_topk(logits, k, want_probs=True)
    assert oracle.count_topk_ties(probs, k) == 0, "seeded input has a probability tie; pick another seed"
    assert np.array_equal(ids[:, :k], ids_o[:, :k])
    assert np.abs(w[:, :k] - w_o[:, :k]).max() <= 1e-6
    tok_o, pw_o, eoff_o, pid_o = oracle.route(ids, w, k, E)
    assert np.array_equal(tok, tok_o) and np.array_equal(eoff, eoff_o) and np.array_equal(pid, pid_o)
    assert np.array_equal(bits(pw), bits(pw_o))
    return ids


@pytest.mark.parametrize("decode_impl", [pkg.DECODE_AUTO, pkg.DECODE_FUSED])
@pytest.mark.parametrize("T", [1, 5])
def test_config2_decode_and_verify(cuda, big_layer, T, decode_impl):
    """Decode (T=1) and verify (T=5) of the benchmark layer with its shared expert: the chained
    GEMV kernels and the one-kernel variant."""
    torch = cuda
    spec = synth.CONFIG2
    logits = synth.make_logits(synth.rng_for(200, T), T, spec.experts)
    xb = synth.make_x(synth.rng_for(200, 9), T, spec.d)
    op = make_op(torch, spec, 16, layer=big_layer, decode_impl=decode_impl)
    y = run_layer(torch, op, spec, xb, logits)
    check_integer_routing(op, logits, spec.topk, spec.experts)
    y_o, _, _ = oracle.moe_forward(spec, big_layer, synth.bf16_bits_to_f32(xb), logits=logits)
    max_abs, mean_rel = assert_output_close(y, y_o, "config 2 T=%d" % T)
    print("config2 T=%d max-abs %.2e mean-rel %.2e" % (T, max_abs, mean_rel))
    op.close()


def test_config3_prefill_chunk_sample(cuda, big_layer):
    """The benchmarked call itself: 16384 tokens, Zipf(1.1) routing, tensor-core path. Routing
    bit-exact on all tokens, output against the oracle on a stratified 256-token sample, and the
    whole output bitwise repeatable."""
    torch = cuda
    spec = synth.CONFIG3
    T = 16384
    logits = synth.make_logits(synth.rng_for(300, 1), T, spec.experts, zipf=True, zipf_rng=synth.rng_for(300, 77))
    xb = synth.make_x(synth.rng_for(300, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=big_layer)
    y = run_layer(torch, op, spec, xb, logits)
    assert np.isfinite(y).all()
    ids = check_integer_routing(op, logits, spec.topk, spec.experts)
    sample, hist = stratified_sample(ids, spec.topk, spec.experts, 256, synth.rng_for(300, 5))
    assert hist.max() > 192 * 16 and (hist == 1).any(), "the chunk should hold a hot expert and single-row experts"
    y_o, _, _ = oracle.moe_forward(spec, big_layer, synth.bf16_bits_to_f32(xb[sample]), logits=logits[sample])
    max_abs, mean_rel = assert_output_close(y[sample], y_o, "config 3 sample")
    print("config3 %d-token sample: max-abs %.2e mean-rel %.2e; pairs max %d, single-row experts %d"
          % (len(sample), max_abs, mean_rel, hist.max(), int((hist == 1).sum())))
    y2 = run_layer(torch, op, spec, xb, logits)
    assert np.array_equal(bits(y), bits(y2)), "prefill path is not bitwise repeatable"
    op.close()


def test_config4_gguf_chunk_sample(cuda):
    """GGUF variant at the benchmark shapes: Q4_K gate/up, Q5_1 down, 8192 tokens, Zipf routing."""
    torch = cuda
    spec = synth.CONFIG4
    layer = synth.make_layer(spec, seed=4)
    T = 8192
    logits = synth.make_logits(synth.rng_for(400, 1), T, spec.experts, zipf=True, zipf_rng=synth.rng_for(400, 77))
    xb = synth.make_x(synth.rng_for(400, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    y = run_layer(torch, op, spec, xb, logits)
    assert np.isfinite(y).all()
    ids = check_integer_routing(op, logits, spec.topk, spec.experts)
    sample, hist = stratified_sample(ids, spec.topk, spec.experts, 128, synth.rng_for(400, 5))
    y_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[sample]), logits=logits[sample])
    max_abs, mean_rel = assert_output_close(y[sample], y_o, "config 4 sample")
    print("config4 %d-token sample: max-abs %.2e mean-rel %.2e" % (len(sample), max_abs, mean_rel))
    # the GEMV path of the same layer (T = 3)
    y3 = run_layer(torch, op, spec, xb[:3], logits[:3])
    y3_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[:3]), logits=logits[:3])
    assert_output_close(y3, y3_o, "config 4 T=3")
    op.close()


# ---------------------------------------------------------------- the engine's own layer shape
def write_hgn(path, tensors):
    from test_file_loaders import write_hgn as w
    w(path, tensors)


@pytest.mark.parametrize("book", ["linear", "random"])
def test_engine_shape_2560_640(cuda, tmp_path, book):
    """d=2560, mid=640: the down tensors' scale records are 40 bytes padded to 48
    (src/hgn.h:230). Dequantised rows bit-exact, and the layer on the GEMV path (T=5) and the
    tensor-core path (T=300), loaded from memory and from an .hgn file."""
    torch = cuda
    spec = synth.LayerSpec(experts=16, topk=4, d=2560, mid=640, shared=True, book=book)
    layer = synth.make_layer(spec, seed=25)
    E, d, mid = spec.experts, spec.d, spec.mid
    assert (mid // 32 * 2) % 16 != 0, "this shape is here for its padded scale records"
    op = make_op(torch, spec, 300, layer=layer)
    for e in (0, E - 1):
        out = torch.empty((d, mid), dtype=torch.float32, device="cuda")
        op.dequant_rows(0, 1, e, 0, d, out)
        want = oracle.q4cp_rows(layer["down"], E * d, mid, e * d, d)
        assert np.array_equal(bits(out.cpu().numpy()), bits(want))
        out = torch.empty((2 * mid, d), dtype=torch.float32, device="cuda")
        op.dequant_rows(0, 0, e, 0, 2 * mid, out)
        want = oracle.q4cp_rows(layer["gate_up"], E * 2 * mid, d, e * 2 * mid, 2 * mid)
        assert np.array_equal(bits(out.cpu().numpy()), bits(want))
    out = torch.empty((d, mid), dtype=torch.float32, device="cuda")
    op.dequant_rows(0, 3, 0, 0, d, out)
    assert np.array_equal(bits(out.cpu().numpy()), bits(oracle.q4cp_rows(layer["sh_down"], d, mid, 0, d)))
    path = str(tmp_path / "engine_shape.hgn")
    write_hgn(path, [
        ("layers.0.mlp.experts.gate_up_proj.weight", 5, (E * 2 * mid, d), layer["gate_up"].tobytes()),
        ("layers.0.mlp.experts.down_proj.weight", 5, (E * d, mid), layer["down"].tobytes()),
        ("layers.0.mlp.shared_expert.gate_proj.weight", 5, (mid, d), layer["sh_gate"].tobytes()),
        ("layers.0.mlp.shared_expert.up_proj.weight", 5, (mid, d), layer["sh_up"].tobytes()),
        ("layers.0.mlp.shared_expert.down_proj.weight", 5, (d, mid), layer["sh_down"].tobytes()),
        ("layers.0.mlp.shared_expert_gate.weight", 0, (1, d), layer["sh_gate_w"].tobytes()),
    ])
    op_file = make_op(torch, spec, 300)
    op_file.load_hgn_file(0, path, model_layer=0)
    for T in (5, 300):
        logits = synth.make_logits(synth.rng_for(25, T), T, E, zipf=T > 16)
        xb = synth.make_x(synth.rng_for(25, 9), T, d)
        y_o, ids_o, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
        y = run_layer(torch, op, spec, xb, logits)
        assert np.array_equal(op.get_routing(T)[0][:, :spec.topk], ids_o[:, :spec.topk])
        max_abs, mean_rel = assert_output_close(y, y_o, "d=2560 mid=640 T=%d" % T)
        print("d=2560 mid=640 book=%s T=%d max-abs %.2e mean-rel %.2e" % (book, T, max_abs, mean_rel))
        assert np.array_equal(bits(run_layer(torch, op_file, spec, xb, logits)), bits(y)), "file path differs from memory path"
    op.close()
    op_file.close()


@pytest.mark.parametrize("mid", [192, 320, 64])
def test_odd_k_block_count_in_down_gemm(cuda, mid):
    """mid = 192 / 320: the down GEMM's K is 3 / 5 blocks of 64 (blocks go in pairs, the last pair
    holds one block); mid = 64 is the single-block case. Tensor-core path against the fp32 path
    on every token and against the oracle; the GEMV path (T=4) too."""
    torch = cuda
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=mid, shared=True, book="random")
    layer = synth.make_layer(spec, seed=61)
    for T in (4, 260):
        logits = synth.make_logits(synth.rng_for(61, T), T, spec.experts, zipf=T > 16)
        xb = synth.make_x(synth.rng_for(61, 9), T, spec.d)
        y_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
        op = make_op(torch, spec, T, layer=layer)
        y = run_layer(torch, op, spec, xb, logits)
        assert_output_close(y, y_o, "mid=%d T=%d" % (mid, T))
        op_simt = make_op(torch, spec, T, impl=pkg.GEMM_SIMT, layer=layer)
        assert_output_close(y, run_layer(torch, op_simt, spec, xb, logits), "mid=%d T=%d vs fp32 path" % (mid, T))
        op.close()
        op_simt.close()


# ---------------------------------------------------------------- invariance audits on the production kernels
@pytest.mark.parametrize("decode_impl", [pkg.DECODE_AUTO, pkg.DECODE_FUSED])
def test_row_invariance_gemv_path(cuda, decode_impl):
    """A token's bytes do not depend on the other tokens of the call on the decode paths either
    (the reference's audit, tools/ktest.cu:920-923, 1152-1271). The one-kernel decode (T <= 8,
    decode_impl = fused) reads an expert once for all the rows that use it: a token alone (T=1, the
    plain path) equals its row inside T=2, 5 and 8 calls bit for bit, which is the reference's
    "dedup == plain" check (tools/moe_gguf_gemv_test.cu:197-223). The chained GEMV kernels
    likewise among themselves (all T <= 16; with the fused implementation 9 <= T <= 16). The routing
    is drawn from 12 experts so that several tokens share experts."""
    torch = cuda
    spec = synth.LayerSpec(experts=12, topk=4, d=512, mid=256, shared=True, book="random")
    layer = synth.make_layer(spec, seed=71)
    logits = synth.make_logits(synth.rng_for(71, 1), 16, spec.experts)
    xb = synth.make_x(synth.rng_for(71, 9), 16, spec.d)
    op = make_op(torch, spec, 16, layer=layer, decode_impl=decode_impl)
    y8 = run_layer(torch, op, spec, xb[:8], logits[:8])
    counts = np.bincount(op.get_routing(8)[0][:, :spec.topk].reshape(-1), minlength=spec.experts)
    assert counts.max() >= 3, "the test wants an expert shared by three or more rows"
    y_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[:8]), logits=logits[:8])
    assert_output_close(y8, y_o, "T=8 decode")
    for T in (2, 5):
        yT = run_layer(torch, op, spec, xb[:T], logits[:T])
        assert np.array_equal(bits(yT), bits(y8[:T])), "T=%d rows differ from the T=8 call" % T
    for t in (0, 4, 7):
        y1 = run_layer(torch, op, spec, xb[t:t + 1], logits[t:t + 1])
        assert np.array_equal(bits(y1[0]), bits(y8[t])), "token %d differs between T=1 and T=8" % t
    y16 = run_layer(torch, op, spec, xb, logits)
    y9 = run_layer(torch, op, spec, xb[:9], logits[:9])
    assert np.array_equal(bits(y9), bits(y16[:9]))
    y_o16, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
    assert_output_close(y16, y_o16, "T=16 decode")
    op.close()


def test_row_invariance_tensor_core_path(cuda):
    """The same on the tensor-core path: a token's row inside a 40-token call equals its row
    inside a 300-token call (other tile widths, other tile positions), bit for bit."""
    torch = cuda
    spec = synth.LayerSpec(experts=16, topk=4, d=512, mid=256, shared=True)
    layer = synth.make_layer(spec, seed=72)
    T = 300
    logits = synth.make_logits(synth.rng_for(72, 1), T, spec.experts, zipf=True)
    xb = synth.make_x(synth.rng_for(72, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    y300 = run_layer(torch, op, spec, xb, logits)
    y40 = run_layer(torch, op, spec, xb[:40], logits[:40])
    assert np.array_equal(bits(y40), bits(y300[:40]))
    sel = np.arange(17, 300, 7)     # 41 tokens from all over the chunk, as a call of their own
    ysel = run_layer(torch, op, spec, xb[sel], logits[sel])
    assert np.array_equal(bits(ysel), bits(y300[sel]))
    op.close()


def test_fp16_range_is_handled_alike_on_both_paths(cuda):
    """The SwiGLU product is stored as fp16 between the two GEMMs on the GEMV path (T <= 16) and
    on the tensor-core path (T > 16) alike. Weights and activations scaled so that many products
    leave the fp16 range: both paths store the largest fp16 number (no infinity), so a token's
    output is finite and the same on both paths (1e-2 of the output's scale: the paths round
    differently), while the fp32 oracle, which has no fp16 intermediate, differs visibly -- the
    proof that the case does saturate. A NaN activation row stays NaN on the tensor-core path
    (it is not clamped to a finite number) and leaves the other rows' bytes untouched."""
    torch = cuda
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=128)
    layer = {"gate_up": synth.make_q4cp(synth.rng_for(81, 1), spec.experts * 2 * spec.mid, spec.d, scale_sigma=2.0),
             "down": synth.make_q4cp(synth.rng_for(81, 2), spec.experts * spec.d, spec.mid, scale_sigma=0.002)}
    T = 40
    logits = synth.make_logits(synth.rng_for(81, 3), T, spec.experts)
    x = synth.rng_for(81, 9).normal(0.0, 16.0, size=(T, spec.d)).astype(np.float32)
    xb = synth.f32_to_bf16_bits(x)
    op = make_op(torch, spec, T, layer=layer)
    y_tc = run_layer(torch, op, spec, xb, logits)
    y_gv = run_layer(torch, op, spec, xb[:4], logits[:4])
    assert np.isfinite(y_tc).all() and np.isfinite(y_gv).all()
    scale = np.abs(y_tc[:4]).max()
    assert np.abs(y_tc[:4] - y_gv).max() <= 1e-2 * scale
    y_o, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[:4]), logits=logits[:4])
    assert np.abs(y_o - y_gv).max() > 5e-2 * scale, "the case does not leave the fp16 range; scale it up"
    # NaN activations on the tensor-core path
    xn = xb.copy()
    xn[3, :] = 0x7FC0
    y_n = run_layer(torch, op, spec, xn, logits)
    assert np.isnan(y_n[3]).all()
    keep = np.arange(T) != 3
    assert np.array_equal(bits(y_n[keep]), bits(y_tc[keep]))
    op.close()


# ---------------------------------------------------------------- non-finite logits, ids out of range
@pytest.mark.parametrize("T", [3, 40])
def test_non_finite_logits_give_valid_ids_and_nan_rows(cuda, T):
    """A NaN (or all -inf) logit row: the router still writes expert ids inside [0, E) -- nothing
    downstream indexes with a wild value -- with NaN weights, so that token's output is NaN and
    every other token's bytes are what they are without it."""
    torch = cuda
    spec = synth.LayerSpec(experts=16, topk=4, d=256, mid=128, shared=True)
    layer = synth.make_layer(spec, seed=73)
    logits = synth.make_logits(synth.rng_for(73, T), T, spec.experts)
    xb = synth.make_x(synth.rng_for(73, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    y_clean = run_layer(torch, op, spec, xb, logits)
    bad = logits.copy()
    bad[1, 5] = np.nan
    bad[2, :] = -np.inf
    y = run_layer(torch, op, spec, xb, bad)
    ids = op.get_routing(T)[0]
    assert ((ids[:, :spec.topk] >= 0) & (ids[:, :spec.topk] < spec.experts)).all()
    assert np.isnan(y[1]).all() and np.isnan(y[2]).all()
    keep = np.array([t for t in range(T) if t not in (1, 2)])
    assert np.array_equal(bits(y[keep]), bits(y_clean[keep]))
    # the oracle behaves the same way (ids in range, NaN output)
    y_o, ids_o, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[1:3]), logits=bad[1:3])
    assert ((ids_o[:, :spec.topk] >= 0) & (ids_o[:, :spec.topk] < spec.experts)).all() and np.isnan(y_o).all()
    op.close()


@pytest.mark.parametrize("T", [3, 40])
def test_caller_ids_out_of_range_are_dropped(cuda, T):
    """b200moe_forward_routed / b200moe_route with an expert id outside [0, E): the pair is
    dropped on the device (never used as an index), the other pairs and tokens are computed as
    usual, and b200moe_synchronize reports B200MOE_ERR_BAD_ARG once. E = 8 and the bad id is 9: even
    without the guard it would stay inside the kernels' 512-entry shared arrays."""
    torch = cuda
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=128)
    layer = synth.make_layer(spec, seed=74)
    logits = synth.make_logits(synth.rng_for(74, T), T, spec.experts)
    xb = synth.make_x(synth.rng_for(74, 9), T, spec.d)
    op = make_op(torch, spec, T, layer=layer)
    y_clean = run_layer(torch, op, spec, xb, logits)
    ids, w = op.get_routing(T)[:2]
    x = bf16_tensor(torch, xb, (T, spec.d))
    ids_bad = ids.copy()
    ids_bad[1, 1] = 9
    out = torch.full((T, spec.d), float("nan"), dtype=torch.bfloat16, device="cuda")
    op.moe_q4w_run(0, x, torch.from_numpy(ids_bad).cuda(), torch.from_numpy(w).cuda(), out)
    with pytest.raises(pkg.B200MoeError) as e:
        op.synchronize()
    assert e.value.status == 1 and "expert id 9" in str(e.value)
    op.synchronize()                                  # reported once, then clear
    y = bf16_out_to_f32(torch, out)
    assert np.isfinite(y).all()
    keep = np.array([t for t in range(T) if t != 1])
    assert np.array_equal(bits(y[keep]), bits(y_clean[keep]))
    _, _, tok, pw, eoff, pid = op.get_routing(T)
    assert eoff[-1] == T * spec.topk - 1 and (pid.reshape(T, -1)[1] == -1).sum() == 1 and (pid >= 0).sum() == T * spec.topk - 1
    # the token's remaining pair alone: the layer with that single expert at its original weight
    w_one = w.copy()
    w_one[1, 1] = 0.0
    out2 = torch.zeros((T, spec.d), dtype=torch.bfloat16, device="cuda")
    op.moe_q4w_run(0, x, torch.from_numpy(ids).cuda(), torch.from_numpy(w_one).cuda(), out2)
    op.synchronize()
    assert np.array_equal(bits(bf16_out_to_f32(torch, out2)[1]), bits(y[1]))
    # the allocation-free bucketing: same rule, the caller sees it in eoff[E]
    tok2 = torch.full((T * 2,), -7, dtype=torch.int32, device="cuda")
    pw2 = torch.zeros((T * 2,), dtype=torch.float32, device="cuda")
    eoff2 = torch.zeros((9,), dtype=torch.int32, device="cuda")
    pid2 = torch.full((T * 2,), -7, dtype=torch.int32, device="cuda")
    ids_dev, w_dev = torch.from_numpy(ids_bad).cuda(), torch.from_numpy(w).cuda()   # (kept alive across the call)
    st = pkg.lib().b200moe_route_static(ids_dev.data_ptr(), w_dev.data_ptr(), 16, T, 2, 8, tok2.data_ptr(), pw2.data_ptr(),
                                        eoff2.data_ptr(), pid2.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(eoff2.cpu().numpy(), eoff) and np.array_equal(pid2.cpu().numpy(), pid)
    assert np.array_equal(tok2.cpu().numpy()[:T * 2 - 1], tok[:T * 2 - 1])
    op.close()


@pytest.mark.parametrize("shape", [dict(experts=64, topk=10, d=512, mid=256, shared=True),
                                   dict(experts=16, topk=4, d=2560, mid=640, shared=True, book="random"),
                                   dict(experts=8, topk=2, d=256, mid=192, shared=False, book="random"),
                                   dict(experts=100, topk=16, d=384, mid=2048, shared=True)])
def test_fused_decode_kernel_shapes(cuda, shape):
    """The one-kernel decode on shapes that exercise its corners: fewer K blocks than warps, an
    intermediate size beyond one 32-group per warp, E not a power of two with k = 16, no shared
    expert; T = 1..8 against the oracle, the caller-ids entry point, and the residual write-back."""
    torch = cuda
    spec = synth.LayerSpec(**shape)
    layer = synth.make_layer(spec, seed=75)
    op = make_op(torch, spec, 8, layer=layer, decode_impl=pkg.DECODE_FUSED)
    for T in (1, 3, 8):
        logits = synth.make_logits(synth.rng_for(75, T), T, spec.experts)
        xb = synth.make_x(synth.rng_for(75, 9), T, spec.d)
        y_o, ids_o, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
        y = run_layer(torch, op, spec, xb, logits)
        ids, w, tok, pw, eoff, pid = op.get_routing(T)
        assert np.array_equal(ids[:, :spec.topk], ids_o[:, :spec.topk])
        tok_o, pw_o, eoff_o, pid_o = oracle.route(ids, w, spec.topk, spec.experts)
        assert np.array_equal(tok, tok_o) and np.array_equal(eoff, eoff_o) and np.array_equal(pid, pid_o)
        assert_output_close(y, y_o, "fused decode %r T=%d" % (shape, T))
        # the seam below the router: caller-supplied ids and weights give the same bytes
        x = bf16_tensor(torch, xb, (T, spec.d))
        out = torch.full((T, spec.d), float("nan"), dtype=torch.bfloat16, device="cuda")
        op.moe_q4w_run(0, x, torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out)
        op.synchronize()
        assert np.array_equal(bits(bf16_out_to_f32(torch, out)), bits(y))
    op.close()


def test_fused_decode_near_tie_takes_the_exact_router(cuda):
    """Two logits of a token's leaders closer than 1e-6: the compact router hands the call to the
    general routing body (the reference's arithmetic); ids and order are the oracle's either way."""
    torch = cuda
    spec = synth.LayerSpec(experts=64, topk=4, d=256, mid=128, shared=True)
    layer = synth.make_layer(spec, seed=76)
    T = 3
    logits = synth.make_logits(synth.rng_for(76, 1), T, spec.experts)
    top = np.argsort(-logits[1])[:2]
    logits[1, top[1]] = np.nextafter(logits[1, top[0]], np.float32(-np.inf))    # one ulp below the leader
    xb = synth.make_x(synth.rng_for(76, 9), T, spec.d)
    y_o, ids_o, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
    _, _, probs = oracle.router_topk(logits, spec.topk, want_probs=True)
    for impl in (pkg.DECODE_AUTO, pkg.DECODE_FUSED):
        op = make_op(torch, spec, 8, layer=layer, decode_impl=impl)
        y = run_layer(torch, op, spec, xb, logits)
        ids = op.get_routing(T)[0]
        if oracle.count_topk_ties(probs, spec.topk) == 0:
            assert np.array_equal(ids[:, :spec.topk], ids_o[:, :spec.topk])
        else:   # the two probabilities are one float: the rule is the lowest id first
            assert sorted(ids[1, :2].tolist()) == sorted(top.tolist()) and ids[1, 0] == min(top)
        assert_output_close(y, y_o, "near tie impl %d" % impl)
        op.close()
