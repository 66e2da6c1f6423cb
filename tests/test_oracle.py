"""CPU: the restated oracle against the golden vectors made by the reference's own code,
and (where the reference build is present) against that code directly."""
import dataclasses
import os

import numpy as np
import pytest

import oracle
from gfx1151_engine_b200 import synth
from helpers import crc, layer_crc


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("cols", [64, 640])
def test_q4cp_rows_golden(golden_dir, cols):
    g = np.load(os.path.join(golden_dir, "q4cp_rows_%d.npz" % cols))
    got = oracle.q4cp_rows(g["blob"], 6, cols, 0, 6)
    assert np.array_equal(bits(got), bits(g["rows"]))
    # a sub-range starts at the right row
    assert np.array_equal(bits(oracle.q4cp_rows(g["blob"], 6, cols, 2, 3)), bits(g["rows"][2:5]))


def test_gguf_rows_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "gguf_rows.npz"))
    assert np.array_equal(bits(oracle.gguf_rows(12, g["q4k"], 512, 3)), bits(g["q4k_rows"]))
    assert np.array_equal(bits(oracle.gguf_rows(7, g["q51"], 256, 3)), bits(g["q51_rows"]))


def test_gguf_iq4_rows_golden(golden_dir):
    """IQ4_NL / IQ4_XS rows against the reference's dequant_row (src/gguf.h:375-406)."""
    g = np.load(os.path.join(golden_dir, "gguf_iq4_rows.npz"))
    assert np.array_equal(bits(oracle.gguf_rows(20, g["iq4nl"], 256, 3)), bits(g["iq4nl_rows"]))
    assert np.array_equal(bits(oracle.gguf_rows(23, g["iq4xs"], 512, 3)), bits(g["iq4xs_rows"]))
    assert np.array_equal(synth.make_iq4nl(synth.rng_for(12, 3), 3, 256), g["iq4nl"])
    assert np.array_equal(synth.make_iq4xs(synth.rng_for(12, 4), 3, 512), g["iq4xs"])
    assert float(np.abs(g["iq4xs_rows"]).max()) > 0 and np.isfinite(g["iq4xs_rows"]).all()


def test_gguf_q5k_rows_golden(golden_dir):
    """Q5_K rows against the reference's dequant_row (src/gguf.h:408-441)."""
    g = np.load(os.path.join(golden_dir, "gguf_q5k_rows.npz"))
    assert np.array_equal(bits(oracle.gguf_rows(13, g["q5k"], 512, 3)), bits(g["q5k_rows"]))
    assert np.array_equal(synth.make_q5k(synth.rng_for(12, 5), 3, 512), g["q5k"])


def test_generators_reproduce_golden_inputs(golden_dir):
    """The synthetic generator must give the bytes the golden outputs were made from."""
    g = np.load(os.path.join(golden_dir, "moe_tiny.npz"))
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=64, shared=True, router=True, book="random")
    layer = synth.make_layer(spec, seed=3)
    assert layer_crc(layer) == g["crc_layer"]
    assert crc(synth.make_x(synth.rng_for(3, 9), 5, spec.d)) == g["crc_x"]


def test_moe_tiny_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe_tiny.npz"))
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=64, shared=True, router=True, book="random")
    layer = synth.make_layer(spec, seed=3)
    x = synth.bf16_bits_to_f32(synth.make_x(synth.rng_for(3, 9), 5, spec.d))
    y, ids, w = oracle.moe_forward(spec, layer, x)
    assert np.array_equal(bits(y), bits(g["y"]))
    assert np.allclose(w[:, :2].sum(1), 1.0, atol=1e-6)


def test_moe_config1_golden(golden_dir):
    """Benchmark configuration 1 (d=2048, 64 experts, top-8, mid=512, 16 tokens, seed 0)."""
    g = np.load(os.path.join(golden_dir, "moe_config1.npz"))
    spec = synth.CONFIG1
    layer = synth.make_layer(spec, seed=0)
    assert layer_crc(layer, ("down", "gate_up", "router_w")) == g["crc_layer"]
    xb = synth.make_x(synth.rng_for(0, 9), 16, spec.d)
    assert crc(xb) == g["crc_x"]
    y, ids, w = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb))
    assert np.array_equal(bits(y), bits(g["y"]))


def test_logits_given_equals_router_weight_path():
    """Feeding the logits the router weight produces must not change anything."""
    spec = synth.LayerSpec(experts=16, topk=4, d=128, mid=64, router=True)
    layer = synth.make_layer(spec, seed=5)
    xb = synth.make_x(synth.rng_for(5, 9), 7, spec.d)
    x = synth.bf16_bits_to_f32(xb)
    y0, ids0, w0 = oracle.moe_forward(spec, layer, x)
    rw = synth.bf16_bits_to_f32(layer["router_w"]).astype(np.float64)
    logits = (x.astype(np.float64) @ rw.T).astype(np.float32)
    # reproduce the reference's sequential double accumulation exactly
    for t in range(x.shape[0]):
        for e in range(spec.experts):
            a = 0.0
            for c in range(spec.d):
                a += float(rw[e, c]) * float(x[t, c])
            logits[t, e] = np.float32(a)
    y1, ids1, w1 = oracle.moe_forward(spec, layer, x, logits=logits)
    assert np.array_equal(ids0, ids1) and np.array_equal(bits(y0), bits(y1))


@pytest.mark.skipif(not oracle.have_ref(), reason="reference build (oracle/_ref) not present")
def test_against_reference_build():
    spec = synth.LayerSpec(experts=8, topk=3, d=128, mid=64, shared=True, router=True, book="random")
    layer = synth.make_layer(spec, seed=21)
    x = synth.bf16_bits_to_f32(synth.make_x(synth.rng_for(21, 9), 6, spec.d))
    yr = oracle.ref_moe_layer(spec, layer, x)
    yo, _, _ = oracle.moe_forward(spec, layer, x)
    assert np.array_equal(bits(yr), bits(yo))
    blob = layer["down"]
    a = oracle.q4cp_rows(blob, spec.experts * spec.d, spec.mid, 5, 9)
    b = oracle.q4cp_rows(blob, spec.experts * spec.d, spec.mid, 5, 9, use_ref=True)
    assert np.array_equal(bits(a), bits(b))


def test_router_and_route_properties():
    rng = synth.rng_for(7, 1)
    T, E, k = 300, 64, 6
    logits = synth.make_logits(rng, T, E, zipf=True)
    ids, w, probs = oracle.router_topk(logits, k, want_probs=True)
    assert oracle.count_topk_ties(probs, k) == 0
    # descending probability, k distinct experts, weights normalised
    p_sel = np.take_along_axis(probs, ids[:, :k], axis=1)
    assert (np.diff(p_sel, axis=1) <= 0).all()
    assert all(len(set(r[:k])) == k for r in ids)
    assert np.allclose(w[:, :k].sum(1), 1, atol=1e-6)
    tok, pw, eoff, pid = oracle.route(ids, w, k, E)
    # eoff is the histogram's prefix sum; rows of one expert hold ascending tokens (stability)
    hist = np.bincount(ids[:, :k].reshape(-1), minlength=E)
    assert np.array_equal(np.diff(eoff), hist) and eoff[-1] == T * k
    for e in range(E):
        seg = tok[eoff[e]:eoff[e + 1]]
        assert (np.diff(seg) > 0).all()
    # pairids: the k rows of a token, in ascending expert order
    row_expert = np.repeat(np.arange(E), hist)
    for t in range(T):
        rows = pid[t * k:(t + 1) * k]
        assert (tok[rows] == t).all() and (np.diff(row_expert[rows]) > 0).all()
    tl = oracle.tiles(eoff, 64)
    assert tl[:, 2].sum() == T * k and (tl[:, 2] <= 64).all() and (tl[:, 2] > 0).all()


def test_empty_and_single_token():
    spec = synth.LayerSpec(experts=8, topk=2, d=128, mid=64)
    layer = synth.make_layer(spec, seed=2)
    lg = synth.make_logits(synth.rng_for(2, 3), 1, 8)
    x = synth.bf16_bits_to_f32(synth.make_x(synth.rng_for(2, 9), 1, spec.d))
    y, ids, w = oracle.moe_forward(spec, layer, x, logits=lg)
    assert y.shape == (1, 128) and np.isfinite(y).all()
    tok, pw, eoff, pid = oracle.route(np.zeros((0, 16), np.int32), np.zeros((0, 16), np.float32), 2, 8)
    assert eoff.tolist() == [0] * 9


def test_q80_rows_match_reference_golden(golden_dir):
    """GGUF Q8_0 rows (the MTP sidecar's experts): the restated dequantiser against rows made by
    the reference's gguf::dequant_row (src/gguf.h:352-359), bit for bit."""
    g = np.load(os.path.join(golden_dir, "gguf_q80_rows.npz"))
    src = synth.make_q80(synth.rng_for(12, 6), 3, 256)
    assert np.array_equal(src, g["q80"]), "generator drifted"
    got = oracle.gguf_rows(8, src, 256, 3)
    assert np.array_equal(got.view(np.uint32), g["q80_rows"].view(np.uint32))


def test_non_finite_logits_keep_ids_in_range():
    """A NaN logit (or a row of -inf) makes every probability NaN (src/ref.cpp:574-582: the maximum
    skips NaN, exp(NaN) poisons the sum): the selection is then arbitrary but the ids are expert
    numbers, the weights NaN and the token's output NaN. The CUDA router is held to the same."""
    spec = synth.LayerSpec(experts=16, topk=4, d=256, mid=64)
    layer = synth.make_layer(spec, seed=5)
    logits = synth.make_logits(synth.rng_for(5, 1), 3, spec.experts)
    logits[0, 3] = np.nan
    logits[1, :] = -np.inf
    ids, w = oracle.router_topk(logits, spec.topk)
    assert ((ids[:, :spec.topk] >= 0) & (ids[:, :spec.topk] < spec.experts)).all()
    assert np.isnan(w[:2, :spec.topk]).all() and np.isfinite(w[2, :spec.topk]).all()
    xb = synth.make_x(synth.rng_for(5, 9), 3, spec.d)
    y, _, _ = oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb), logits=logits)
    assert np.isnan(y[:2]).all() and np.isfinite(y[2]).all()


def test_i4r_oracle_matches_reference_converter_golden(golden_dir):
    """hgn v2 i4r: rows of the rotated-domain matrices equal the reference converter's decode bit
    for bit, and the rotated dataflow of oracle/i4r.py reproduces (1e-5 of the output's scale) the
    float64 output of an ordinary SwiGLU MoE over the reference's UN-rotated weights
    (tests/golden/make_golden.py::i4r_layer; tools/v2repro/v2enc.py of the reference)."""
    from oracle import i4r
    c = dict(experts=4, topk=2, d=256, mid=128, tokens=6, seed=13)   # I4R_SHAPE of tests/golden/make_golden.py
    g = np.load(os.path.join(golden_dir, "i4r_layer.npz"))
    E, k, d, mid, T = c["experts"], c["topk"], c["d"], c["mid"], c["tokens"]
    L = synth.make_i4r_layer(E, d, mid, seed=c["seed"])
    xb = synth.make_x(synth.rng_for(c["seed"], 9), T, d)
    logits = synth.make_logits(synth.rng_for(c["seed"], 10), T, E)
    assert layer_crc(L) == g["crc_layer"] and crc(xb) == g["crc_x"] and crc(logits) == g["crc_logits"], "generator drifted"
    r = i4r.dequant_rot(L["gate_up"], E * 2 * mid, d, 1 * 2 * mid + 126, 4)
    assert np.array_equal(r.view(np.uint32), g["gu_rows"].view(np.uint32))
    r = i4r.dequant_rot(L["down"], E * d, mid, 2 * d, 3)
    assert np.array_equal(r.view(np.uint32), g["dn_rows"].view(np.uint32))
    ids, w = oracle.router_topk(logits, k)
    y = i4r.moe_forward(E, d, mid, L, synth.bf16_bits_to_f32(xb), ids, w, k)
    assert np.abs(y - g["y"]).max() <= 1e-5 * np.abs(g["y"]).max()
