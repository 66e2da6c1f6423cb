"""Generates the golden vectors in this directory from the REFERENCE'S OWN CPU code.

Run in a container where the reference tree is mounted:
    make -C oracle REF_DIR=<checkout of the reference> && python tests/golden/make_golden.py
(`--i4r-only` regenerates the hgn v2 i4r fixture alone; REF_DIR in the environment names the
checkout, default: reference/ next to the repository.)
It calls oracle/_ref/libref.so, i.e. the unmodified Model::moe (src/ref.cpp:563-637),
Checkpoint::q4cp_row (src/hgn.h:249-261) and gguf::dequant_row (src/gguf.h:339-443) of
the reference, on seeded synthetic inputs, and stores the outputs together with CRC32
checksums of the inputs (the inputs are re-created from the seed by
gfx1151_engine_b200/synth.py; the checksum catches a drifting generator).
"""
import dataclasses
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from gfx1151_engine_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def crc(*arrays):
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes(), c)
    return np.uint32(c)


def layer_crc(layer):
    return crc(*[layer[k] for k in sorted(layer)])


def gguf_iq4():
    """GGUF IQ4_NL / IQ4_XS / Q8_0 / Q5_K rows through the reference's dequant_row (src/gguf.h:352-359, 375-441)."""
    nl = synth.make_iq4nl(synth.rng_for(12, 3), 3, 256)
    xs = synth.make_iq4xs(synth.rng_for(12, 4), 3, 512)
    np.savez_compressed(os.path.join(OUT, "gguf_iq4_rows.npz"), iq4nl=nl, iq4nl_rows=oracle.gguf_rows(20, nl, 256, 3, use_ref=True),
                        iq4xs=xs, iq4xs_rows=oracle.gguf_rows(23, xs, 512, 3, use_ref=True))
    q80 = synth.make_q80(synth.rng_for(12, 6), 3, 256)
    np.savez_compressed(os.path.join(OUT, "gguf_q80_rows.npz"), q80=q80, q80_rows=oracle.gguf_rows(8, q80, 256, 3, use_ref=True))
    q5k = synth.make_q5k(synth.rng_for(12, 5), 3, 512)
    np.savez_compressed(os.path.join(OUT, "gguf_q5k_rows.npz"), q5k=q5k, q5k_rows=oracle.gguf_rows(13, q5k, 512, 3, use_ref=True))


I4R_SHAPE = dict(experts=4, topk=2, d=256, mid=128, tokens=6, seed=13)


def i4r_layer(ref_dir):
    """hgn v2 i4r: the reference has no CPU code for this format; its Python converter
    (tools/v2repro/v2enc.py) holds the decode and the rotation. Stored: rows of the rotated-domain
    matrices from i4r_decode_rot, and the output of an ORDINARY SwiGLU MoE in float64 over the
    un-rotated weights unrotate(i4r_decode_rot(...), suh, svh) -- what the rotated dataflow of
    the engine (and of oracle/i4r.py) must reproduce."""
    import math
    if not hasattr(math, "fma"):
        # v2enc builds its table for the "ht" format at import time with math.fma (Python >= 3.13);
        # that table is not used here, so an unfused stand-in is enough to import the module
        math.fma = lambda a, b, c: a * b + c
    sys.path.insert(0, os.path.join(ref_dir, "tools", "v2repro"))
    import v2enc
    c = I4R_SHAPE
    E, k, d, mid, T = c["experts"], c["topk"], c["d"], c["mid"], c["tokens"]
    L = synth.make_i4r_layer(E, d, mid, seed=c["seed"])
    G_gu = v2enc.i4r_decode_rot(*v2enc.i4r_split(L["gate_up"].tobytes(), E, 2 * mid, d))
    G_dn = v2enc.i4r_decode_rot(*v2enc.i4r_split(L["down"].tobytes(), E, d, mid))
    W_gu = v2enc.unrotate(G_gu, L["gu_suh"].astype(np.float32), L["gu_svh"].astype(np.float32)).astype(np.float64)
    W_dn = v2enc.unrotate(G_dn, L["dn_suh"].astype(np.float32), L["dn_svh"].astype(np.float32)).astype(np.float64)
    xb = synth.make_x(synth.rng_for(c["seed"], 9), T, d)
    x = synth.bf16_bits_to_f32(xb).astype(np.float64)
    logits = synth.make_logits(synth.rng_for(c["seed"], 10), T, E)
    ids, w = oracle.router_topk(logits, k)
    y = np.zeros((T, d))
    for t in range(T):
        for s in range(k):
            e = int(ids[t, s])
            gu = W_gu[e] @ x[t]
            g, u = gu[:mid], gu[mid:]
            y[t] += float(w[t, s]) * (W_dn[e] @ (g / (1.0 + np.exp(-g)) * u))
    np.savez_compressed(os.path.join(OUT, "i4r_layer.npz"), y=y, gu_rows=G_gu[1, 126:130].astype(np.float32),
                        dn_rows=G_dn[2, :3].astype(np.float32), crc_layer=layer_crc(L), crc_x=crc(xb), crc_logits=crc(logits))


def main():
    ref_dir = os.environ.get("REF_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    if "--i4r-only" in sys.argv:
        i4r_layer(ref_dir)
        return
    assert oracle.have_ref(), "build oracle/_ref/libref.so first (needs the reference tree)"
    # 1. q4cp rows, including a width whose scale record is padded (640 -> 40 B -> 48 B)
    for cols in (64, 640):
        blob = synth.make_q4cp(synth.rng_for(11, cols), 6, cols, "random")
        rows = oracle.q4cp_rows(blob, 6, cols, 0, 6, use_ref=True)
        np.savez_compressed(os.path.join(OUT, "q4cp_rows_%d.npz" % cols), blob=blob, rows=rows)
    # 2. GGUF rows
    q4k = synth.make_q4k(synth.rng_for(12, 1), 3, 512)
    q51 = synth.make_q51(synth.rng_for(12, 2), 3, 256)
    np.savez_compressed(os.path.join(OUT, "gguf_rows.npz"), q4k=q4k, q4k_rows=oracle.gguf_rows(12, q4k, 512, 3, use_ref=True),
                        q51=q51, q51_rows=oracle.gguf_rows(7, q51, 256, 3, use_ref=True))
    gguf_iq4()
    # 3. tiny layer with shared expert and a random non-uniform code book
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=64, shared=True, router=True, book="random")
    layer = synth.make_layer(spec, seed=3)
    xb = synth.make_x(synth.rng_for(3, 9), 5, spec.d)
    y = oracle.ref_moe_layer(spec, layer, synth.bf16_bits_to_f32(xb))
    np.savez_compressed(os.path.join(OUT, "moe_tiny.npz"), y=y, crc_layer=layer_crc(layer), crc_x=crc(xb))
    # 4. configuration 1 of the benchmark (d=2048, 64 experts, top-8, mid=512, 16 tokens, seed 0).
    #    The reference always evaluates a shared expert; zero scales on its down projection
    #    switch it off exactly (its contribution is 0.0).
    spec1 = dataclasses.replace(synth.CONFIG1, shared=True)
    layer1 = synth.make_layer(spec1, seed=0)
    layer1["sh_down"] = synth.make_q4cp(synth.rng_for(0, 6), spec1.d, spec1.mid, zero_scales=True)
    xb1 = synth.make_x(synth.rng_for(0, 9), 16, spec1.d)
    y1 = oracle.ref_moe_layer(spec1, layer1, synth.bf16_bits_to_f32(xb1))
    routed = {k: layer1[k] for k in ("gate_up", "down", "router_w")}
    np.savez_compressed(os.path.join(OUT, "moe_config1.npz"), y=y1, crc_layer=layer_crc(routed), crc_x=crc(xb1))
    # 5. hgn v2 i4r layer from the reference's converter math
    i4r_layer(ref_dir)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
