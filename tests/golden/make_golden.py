"""Generates the golden vectors in this directory from the REFERENCE'S OWN CPU code.

Run in a container where the reference tree is mounted:
    make -C oracle REF_DIR=<checkout of the reference> && python tests/golden/make_golden.py
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


def main():
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
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
