"""Seeded synthetic tensors in the reference's on-disk formats (numpy only).

Test and benchmark data only: the product library (libb200moe.so) and its ctypes binding never
import this module; it sits in the package so that tests, the smoke check and the benchmark find
one generator.

Stand-ins for real checkpoints, with the shapes and value distributions of the
benchmark configurations:
  * hgn q4cp tensors (layout: src/hgn.h:5-9 of the reference): 16 x f32 code book, 4-bit
    codes uniform in [0,15], fp16 scales |N(0, 0.02)| per (row, 32 columns);
  * GGUF Q4_K / Q5_K / Q5_1 / Q8_0 / IQ4_NL / IQ4_XS blocks (layout: src/gguf.h:360-441) with uniform codes and
    block scales normalised so that dequantised magnitudes match the q4cp case;
  * hgn v2 i4r tensors (4-bit codes, fp16 scale per 128 columns) with their sign-scale planes;
  * bf16 activations ~ N(0,1), router logits ~ N(0,1) with an optional per-expert
    Zipf(1.1) bias under a seeded permutation of the expert ids.
The generator is Philox (counter based): the same seed gives the same bytes on every
machine with the same numpy.
"""
from dataclasses import dataclass

import numpy as np

GGML_Q5_1 = 7
GGML_Q4_K = 12


def rng_for(seed, stream=0):
    return np.random.Generator(np.random.Philox(key=[int(seed), int(stream)]))


def f32_to_bf16_bits(a):
    """Round-to-nearest-even conversion of float32 to bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return u.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def q4cp_nbytes(rows, cols):
    return 64 + rows * cols // 2 + rows * (((cols // 32 * 2) + 15) & ~15)


LINEAR_BOOK = ((2.0 * np.arange(16) - 15.0) / 15.0).astype("<f4")


def make_q4cp(rng, rows, cols, book="linear", scale_sigma=0.02, zero_scales=False):
    """One q4cp tensor blob as a uint8 array (16-byte aligned when allocated by numpy)."""
    if isinstance(book, str):
        cb = LINEAR_BOOK if book == "linear" else rng.uniform(-2.0, 2.0, 16).astype("<f4")
    else:
        cb = np.asarray(book, dtype="<f4")
    stride = ((cols // 32 * 2) + 15) & ~15
    out = np.zeros(q4cp_nbytes(rows, cols), dtype=np.uint8)
    out[:64] = cb.view(np.uint8)
    ncode = rows * cols // 2
    out[64:64 + ncode] = rng.integers(0, 256, size=ncode, dtype=np.uint8)
    sc = np.zeros((rows, stride), dtype=np.uint8)
    if not zero_scales:
        s = np.abs(rng.normal(0.0, scale_sigma, size=(rows, cols // 32))).astype("<f2")
        sc[:, : cols // 32 * 2] = s.view(np.uint8).reshape(rows, -1)
    out[64 + ncode:] = sc.reshape(-1)
    return out


def make_q4k(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF Q4_K blocks (144 bytes per 256 elements)."""
    nb = nrows * (k // 256)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 144), dtype=np.uint8)
    blk[:, 0:2] = (a / (63.0 * 15.0)).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:4] = (a / (63.0 * 2.0)).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 4:] = rng.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    return blk.reshape(-1)


def make_q51(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF Q5_1 blocks (24 bytes per 32 elements)."""
    nb = nrows * (k // 32)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 24), dtype=np.uint8)
    blk[:, 0:2] = (a / 31.0).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:4] = (-a / 2.0).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 4:] = rng.integers(0, 256, size=(nb, 20), dtype=np.uint8)
    return blk.reshape(-1)


def zipf_bias(rng, experts, s=1.1, strength=1.0):
    """ln of a Zipf(s) pmf over expert ranks, ranks assigned by a seeded permutation."""
    ranks = rng.permutation(experts) + 1
    pmf = ranks.astype(np.float64) ** (-s)
    pmf /= pmf.sum()
    return (strength * np.log(pmf)).astype(np.float32)


def make_logits(rng, T, experts, zipf=False, zipf_rng=None, strength=1.0):
    lg = rng.normal(0.0, 1.0, size=(T, experts)).astype(np.float32)
    if zipf:
        lg = lg + zipf_bias(zipf_rng if zipf_rng is not None else rng, experts, strength=strength)[None, :]
    return np.ascontiguousarray(lg, dtype=np.float32)


def make_x(rng, T, d):
    """bf16 activations ~ N(0,1) as uint16 bit patterns."""
    return f32_to_bf16_bits(rng.normal(0.0, 1.0, size=(T, d)).astype(np.float32))
def make_q5k(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF Q5_K blocks (176 bytes per 256 elements: d, dmin, 12 packed scale bytes,
    32 bytes of fifth bits, 128 nibble bytes; src/gguf.h:408-441)."""
    nb = nrows * (k // 256)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 176), dtype=np.uint8)
    blk[:, 0:2] = (a / (63.0 * 31.0)).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:4] = (a / (63.0 * 2.0)).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 4:] = rng.integers(0, 256, size=(nb, 172), dtype=np.uint8)
    return blk.reshape(-1)


def make_iq4nl(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF IQ4_NL blocks (18 bytes per 32 elements: fp16 d, 16 code bytes;
    src/gguf.h:375-387). |w| <= a with a = |N(0, sigma)| per block, as for the other formats."""
    nb = nrows * (k // 32)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 18), dtype=np.uint8)
    blk[:, 0:2] = (a / 127.0).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    return blk.reshape(-1)


def make_iq4xs(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF IQ4_XS blocks (136 bytes per 256 elements: fp16 d, u16 + 4 bytes of 6-bit
    sub-block scales, 128 code bytes; src/gguf.h:388-406). d = a / (32 * 127) lands in the fp16
    subnormal range, as in real files."""
    nb = nrows * (k // 256)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 136), dtype=np.uint8)
    blk[:, 0:2] = (a / (32.0 * 127.0)).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, size=(nb, 134), dtype=np.uint8)
    return blk.reshape(-1)


def make_q80(rng, nrows, k, sigma=0.02):
    """nrows rows of GGUF Q8_0 blocks (34 bytes per 32 elements: fp16 d, 32 int8 codes; src/gguf.h:352-359).
    |w| <= a with a = |N(0, sigma)| per block, as for the other formats."""
    nb = nrows * (k // 32)
    a = np.abs(rng.normal(0.0, sigma, size=nb))
    blk = np.zeros((nb, 34), dtype=np.uint8)
    blk[:, 0:2] = (a / 127.0).astype("<f2").view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, size=(nb, 32), dtype=np.uint8)
    return blk.reshape(-1)


def i4r_nbytes(rows, cols):
    return rows * cols // 2 + rows * (cols // 128) * 2


def make_i4r(rng, rows, cols, sigma=0.02):
    """One hgn v2 i4r tensor blob (dtype 23; src/gpu/parts/30_host_util.inc:885-887 and
    40_model.inc:1593-1600 of the reference): rows*cols/2 code bytes (low nibble = even column), then
    one fp16 scale per (row, 128 columns), w = (nib - 8) * scale. Scales are signed, as the
    reference's encoder writes them; |w| <= ~8 * |N(0, sigma / 8)|."""
    out = np.zeros(i4r_nbytes(rows, cols), dtype=np.uint8)
    ncode = rows * cols // 2
    out[:ncode] = rng.integers(0, 256, size=ncode, dtype=np.uint8)
    sc = (rng.normal(0.0, sigma / 8.0, size=(rows, cols // 128))).astype("<f2")
    out[ncode:] = sc.view(np.uint8).reshape(-1)
    return out


def make_i4r_planes(rng, n):
    """A sign-scale plane (.suh / .svh sidecar): fp16, random sign, magnitude around 1."""
    return (rng.choice([-1.0, 1.0], size=n) * rng.uniform(0.5, 1.5, size=n)).astype("<f2")


def make_i4r_layer(experts, d, mid, seed=0):
    """All tensors of one hgn v2 i4r MoE layer: the two blobs and the four planes."""
    return {"gate_up": make_i4r(rng_for(seed, 1), experts * 2 * mid, d),
            "down": make_i4r(rng_for(seed, 2), experts * d, mid),
            "gu_suh": make_i4r_planes(rng_for(seed, 11), d), "gu_svh": make_i4r_planes(rng_for(seed, 12), 2 * mid),
            "dn_suh": make_i4r_planes(rng_for(seed, 13), mid), "dn_svh": make_i4r_planes(rng_for(seed, 14), d)}


GGML_Q5_1, GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_IQ4_NL, GGML_IQ4_XS = 7, 8, 12, 13, 20, 23
_GG_MAKERS = {GGML_Q8_0: make_q80, GGML_Q5_1: make_q51, GGML_Q4_K: make_q4k, GGML_Q5_K: make_q5k, GGML_IQ4_NL: make_iq4nl, GGML_IQ4_XS: make_iq4xs}


def gg_row_bytes(gtype, k):
    """Bytes of one row of k elements in GGUF block type `gtype` (src/gguf.h:49-62)."""
    per, nbytes = {GGML_Q8_0: (32, 34), GGML_Q5_1: (32, 24), GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_IQ4_NL: (32, 18), GGML_IQ4_XS: (256, 136)}[gtype]
    assert k % per == 0
    return k // per * nbytes


@dataclass
class LayerSpec:
    experts: int
    topk: int
    d: int
    mid: int
    shared: bool = False
    fmt: str = "q4cp"      # "q4cp" or "gguf"
    book: str = "linear"   # "linear" or "random" (q4cp only)
    router: bool = False   # also make a bf16 router weight [E][d]
    gg_gu: int = 12        # GGUF block type of gate/up (fmt "gguf"): Q4_K 12, Q5_K 13, IQ4_NL 20, IQ4_XS 23
    gg_dn: int = 7         # GGUF block type of down: Q5_1 7, IQ4_NL 20, IQ4_XS 23


# The benchmark configurations (shapes only; see BASELINE.json `configs`).
CONFIG1 = LayerSpec(experts=64, topk=8, d=2048, mid=512, router=True)
CONFIG2 = LayerSpec(experts=512, topk=10, d=4096, mid=1024, shared=True)
CONFIG3 = LayerSpec(experts=512, topk=10, d=4096, mid=1024)
CONFIG4 = LayerSpec(experts=512, topk=10, d=4096, mid=1024, fmt="gguf")


def make_layer(spec, seed=0):
    """All weight tensors of one MoE layer, as a dict of uint8 / uint16 numpy arrays."""
    E, d, mid = spec.experts, spec.d, spec.mid
    out = {}
    if spec.fmt == "q4cp":
        out["gate_up"] = make_q4cp(rng_for(seed, 1), E * 2 * mid, d, spec.book)
        out["down"] = make_q4cp(rng_for(seed, 2), E * d, mid, spec.book)
    else:
        out["gate"] = _GG_MAKERS[spec.gg_gu](rng_for(seed, 1), E * mid, d)
        out["up"] = _GG_MAKERS[spec.gg_gu](rng_for(seed, 3), E * mid, d)
        out["down"] = _GG_MAKERS[spec.gg_dn](rng_for(seed, 2), E * d, mid)
    if spec.shared:
        out["sh_gate"] = make_q4cp(rng_for(seed, 4), mid, d, spec.book)
        out["sh_up"] = make_q4cp(rng_for(seed, 5), mid, d, spec.book)
        out["sh_down"] = make_q4cp(rng_for(seed, 6), d, mid, spec.book)
        out["sh_gate_w"] = f32_to_bf16_bits(rng_for(seed, 7).normal(0.0, 0.02, size=d).astype(np.float32))
    if spec.router:
        out["router_w"] = f32_to_bf16_bits(rng_for(seed, 8).normal(0.0, 0.02, size=(E, d)).astype(np.float32))
    return out
