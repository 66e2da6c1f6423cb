"""hgn v2 "i4r" routed experts on the CPU (numpy) -- TEST INFRASTRUCTURE ONLY.

A restatement of the reference's i4r MoE layer in its fp32 form (the grouped-GEMV branch of
moe_b_v2, src/gpu/parts/40_model.inc:4640-4672: k_v2_rot, k_q4cp_gemv_gg<2>, k_i4r_mid,
k_q4cp_gemv_gd<2>, k_v2_rot), with the format as the engine and its converter read it
(src/gpu/parts/30_host_util.inc:885-887, 40_model.inc:1593-1600, tools/v2repro/v2enc.py:86-96):

    blob   = rows*cols/2 code bytes (low nibble = even column), then fp16 scale[row][cols/128]
    G[r,c] = (nib - 8) * scale[r][c / 128]                       weights in the rotated domain
    W      = diag(svh) . Hn . G . Hn . diag(suh)                 Hn = H128 / sqrt(128), block-diagonal
    layer  : xr = Hn(suh_gu * x);  z = G_gu[e] xr;  g|u = svh_gu * Hn(z);  h = silu(g) * u
             hr = Hn(suh_dn * h);  p = G_dn[e] hr;  y = svh_dn * Hn(sum_e w_e p_e)

The reference has no CPU implementation of this format (src/ref.cpp reads hgn v1 and GGUF only);
parity is pinned on its Python converter instead: tests/golden/i4r_layer.npz holds rows decoded
by tools/v2repro/v2enc.py::i4r_decode_rot and a layer output computed in float64 from the
UN-rotated weights v2enc.unrotate(...) as an ordinary SwiGLU MoE -- which the rotated dataflow
below must reproduce. Only tests may import this module.
"""
import numpy as np


def split(blob, rows, cols):
    b = np.ascontiguousarray(blob, dtype=np.uint8)
    nc = rows * cols // 2
    return b[:nc].reshape(rows, cols // 2), b[nc:nc + rows * (cols // 128) * 2].view("<f2").reshape(rows, cols // 128)


def dequant_rot(blob, rows, cols, row0=0, n=None):
    """Rows row0 .. row0+n-1 of the rotated-domain matrix G as float32 (one fp32 multiply per
    element, exact: a 4-bit integer times an fp16 number)."""
    codes, scales = split(blob, rows, cols)
    n = rows - row0 if n is None else n
    c = codes[row0:row0 + n]
    q = np.stack([c & 15, c >> 4], -1).reshape(n, cols).astype(np.float32) - 8.0
    s = np.repeat(scales[row0:row0 + n].astype(np.float32), 128, axis=1)
    return q * s


def hadamard128():
    """Sylvester Hadamard matrix of order 128 in natural order, divided by sqrt(128)."""
    H = np.array([[1.0]], np.float32)
    while H.shape[0] < 128:
        H = np.block([[H, H], [H, -H]])
    return (H / np.sqrt(np.float32(128.0))).astype(np.float32)


_HN = hadamard128()


def rot(v, pre=None, post=None):
    """post * Hn(pre * v) per 128-block of the last axis (k_v2_rot, 28_kernels_hgn_v2.inc:63-96)."""
    v = np.asarray(v, np.float32)
    if pre is not None:
        v = v * pre
    sh = v.shape
    o = (v.reshape(-1, sh[-1] // 128, 128) @ _HN.T).reshape(sh).astype(np.float32)
    return o * post if post is not None else o


def silu(g):
    g = np.asarray(g, np.float32)
    return (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32)


def moe_forward(experts, d, mid, layer, x_f32, ids, w, k):
    """y [T][d] float32. ids / w: the router's top-k (first k columns used), layer: the dict of
    gfx1151_engine_b200.synth.make_i4r_layer (blobs and fp16 planes)."""
    x = np.asarray(x_f32, np.float32)
    T = x.shape[0]
    su_gu, sv_gu = layer["gu_suh"].astype(np.float32), layer["gu_svh"].astype(np.float32)
    su_dn, sv_dn = layer["dn_suh"].astype(np.float32), layer["dn_svh"].astype(np.float32)
    xr = rot(x, pre=su_gu)
    acc = np.zeros((T, d), np.float32)
    cache = {}
    for t in range(T):
        for s in range(k):
            e = int(ids[t, s])
            if e not in cache:
                cache[e] = (dequant_rot(layer["gate_up"], experts * 2 * mid, d, e * 2 * mid, 2 * mid),
                            dequant_rot(layer["down"], experts * d, mid, e * d, d))
            G_gu, G_dn = cache[e]
            z = G_gu @ xr[t]
            gu = rot(z, post=sv_gu)
            h = silu(gu[:mid]) * gu[mid:]
            hr = rot(h, pre=su_dn)
            acc[t] += np.float32(w[t, s]) * (G_dn @ hr)
    return rot(acc, post=sv_dn)
