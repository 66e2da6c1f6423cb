"""CPU checker for the MoE path -- TEST INFRASTRUCTURE ONLY.

ctypes bindings of oracle/liboracle.so (the restated oracle, moe_oracle.cpp) and, when
it has been built, oracle/_ref/libref.so (the reference's own CPU code compiled from its
sources, ref_adapter.cpp). Only tests, the smoke check and the benchmark's CPU-baseline
leg may import this package; the product library never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libref.so")

_P = ctypes.c_void_p


class OrcLayer(ctypes.Structure):
    _fields_ = [("experts", ctypes.c_int32), ("topk", ctypes.c_int32), ("d", ctypes.c_int32),
                ("mid", ctypes.c_int32), ("format", ctypes.c_int32), ("gg_type_gu", ctypes.c_int32),
                ("gg_type_dn", ctypes.c_int32), ("has_shared", ctypes.c_int32),
                ("gate_up", _P), ("down", _P), ("gg_gate", _P), ("gg_up", _P), ("router_w", _P),
                ("sh_gate", _P), ("sh_up", _P), ("sh_down", _P), ("sh_gate_w", _P)]


def build(ref_dir=None):
    """Compile the checker libraries (make -C oracle). The reference tree is looked for in
    `ref_dir`, else in the environment's REF_DIR, else in reference/ next to the repository and
    in baseline/_ref/ inside it; without one only the restated oracle is built."""
    cmd = ["make", "-C", _HERE]
    ref_dir = ref_dir or os.environ.get("REF_DIR")
    if ref_dir:
        cmd.append("REF_DIR=" + ref_dir)
    subprocess.run(cmd, check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


_orc = None
_ref = None


def orc():
    global _orc
    if _orc is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        L.orc_moe_forward.restype = ctypes.c_int
        L.orc_gguf_rows.restype = ctypes.c_int
        L.orc_tiles.restype = ctypes.c_int
        L.orc_count_topk_ties.restype = ctypes.c_int
        L.orc_threads.restype = ctypes.c_int
        _orc = L
    return _orc


def have_ref():
    return os.path.exists(REF_SO)


def ref():
    global _ref
    if _ref is None:
        L = ctypes.CDLL(REF_SO)
        for n in ("ref_moe_layer", "ref_q4cp_rows", "ref_gguf_rows", "ref_hgn_tensor", "ref_gguf_tensor"):
            getattr(L, n).restype = ctypes.c_int
        _ref = L
    return _ref


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _u64(v):
    return ctypes.c_uint64(int(v))


def q4cp_rows(blob, rows, cols, row0, n, use_ref=False):
    out = np.empty((n, cols), np.float32)
    f = ref().ref_q4cp_rows if use_ref else orc().orc_q4cp_rows
    f(_p(blob), _u64(rows), _u64(cols), _u64(row0), _u64(n), _p(out))
    return out


def gguf_rows(gtype, src, k, n, use_ref=False):
    out = np.empty((n, k), np.float32)
    f = ref().ref_gguf_rows if use_ref else orc().orc_gguf_rows
    rc = f(ctypes.c_uint32(gtype), _p(src), _u64(k), _u64(n), _p(out))
    assert rc == 0
    return out


def router_topk(logits, k, stride=16, want_probs=False):
    T, E = logits.shape
    ids = np.zeros((T, stride), np.int32)
    w = np.zeros((T, stride), np.float32)
    probs = np.zeros((T, E), np.float32) if want_probs else None
    orc().orc_router_topk(_p(np.ascontiguousarray(logits, np.float32)), T, E, k, stride, _p(ids), _p(w),
                          _p(probs))
    return (ids, w, probs) if want_probs else (ids, w)


def router_logits(router_w_bits, x_f32):
    """logits[T][E] of the reference's router matvec (bf16 weight bits [E][d], fp32 activations)."""
    E, d = router_w_bits.shape
    T = x_f32.shape[0]
    out = np.zeros((T, E), np.float32)
    orc().orc_router_logits(_p(np.ascontiguousarray(router_w_bits, np.uint16)),
                            _p(np.ascontiguousarray(x_f32, np.float32)), T, E, d, _p(out))
    return out


def count_topk_ties(probs, k):
    T, E = probs.shape
    return orc().orc_count_topk_ties(_p(np.ascontiguousarray(probs, np.float32)), T, E, k)


def route(ids, w, k, E):
    T, stride = ids.shape
    tok = np.zeros(T * k, np.int32)
    pw = np.zeros(T * k, np.float32)
    eoff = np.zeros(E + 1, np.int32)
    pid = np.zeros(T * k, np.int32)
    orc().orc_route(_p(ids), _p(w), T, k, E, stride, _p(tok), _p(pw), _p(eoff), _p(pid))
    return tok, pw, eoff, pid


def tiles(eoff, cap):
    E = len(eoff) - 1
    buf = np.zeros((int(eoff[-1]) // cap + E + 1, 3), np.int32)
    n = orc().orc_tiles(_p(np.ascontiguousarray(eoff, np.int32)), E, cap, _p(buf))
    return buf[:n]


def moe_forward(spec, layer, x_f32, logits=None, threads=0):
    """Restated oracle on T tokens. layer: dict from synth.make_layer; x_f32: [T][d] float32
    (bf16-valued). Returns (y[T][d] f32, ids[T][16], w[T][16])."""
    L = OrcLayer()
    L.experts, L.topk, L.d, L.mid = spec.experts, spec.topk, spec.d, spec.mid
    L.format = 0 if spec.fmt == "q4cp" else 1
    L.gg_type_gu, L.gg_type_dn = getattr(spec, "gg_gu", 12), getattr(spec, "gg_dn", 7)
    L.has_shared = int(spec.shared)
    keep = []

    def addr(name):
        a = layer.get(name)
        if a is None:
            return None
        keep.append(a)
        return a.ctypes.data
    if spec.fmt == "q4cp":
        L.gate_up, L.down = addr("gate_up"), addr("down")
    else:
        L.gg_gate, L.gg_up, L.down = addr("gate"), addr("up"), addr("down")
    L.router_w = addr("router_w") if logits is None else None
    if spec.shared:
        L.sh_gate, L.sh_up, L.sh_down, L.sh_gate_w = (addr("sh_gate"), addr("sh_up"), addr("sh_down"),
                                                        addr("sh_gate_w"))
    x_f32 = np.ascontiguousarray(x_f32, np.float32)
    T = x_f32.shape[0]
    y = np.zeros((T, spec.d), np.float32)
    ids = np.zeros((T, 16), np.int32)
    w = np.zeros((T, 16), np.float32)
    lg = None if logits is None else np.ascontiguousarray(logits, np.float32)
    rc = orc().orc_moe_forward(ctypes.byref(L), _p(x_f32), _p(lg), T, _p(y), _p(ids), _p(w), threads)
    assert rc == 0, rc
    return y, ids, w


def ref_moe_layer(spec, layer, x_f32, threads=0):
    """The reference's unmodified Model::moe on T tokens (router weight required)."""
    x_f32 = np.ascontiguousarray(x_f32, np.float32)
    T = x_f32.shape[0]
    y = np.zeros((T, spec.d), np.float32)
    rc = ref().ref_moe_layer(spec.d, spec.experts, spec.topk, spec.mid, _p(layer["router_w"]),
                             _p(layer["gate_up"]), _p(layer["down"]), _p(layer["sh_gate_w"]),
                             _p(layer["sh_gate"]), _p(layer["sh_up"]), _p(layer["sh_down"]),
                             _p(x_f32), T, _p(y), threads)
    assert rc == 0
    return y


def ref_file_tensor(kind, path, name):
    """Tensor `name` of a model file as the reference's own reader sees it (hgn::Checkpoint /
    gguf::File): dict with dtype, ndims, dims, size, crc32; None when the file has no such tensor.
    Raises when the reference refuses the file."""
    meta = np.zeros(8, np.uint64)
    f = ref().ref_hgn_tensor if kind == "hgn" else ref().ref_gguf_tensor
    rc = f(path.encode(), name.encode(), _p(meta))
    if rc == 1:
        return None
    if rc != 0:
        raise RuntimeError("the reference reader refused %s" % path)
    return {"dtype": int(meta[0]), "ndims": int(meta[1]), "dims": [int(v) for v in meta[2:6]],
            "size": int(meta[6]), "crc32": int(meta[7])}


def threads():
    return orc().orc_threads()
