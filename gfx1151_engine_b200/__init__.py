"""B200 (sm_100a) routed-expert MoE FFN operator: Python face of the C-ABI library.

The product is `libb200moe.so` (CUDA C++, declared in include/b200moe.h). This module
only binds it with ctypes and mirrors the reference engine's MoE operator surface
(GpuModel::moe / moe_b / moe_q4w_run / router_topk_b, src/gpu/parts/40_model.inc of the
reference) for Python callers and tests. There is no CPU or PyTorch fallback: if the
library is missing or fails, calls raise.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200moe.so")

GEMM_AUTO, GEMM_SIMT, GEMM_TC = 0, 1, 2
DECODE_AUTO, DECODE_FUSED = 0, 1
GGML_Q5_1, GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_IQ4_NL, GGML_IQ4_XS = 7, 8, 12, 13, 20, 23

STATUS = {0: "ok", 1: "bad argument", 2: "unsupported", 3: "CUDA error", 4: "not loaded",
          5: "device timeout", 6: "NCCL error", 7: "out of memory", 8: "too large for the static scratch"}

# Every symbol include/b200moe.h declares: name -> (restype, argtypes)
_P, _I, _SZ = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t


class Config(ctypes.Structure):
    """Field-for-field mirror of b200moe_config."""
    _fields_ = [(n, ctypes.c_int32) for n in (
        "experts", "topk", "d_model", "d_mid", "n_layers", "max_tokens", "has_shared", "device",
        "gemm_impl", "decode_max_tokens", "ep_rank", "ep_size", "ep_sm_margin", "decode_impl")] + [("reserved", ctypes.c_int32 * 2)]


SYMBOLS = {
    "b200moe_create": (_I, [ctypes.POINTER(Config), ctypes.POINTER(_P)]),
    "b200moe_destroy": (_I, [_P]),
    "b200moe_status_string": (ctypes.c_char_p, [_I]),
    "b200moe_last_error": (ctypes.c_char_p, [_P]),
    "b200moe_load_q4cp": (_I, [_P, _I, _P, _SZ, _P, _SZ]),
    "b200moe_load_i4r": (_I, [_P, _I, _P, _SZ, _P, _SZ, _P, _P, _P, _P]),
    "b200moe_load_gguf": (_I, [_P, _I, _P, _P, _P, _I, _I]),
    "b200moe_load_shared_q4cp": (_I, [_P, _I, _P, _P, _P, _P]),
    "b200moe_forward": (_I, [_P, _I, _P, _I, _P, _P, _P]),
    "b200moe_forward_hc": (_I, [_P, _I, _P, _I, _P, _P, _P, _P]),
    "b200moe_forward_routed": (_I, [_P, _I, _P, _I, _P, _P, _I, _P, _P]),
    "b200moe_forward_host": (_I, [_P, _I, _P, _I, _P, _P, _P]),
    "b200moe_router_topk": (_I, [_P, _P, _I, _P, _P, _I, _P]),
    "b200moe_load_router": (_I, [_P, _I, _P]),
    "b200moe_get_config": (_I, [_P, _P]),
    "b200moe_load_hgn_file": (_I, [_P, _I, ctypes.c_char_p, _I]),
    "b200moe_load_gguf_file": (_I, [_P, _I, ctypes.c_char_p, _I]),
    "b200moe_router_logits": (_I, [_P, _I, _P, _I, _P, _P]),
    "b200moe_forward_hidden": (_I, [_P, _I, _P, _I, _P, _P]),
    "b200moe_route": (_I, [_P, _P, _P, _I, _I, _P]),
    "b200moe_route_static": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "b200moe_ep_set_placement": (_I, [_P, _P]),
    "b200moe_share_weights": (_I, [_P, _P]),
    "b200moe_ep_attach": (_I, [_P, _P, _P, _P, _P, ctypes.c_int64]),
    "b200moe_ep_route": (_I, [_P, _I, _P, _I, _P, _P, _P]),
    "b200moe_ep_offsets": (_I, [_P, ctypes.POINTER(_P)]),
    "b200moe_ep_experts": (_I, [_P, _I, _P, _P]),
    "b200moe_ep_experts_part": (_I, [_P, _I, _P, _I, _P]),
    "b200moe_ep_combine": (_I, [_P, _I, _P, _P]),
    "b200moe_ep_wait_flags": (_I, [_P, _P, _I, _I, _P]),
    "b200moe_ep_unique_id": (_I, [_P]),
    "b200moe_ep_init": (_I, [_P, _P, ctypes.c_double]),
    "b200moe_ep_forward": (_I, [_P, _I, _P, _I, _P, _P, _P]),
    "b200moe_ep_shutdown": (_I, [_P]),
    "b200moe_ep_last_error": (ctypes.c_char_p, [_P]),
    "b200moe_debug_get_routing": (_I, [_P, _I, _P, _P, _P, _P, _P, _P]),
    "b200moe_dequant_rows": (_I, [_P, _I, _I, _I, _I, _I, _P, _P]),
    "b200moe_synchronize": (_I, [_P, _P]),
    "b200moe_profile_enable": (_I, [_P, _I]),
    "b200moe_profile_read": (_I, [_P, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_I)]),
    "b200moe_launch_count": (ctypes.c_int64, [_P]),
    "b200moe_version": (ctypes.c_char_p, []),
}

_lib = None


class B200MoeError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        super().__init__("b200moe status %d (%s) %s" % (status, STATUS.get(status, "?"), detail))


def lib():
    """Load libb200moe.so and declare its entry points. Raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s not found: build it with `python -m gfx1151_engine_b200.build` "
                "(there is no fallback implementation)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ptr(obj):
    """Address of a torch tensor / numpy array / int; None -> NULL."""
    if obj is None:
        return None
    if isinstance(obj, int):
        return obj
    if hasattr(obj, "data_ptr"):
        return obj.data_ptr()
    if hasattr(obj, "ctypes"):
        return obj.ctypes.data
    raise TypeError("cannot take the address of %r" % type(obj))


def _stream(stream):
    if stream is None:
        return None
    return getattr(stream, "cuda_stream", stream)


class MoeOperator:
    """One handle = the MoE layers of one GPU, with shared workspaces.

    Method names follow the reference's host functions for this path; arguments are
    device tensors (torch) or raw device addresses.
    """

    def __init__(self, experts, topk, d_model, d_mid, max_tokens, n_layers=1, has_shared=False,
                 device=0, gemm_impl=GEMM_AUTO, decode_max_tokens=0, ep_rank=0, ep_size=1, ep_sm_margin=0,
                 decode_impl=DECODE_AUTO):
        self.cfg = Config(experts, topk, d_model, d_mid, n_layers, max_tokens, int(has_shared), device,
                          gemm_impl, decode_max_tokens, ep_rank, ep_size, ep_sm_margin, decode_impl)
        self._h = _P()
        st = lib().b200moe_create(ctypes.byref(self.cfg), ctypes.byref(self._h))
        if st != 0:
            self._h = _P()
            raise B200MoeError(st, "b200moe_create")

    # -- plumbing ---------------------------------------------------------------------
    def _check(self, st):
        if st != 0:
            raise B200MoeError(st, (lib().b200moe_last_error(self._h) or b"").decode())

    def close(self):
        if self._h:
            lib().b200moe_destroy(self._h)
            self._h = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def launches(self):
        return lib().b200moe_launch_count(self._h)

    # -- weights (wview / gguf_experts_open of the reference) ------------------------------
    def load_q4cp(self, layer, gate_up, down):
        self._check(lib().b200moe_load_q4cp(self._h, layer, _ptr(gate_up), _nbytes(gate_up),
                                            _ptr(down), _nbytes(down)))

    def load_i4r(self, layer, gate_up, down, gu_suh, gu_svh, dn_suh, dn_svh):
        """hgn v2 i4r experts (dtype 23 blobs) with their four fp16 sign-scale planes
        (moe_b_v2, src/gpu/parts/40_model.inc:4559-4680 of the reference)."""
        self._check(lib().b200moe_load_i4r(self._h, layer, _ptr(gate_up), _nbytes(gate_up), _ptr(down), _nbytes(down),
                                           _ptr(gu_suh), _ptr(gu_svh), _ptr(dn_suh), _ptr(dn_svh)))

    def load_gguf(self, layer, gate, up, down, type_gu=GGML_Q4_K, type_dn=GGML_Q5_1):
        self._check(lib().b200moe_load_gguf(self._h, layer, _ptr(gate), _ptr(up), _ptr(down),
                                            type_gu, type_dn))

    def load_hgn_file(self, layer, path, model_layer=0):
        """Expert (+ shared expert, router) tensors of layers.<model_layer> from an .hgn file."""
        self._check(lib().b200moe_load_hgn_file(self._h, layer, os.fsencode(path), model_layer))

    def load_gguf_file(self, layer, path, model_layer=0):
        """blk.<model_layer>.ffn_{gate,up,down}_exps.weight from a GGUF file or shard set."""
        self._check(lib().b200moe_load_gguf_file(self._h, layer, os.fsencode(path), model_layer))

    def load_router(self, layer, gate_weight_bf16):
        """layers.L.mlp.gate.weight, bf16 [experts][d_model] (tensor or numpy uint16 bits)."""
        self._check(lib().b200moe_load_router(self._h, layer, _ptr(gate_weight_bf16)))

    def router_logits(self, layer, x, logits, T=None, stream=None):
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_router_logits(self._h, layer, _ptr(x), T, _ptr(logits), _stream(stream)))

    def moe_hidden(self, layer, x, out, T=None, stream=None):
        """out[T][d] (bf16) = MoE(x) with the router logits computed from x; asynchronous."""
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_forward_hidden(self._h, layer, _ptr(x), T, _ptr(out), _stream(stream)))

    def load_shared_q4cp(self, layer, gate, up, down, gate_w_bf16):
        self._check(lib().b200moe_load_shared_q4cp(self._h, layer, _ptr(gate), _ptr(up), _ptr(down),
                                                   _ptr(gate_w_bf16)))

    # -- forward (moe / moe_b of the reference) ---------------------------------------------
    def moe_b(self, layer, x, logits, out, T=None, stream=None):
        """out[T][d] (bf16) = MoE(x[T][d] bf16, router logits[T][E] f32); asynchronous."""
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_forward(self._h, layer, _ptr(x), T, _ptr(logits), _ptr(out),
                                          _stream(stream)))

    def moe_b_hc(self, layer, x, logits, inject_w4, state, T=None, stream=None):
        """As moe_b, but the result is added into the bf16 residual state [T][4][d] with the gates
        2*sigmoid(inject_w4[t][b] / 4) (k_moe_reduce_pw_sg_hc of the reference) instead of stored."""
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_forward_hc(self._h, layer, _ptr(x), T, _ptr(logits), _ptr(inject_w4),
                                             _ptr(state), _stream(stream)))

    moe = moe_b  # the single-token entry point of the reference is the same call with T = 1

    def moe_q4w_run(self, layer, x, topids, topw, out, stride=16, T=None, stream=None):
        """The seam below the router: caller-supplied top-k ids / weights."""
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_forward_routed(self._h, layer, _ptr(x), T, _ptr(topids), _ptr(topw),
                                                 stride, _ptr(out), _stream(stream)))

    def moe_b_host(self, layer, x_host, logits_host, out_host, T, stream=None):
        """Host buffers in, host buffer out; returns when the result is in out_host."""
        self._check(lib().b200moe_forward_host(self._h, layer, _ptr(x_host), T, _ptr(logits_host),
                                               _ptr(out_host), _stream(stream)))

    def router_topk_b(self, logits, topids, topw, stride=16, T=None, stream=None):
        T = logits.shape[0] if T is None else T
        self._check(lib().b200moe_router_topk(self._h, _ptr(logits), T, _ptr(topids), _ptr(topw),
                                              stride, _stream(stream)))

    def route(self, topids, topw, T, stride=16, stream=None):
        self._check(lib().b200moe_route(self._h, _ptr(topids), _ptr(topw), stride, T, _stream(stream)))

    # -- expert parallelism: library phases; the exchanges in between belong to the caller ------
    def ep_set_placement(self, placed_id_of_expert):
        self._check(lib().b200moe_ep_set_placement(self._h, _ptr(placed_id_of_expert)))

    def share_weights(self, owner):
        """Use `owner`'s repacked weights; keep a reference so that it outlives this handle."""
        self._check(lib().b200moe_share_weights(self._h, owner._h))
        self._weights_owner = owner

    def ep_attach(self, x_send, x_recv, pairs_recv, pairs_back, cap_rows):
        self._check(lib().b200moe_ep_attach(self._h, _ptr(x_send), _ptr(x_recv), _ptr(pairs_recv),
                                            _ptr(pairs_back), cap_rows))

    def ep_route(self, layer, x, logits, eoff_out=None, T=None, stream=None):
        T = x.shape[0] if T is None else T
        self._check(lib().b200moe_ep_route(self._h, layer, _ptr(x), T, _ptr(logits), _ptr(eoff_out),
                                           _stream(stream)))

    def ep_offsets_ptr(self):
        p = _P()
        self._check(lib().b200moe_ep_offsets(self._h, ctypes.byref(p)))
        return p.value

    def ep_experts(self, layer, eoff_all, stream=None, part=0):
        """part 0: all received rows; 1: the rows this rank sent to itself; 2: the other ranks' rows."""
        self._check(lib().b200moe_ep_experts_part(self._h, layer, _ptr(eoff_all), part, _stream(stream)))

    def ep_combine(self, out, T, stream=None):
        self._check(lib().b200moe_ep_combine(self._h, T, _ptr(out), _stream(stream)))

    def ep_wait_flags(self, flags, n, expected, stream=None):
        """Enqueue a bounded wait until flags[0..n) (int32, written by peer GPUs) reach `expected`."""
        self._check(lib().b200moe_ep_wait_flags(self._h, _ptr(flags), n, expected, _stream(stream)))

    # -- expert parallelism with the host inside the library (NCCL, no torch.distributed) --------
    def ep_init(self, unique_id, cap_factor=2.0):
        """Collective over the ranks: communicator from the 128-byte id (ep_unique_id() on rank 0,
        carried to the others by the caller), row buffers allocated and attached."""
        buf = (ctypes.c_char * 128).from_buffer_copy(bytes(unique_id))
        self._check(lib().b200moe_ep_init(self._h, ctypes.addressof(buf), float(cap_factor)))

    def ep_forward(self, layer, x, logits, out, T=None, stream=None):
        T = x.shape[0] if T is None else T
        st = lib().b200moe_ep_forward(self._h, layer, _ptr(x), T, _ptr(logits), _ptr(out), _stream(stream))
        if st != 0:
            detail = (lib().b200moe_ep_last_error(self._h) or b"").decode() or (lib().b200moe_last_error(self._h) or b"").decode()
            raise B200MoeError(st, detail)

    def ep_shutdown(self):
        self._check(lib().b200moe_ep_shutdown(self._h))

    def synchronize(self, stream=None):
        """Wait for the stream and raise if a device-side wait gave up."""
        self._check(lib().b200moe_synchronize(self._h, _stream(stream)))

    def profile_enable(self, on=True):
        self._check(lib().b200moe_profile_enable(self._h, int(on)))

    def profile_read(self):
        """Mean stage times in ms since the last read: dict with route, gather, up, down,
        combine, total and the number of calls averaged."""
        ms = (ctypes.c_float * 6)()
        n = _I(0)
        self._check(lib().b200moe_profile_read(self._h, ms, ctypes.byref(n)))
        names = ("route", "gather", "up", "down", "combine", "total")
        out = {k: float(v) for k, v in zip(names, ms)}
        out["calls"] = n.value
        return out

    # -- inspection ---------------------------------------------------------------------------
    def get_routing(self, T):
        """(topids[T,16], topw[T,16], tokidx[T*k], pw[T*k], eoff[E+1], pairids[T*k]) as numpy."""
        import numpy as np
        k, E = self.cfg.topk, self.cfg.experts
        ids = np.zeros((T, 16), np.int32)
        w = np.zeros((T, 16), np.float32)
        tok = np.zeros(T * k, np.int32)
        pw = np.zeros(T * k, np.float32)
        eoff = np.zeros(E + 1, np.int32)
        pid = np.zeros(T * k, np.int32)
        self._check(lib().b200moe_debug_get_routing(self._h, T, _ptr(ids), _ptr(w), _ptr(tok), _ptr(pw),
                                                    _ptr(eoff), _ptr(pid)))
        return ids, w, tok, pw, eoff, pid

    def dequant_rows(self, layer, which, expert, row0, nrows, out, stream=None):
        self._check(lib().b200moe_dequant_rows(self._h, layer, which, expert, row0, nrows, _ptr(out),
                                               _stream(stream)))


def _nbytes(obj):
    if hasattr(obj, "nbytes"):
        return int(obj.nbytes)
    if hasattr(obj, "numel"):
        return int(obj.numel() * obj.element_size())
    raise TypeError("cannot size %r" % type(obj))


def ep_unique_id():
    """The 128-byte NCCL id of a new expert-parallel group (make it on one rank, hand it to the rest)."""
    buf = (ctypes.c_char * 128)()
    st = lib().b200moe_ep_unique_id(ctypes.addressof(buf))
    if st != 0:
        raise B200MoeError(st, "b200moe_ep_unique_id")
    return bytes(buf)


def version():
    return lib().b200moe_version().decode()
