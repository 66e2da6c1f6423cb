"""Shared pieces of the test-suite: checksums, comparison metrics, device upload."""
import zlib

import numpy as np


def crc(*arrays):
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes(), c)
    return np.uint32(c)


def layer_crc(layer, keys=None):
    keys = sorted(layer) if keys is None else keys
    return crc(*[layer[k] for k in keys])


def to_bf16_f32(a):
    """Round a float32 array to bf16 (nearest even) and return it as float32."""
    from gfx1151_engine_b200 import synth
    return synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(a))


# Tolerance of the layer output against the CPU reference, both rounded to bf16:
# max |diff| <= 2e-2 and mean |diff| / mean |ref| <= 1e-3.
MAX_ABS_TOL = 2e-2
MEAN_REL_TOL = 1e-3


def output_errors(y_gpu_bf16_as_f32, y_ref_f32):
    ref = to_bf16_f32(y_ref_f32)
    diff = np.abs(y_gpu_bf16_as_f32.astype(np.float64) - ref.astype(np.float64))
    return float(diff.max()), float(diff.mean() / max(np.abs(ref).mean(), 1e-30))


def assert_output_close(y_gpu, y_ref, what=""):
    max_abs, mean_rel = output_errors(y_gpu, y_ref)
    assert np.isfinite(y_gpu).all(), what + ": non-finite output"
    assert max_abs <= MAX_ABS_TOL and mean_rel <= MEAN_REL_TOL, (
        "%s: max-abs %.3e (tol %.0e), mean-rel %.3e (tol %.0e)" % (what, max_abs, MAX_ABS_TOL, mean_rel, MEAN_REL_TOL))
    return max_abs, mean_rel


def dev_bytes(torch, arr):
    """numpy array -> CUDA uint8 tensor (16-byte aligned by the allocator)."""
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).cuda()


def bf16_tensor(torch, bits, shape):
    """uint16 bf16 bit patterns -> CUDA bf16 tensor."""
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).reshape(shape)).cuda()
    return t.view(torch.bfloat16)


def bf16_out_to_f32(torch, t):
    return t.float().cpu().numpy()
