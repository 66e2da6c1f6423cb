"""Loading the expert tensors from model files: synthetic .hgn and (sharded) GGUF files written
here in the layouts the reference reads (src/hgn.h:48-62, 295-363; src/gguf.h:1-11, 136-314)
give the same bytes out as loading the same tensors from memory."""
import struct

import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
from gfx1151_engine_b200 import synth

from test_gpu_parity import bf16_out_to_f32, bits, make_op, run_layer


def write_hgn(path, tensors):
    """tensors: list of (name, dtype, dims, bytes)."""
    hdr, rec = 104, 160
    data_off = hdr + rec * len(tensors)
    blobs, records, off = [], [], data_off
    for name, dtype, dims, raw in tensors:
        raw = bytes(raw)
        pad = (-off) % 64
        off += pad
        blobs.append(b"\0" * pad + raw)
        d4 = list(dims) + [0] * (4 - len(dims))
        records.append(struct.pack("<96sII4QQQQ", name.encode(), dtype, len(dims), *d4, off, len(raw), 0))
        off += len(raw)
    header = struct.pack("<4sIIIQQQ64s", b"HGN1", 1, len(tensors), 0, hdr, data_off, off, b"synthetic")
    with open(path, "wb") as f:
        f.write(header + b"".join(records) + b"".join(blobs))


def gguf_str(s):
    return struct.pack("<Q", len(s)) + s.encode()


def write_gguf(path, tensors, alignment=32, extra_kv=True):
    """tensors: list of (name, ne, ggml_type, bytes)."""
    kv = [gguf_str("general.architecture") + struct.pack("<I", 8) + gguf_str("synthetic"),
          gguf_str("general.alignment") + struct.pack("<II", 4, alignment)]
    if extra_kv:   # an array of strings and an array of floats in front of the tensor infos
        kv.append(gguf_str("tokenizer.tokens") + struct.pack("<IIQ", 9, 8, 3) + b"".join(gguf_str(t) for t in ("a", "bc", "")))
        kv.append(gguf_str("x.scores") + struct.pack("<IIQ", 9, 6, 2) + struct.pack("<2f", 1.0, 2.0))
    infos, blobs, off = [], [], 0
    for name, ne, typ, raw in tensors:
        raw = bytes(raw)
        pad = (-off) % alignment
        off += pad
        blobs.append(b"\0" * pad + raw)
        infos.append(gguf_str(name) + struct.pack("<I", len(ne)) + struct.pack("<%dQ" % len(ne), *ne) + struct.pack("<IQ", typ, off))
        off += len(raw)
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head + b"".join(blobs))


def hgn_tensors(spec, layer, L):
    E, d, mid = spec.experts, spec.d, spec.mid
    return [
        ("tok_embeddings.weight", 0, (4, d), np.zeros(4 * d, np.uint16).tobytes()),
        ("layers.%d.mlp.gate.weight" % L, 0, (E, d), layer["router_w"].tobytes()),
        ("layers.%d.mlp.experts.gate_up_proj.weight" % L, 5, (E * 2 * mid, d), layer["gate_up"].tobytes()),
        ("layers.%d.mlp.experts.down_proj.weight" % L, 5, (E * d, mid), layer["down"].tobytes()),
        ("layers.%d.mlp.shared_expert.gate_proj.weight" % L, 5, (mid, d), layer["sh_gate"].tobytes()),
        ("layers.%d.mlp.shared_expert.up_proj.weight" % L, 5, (mid, d), layer["sh_up"].tobytes()),
        ("layers.%d.mlp.shared_expert.down_proj.weight" % L, 5, (d, mid), layer["sh_down"].tobytes()),
        ("layers.%d.mlp.shared_expert_gate.weight" % L, 0, (1, d), layer["sh_gate_w"].tobytes()),
    ]


needs_ref = pytest.mark.skipif(not __import__("oracle").have_ref(),
                               reason="oracle/_ref/libref.so (the reference compiled from its sources) is not built here")


@needs_ref
def test_reference_reader_accepts_the_synthetic_hgn_file(tmp_path):
    """The .hgn files these tests write are files the reference's own hgn::Checkpoint(path)
    (src/hgn.h:295-363) opens, and it sees the tensors with the dtype, dims and bytes written."""
    import zlib

    import oracle
    spec = synth.LayerSpec(experts=4, topk=2, d=256, mid=64, shared=True, router=True)
    layer = synth.make_layer(spec, seed=21)
    path = str(tmp_path / "model.hgn")
    tensors = hgn_tensors(spec, layer, 3)
    write_hgn(path, tensors)
    for name, dtype, dims, raw in tensors:
        t = oracle.ref_file_tensor("hgn", path, name)
        assert t is not None, name
        assert t["dtype"] == dtype and t["ndims"] == len(dims) and t["dims"][:len(dims)] == list(dims)
        assert t["size"] == len(raw) and t["crc32"] == zlib.crc32(raw)
    assert oracle.ref_file_tensor("hgn", path, "layers.4.mlp.gate.weight") is None
    with open(path, "r+b") as f:     # a file whose header size field is wrong is refused
        f.seek(32)
        f.write(struct.pack("<Q", 12345))
    with pytest.raises(RuntimeError):
        oracle.ref_file_tensor("hgn", path, tensors[0][0])


@needs_ref
@pytest.mark.parametrize("sharded", [False, True])
def test_reference_reader_accepts_the_synthetic_gguf_files(tmp_path, sharded):
    """The same for GGUF through the reference's gguf::File(path) (src/gguf.h:136-314), sharded or
    not, with the key/value section these tests put in front of the tensor infos."""
    import zlib

    import oracle
    spec = synth.LayerSpec(experts=4, topk=2, d=512, mid=256, fmt="gguf", gg_gu=12, gg_dn=7)
    layer = synth.make_layer(spec, seed=22)
    E, d, mid = spec.experts, spec.d, spec.mid
    t_gate = ("blk.1.ffn_gate_exps.weight", (d, mid, E), 12, layer["gate"].tobytes())
    t_up = ("blk.1.ffn_up_exps.weight", (d, mid, E), 12, layer["up"].tobytes())
    t_down = ("blk.1.ffn_down_exps.weight", (mid, d, E), 7, layer["down"].tobytes())
    t_other = ("blk.1.attn_norm.weight", (d,), 0, np.ones(d, np.float32).tobytes())
    if sharded:
        write_gguf(str(tmp_path / "m-00001-of-00002.gguf"), [t_other, t_gate])
        write_gguf(str(tmp_path / "m-00002-of-00002.gguf"), [t_down, t_up], alignment=64, extra_kv=False)
        path = str(tmp_path / "m-00002-of-00002.gguf")
    else:
        write_gguf(str(tmp_path / "m.gguf"), [t_other, t_gate, t_up, t_down])
        path = str(tmp_path / "m.gguf")
    for name, ne, typ, raw in (t_gate, t_up, t_down, t_other):
        t = oracle.ref_file_tensor("gguf", path, name)
        assert t is not None, name
        assert t["dtype"] == typ and t["ndims"] == len(ne) and t["dims"][:len(ne)] == list(ne)
        assert t["size"] == len(raw) and t["crc32"] == zlib.crc32(raw)
    assert oracle.ref_file_tensor("gguf", path, "blk.0.ffn_up_exps.weight") is None


@pytest.mark.gpu
def test_hgn_file_with_a_short_shared_tensor_is_refused(cuda, tmp_path):
    """A shared-expert tensor whose size or shape does not match the handle is refused with a
    status code before anything reads past the mapping."""
    torch = cuda
    spec = synth.LayerSpec(experts=4, topk=2, d=256, mid=64, shared=True, router=True)
    layer = synth.make_layer(spec, seed=23)
    good = hgn_tensors(spec, layer, 0)
    op = make_op(torch, spec, 8)
    for victim, cut in (("shared_expert.gate_proj", 64), ("shared_expert.down_proj", 16), ("shared_expert.up_proj", 0)):
        tensors = []
        for name, dtype, dims, raw in good:
            if victim in name:
                if cut:
                    raw = raw[:len(raw) - cut]                  # truncated blob, dims unchanged
                else:
                    dims = (dims[0] // 2, dims[1] * 2)          # same bytes, another shape
            tensors.append((name, dtype, dims, raw))
        path = str(tmp_path / ("bad_%s.hgn" % victim))
        write_hgn(path, tensors)
        with pytest.raises(pkg.B200MoeError) as e:
            op.load_hgn_file(0, path, model_layer=0)
        assert e.value.status in (1, 2)
    path = str(tmp_path / "good.hgn")
    write_hgn(path, good)
    op.load_hgn_file(0, path, model_layer=0)                    # the untouched file still loads
    op.close()


@pytest.mark.gpu
def test_hgn_file_with_shared_expert_and_router(cuda, tmp_path):
    torch = cuda
    spec = synth.LayerSpec(experts=8, topk=2, d=256, mid=64, shared=True, router=True, book="random")
    layer = synth.make_layer(spec, seed=21)
    E, d, mid = spec.experts, spec.d, spec.mid
    path = str(tmp_path / "model.hgn")
    write_hgn(path, [
        ("tok_embeddings.weight", 0, (4, d), np.zeros(4 * d, np.uint16).tobytes()),
        ("layers.3.mlp.gate.weight", 0, (E, d), layer["router_w"].tobytes()),
        ("layers.3.mlp.experts.gate_up_proj.weight", 5, (E * 2 * mid, d), layer["gate_up"].tobytes()),
        ("layers.3.mlp.experts.down_proj.weight", 5, (E * d, mid), layer["down"].tobytes()),
        ("layers.3.mlp.shared_expert.gate_proj.weight", 5, (mid, d), layer["sh_gate"].tobytes()),
        ("layers.3.mlp.shared_expert.up_proj.weight", 5, (mid, d), layer["sh_up"].tobytes()),
        ("layers.3.mlp.shared_expert.down_proj.weight", 5, (d, mid), layer["sh_down"].tobytes()),
        ("layers.3.mlp.shared_expert_gate.weight", 0, (1, d), layer["sh_gate_w"].tobytes()),
    ])
    T = 40
    xb = synth.make_x(synth.rng_for(21, 9), T, d)
    logits = synth.make_logits(synth.rng_for(21, 1), T, E)
    y_mem = run_layer(torch, make_op(torch, spec, T, layer=layer), spec, xb, logits)
    op = make_op(torch, spec, T)
    op.load_hgn_file(0, path, model_layer=3)
    assert np.array_equal(bits(run_layer(torch, op, spec, xb, logits)), bits(y_mem))
    # the router weight came along: forward from hidden states works
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16).reshape(T, d)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    op.moe_hidden(0, x, out)
    op.synchronize()
    assert np.isfinite(bf16_out_to_f32(torch, out)).all()
    with pytest.raises(pkg.B200MoeError):
        op.load_hgn_file(0, path, model_layer=4)            # no such layer in the file
    with pytest.raises(pkg.B200MoeError):
        op.load_hgn_file(0, str(tmp_path / "missing.hgn"))


def i4r_hgn_tensors(L, E, d, mid, layer_no, shared_su):
    """An hgn v2 layer: dtype 23 expert tensors [E, O, K] and their fp16 planes; the input plane of
    gate_up under its own name or as experts.su (src/gpu/parts/30_host_util.inc:852-856)."""
    ex = "layers.%d.mlp.experts" % layer_no
    return [
        (ex + ".gate_up_proj.weight", 23, (E, 2 * mid, d), L["gate_up"].tobytes()),
        (ex + ".down_proj.weight", 23, (E, d, mid), L["down"].tobytes()),
        (ex + (".su" if shared_su else ".gate_up_proj.suh"), 2, (d,), L["gu_suh"].tobytes()),
        (ex + ".gate_up_proj.svh", 2, (2 * mid,), L["gu_svh"].tobytes()),
        (ex + ".down_proj.suh", 2, (mid,), L["dn_suh"].tobytes()),
        (ex + ".down_proj.svh", 2, (d,), L["dn_svh"].tobytes()),
    ]


@needs_ref
def test_reference_reader_accepts_the_synthetic_i4r_file(tmp_path):
    import zlib

    import oracle
    E, d, mid = 4, 256, 128
    L = synth.make_i4r_layer(E, d, mid, seed=29)
    path = str(tmp_path / "v2.hgn")
    tensors = i4r_hgn_tensors(L, E, d, mid, 2, True)
    write_hgn(path, tensors)
    for name, dtype, dims, raw in tensors:
        t = oracle.ref_file_tensor("hgn", path, name)
        assert t is not None and t["dtype"] == dtype and t["dims"][:len(dims)] == list(dims)
        assert t["size"] == len(raw) and t["crc32"] == zlib.crc32(raw)


@pytest.mark.gpu
@pytest.mark.parametrize("shared_su", [False, True])
def test_hgn_v2_file_with_i4r_experts(cuda, tmp_path, shared_su):
    """dtype 23 experts and their planes from a file give the bytes of the in-memory load."""
    torch = cuda
    E, k, d, mid, T = 4, 2, 256, 128, 40
    L = synth.make_i4r_layer(E, d, mid, seed=29)
    path = str(tmp_path / "v2.hgn")
    write_hgn(path, i4r_hgn_tensors(L, E, d, mid, 2, shared_su))
    xb = synth.make_x(synth.rng_for(29, 9), T, d)
    logits = synth.make_logits(synth.rng_for(29, 1), T, E)
    spec = synth.LayerSpec(experts=E, topk=k, d=d, mid=mid)
    op_mem = pkg.MoeOperator(E, k, d, mid, T)
    op_mem.load_i4r(0, L["gate_up"], L["down"], L["gu_suh"], L["gu_svh"], L["dn_suh"], L["dn_svh"])
    y_mem = run_layer(torch, op_mem, spec, xb, logits)
    op = pkg.MoeOperator(E, k, d, mid, T)
    op.load_hgn_file(0, path, model_layer=2)
    assert np.isfinite(y_mem).all() and np.array_equal(bits(run_layer(torch, op, spec, xb, logits)), bits(y_mem))
    with open(path, "r+b") as f:     # a plane of the wrong length is refused
        raw = f.read()
    bad = str(tmp_path / "bad.hgn")
    tensors = i4r_hgn_tensors(L, E, d, mid, 2, shared_su)
    tensors[3] = (tensors[3][0], 2, (2 * mid - 1,), tensors[3][3][:-2])
    write_hgn(bad, tensors)
    with pytest.raises(pkg.B200MoeError):
        op.load_hgn_file(0, bad, model_layer=2)
    op.close()
    op_mem.close()


@pytest.mark.gpu
@pytest.mark.parametrize("sharded,gu,dn", [(False, 12, 7), (True, 12, 7), (False, 20, 23), (True, 23, 20), (False, 13, 7), (True, 8, 8)])
def test_gguf_file(cuda, tmp_path, sharded, gu, dn):
    torch = cuda
    spec = synth.LayerSpec(experts=8, topk=2, d=512, mid=256, fmt="gguf", gg_gu=gu, gg_dn=dn)
    layer = synth.make_layer(spec, seed=22)
    E, d, mid = spec.experts, spec.d, spec.mid
    t_gate = ("blk.1.ffn_gate_exps.weight", (d, mid, E), gu, layer["gate"].tobytes())
    t_up = ("blk.1.ffn_up_exps.weight", (d, mid, E), gu, layer["up"].tobytes())
    t_down = ("blk.1.ffn_down_exps.weight", (mid, d, E), dn, layer["down"].tobytes())
    t_other = ("blk.1.attn_norm.weight", (d,), 0, np.ones(d, np.float32).tobytes())
    if sharded:
        write_gguf(str(tmp_path / "m-00001-of-00002.gguf"), [t_other, t_gate])
        write_gguf(str(tmp_path / "m-00002-of-00002.gguf"), [t_down, t_up], alignment=64, extra_kv=False)
        path = str(tmp_path / "m-00002-of-00002.gguf")
    else:
        write_gguf(str(tmp_path / "m.gguf"), [t_other, t_gate, t_up, t_down])
        path = str(tmp_path / "m.gguf")
    T = 40
    xb = synth.make_x(synth.rng_for(22, 9), T, d)
    logits = synth.make_logits(synth.rng_for(22, 1), T, E)
    y_mem = run_layer(torch, make_op(torch, spec, T, layer=layer), spec, xb, logits)
    op = make_op(torch, spec, T)
    op.load_gguf_file(0, path, model_layer=1)
    assert np.array_equal(bits(run_layer(torch, op, spec, xb, logits)), bits(y_mem))
    with pytest.raises(pkg.B200MoeError):
        op.load_gguf_file(0, path, model_layer=0)
