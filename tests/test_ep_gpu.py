"""The expert-parallel phases of the library (b200moe_ep_route / ep_experts(_part) / ep_combine) on ONE
GPU: the ranks are handles of one process that run one after the other, and the two exchanges are plain
device copies laid out by ep.p2p_plan -- the copy lists the multi-GPU transport uses. Nothing waits on
another rank, so no kernel depends on a concurrent one. The result must equal the single-GPU operator on
the same tokens up to the order of the combine's additions, and the split into an in-place own-rows
pass (no copy of the rows that stay on a rank; the shared expert rides along) plus an other-rows pass
must give the bytes of the single pass."""
import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
from gfx1151_engine_b200 import ep, synth
from helpers import bf16_out_to_f32, bf16_tensor, dev_bytes, output_errors

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def run_ranks(torch, spec, layer, xs, lgs, world, split, placement=None, merged=False):
    T = xs[0].shape[0]
    pairs = T * spec.topk
    own_rows = pairs + (T if spec.shared else 0)
    cap = world * pairs
    ops, bufs = [], []
    for r in range(world):
        op = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=spec.shared, ep_rank=r, ep_size=world)
        if placement is not None:
            op.ep_set_placement(np.ascontiguousarray(placement, dtype=np.int32))
        op.load_q4cp(0, dev_bytes(torch, layer["gate_up"]), dev_bytes(torch, layer["down"]))
        if spec.shared:
            op.load_shared_q4cp(0, dev_bytes(torch, layer["sh_gate"]), dev_bytes(torch, layer["sh_up"]),
                                dev_bytes(torch, layer["sh_down"]), dev_bytes(torch, layer["sh_gate_w"]))
        b = {"x_send": torch.zeros(own_rows, spec.d, dtype=torch.float16, device="cuda"),
             "x_recv": torch.zeros(cap, spec.d, dtype=torch.float16, device="cuda"),
             "pairs_recv": torch.zeros(cap, spec.d, dtype=torch.float16, device="cuda"),
             "pairs_back": torch.full((own_rows, spec.d), float("nan"), dtype=torch.float16, device="cuda"),
             "eoff": torch.zeros(spec.experts + 1, dtype=torch.int32, device="cuda")}
        op.ep_attach(b["x_send"], b["x_recv"], b["pairs_recv"], b["pairs_back"], cap)
        ops.append(op)
        bufs.append(b)
    for r in range(world):
        ops[r].ep_route(0, xs[r], lgs[r], eoff_out=bufs[r]["eoff"])
    torch.cuda.synchronize()
    eoff_all = torch.cat([b["eoff"] for b in bufs]).contiguous()
    eo = eoff_all.cpu().numpy()
    assert int(ep.recv_rows_all(eo, world).sum()) == world * pairs
    plans = [ep.p2p_plan(eo, r, world) for r in range(world)]
    for r in range(world):                      # dispatch (with the split the own rows stay where they are)
        for p, src0, dst0, n in plans[r][0]:
            if n and not (split and p == r):
                bufs[p]["x_recv"][dst0:dst0 + n].copy_(bufs[r]["x_send"][src0:src0 + n])
    for r in range(world):                      # experts
        if split:
            ops[r].ep_experts(0, eoff_all, part=3)
            ops[r].ep_experts(0, eoff_all, part=4 if merged else 2)
        else:
            ops[r].ep_experts(0, eoff_all)
    torch.cuda.synchronize()
    for r in range(world):                      # results back to their owners
        for s, src0, dst0, n in plans[r][1]:
            if n and not (split and s == r):
                bufs[s]["pairs_back"][dst0:dst0 + n].copy_(bufs[r]["pairs_recv"][src0:src0 + n])
    outs = []
    for r in range(world):
        out = torch.full((T, spec.d), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops[r].ep_combine(out, T)
        ops[r].synchronize()
        outs.append(bf16_out_to_f32(torch, out))
    return outs, [p[2] for p in plans]


def make_inputs(torch, spec, layer, world, T):
    xs, lgs, want = [], [], []
    single = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=spec.shared)
    single.load_q4cp(0, dev_bytes(torch, layer["gate_up"]), dev_bytes(torch, layer["down"]))
    if spec.shared:
        single.load_shared_q4cp(0, dev_bytes(torch, layer["sh_gate"]), dev_bytes(torch, layer["sh_up"]),
                                dev_bytes(torch, layer["sh_down"]), dev_bytes(torch, layer["sh_gate_w"]))
    for r in range(world):
        xb = synth.make_x(synth.rng_for(120, 10 + r), T, spec.d)
        lg = synth.make_logits(synth.rng_for(120, 20 + r), T, spec.experts, zipf=True, zipf_rng=synth.rng_for(120, 77))
        xs.append(bf16_tensor(torch, xb, (T, spec.d)))
        lgs.append(torch.from_numpy(np.ascontiguousarray(lg, np.float32)).cuda())
        out = torch.empty((T, spec.d), dtype=torch.bfloat16, device="cuda")
        single.moe_b(0, xs[r], lgs[r], out)
        single.synchronize()
        want.append(bf16_out_to_f32(torch, out))
    return xs, lgs, want


@pytest.mark.parametrize("world,placed", [(2, False), (4, True)])
def test_ep_phases_match_single_gpu(cuda, world, placed):
    torch = cuda
    spec = synth.LayerSpec(experts=16, topk=4, d=512, mid=128)
    layer = synth.make_layer(spec, seed=120)
    T = 300
    placement = None
    if placed:
        placement = synth.rng_for(120, 50).permutation(spec.experts)
    xs, lgs, want = make_inputs(torch, spec, layer, world, T)
    plain, recv = run_ranks(torch, spec, layer, xs, lgs, world, split=False, placement=placement)
    assert sum(recv) == world * T * spec.topk          # every pair lands on exactly one rank
    for r in range(world):
        assert np.isfinite(plain[r]).all()
        max_abs, mean_rel = output_errors(plain[r], want[r])
        # same products and fp32 accumulators; only the combine adds in placed-id order
        assert max_abs <= 4e-3 and mean_rel <= 1e-5, (r, max_abs, mean_rel)
    halves, _ = run_ranks(torch, spec, layer, xs, lgs, world, split=True, placement=placement)
    for r in range(world):
        assert np.array_equal(bits(halves[r]), bits(plain[r]))
    # the other ranks' rows merged by expert before their GEMMs (part 4): other tiles, same rows, same bytes
    merged, _ = run_ranks(torch, spec, layer, xs, lgs, world, split=True, placement=placement, merged=True)
    for r in range(world):
        assert np.array_equal(bits(merged[r]), bits(plain[r]))


@pytest.mark.parametrize("world", [2, 4])
def test_ep_with_shared_expert(cuda, world):
    """The shared expert is not sharded: every rank runs it for its own tokens inside the in-place
    own-rows pass. Result against the single-GPU operator with the same shared expert."""
    torch = cuda
    spec = synth.LayerSpec(experts=16, topk=4, d=512, mid=128, shared=True)
    layer = synth.make_layer(spec, seed=121)
    T = 300
    placement = synth.rng_for(121, 50).permutation(spec.experts)
    xs, lgs, want = make_inputs(torch, spec, layer, world, T)
    got, _ = run_ranks(torch, spec, layer, xs, lgs, world, split=True, placement=placement)
    for r in range(world):
        assert np.isfinite(got[r]).all()
        max_abs, mean_rel = output_errors(got[r], want[r])
        assert max_abs <= 4e-3 and mean_rel <= 1e-5, (r, max_abs, mean_rel)
    merged, _ = run_ranks(torch, spec, layer, xs, lgs, world, split=True, placement=placement, merged=True)
    for r in range(world):
        assert np.array_equal(bits(merged[r]), bits(got[r]))
    # without the in-place pass the library refuses the combination instead of dropping the expert
    op = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=True, ep_rank=0, ep_size=world)
    op.load_q4cp(0, dev_bytes(torch, layer["gate_up"]), dev_bytes(torch, layer["down"]))
    op.load_shared_q4cp(0, dev_bytes(torch, layer["sh_gate"]), dev_bytes(torch, layer["sh_up"]),
                        dev_bytes(torch, layer["sh_down"]), dev_bytes(torch, layer["sh_gate_w"]))
    rows = T * spec.topk + T
    bufs = [torch.zeros(rows if i in (0, 3) else world * rows, spec.d, dtype=torch.float16, device="cuda") for i in range(4)]
    op.ep_attach(bufs[0], bufs[1], bufs[2], bufs[3], world * rows)
    op.ep_route(0, xs[0], lgs[0])
    eoff_all = torch.zeros(world * (spec.experts + 1), dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.B200MoeError) as e:
        op.ep_experts(0, eoff_all, part=0)
    assert e.value.status == 2
    op.close()
