"""GPU: b200moe_route_static, the bucketing entry point that allocates nothing.

It exists for hosts that cannot call cudaMalloc when they reach the MoE layer (device memory
already handed to their own pool, or a section where an allocation's implicit sync is not
acceptable) and so cannot create a handle. Its scratch is a fixed __device__ array inside
the library, shared by every call on a GPU and never cleared, so this test makes two calls
in a row (the second smaller, so stale entries from the first would show) and compares each
with the handle-based b200moe_route, bit for bit. Collected last on purpose: a failure here
cannot hide another test's result in a stop-at-first-failure run.
"""
import numpy as np
import pytest

import gfx1151_engine_b200 as pkg
from gfx1151_engine_b200 import synth

pytestmark = pytest.mark.gpu


def route_both_ways(torch, T, E, k, seed, stride=16):
    logits = synth.make_logits(synth.rng_for(seed, 1), T, E, zipf=True)
    op = pkg.MoeOperator(E, k, 128, 64, T)
    ids = torch.zeros((T, stride), dtype=torch.int32, device="cuda")
    w = torch.zeros((T, stride), dtype=torch.float32, device="cuda")
    op.router_topk_b(torch.from_numpy(logits).cuda(), ids, w, stride=stride)
    op.route(ids, w, T, stride=stride)
    _, _, tok, pw, eoff, pid = op.get_routing(T)
    # the allocation-free entry point, straight through the C ABI, caller-owned outputs
    tok2 = torch.full((T * k,), -1, dtype=torch.int32, device="cuda")
    pw2 = torch.full((T * k,), -1.0, dtype=torch.float32, device="cuda")
    eoff2 = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
    pid2 = torch.full((T * k,), -1, dtype=torch.int32, device="cuda")
    st = pkg.lib().b200moe_route_static(ids.data_ptr(), w.data_ptr(), stride, T, k, E, tok2.data_ptr(),
                                        pw2.data_ptr(), eoff2.data_ptr(), pid2.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(tok2.cpu().numpy(), tok)
    assert np.array_equal(eoff2.cpu().numpy(), eoff)
    assert np.array_equal(pid2.cpu().numpy(), pid)
    assert np.array_equal(pw2.cpu().numpy().view(np.uint32), pw.view(np.uint32))
    op.close()


def test_route_static_matches_route_twice_in_a_row(cuda):
    torch = cuda
    route_both_ways(torch, 6000, 512, 10, seed=5)   # 60000 pairs: close to the 65536 limit
    route_both_ways(torch, 37, 64, 8, seed=6)       # a smaller call on the same, uncleared scratch
    route_both_ways(torch, 1, 8, 2, seed=7)


def test_route_static_refuses_what_does_not_fit(cuda):
    torch = cuda
    L = pkg.lib()
    buf = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    assert L.b200moe_route_static(p, p, 16, 6554, 10, 512, p, p, p, p, None) == 8   # 65540 pairs
    assert L.b200moe_route_static(p, p, 16, 4, 2, 513, p, p, p, p, None) == 8        # too many experts
    assert L.b200moe_route_static(None, p, 16, 4, 2, 8, p, p, p, p, None) == 1
    assert L.b200moe_route_static(p, p, 1, 4, 2, 8, p, p, p, p, None) == 1           # stride < topk
    assert L.b200moe_status_string(8).startswith(b"request exceeds")
