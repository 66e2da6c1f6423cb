"""CPU: host logic of the expert-parallel path -- placement, exchange split sizes -- and a
world-size-2 gloo run of the same exchange pattern on CPU tensors, checked row by row."""
import os
import socket
import sys

import numpy as np
import pytest

import oracle
from gfx1151_engine_b200 import ep, synth


def test_greedy_placement_balances_zipf_load():
    E, world, k = 512, 8, 10
    # the load that matters is how often an expert is SELECTED (at most once per token), not
    # its router prior: take the top-k histogram of a calibration batch
    logits = synth.make_logits(synth.rng_for(0, 10), 2048, E, zipf=True, zipf_rng=synth.rng_for(0, 77))
    ids, _ = oracle.router_topk(logits, k)
    load = np.bincount(ids[:, :k].reshape(-1), minlength=E).astype(np.float64)
    placed = ep.greedy_placement(load, world)
    assert sorted(placed.tolist()) == list(range(E))                 # a permutation
    assert np.bincount(placed // (E // world)).tolist() == [E // world] * world
    contiguous = np.arange(E, dtype=np.int32)
    assert ep.imbalance(load, placed, world) < 1.02 and ep.imbalance(load, contiguous, world) > 1.3


def test_exchange_splits_match_a_direct_count():
    E, world, k, T = 64, 4, 6, 200
    tables, owners = [], []
    for r in range(world):
        logits = synth.make_logits(synth.rng_for(3, r), T, E, zipf=True, zipf_rng=synth.rng_for(3, 99))
        ids, w = oracle.router_topk(logits, k)
        tok, pw, eoff, pid = oracle.route(ids, w, k, E)
        tables.append(eoff)
        owners.append(np.sort(ids[:, :k].reshape(-1)) // (E // world))
    for r in range(world):
        send, recv = ep.exchange_splits(np.stack(tables), r, world)
        assert send == np.bincount(owners[r], minlength=world).tolist()
        assert recv == [int((owners[s] == r).sum()) for s in range(world)]
    assert sum(sum(ep.exchange_splits(np.stack(tables), r, world)[0]) for r in range(world)) == world * T * k


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_gloo_two_ranks_exchange_round_trip():
    """Two CPU ranks (gloo) run the dispatch and combine exchanges of ep_gloo_worker.py."""
    import subprocess
    port = _free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ep_gloo_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "EXCHANGE OK" in o, "rank %d failed:\n%s" % (r, o)
