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


def test_p2p_plan_moves_every_row_there_and_back():
    """The copy lists of the copy-engine transport: applying every rank's dispatch copies leaves
    each receive buffer exactly as the all-to-all would (sources in rank order, experts ascending
    inside a source), and the return copies bring every row back to where it started."""
    world, E, k = 3, 12, 2
    rng = np.random.default_rng(5)
    eoffs, sends = [], []
    for r in range(world):
        counts = rng.integers(0, 6, size=E)
        counts[rng.integers(0, E)] = 0
        eoff = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        eoffs.append(eoff)
        # a send row is labelled (source rank, row index, expert)
        experts = np.repeat(np.arange(E), counts)
        sends.append(np.stack([np.full(eoff[-1], r), np.arange(eoff[-1]), experts], axis=1))
    eoff_all = np.stack(eoffs)
    plans = [ep.p2p_plan(eoff_all, r, world) for r in range(world)]
    recv = [np.full((plans[r][2], 3), -1) for r in range(world)]
    for r in range(world):
        assert sorted(p for p, _, _, _ in plans[r][0]) == list(range(world))
        for p, src0, dst0, n in plans[r][0]:
            recv[p][dst0:dst0 + n] = sends[r][src0:src0 + n]
    per = E // world
    for r in range(world):
        send_splits, recv_splits = ep.exchange_splits(eoff_all, r, world)
        assert sum(recv_splits) == plans[r][2] and (recv[r] >= 0).all()
        # sources in rank order, every row an expert of this rank, experts ascending per source
        assert np.array_equal(recv[r][:, 0], np.repeat(np.arange(world), recv_splits))
        assert ((recv[r][:, 2] // per) == r).all()
        for s in range(world):
            seg = recv[r][recv[r][:, 0] == s]
            assert (np.diff(seg[:, 2]) >= 0).all() and (np.diff(seg[:, 1]) == 1).all()
    back = [np.full((len(sends[r]), 3), -1) for r in range(world)]
    for r in range(world):
        for s, src0, dst0, n in plans[r][1]:
            back[s][dst0:dst0 + n] = recv[r][src0:src0 + n]
    for r in range(world):
        assert np.array_equal(back[r], sends[r])


def test_sequence_numbers_wrap_and_stay_comparable():
    """The copy-engine transport numbers its forwards with a signed 32-bit value that wraps; the
    device-side wait compares `flag - expected >= 0` in 32-bit arithmetic. Far more forwards than
    the 65535 an earlier version allowed, and across the wrap the newer number still compares as
    reached while an older one does not."""
    from gfx1151_engine_b200 import ep

    def reached(flag, expected):          # the kernel's comparison, in int32 arithmetic
        return np.int32(np.uint32(flag & 0xFFFFFFFF) - np.uint32(expected & 0xFFFFFFFF)) >= 0

    seq = 0
    for _ in range(70000):
        nxt = ep.next_seq(seq)
        assert nxt == seq + 1 and reached(nxt, nxt) and reached(nxt, seq) and not reached(seq, nxt)
        seq = nxt
    seq = 2 ** 31 - 3
    for _ in range(8):
        nxt = ep.next_seq(seq)
        assert -2 ** 31 <= nxt < 2 ** 31
        assert reached(nxt, nxt) and reached(nxt, seq) and not reached(seq, nxt)
        seq = nxt
    assert seq < 0                         # the numbers went through the wrap


def test_every_rank_sees_every_receive_count():
    """recv_rows_all gives all ranks' receive counts from the table every rank holds, so that an
    overflow of one rank's buffer stops all ranks together (no rank is left waiting for rows)."""
    from gfx1151_engine_b200 import ep
    world, E, k, T = 4, 16, 2, 50
    rng = np.random.default_rng(3)
    tables = []
    for r in range(world):
        ids = rng.integers(0, E, size=T * k)
        tables.append(np.concatenate([[0], np.cumsum(np.bincount(ids, minlength=E))]))
    eo = np.stack(tables)
    need = ep.recv_rows_all(eo, world)
    assert need.sum() == world * T * k
    for r in range(world):
        assert need[r] == ep.p2p_plan(eo, r, world)[2] == sum(ep.exchange_splits(eo, r, world)[1])


def test_chunk_sizes_and_spans():
    """Unequal chunks: sizes follow the weights, add up to the capacity, and a shorter forward fills
    the chunks in order."""
    assert ep.chunk_sizes(16384, 2) == [8192, 8192]
    assert ep.chunk_sizes(10, 3) == [4, 4, 4]
    s = ep.chunk_sizes(16384, 4, (1, 3, 3, 1))
    assert s == [2048, 6144, 6144, 2048] and sum(s) == 16384
    s = ep.chunk_sizes(1000, 3, (1, 2, 1))
    assert sum(s) == 1000 and s[1] == max(s) and min(s) >= 1
    assert ep.chunk_spans(16384, [2048, 6144, 6144, 2048]) == [(0, 2048), (2048, 8192), (8192, 14336), (14336, 16384)]
    assert ep.chunk_spans(3000, [2048, 6144, 6144, 2048]) == [(0, 2048), (2048, 3000)]
    assert ep.chunk_spans(5, [4, 4, 4]) == [(0, 4), (4, 5)]
    with pytest.raises(ValueError):
        ep.chunk_sizes(100, 2, (1, 0))
