"""One CPU rank (gloo) of the expert-parallel exchange test: python ep_gloo_worker.py RANK WORLD PORT.

Builds this rank's routing with the CPU oracle, exchanges expert offset tables, sends its
expert-sorted rows to the owning ranks with all-to-all, checks what arrives (only this rank's
experts, source-major, ascending expert inside a source), sends the rows back and checks that
they return in the sender's own order."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from gfx1151_engine_b200 import ep, synth  # noqa: E402


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    E, k, T, d = 16, 3, 40, 8
    logits = synth.make_logits(synth.rng_for(5, rank), T, E, zipf=True, zipf_rng=synth.rng_for(5, 99))
    ids, w = oracle.router_topk(logits, k)
    tok, pw, eoff, pid = oracle.route(ids, w, k, E)
    expert_of_row = np.repeat(np.arange(E), np.diff(eoff))
    x_send = torch.zeros(T * k, d)
    x_send[:, 0] = rank
    x_send[:, 1] = torch.arange(T * k)
    x_send[:, 2] = torch.from_numpy(expert_of_row)
    gathered = [torch.zeros(E + 1, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(eoff.astype(np.int32)))
    send, recv = ep.exchange_splits(torch.stack(gathered).numpy(), rank, world)
    x_recv = torch.zeros(sum(recv), d)
    dist.all_to_all_single(x_recv, x_send, recv, send)
    per = E // world
    ok = bool(((x_recv[:, 2] // per) == rank).all())
    src = np.repeat(np.arange(world), recv)
    ok &= bool((x_recv[:, 0].numpy() == src).all())
    for s in range(world):
        ok &= bool((np.diff(x_recv[src == s, 2].numpy()) >= 0).all())
    back = torch.zeros(T * k, d)
    dist.all_to_all_single(back, x_recv + 100, send, recv)
    ok &= bool(torch.equal(back, x_send + 100))
    dist.destroy_process_group()
    print("EXCHANGE OK" if ok else "EXCHANGE WRONG")
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
