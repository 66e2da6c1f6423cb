"""Expert parallelism over one node's GPUs: host side.

One process per GPU (torch.distributed, NCCL). The 512 experts are partitioned evenly; a
forward is three library phases (route+gather, grouped GEMMs on the received rows, combine)
with two NCCL all-to-all exchanges of fp16 rows in between. The reference engine is a
single-device program and has no counterpart of this file.

Placement: under a skewed router a contiguous split of the expert ids leaves the ranks with
very different loads, so experts are renumbered ("placed") by a greedy longest-first
assignment of an expected-load histogram to ranks with equal expert counts.
"""
import numpy as np


def greedy_placement(load, world):
    """placed id of every expert: rank r owns placed ids [r*E/world, (r+1)*E/world).
    Experts are taken by descending load and given to the least-loaded rank with room."""
    load = np.asarray(load, dtype=np.float64)
    E = load.shape[0]
    assert E % world == 0
    per = E // world
    order = np.argsort(-load, kind="stable")
    rank_load = np.zeros(world)
    rank_fill = np.zeros(world, dtype=np.int64)
    placed = np.empty(E, dtype=np.int32)
    for e in order:
        free = np.where(rank_fill < per)[0]
        r = free[np.argmin(rank_load[free])]
        placed[e] = r * per + rank_fill[r]
        rank_fill[r] += 1
        rank_load[r] += load[e]
    return placed


def imbalance(load, placed, world):
    """max / mean of the per-rank load under a placement."""
    load = np.asarray(load, dtype=np.float64)
    per = load.shape[0] // world
    rank_load = np.bincount(np.asarray(placed) // per, weights=load, minlength=world)
    return float(rank_load.max() / max(rank_load.mean(), 1e-30))


def exchange_splits(eoff_all, rank, world):
    """Row counts of the two all-to-all exchanges from every rank's expert offset table.

    eoff_all: [world][E+1] integer array, row s = rank s's exclusive prefix of its pairs per
    placed expert id. Returns (send_splits, recv_splits): rows this rank sends to / receives
    from each rank, in rank order (which is also the row order inside the buffers)."""
    eoff_all = np.asarray(eoff_all).reshape(world, -1)
    E = eoff_all.shape[1] - 1
    per = E // world
    bounds = eoff_all[:, ::per]                      # [world][world+1]
    send = (bounds[rank, 1:] - bounds[rank, :-1]).astype(np.int64)
    recv = (bounds[:, rank + 1] - bounds[:, rank]).astype(np.int64)
    return send.tolist(), recv.tolist()


class ExpertParallelMoe:
    """The MoE layer sharded by expert over the ranks of a torch.distributed group."""

    def __init__(self, experts, topk, d_model, d_mid, max_tokens, rank, world, device,
                 cap_factor=2.0, placement=None, group=None):
        import torch
        import gfx1151_engine_b200 as pkg
        self.torch, self.group = torch, group
        self.E, self.k, self.d, self.rank, self.world = experts, topk, d_model, rank, world
        self.op = pkg.MoeOperator(experts, topk, d_model, d_mid, max_tokens, device=device,
                                  ep_rank=rank, ep_size=world)
        if placement is not None:
            self.op.ep_set_placement(np.ascontiguousarray(placement, dtype=np.int32))
        pairs = max_tokens * topk
        self.cap = int(cap_factor * pairs)
        dev = torch.device("cuda", device)
        self.x_send = torch.empty(pairs, d_model, dtype=torch.float16, device=dev)
        self.x_recv = torch.empty(self.cap, d_model, dtype=torch.float16, device=dev)
        self.pairs_recv = torch.empty(self.cap, d_model, dtype=torch.float16, device=dev)
        self.pairs_back = torch.empty(pairs, d_model, dtype=torch.float16, device=dev)
        self.op.ep_attach(self.x_send, self.x_recv, self.pairs_recv, self.pairs_back, self.cap)
        self.eoff = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        self.eoff_all = torch.empty(world * (experts + 1), dtype=torch.int32, device=dev)
        self.last_recv_rows = 0

    def load_q4cp(self, layer, gate_up, down):
        """Every rank passes the full tensors; the library keeps this rank's experts."""
        self.op.load_q4cp(layer, gate_up, down)

    def forward(self, layer, x, logits, out):
        torch, dist = self.torch, self.torch.distributed
        T = x.shape[0]
        st = torch.cuda.current_stream()
        self.op.ep_route(layer, x, logits, eoff_out=self.eoff, stream=st)
        dist.all_gather_into_tensor(self.eoff_all, self.eoff, group=self.group)
        send, recv = exchange_splits(self.eoff_all.cpu().numpy(), self.rank, self.world)
        R = int(sum(recv))
        if R > self.cap:
            raise RuntimeError("expert-parallel receive buffer too small: %d rows > capacity %d" % (R, self.cap))
        self.last_recv_rows = R
        dist.all_to_all_single(self.x_recv[:R], self.x_send[:T * self.k], recv, send, group=self.group)
        self.op.ep_experts(layer, self.eoff_all, stream=st)
        dist.all_to_all_single(self.pairs_back[:T * self.k], self.pairs_recv[:R], send, recv, group=self.group)
        self.op.ep_combine(out, T, stream=st)
