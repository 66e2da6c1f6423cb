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
    """The MoE layer sharded by expert over the ranks of a torch.distributed group.

    chunks > 1 splits a forward's tokens into that many chunks, each with its own library
    handle (workspaces) sharing one set of repacked weights; the all-to-all exchanges of a
    chunk run on a communication stream while the grouped GEMMs of its neighbours run on the
    compute stream, so the NVLink time hides behind the tensor-core time."""

    def __init__(self, experts, topk, d_model, d_mid, max_tokens, rank, world, device,
                 cap_factor=2.0, placement=None, group=None, chunks=1, sm_margin=16):
        import torch
        import gfx1151_engine_b200 as pkg
        self.torch, self.group = torch, group
        self.E, self.k, self.d, self.rank, self.world = experts, topk, d_model, rank, world
        self.chunks = chunks
        self.tc = (max_tokens + chunks - 1) // chunks            # tokens per chunk
        dev = torch.device("cuda", device)
        self.ops, self.buf = [], []
        for c in range(chunks):
            op = pkg.MoeOperator(experts, topk, d_model, d_mid, self.tc, device=device,
                                 ep_rank=rank, ep_size=world, ep_sm_margin=sm_margin if chunks > 1 else 0)
            if c == 0:
                if placement is not None:
                    op.ep_set_placement(np.ascontiguousarray(placement, dtype=np.int32))
            else:
                op.share_weights(self.ops[0])
            pairs = self.tc * topk
            cap = int(cap_factor * pairs)
            b = {"cap": cap,
                 "x_send": torch.empty(pairs, d_model, dtype=torch.float16, device=dev),
                 "x_recv": torch.empty(cap, d_model, dtype=torch.float16, device=dev),
                 "pairs_recv": torch.empty(cap, d_model, dtype=torch.float16, device=dev),
                 "pairs_back": torch.empty(pairs, d_model, dtype=torch.float16, device=dev),
                 "eoff": torch.empty(experts + 1, dtype=torch.int32, device=dev),
                 "eoff_all": torch.empty(world * (experts + 1), dtype=torch.int32, device=dev)}
            op.ep_attach(b["x_send"], b["x_recv"], b["pairs_recv"], b["pairs_back"], cap)
            self.ops.append(op)
            self.buf.append(b)
        self.op = self.ops[0]
        self.comm = torch.cuda.Stream(device=dev)
        self.last_recv_rows = 0

    def load_q4cp(self, layer, gate_up, down):
        """Every rank passes the full tensors; the library keeps this rank's experts."""
        self.ops[0].load_q4cp(layer, gate_up, down)
        for op in self.ops[1:]:
            op.share_weights(self.ops[0])

    @property
    def launches(self):
        return sum(op.launches for op in self.ops)

    def forward(self, layer, x, logits, out):
        torch, dist = self.torch, self.torch.distributed
        T = x.shape[0]
        main = torch.cuda.current_stream()
        C = min(self.chunks, (T + self.tc - 1) // self.tc)
        span = [(c * self.tc, min(T, (c + 1) * self.tc)) for c in range(C)]
        # 1. routing + gather of every chunk, expert offsets of all ranks
        for c, (a, b) in enumerate(span):
            B = self.buf[c]
            self.ops[c].ep_route(layer, x[a:b], logits[a:b], eoff_out=B["eoff"], stream=main)
            dist.all_gather_into_tensor(B["eoff_all"], B["eoff"], group=self.group)
        routed = torch.cuda.Event()
        routed.record(main)
        splits, rows = [], 0
        for c in range(C):
            send, recv = exchange_splits(self.buf[c]["eoff_all"].cpu().numpy(), self.rank, self.world)
            if sum(recv) > self.buf[c]["cap"]:
                raise RuntimeError("expert-parallel receive buffer too small: %d rows > capacity %d"
                                   % (sum(recv), self.buf[c]["cap"]))
            splits.append((send, recv))
            rows += sum(recv)
        self.last_recv_rows = rows
        # 2. dispatch / experts / combine, exchanges on the communication stream
        self.comm.wait_event(routed)
        disp = [torch.cuda.Event() for _ in range(C)]
        done = [torch.cuda.Event() for _ in range(C)]
        back = [torch.cuda.Event() for _ in range(C)]

        def dispatch(c):
            (a, b), (send, recv), B = span[c], splits[c], self.buf[c]
            with torch.cuda.stream(self.comm):
                dist.all_to_all_single(B["x_recv"][:sum(recv)], B["x_send"][:(b - a) * self.k], recv, send,
                                       group=self.group)
                disp[c].record(self.comm)

        def combine_exchange(c):
            (a, b), (send, recv), B = span[c], splits[c], self.buf[c]
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(done[c])
                dist.all_to_all_single(B["pairs_back"][:(b - a) * self.k], B["pairs_recv"][:sum(recv)], send, recv,
                                       group=self.group)
                back[c].record(self.comm)

        dispatch(0)
        for c in range(C):
            if c + 1 < C:
                dispatch(c + 1)
            main.wait_event(disp[c])
            self.ops[c].ep_experts(layer, self.buf[c]["eoff_all"], stream=main)
            done[c].record(main)
            combine_exchange(c)
            if c >= 1:
                main.wait_event(back[c - 1])
                a, b = span[c - 1]
                self.ops[c - 1].ep_combine(out[a:b], b - a, stream=main)
        main.wait_event(back[C - 1])
        a, b = span[C - 1]
        self.ops[C - 1].ep_combine(out[a:b], b - a, stream=main)
