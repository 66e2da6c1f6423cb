"""Expert parallelism over one node's GPUs: host side.

One process per GPU (torch.distributed, NCCL). The 512 experts are partitioned evenly; a
forward is three library phases (route+gather, grouped GEMMs on the received rows, combine)
with two exchanges of fp16 rows in between: NCCL all-to-all (transport "nccl") or peer copies
by the copy engines into symmetric-memory buffers (transport "p2p"), which overlap the GEMMs
because they need no SM. The reference engine is a single-device program and has no
counterpart of this file.

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


def p2p_plan(eoff_all, rank, world):
    """Copy lists of the copy-engine transport from every rank's expert offset table.

    Returns (dispatch, back, recv_rows): dispatch = [(peer, src_row, dst_row, n)] copies of this
    rank's send rows into the peers' receive buffers (a receive buffer holds the sources' rows in
    rank order, exactly as all_to_all_single would leave them); back = [(peer, src_row, dst_row,
    n)] copies of this rank's result rows into the peers' result buffers (which are in the
    peers' own send order); recv_rows = rows this rank receives."""
    eo = np.asarray(eoff_all).reshape(world, -1)
    per = (eo.shape[1] - 1) // world
    bd = eo[:, ::per].astype(np.int64)          # [source][dest] row offsets in the source's send buffer
    cnt = bd[:, 1:] - bd[:, :-1]                # rows source s sends to dest p
    order = [(rank + i) % world for i in range(1, world + 1)]   # peers first, myself last
    dispatch = [(p, int(bd[rank, p]), int(cnt[:rank, p].sum()), int(cnt[rank, p])) for p in order]
    back = [(s, int(cnt[:s, rank].sum()), int(bd[s, rank]), int(cnt[s, rank])) for s in order]
    return dispatch, back, int(cnt[:, rank].sum())


def recv_rows_all(eoff_all, world):
    """Rows every rank receives (all sources), from the offset tables every rank holds: each rank
    can therefore see an overflow of ANY rank's receive buffer and all of them stop together,
    before a single row has been copied."""
    eo = np.asarray(eoff_all).reshape(world, -1)
    per = (eo.shape[1] - 1) // world
    bd = eo[:, ::per].astype(np.int64)
    return (bd[:, 1:] - bd[:, :-1]).sum(axis=0)


def next_seq(seq):
    """Sequence number of the next forward as a signed 32-bit value that wraps around: the
    device-side wait compares `flag - expected >= 0` in 32-bit arithmetic, which stays right
    across the wrap as long as two live numbers are less than 2^31 apart."""
    seq = (seq + 1) & 0xFFFFFFFF
    return seq - (1 << 32) if seq >= (1 << 31) else seq


def chunk_sizes(max_tokens, chunks, weights=None):
    """Tokens per chunk: equal parts (rounded up), or proportional to `weights` with every chunk at
    least one token and the sizes adding up to max_tokens."""
    if weights is None:
        return [(max_tokens + chunks - 1) // chunks] * chunks
    w = [float(v) for v in weights]
    if len(w) != chunks or min(w) <= 0:
        raise ValueError("chunk_weights: one positive weight per chunk")
    total = sum(w)
    sizes = [max(1, int(max_tokens * v / total)) for v in w]
    sizes[w.index(max(w))] += max_tokens - sum(sizes)   # the rounding remainder goes to the largest chunk
    if min(sizes) <= 0:
        raise ValueError("chunk_weights: too many chunks for %d tokens" % max_tokens)
    return sizes


def chunk_spans(T, sizes):
    """[(first, end)] token ranges of a forward of T tokens over chunks of at most `sizes` tokens,
    in order; chunks that get no token are left out."""
    span, a = [], 0
    for n in sizes:
        if a >= T:
            break
        span.append((a, min(T, a + n)))
        a += n
    return span


class ExpertParallelMoe:
    """The MoE layer sharded by expert over the ranks of a torch.distributed group.

    chunks > 1 splits a forward's tokens into that many chunks, each with its own library
    handle (workspaces) sharing one set of repacked weights; the all-to-all exchanges of a
    chunk run on a communication stream while the grouped GEMMs of its neighbours run on the
    compute stream, so the NVLink time hides behind the tensor-core time."""

    def __init__(self, experts, topk, d_model, d_mid, max_tokens, rank, world, device,
                 cap_factor=2.0, placement=None, group=None, chunks=1, sm_margin=16, transport="nccl", split_local=False,
                 has_shared=False, own_order="ends", chunk_weights=None, merge_sources=None):
        import torch
        import gfx1151_engine_b200 as pkg
        self.torch, self.group = torch, group
        self.transport = transport
        # p2p transport only: GEMMs over the rows a rank sent to itself run apart from those over the
        # other ranks' rows -- first chunk: own rows first (while the others still arrive), last
        # chunk: own rows last (while the others' results already travel back)
        self.split_local = (split_local or has_shared) and transport == "p2p"
        if has_shared and transport != "p2p":
            raise ValueError("a shared expert under expert parallelism needs the p2p transport (its rows run in the in-place own-rows pass)")
        # where the own-rows passes (which need no exchange) go: "first" = all of them up front, while
        # the first rows travel; "ends" = first chunk's up front, last chunk's at the very end, while
        # the last results travel back
        self.own_order = own_order
        # the other ranks' rows merged by expert before their GEMMs (b200moe_ep_experts_part part 4): one
        # extra memory pass per chunk against far fewer ragged tiles; pays from about four ranks on
        self.merge_sources = (world >= 4) if merge_sources is None else bool(merge_sources)
        self.has_shared = has_shared
        self.E, self.k, self.d, self.rank, self.world = experts, topk, d_model, rank, world
        # chunk sizes: equal, or in the proportions of chunk_weights (e.g. (1, 3, 3, 1): what no GEMM
        # hides is the dispatch of the FIRST chunk and the return of the LAST one, so those two are
        # best short)
        if chunk_weights is not None:
            chunks = len(chunk_weights)
        self.chunks = chunks
        self.chunk_tokens = chunk_sizes(max_tokens, chunks, chunk_weights)
        dev = torch.device("cuda", device)
        self.ops, self.buf = [], []
        for c in range(chunks):
            tc = self.chunk_tokens[c]
            op = pkg.MoeOperator(experts, topk, d_model, d_mid, tc, device=device, has_shared=has_shared,
                                 ep_rank=rank, ep_size=world,
                                 ep_sm_margin=sm_margin if (chunks > 1 and transport == "nccl") else 0)
            if c == 0:
                if placement is not None:
                    op.ep_set_placement(np.ascontiguousarray(placement, dtype=np.int32))
            else:
                op.share_weights(self.ops[0])
            pairs = tc * topk
            cap = int(cap_factor * pairs)
            own_rows = pairs + (tc if has_shared else 0)   # the shared expert's rows sit behind the routed ones
            if transport == "p2p":
                # written by the peers' copy engines: symmetric memory (mapped into every rank)
                import torch.distributed._symmetric_memory as symm_mem
                remote = lambda *shape, dtype=torch.float16: symm_mem.empty(*shape, dtype=dtype, device=dev)
            else:
                remote = lambda *shape, dtype=torch.float16: torch.empty(*shape, dtype=dtype, device=dev)
            b = {"cap": cap,
                 "x_send": torch.empty(own_rows, d_model, dtype=torch.float16, device=dev),
                 "x_recv": remote(cap, d_model),
                 "pairs_recv": torch.empty(cap, d_model, dtype=torch.float16, device=dev),
                 "pairs_back": remote(own_rows, d_model),
                 "eoff": torch.empty(experts + 1, dtype=torch.int32, device=dev),
                 "eoff_all": torch.empty(world * (experts + 1), dtype=torch.int32, device=dev),
                 "eoff_host": torch.empty(world * (experts + 1), dtype=torch.int32).pin_memory()}
            op.ep_attach(b["x_send"], b["x_recv"], b["pairs_recv"], b["pairs_back"], cap)
            self.ops.append(op)
            self.buf.append(b)
        self.op = self.ops[0]
        self.comm = torch.cuda.Stream(device=dev)
        self.last_recv_rows = 0
        if transport == "p2p":
            self._p2p_setup(dev)

    # ---- copy-engine transport -------------------------------------------------------------
    # The exchanges are peer copies (DMA over NVLink, no SM) straight into the destination
    # rank's receive buffer, so that they overlap the grouped GEMMs, which occupy every SM.
    # The receive buffers are symmetric memory (torch.distributed._symmetric_memory: mapped into
    # every rank through the driver's virtual-memory interface; plain cudaIpc mappings reached
    # only 23 GB/s here, these 685 GB/s per direction). "The rows of rank s have
    # arrived" is a flag in the receiver's memory: s copies its sequence number there behind
    # its data on the same stream (the copy engine runs a stream's copies in order), and the
    # receiver enqueues a bounded device-side wait on its flags (b200moe_ep_wait_flags).
    def _p2p_setup(self, dev):
        torch, dist = self.torch, self.torch.distributed
        import torch.distributed._symmetric_memory as symm_mem
        group = self.group if self.group is not None else dist.group.WORLD
        self.comm2 = torch.cuda.Stream(device=dev)
        self.seq = 0
        # the flag value of a forward: a one-element tensor filled on the copy stream; a small ring of
        # them, because the result copies of forward n may still read theirs when forward n+1 starts
        self.seq_ring = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(4)]
        self._handles = []
        for b in self.buf:
            b["flags"] = symm_mem.empty(2, 32, dtype=torch.int32, device=dev)  # [dispatch | return][source rank]
            b["flags"].zero_()
            torch.cuda.synchronize(dev)
            b["peer_x_recv"], b["peer_back"], b["peer_flags"] = [], [], []
            for key, dst in (("x_recv", "peer_x_recv"), ("pairs_back", "peer_back"), ("flags", "peer_flags")):
                hdl = symm_mem.rendezvous(b[key], group)
                self._handles.append(hdl)
                for r in range(self.world):
                    b[dst].append(b[key] if r == self.rank else hdl.get_buffer(r, list(b[key].shape), b[key].dtype))
        dist.barrier(group=self.group)

    def _forward_p2p(self, layer, x, logits, out, in_ready=None, out_done=None):
        torch, dist = self.torch, self.torch.distributed
        T = x.shape[0]
        main = torch.cuda.current_stream()
        span = chunk_spans(T, self.chunk_tokens)
        C = len(span)
        self.seq = next_seq(self.seq)
        seq = self.seq
        seq_t = self.seq_ring[seq & 3]
        # 1. routing of every chunk; the offset tables of all ranks travel to the host one chunk at a
        #    time, so that the host can plan (and start) chunk 0's copies while chunk 1 still routes
        routed, tables = [], []
        for c, (a, b) in enumerate(span):
            B = self.buf[c]
            if in_ready is not None:
                main.wait_event(in_ready[c])     # the chunk's x and logits (a host copy on another stream) are there
            self.ops[c].ep_route(layer, x[a:b], logits[a:b], eoff_out=B["eoff"], stream=main)
            ev = torch.cuda.Event()
            ev.record(main)
            routed.append(ev)
            dist.all_gather_into_tensor(B["eoff_all"], B["eoff"], group=self.group)
            B["eoff_host"].copy_(B["eoff_all"], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(main)
            tables.append(ev)
        in_place = self.split_local
        if in_place:
            # the rows that stay on this GPU (and the shared expert's) need no exchange: their GEMMs read
            # the send buffer and write the result buffer in place, while the first rows travel
            first_own = range(C) if self.own_order == "first" or C == 1 else range(C - 1)
            for c in first_own:
                self.ops[c].ep_experts(layer, self.buf[c]["eoff_all"], stream=main, part=3)
        plans, rows = [], 0
        with torch.cuda.stream(self.comm):
            seq_t.fill_(seq)
            seq_ready = torch.cuda.Event()
            seq_ready.record(self.comm)
        for c in range(C):
            tables[c].synchronize()
            eo = self.buf[c]["eoff_host"].numpy()
            need = recv_rows_all(eo, self.world)
            if int(need.max()) > self.buf[c]["cap"]:
                # every rank sees the same table and stops here, before any copy has been issued
                raise RuntimeError("expert-parallel receive buffer too small: rank %d would receive %d rows, capacity %d"
                                   % (int(need.argmax()), int(need.max()), self.buf[c]["cap"]))
            plan = p2p_plan(eo, self.rank, self.world)
            plans.append(plan)
            rows += plan[2]
            # 2. dispatch of the chunk: my rows for rank p go behind the rows of the ranks before me in
            #    p's buffer. (p has finished reading that buffer: I waited for p's results of the
            #    previous forward, which p sent after its GEMMs.)
            B = self.buf[c]
            self.comm.wait_event(routed[c])
            with torch.cuda.stream(self.comm):
                for p, src0, dst0, n in plan[0]:
                    if n and not (in_place and p == self.rank):
                        B["peer_x_recv"][p][dst0:dst0 + n].copy_(B["x_send"][src0:src0 + n], non_blocking=True)
                    B["peer_flags"][p][0, self.rank:self.rank + 1].copy_(seq_t, non_blocking=True)
        self.last_recv_rows = rows
        self.comm2.wait_event(seq_ready)

        def send_back(c):
            B = self.buf[c]
            done = torch.cuda.Event()
            done.record(main)
            self.comm2.wait_event(done)
            with torch.cuda.stream(self.comm2):
                for s, src0, dst0, n in plans[c][1]:
                    if n and not (in_place and s == self.rank):
                        B["peer_back"][s][dst0:dst0 + n].copy_(B["pairs_recv"][src0:src0 + n], non_blocking=True)
                    B["peer_flags"][s][1, self.rank:self.rank + 1].copy_(seq_t, non_blocking=True)

        def combine(c):
            a, b = span[c]
            B = self.buf[c]
            self.ops[c].ep_wait_flags(B["flags"][1], self.world, seq, stream=main)
            self.ops[c].ep_combine(out[a:b], b - a, stream=main)
            if out_done is not None:
                out_done[c].record(main)

        # 3. experts per chunk once its rows have arrived; results go straight back to their owners.
        #    With out_done given (a caller that copies each chunk's output away as soon as it is
        #    there), a chunk is combined right behind the NEXT chunk's GEMMs -- its results came back
        #    while those ran -- instead of at the very end.
        early = out_done is not None
        for c in range(C):
            B = self.buf[c]
            self.ops[c].ep_wait_flags(B["flags"][0], self.world, seq, stream=main)
            self.ops[c].ep_experts(layer, B["eoff_all"], stream=main,
                                   part=(4 if self.merge_sources else 2) if in_place else 0)
            send_back(c)
            if early and c >= 1:
                combine(c - 1)
        if in_place and self.own_order != "first" and C > 1:
            self.ops[C - 1].ep_experts(layer, self.buf[C - 1]["eoff_all"], stream=main, part=3)
        # 4. combine
        for c in range(C - 1 if early else 0, C):
            combine(c)

    def load_q4cp(self, layer, gate_up, down):
        """Every rank passes the full tensors; the library keeps this rank's experts."""
        self.ops[0].load_q4cp(layer, gate_up, down)
        for op in self.ops[1:]:
            op.share_weights(self.ops[0])

    def load_shared_q4cp(self, layer, gate, up, down, gate_w_bf16):
        """The shared expert is not sharded: every rank holds it and runs it for its own tokens."""
        self.ops[0].load_shared_q4cp(layer, gate, up, down, gate_w_bf16)
        for op in self.ops[1:]:
            op.share_weights(self.ops[0])

    @property
    def launches(self):
        return sum(op.launches for op in self.ops)

    def forward(self, layer, x, logits, out, in_ready=None, out_done=None):
        """in_ready / out_done (p2p transport): one CUDA event per chunk (chunk_spans(T, self.chunk_tokens)).
        The routing of chunk c waits for in_ready[c] -- the caller's copy of that chunk's x and logits
        into device memory -- and out_done[c] is recorded when the chunk's rows of `out` are final, so
        that host copies in and out overlap the other chunks' work."""
        if self.transport == "p2p":
            return self._forward_p2p(layer, x, logits, out, in_ready, out_done)
        if in_ready is not None:
            for ev in in_ready:
                self.torch.cuda.current_stream().wait_event(ev)
        torch, dist = self.torch, self.torch.distributed
        T = x.shape[0]
        main = torch.cuda.current_stream()
        span = chunk_spans(T, self.chunk_tokens)
        C = len(span)
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
