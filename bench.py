"""Benchmark of the routed-expert MoE FFN path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[2], "config 3"): one 512-expert top-10 q4cp MoE layer
(d_model 4096, expert intermediate 1024, group 32, fp16 scales), a 16384-token prefill
chunk per step and per GPU, bf16 activations ~ N(0,1), router logits ~ N(0,1) plus a
per-expert Zipf(1.1) bias. Weights and inputs are synthetic (seeded); a step is one
b200moe_forward call: router top-k, bucketing, activation gather, tcgen05 gate/up GEMM
+ SwiGLU, down GEMM, weighted combine.

Prints ONE JSON line: value = tokens/s with inputs resident in HBM (CUDA events on the
launching stream, max over ranks); e2e = the same call through b200moe_forward_host with
pinned host buffers (host<->device copies inside the timed region); roofline = the gate/up
GEMM kernel's algorithmic FLOP/s against the measured dense 16-bit peak; cpu_baseline =
the CPU oracle timed on this host on a bounded token sample; decode = the T=1 / T=5 GEMV
path (configs[1]) with rotated routings. `--impl reference` times the reference's own CPU
code (oracle/_ref, built from the reference sources) instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E, K_TOP, D, MID, T_CHUNK = 512, 10, 4096, 1024, 16384   # E is overridable for small profiling cases
FLOP_PER_TOKEN = K_TOP * (2 * (2 * MID) * D + 2 * D * MID)          # 251,658,240
FLOP_UP_PER_TOKEN = K_TOP * 2 * (2 * MID) * D                        # gate/up GEMM share
BYTES_PER_EXPERT = 3 * MID * D * 9 // 16                             # 7,077,888 (0.5625 B / weight)
WORKLOAD = "config3: 16384-token prefill, 512 experts top-10, d=4096, mid=1024, q4cp g32, Zipf(1.1) routing"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["bf16_tflops"]), float(j["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples (every 25 ms, with nvidia-smi's own time
    stamps); stop(t0, t1) keeps the samples that fall inside the timed region."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            deadline = time.time() + 3.0          # nvidia-smi needs a moment before its first line
            while not self.rows and time.time() < deadline:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    @staticmethod
    def _epoch(stamp):
        import datetime
        try:
            return datetime.datetime.strptime(stamp, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self, t0=None, t1=None):
        if self.proc:
            time.sleep(0.06)                      # let the last samples of the region arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, power, reasons, total = [], 0, [], set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                total += 1
                ts = self._epoch(r[0])
                if t0 is not None and ts is not None and not (t0 - 0.005 <= ts <= t1 + 0.03):
                    continue
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
                power.append(float(r[3]))
                for n, v in zip(names, r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "power_w": float(np.median(power)) if power else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_total": total}


# ------------------------------------------------------------------ synthetic layer on the GPU
def q4cp_blob_device(torch, rows, cols, gen):
    """A q4cp tensor blob built in device memory: linear symmetric code book, uniform codes,
    fp16 scales |N(0, 0.02)| (no padding at these widths: the scale record is cols/16 bytes)."""
    assert (cols // 32 * 2) % 16 == 0
    ncode, nscale = rows * cols // 2, rows * (cols // 32)
    blob = torch.empty(64 + ncode + nscale * 2, dtype=torch.uint8, device="cuda")
    book = ((2.0 * torch.arange(16, dtype=torch.float32) - 15.0) / 15.0)
    blob[:64] = book.view(torch.uint8).cuda()
    step = 1 << 28
    for o in range(0, ncode, step):
        n = min(step, ncode - o)
        blob[64 + o:64 + o + n] = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=gen)
    sc = (torch.randn(nscale, device="cuda", generator=gen) * 0.02).abs().to(torch.float16)
    blob[64 + ncode:] = sc.view(torch.uint8)
    return blob


def gguf_blocks_device(torch, rows, cols, kind, gen):
    """GGUF blocks built in device memory with the magnitudes of the q4cp configs: per block
    a = |N(0, 0.02)|; Q4_K (144 B / 256): d = a/(63*15), dmin = a/(63*2), the other 140 bytes
    uniform; Q5_1 (24 B / 32): d = a/31, m = -a/2, the other 20 bytes uniform."""
    per, bb = (256, 144) if kind == "q4k" else (32, 24)
    nb = rows * cols // per
    blob = torch.empty(nb, bb, dtype=torch.uint8, device="cuda")
    step = 1 << 22
    for o in range(0, nb, step):
        n = min(step, nb - o)
        blob[o:o + n] = torch.randint(0, 256, (n, bb), dtype=torch.uint8, device="cuda", generator=gen)
        a = (torch.randn(n, device="cuda", generator=gen) * 0.02).abs()
        if kind == "q4k":
            hdr = torch.stack([a / (63.0 * 15.0), a / (63.0 * 2.0)], dim=1)
        else:
            hdr = torch.stack([a / 31.0, -a / 2.0], dim=1)
        blob[o:o + n, 0:4] = hdr.to(torch.float16).view(torch.uint8).reshape(n, 4)
    return blob.reshape(-1)


ZIPF_STRENGTH = 1.0  # --zipf-strength: 1.0 = the benchmark's Zipf(1.1) bias, 0.5 = the milder sensitivity run


def zipf_logits(torch, T, gen, seed):
    from gfx1151_engine_b200 import synth
    bias = synth.zipf_bias(synth.rng_for(seed, 77), E, strength=ZIPF_STRENGTH)
    return (torch.randn(T, E, device="cuda", generator=gen) + torch.from_numpy(bias).cuda()[None, :]).contiguous()


# ------------------------------------------------------------------ CPU legs
def cpu_leg(layer_host, x_bits, logits, threads, spec=None):
    """Runs and times the CPU oracle on the given tokens of the workload.
    Returns (tokens/s, y[n][d] f32, ids[n][16])."""
    import oracle
    from gfx1151_engine_b200 import synth
    spec = spec or synth.CONFIG3
    x = synth.bf16_bits_to_f32(x_bits)
    t0 = time.perf_counter()
    y, ids, _ = oracle.moe_forward(spec, layer_host, x, logits=logits, threads=threads)
    return x.shape[0] / (time.perf_counter() - t0), y, ids


def parity(y_gpu_f32, y_ref_f32, ids_gpu, ids_ref, k):
    """The CUDA result against the CPU oracle on the same tokens, both rounded to bf16."""
    from gfx1151_engine_b200 import synth
    ref = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(y_ref_f32)).astype(np.float64)
    diff = np.abs(y_gpu_f32.astype(np.float64) - ref)
    max_abs, mean_rel = float(diff.max()), float(diff.mean() / max(np.abs(ref).mean(), 1e-30))
    ids_equal = bool(np.array_equal(ids_gpu[:, :k], ids_ref[:, :k]))
    return {"tokens": int(ref.shape[0]), "max_abs": max_abs, "mean_rel": mean_rel, "ids_equal": ids_equal,
            "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-3},
            "ok": bool(ids_equal and max_abs <= 2e-2 and mean_rel <= 1e-3 and np.isfinite(y_gpu_f32).all())}


def stratified_tokens(ids, k, n, seed=5):
    """n token indices of the chunk: a third with a pair on the most loaded expert, a third with
    a pair on a single-row expert (as far as such tokens exist), the rest at random."""
    rng = np.random.Generator(np.random.Philox(key=[seed, 0]))
    T = ids.shape[0]
    hist = np.bincount(ids[:, :k].reshape(-1), minlength=E)
    on_hot = np.flatnonzero((ids[:, :k] == int(np.argmax(hist))).any(axis=1))
    on_single = np.flatnonzero(np.isin(ids[:, :k], np.flatnonzero(hist == 1)).any(axis=1))
    pick = set(int(t) for t in rng.permutation(on_hot)[: n // 3])
    pick |= set(int(t) for t in rng.permutation(on_single)[: n // 3])
    for t in rng.permutation(T):
        if len(pick) >= n:
            break
        pick.add(int(t))
    sel = np.array(sorted(pick), dtype=np.int64)
    return sel, {"on_most_loaded_expert": int(np.isin(sel, on_hot).sum()), "on_single_row_experts": int(np.isin(sel, on_single).sum())}


def reference_arm(args):
    """The reference's own CPU path (Model::moe, src/ref.cpp) on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from gfx1151_engine_b200 import synth
    cores = os.cpu_count() or 1
    kind = "reference" if oracle.have_ref() else "port"
    spec = synth.CONFIG3
    layer = {"gate_up": synth.make_q4cp(synth.rng_for(0, 1), E * 2 * MID, D),
             "down": synth.make_q4cp(synth.rng_for(0, 2), E * D, MID)}
    n_tok = max(cores, 8) * 2     # per step: about 0.3 core-seconds per token
    total = n_tok * (args.steps + args.warmup)
    xb = synth.make_x(synth.rng_for(0, 9), total, D)
    logits = synth.make_logits(synth.rng_for(0, 10), total, E, zipf=True, zipf_rng=synth.rng_for(0, 77))
    if kind == "reference":
        # Model::moe derives its logits from a router weight and always evaluates a shared
        # expert: give it a random router weight and a shared expert with zero down scales.
        layer["router_w"] = synth.f32_to_bf16_bits(synth.rng_for(0, 8).normal(0, 0.02, (E, D)).astype(np.float32))
        layer["sh_gate"] = synth.make_q4cp(synth.rng_for(0, 4), MID, D)
        layer["sh_up"] = synth.make_q4cp(synth.rng_for(0, 5), MID, D)
        layer["sh_down"] = synth.make_q4cp(synth.rng_for(0, 6), D, MID, zero_scales=True)
        layer["sh_gate_w"] = synth.f32_to_bf16_bits(np.zeros(D, np.float32))
    times = []
    for s in range(args.steps + args.warmup):
        sl = slice(s * n_tok, (s + 1) * n_tok)
        t0 = time.perf_counter()
        if kind == "reference":
            import dataclasses
            oracle.ref_moe_layer(dataclasses.replace(spec, shared=True), layer,
                                 synth.bf16_bits_to_f32(xb[sl]), threads=cores)
        else:
            oracle.moe_forward(spec, layer, synth.bf16_bits_to_f32(xb[sl]), logits=logits[sl], threads=cores)
        if s >= args.warmup:
            times.append(time.perf_counter() - t0)
    value = n_tok * len(times) / sum(times)
    sample = ("%d tokens per step of the config-3 layer on %d host threads (OpenMP over tokens)" % (n_tok, cores))
    if kind == "reference":
        sample += "; unmodified Model::moe, logits from a random bf16 router weight, shared expert evaluated with zero down scales"
    print(json.dumps({
        "impl": "reference", "metric": "moe_prefill_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": n_tok},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# ------------------------------------------------------------------ GPU arm
def main():
    global E, ZIPF_STRENGTH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--tokens", type=int, default=T_CHUNK)
    ap.add_argument("--experts", type=int, default=E, help="smaller layer for profiler captures (not a bench line)")
    ap.add_argument("--format", default="q4cp", choices=["q4cp", "gguf"],
                    help="expert tensors: hgn q4cp (the benchmark workload) or GGUF Q4_K gate/up + Q5_1 down "
                         "(the GGUF variant; with --tokens 8192 --no-decode --no-cpu, single GPU)")
    ap.add_argument("--chunks", type=int, default=0,
                    help="N>1: token chunks whose exchanges overlap the GEMMs; 0 (default) = 2 up to 4 GPUs, 3 from 8 on "
                         "(measured at 8 GPUs: 2 chunks 6.84 ms, 3 chunks 6.46 ms, 4 chunks 6.72 ms)")
    ap.add_argument("--chunk-weights", default="", help="N>1: relative chunk sizes, e.g. 1,3,3,1 (overrides --chunks)")
    ap.add_argument("--sm-margin", type=int, default=32, help="N>1: SMs left free for the NCCL kernels")
    ap.add_argument("--transport", default="p2p", choices=["nccl", "p2p"],
                    help="N>1: exchanges by NCCL all-to-all or by peer copies (copy engines) through CUDA IPC")
    ap.add_argument("--zipf-strength", type=float, default=1.0,
                    help="scale of the per-expert Zipf(1.1) log-bias (1.0 = benchmark workload; 0.5 / 0 = sensitivity runs)")
    ap.add_argument("--ep-split", type=int, default=1,
                    help="N>1, p2p transport: 1 (default) = the rows a rank keeps are multiplied in place (no copy), apart from the other ranks' rows; 0 = one GEMM pass per chunk over copied rows")
    ap.add_argument("--ep-merge", type=int, default=-1,
                    help="N>1: 1 = the other ranks' rows are merged by expert before their GEMMs (one run per expert instead of "
                         "one per source rank and expert), 0 = not, -1 (default) = from 4 GPUs on")
    ap.add_argument("--own-order", default="ends", choices=["first", "ends"],
                    help="N>1, --ep-split 1: the in-place own-rows passes all up front, or the last chunk's at the very end")
    ap.add_argument("--check", type=int, default=1,
                    help="N>1: 1 (default) = compare rank 0's output with the single-GPU operator on the same tokens; 0 = skip")
    ap.add_argument("--no-gguf", action="store_true", help="skip the GGUF-variant leg (Q4_K gate/up, Q5_1 down, 8192 tokens)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode / verify measurements")
    ap.add_argument("--decode-only", action="store_true",
                    help="profiling aid: only the decode / verify leg, prints its numbers")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    E = args.experts
    ZIPF_STRENGTH = args.zipf_strength
    if args.chunks <= 0:
        args.chunks = 3 if args.gpus >= 8 else 2

    import torch
    import torch.distributed as dist
    import gfx1151_engine_b200 as pkg
    from gfx1151_engine_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    T = args.tokens
    peak_tf, peak_hbm, peak_kind = measured_peaks()

    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)            # one weight set shared by all ranks
    gguf = args.format == "gguf"
    if gguf:
        if world > 1:
            raise SystemExit("--format gguf is a single-GPU measurement")
        args.no_decode = args.no_cpu = True
        gu = (gguf_blocks_device(torch, E * MID, D, "q4k", gen), gguf_blocks_device(torch, E * MID, D, "q4k", gen))
        dn = gguf_blocks_device(torch, E * D, MID, "q51", gen)
    else:
        gu = q4cp_blob_device(torch, E * 2 * MID, D, gen)
        dn = q4cp_blob_device(torch, E * D, MID, gen)
    epm = None
    if world > 1:
        # expert parallelism: E/world experts per GPU, placed by a calibration histogram of the
        # router (same seeded batch on every rank), NCCL all-to-all for dispatch and combine
        from gfx1151_engine_b200 import ep
        gcal = torch.Generator(device="cuda")
        gcal.manual_seed(4321)
        cal = torch.topk(zipf_logits(torch, 4096, gcal, 0), K_TOP, dim=1).indices.reshape(-1)
        load = torch.bincount(cal, minlength=E).cpu().numpy()
        placement = ep.greedy_placement(load, world)
        epm = ep.ExpertParallelMoe(E, K_TOP, D, MID, T, rank, world, local, cap_factor=2.0, placement=placement,
                                   chunks=args.chunks, sm_margin=args.sm_margin, transport=args.transport,
                                   chunk_weights=[float(v) for v in args.chunk_weights.split(",")] if args.chunk_weights else None,
                                   split_local=args.ep_split == 1, own_order=args.own_order,
                                   merge_sources=None if args.ep_merge < 0 else bool(args.ep_merge))
        epm.load_q4cp(0, gu, dn)
        op = epm.op
    else:
        op = pkg.MoeOperator(E, K_TOP, D, MID, T, device=local)
        if gguf:
            op.load_gguf(0, gu[0], gu[1], dn)
        else:
            op.load_q4cp(0, gu, dn)
    if args.decode_only:
        args.no_cpu = True
    want_cpu = rank == 0 and world == 1 and not args.no_cpu
    layer_host = {"gate_up": gu.cpu().numpy(), "down": dn.cpu().numpy()} if want_cpu else None
    op_dec = None
    if rank == 0 and world == 1 and not args.no_decode:
        gen2 = torch.Generator(device="cuda")
        gen2.manual_seed(99)
        op_dec = pkg.MoeOperator(E, K_TOP, D, MID, 16, has_shared=True, device=local)
        op_dec.load_q4cp(0, gu, dn)
        sh = [q4cp_blob_device(torch, MID, D, gen2), q4cp_blob_device(torch, MID, D, gen2),
              q4cp_blob_device(torch, D, MID, gen2)]
        sh_gw = (torch.randn(D, device="cuda", generator=gen2) * 0.02).to(torch.bfloat16)
        op_dec.load_shared_q4cp(0, sh[0], sh[1], sh[2], sh_gw)
        if layer_host is not None:
            layer_host.update({"sh_gate": sh[0].cpu().numpy(), "sh_up": sh[1].cpu().numpy(), "sh_down": sh[2].cpu().numpy(),
                               "sh_gate_w": sh_gw.view(torch.int16).cpu().numpy().view(np.uint16)})
    if args.decode_only and op_dec is not None:
        del gu, dn
        print(json.dumps({"decode": decode_leg(torch, op_dec, peak_hbm, torch.cuda.current_stream(), graph=True,
                                               layer_host=layer_host)}))
        return
    op_ref = None
    if world > 1 and args.check == 1 and rank == 0:
        op_ref = pkg.MoeOperator(E, K_TOP, D, MID, T, device=local)   # whole layer on one GPU, for the check
        op_ref.load_q4cp(0, gu, dn)
    del gu, dn
    torch.cuda.empty_cache()

    gen_in = torch.Generator(device="cuda")
    gen_in.manual_seed(1000 + rank)  # per-rank inputs
    x = torch.randn(T, D, device="cuda", generator=gen_in).to(torch.bfloat16)
    logits = zipf_logits(torch, T, gen_in, 0)
    out = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream()
    # realised routing histogram of this rank's chunk (pairs per expert)
    hist = torch.bincount(torch.topk(logits, K_TOP, dim=1).indices.reshape(-1), minlength=E).cpu().numpy()
    routing = {"zipf_strength": ZIPF_STRENGTH, "pairs_max": int(hist.max()), "pairs_median": float(np.median(hist)),
               "experts_below_64_pairs": int((hist < 64).sum()), "experts_unused": int((hist == 0).sum())}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if epm is not None:
            epm.forward(0, x, logits, out)
        else:
            op.moe_b(0, x, logits, out, stream=stream)

    for _ in range(args.warmup):
        step()
    op.synchronize(stream)
    check = None
    if op_ref is not None:
        ref_out = torch.empty_like(out)
        op_ref.moe_b(0, x, logits, ref_out, stream=stream)
        op_ref.synchronize(stream)
        a, b = out.float(), ref_out.float()
        check = {"max_abs": float((a - b).abs().max()), "mean_rel": float((a - b).abs().mean() / b.abs().mean())}
        op_ref.close()
    if world == 1:
        op.profile_enable(True)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    barrier()   # the sampler's start-up must not skew the ranks against each other
    counter = epm if epm is not None else op
    l0 = counter.launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    wall1 = time.time()
    launches = counter.launches - l0
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    op.synchronize(stream)
    ms = ev0.elapsed_time(ev1)
    stages = op.profile_read() if world == 1 else {"up": 0.0}
    if world == 1:
        op.profile_enable(False)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * T * args.steps / (ms * 1e-3)

    # end to end with HOST buffers (pinned), host<->device copies inside the timed region
    xh = torch.empty(T, D, dtype=torch.bfloat16).pin_memory()
    xh.copy_(x)
    lh = torch.empty(T, E, dtype=torch.float32).pin_memory()
    lh.copy_(logits)
    oh = torch.empty(T, D, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    if epm is not None and args.transport == "p2p":
        # host copies per chunk on their own streams: chunk c+1 comes in while chunk c is routed and
        # multiplied, chunk c goes out while chunk c+1 is multiplied
        from gfx1151_engine_b200 import ep as ep_mod
        spans = ep_mod.chunk_spans(T, epm.chunk_tokens)
        ev_in = [torch.cuda.Event() for _ in spans]
        ev_out = [torch.cuda.Event() for _ in spans]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        if epm is not None and args.transport == "p2p":
            s_in.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s_in):
                for c, (a, b) in enumerate(spans):
                    logits[a:b].copy_(lh[a:b], non_blocking=True)
                    x[a:b].copy_(xh[a:b], non_blocking=True)
                    ev_in[c].record(s_in)
            epm.forward(0, x, logits, out, in_ready=ev_in, out_done=ev_out)
            with torch.cuda.stream(s_out):
                for c, (a, b) in enumerate(spans):
                    s_out.wait_event(ev_out[c])
                    oh[a:b].copy_(out[a:b], non_blocking=True)
            torch.cuda.synchronize()
        elif epm is not None:
            x.copy_(xh, non_blocking=True)
            logits.copy_(lh, non_blocking=True)
            epm.forward(0, x, logits, out)
            oh.copy_(out, non_blocking=True)
            torch.cuda.synchronize()
        else:
            op.moe_b_host(0, xh, lh, oh, T, stream=stream)   # the C-ABI entry point with host buffers

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": world * T * e2e_steps / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": T * D * 2 + T * E * 4, "d2h_bytes_per_step": T * D * 2,
           "checksum": float(oh.float().abs().mean())}
    ep_info = None
    if epm is not None:
        rows = torch.tensor([float(epm.last_recv_rows)], device="cuda")
        mx = rows.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows, op=dist.ReduceOp.SUM)
        ep_info = {"experts_per_gpu": E // world, "placement": "greedy by calibration histogram",
                   "recv_rows_max_over_mean": float(mx.item() / (rows.item() / world)),
                   "exchange": ("peer copies by the copy engines into symmetric-memory receive buffers, arrival flags + bounded device-side wait"
                                if args.transport == "p2p" else "NCCL all_to_all_single (dispatch, combine)") + "; NCCL all_gather of expert offsets",
                   "chunks": args.chunks, "chunk_weights": args.chunk_weights or None, "transport": args.transport,
                   "own_rows": "in place, own passes at the %s of the chunk pipeline" % ("ends" if args.own_order == "ends" else "front") if args.ep_split == 1 else "copied like the others",
                   "tails_merged_by_expert": bool(epm.merge_sources),
                   "check_vs_single_gpu": check}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    if world == 1:
        up_s = stages["up"] * 1e-3
        achieved = FLOP_UP_PER_TOKEN * T / up_s / 1e12 if up_s > 0 else 0.0
        roof_kernel = "k_expert_tc<up> (gate/up GEMM + SwiGLU)"
    else:
        # per GPU, over the whole step including both all-to-all exchanges
        achieved = FLOP_PER_TOKEN * T * args.steps / (ms * 1e-3) / 1e12
        roof_kernel = ("whole expert-parallel step per GPU (grouped GEMMs + dispatch / combine exchanges by %s)"
                       % ("peer copies of the copy engines" if args.transport == "p2p" else "NCCL all-to-all"))
        stages = {}
    result = {
        "metric": "moe_prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": ("GGUF variant (Q4_K gate/up, Q5_1 down), not the benchmark workload" if gguf else
                                "sensitivity run with a scaled routing bias (not the benchmark workload)" if ZIPF_STRENGTH != 1.0 else
                                WORKLOAD if (E, T) == (512, T_CHUNK) else "reduced case for profiling (not the benchmark workload)"), "tokens_per_gpu": T, "experts": E, "topk": K_TOP, "d_model": D,
                   "d_mid": MID, "routing": routing, "parallelism": "expert-parallel x%d" % world if world > 1 else "single GPU",
                   "l2": "inputs larger than L2: 3.6 GB of expert weights + 168 MB of activations per step"},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "expert_parallel": ep_info,
        "stage_ms": {k: round(v, 4) for k, v in stages.items()},
        "layer_tflops": FLOP_PER_TOKEN * T * args.steps / (ms * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "kernel": roof_kernel,
                     "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_kind": peak_kind + " dense 16-bit burst",
                     "traffic": 4.98e9 if (world == 1 and (E, T) == (512, T_CHUNK)) else None,
                     "traffic_note": "bytes per gate/up launch, scaled from an ncu capture of a reduced case by algorithmic bytes"},
    }

    if op_dec is not None:
        result["decode"] = decode_leg(torch, op_dec, peak_hbm, stream, layer_host=layer_host)
    if world == 1 and not gguf:
        # the step in front of the path: router logits from hidden states (random router weight)
        gw = torch.Generator(device="cuda")
        gw.manual_seed(77)
        op.load_router(0, (torch.randn(E, D, device="cuda", generator=gw) * 0.02).to(torch.bfloat16))
        lg2 = torch.empty(T, E, dtype=torch.float32, device="cuda")
        for _ in range(3):
            op.router_logits(0, x, lg2, stream=stream)
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record(stream)
        for _ in range(10):
            op.router_logits(0, x, lg2, stream=stream)
        r1.record(stream)
        op.synchronize(stream)
        rms = r0.elapsed_time(r1) / 10
        result["router_from_hidden"] = {"ms": rms, "tflops": 2.0 * T * E * D / (rms * 1e-3) / 1e12,
                                        "what": "b200moe_router_logits: bf16 tcgen05 GEMM + near-tie recomputation in the reference's arithmetic; not part of `value`"}
    if want_cpu:
        # The CPU oracle on a sample of the very chunk the GPU just computed: its time is the CPU
        # baseline, its output the parity check of the benchmarked call (`out` still holds the
        # result of the last timed step).
        cores = os.cpu_count() or 1
        n_tok = max(64, min(256, cores * 8))
        op.moe_b(0, x, logits, out, stream=stream)   # (the host-buffer leg above left the routing of its last token range)
        op.synchronize(stream)
        ids_gpu = op.get_routing(T)[0]
        sel, strata = stratified_tokens(ids_gpu, K_TOP, n_tok)
        sel_dev = torch.from_numpy(sel).cuda()
        xb = x[sel_dev].view(torch.int16).cpu().numpy().view(np.uint16)
        lg = logits[sel_dev].cpu().numpy()
        v, y_ref, ids_ref = cpu_leg(layer_host, xb, lg, cores)
        result["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                                  "sample": "%d tokens of the same chunk (stratified: hot-expert, single-row-expert and random tokens), "
                                            "CPU oracle with OpenMP over tokens" % len(sel)}
        result["parity"] = parity(out[sel_dev].float().cpu().numpy(), y_ref, ids_gpu[sel], ids_ref, K_TOP)
        result["parity"].update(strata)
        result["parity"]["what"] = "output of the timed 16384-token call against the CPU oracle on a stratified token sample, both rounded to bf16"
    if world == 1 and not gguf and not args.no_gguf and (E, T) == (512, T_CHUNK):
        op.close()
        del op
        torch.cuda.empty_cache()
        result["gguf"] = gguf_leg(torch, pkg, peak_tf, stream, local)
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def gguf_leg(torch, pkg, peak_tf, stream, device, T=8192, steps=10):
    """configs[3]: the GGUF variant of the layer (Q4_K gate/up, Q5_1 down) at 8192 tokens."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4321)
    gate = gguf_blocks_device(torch, E * MID, D, "q4k", gen)
    up = gguf_blocks_device(torch, E * MID, D, "q4k", gen)
    dn = gguf_blocks_device(torch, E * D, MID, "q51", gen)
    op = pkg.MoeOperator(E, K_TOP, D, MID, T, device=device)
    op.load_gguf(0, gate, up, dn)
    del gate, up, dn
    torch.cuda.empty_cache()
    x = torch.randn(T, D, device="cuda", generator=gen).to(torch.bfloat16)
    logits = zipf_logits(torch, T, gen, 0)
    out = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        op.moe_b(0, x, logits, out, stream=stream)
    op.synchronize(stream)
    op.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        op.moe_b(0, x, logits, out, stream=stream)
    e1.record(stream)
    op.synchronize(stream)
    ms = e0.elapsed_time(e1) / steps
    stages = op.profile_read()
    op.close()
    tf = FLOP_PER_TOKEN * T / (ms * 1e-3) / 1e12
    return {"workload": "config4: 8192-token prefill, Q4_K gate/up + Q5_1 down, same layer shapes and routing bias",
            "ms": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": tf, "frac": tf / peak_tf,
            "stage_ms": {k: round(v, 4) for k, v in stages.items() if k != "calls"},
            "finite": bool(torch.isfinite(out.float()).all().item())}


def decode_leg(torch, op, peak_hbm, stream, graph=True, layer_host=None):
    """configs[1]: T = 1 and T = 5 with the shared expert; 64 rotated routings so that the
    selected experts are not resident in L2 from the previous call. With the layer's host
    copy, the first routing of each T is also checked against the CPU oracle."""
    out = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    for T in (1, 5):
        sets = 64
        xs = torch.randn(sets, T, D, device="cuda", generator=gen).to(torch.bfloat16)
        lgs = torch.randn(sets, T, E, device="cuda", generator=gen)
        o = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
        for i in range(8):
            op.moe_b(0, xs[i], lgs[i], o, stream=stream)
        op.synchronize(stream)
        par = None
        if layer_host is not None and "sh_gate" in layer_host:
            from gfx1151_engine_b200 import synth
            op.moe_b(0, xs[0], lgs[0], o, stream=stream)
            op.synchronize(stream)
            _, y_ref, ids_ref = cpu_leg(layer_host, xs[0].view(torch.int16).cpu().numpy().view(np.uint16),
                                        lgs[0].cpu().numpy(), os.cpu_count() or 1, spec=synth.CONFIG2)
            par = parity(o.float().cpu().numpy(), y_ref, op.get_routing(T)[0], ids_ref, K_TOP)
        uniq = []
        for i in range(sets):
            ids = torch.topk(lgs[i], K_TOP, dim=1).indices
            uniq.append(int(torch.unique(ids).numel()))
        op.profile_enable(True)
        for i in range(16):
            op.moe_b(0, xs[i], lgs[i], o, stream=stream)
        stages = op.profile_read()
        op.profile_enable(False)
        # the engine replays decode as a captured graph (no host work between kernels): capture
        # one pass over the 64 rotated routings and replay it
        if graph:
            side = torch.cuda.Stream()
            side.wait_stream(stream)
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(cg, stream=side):
                    for i in range(sets):
                        op.moe_b(0, xs[i], lgs[i], o, stream=side)
            stream.wait_stream(side)
            reps = 4
            cg.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                cg.replay()
            e1.record()
            torch.cuda.synchronize()
            op.synchronize(stream)
            us = e0.elapsed_time(e1) * 1e3 / (reps * sets)
        else:
            us = stages["total"] * 1e3
        nbytes = (float(np.mean(uniq)) + 1) * BYTES_PER_EXPERT
        gbs = nbytes / (us * 1e-6) / 1e9
        out["T%d" % T] = {"us_per_call": us, "us_per_token": us / T, "unique_experts": float(np.mean(uniq)),
                          "algorithmic_bytes": nbytes, "hbm_gbs": gbs, "frac_of_hbm_peak": gbs / peak_hbm,
                          "timing": "CUDA graph replay of 64 rotated routings" if graph else "eager launches, stage timer",
                          "stage_us_eager": {k: round(v * 1e3, 2) for k, v in stages.items() if k != "calls"},
                          "parity": par}
    return out


if __name__ == "__main__":
    main()
