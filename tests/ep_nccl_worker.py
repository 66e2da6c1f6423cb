"""Worker of tests/test_ep_nccl_gpu.py: one rank of the library-side expert-parallel host
(b200moe_ep_init / b200moe_ep_forward, NCCL inside the library, no torch.distributed).
Usage: python ep_nccl_worker.py <rank> <world> <dir> <shared 0|1>"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank, world, work, shared = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4] == "1"
    import torch
    import gfx1151_engine_b200 as pkg
    from gfx1151_engine_b200 import synth
    from helpers import bf16_tensor, dev_bytes, output_errors
    torch.cuda.set_device(rank)
    id_path = os.path.join(work, "nccl_id.bin")
    if rank == 0:
        uid = pkg.ep_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(id_path):
            if time.time() > deadline:
                raise SystemExit("rank %d: no NCCL id from rank 0" % rank)
            time.sleep(0.05)
        uid = open(id_path, "rb").read()
    spec = synth.LayerSpec(experts=16, topk=4, d=512, mid=128, shared=shared)
    layer = synth.make_layer(spec, seed=130)
    T = 300
    placement = synth.rng_for(130, 50).permutation(spec.experts).astype(np.int32)

    def load(op):
        op.load_q4cp(0, dev_bytes(torch, layer["gate_up"]), dev_bytes(torch, layer["down"]))
        if shared:
            op.load_shared_q4cp(0, dev_bytes(torch, layer["sh_gate"]), dev_bytes(torch, layer["sh_up"]),
                                dev_bytes(torch, layer["sh_down"]), dev_bytes(torch, layer["sh_gate_w"]))

    op = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=shared, device=rank, ep_rank=rank, ep_size=world)
    op.ep_set_placement(placement)
    load(op)
    op.ep_init(uid, cap_factor=float(world))
    xb = synth.make_x(synth.rng_for(130, 10 + rank), T, spec.d)
    lg = synth.make_logits(synth.rng_for(130, 20 + rank), T, spec.experts, zipf=True, zipf_rng=synth.rng_for(130, 77))
    x = bf16_tensor(torch, xb, (T, spec.d))
    logits = torch.from_numpy(np.ascontiguousarray(lg, np.float32)).cuda()
    out = torch.full((T, spec.d), float("nan"), dtype=torch.bfloat16, device="cuda")
    res = {}
    for it in range(2):                       # the second call reuses every buffer
        out.fill_(float("nan"))
        op.ep_forward(0, x, logits, out)
        op.synchronize()
    single = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=shared, device=rank)
    load(single)
    want = torch.empty_like(out)
    single.moe_b(0, x, logits, want)
    single.synchronize()
    max_abs, mean_rel = output_errors(out.float().cpu().numpy(), want.float().cpu().numpy())
    res.update(max_abs=max_abs, mean_rel=mean_rel, finite=bool(torch.isfinite(out.float()).all().item()))
    # a receive buffer that is too small stops every rank with the same status, before anything moves
    small = pkg.MoeOperator(spec.experts, spec.topk, spec.d, spec.mid, T, has_shared=shared, device=rank, ep_rank=rank, ep_size=world)
    small.ep_set_placement(placement)
    load(small)
    uid2_path = os.path.join(work, "nccl_id2.bin")
    if rank == 0:
        with open(uid2_path + ".tmp", "wb") as f:
            f.write(pkg.ep_unique_id())
        os.replace(uid2_path + ".tmp", uid2_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(uid2_path):
            if time.time() > deadline:
                raise SystemExit("rank %d: no second NCCL id" % rank)
            time.sleep(0.05)
    small.ep_init(open(uid2_path, "rb").read(), cap_factor=1.0)   # the skewed routing needs more than 1.0 on some rank
    try:
        small.ep_forward(0, x, logits, out)
        small.synchronize()
        res["overflow_status"] = 0
    except pkg.B200MoeError as e:
        res["overflow_status"] = e.status
    small.ep_shutdown()
    op.ep_shutdown()
    with open(os.path.join(work, "rank%d.json" % rank), "w") as f:
        json.dump(res, f)


if __name__ == "__main__":
    main()
