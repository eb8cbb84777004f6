"""Multi-GPU check of the data-parallel MLP step.  Not collected by pytest (it needs one process
per GPU); run it as

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 tests/dp_check.py [--dim 1024 --batch 2048 --layers 3 --steps 3]

Every rank trains the same seeded model on its shard of a seeded global batch with these drivers
("multimem-exclusive" is "multimem" with the exchange kernel on SMs of its own):
copy-engine transfers around a local sum-and-update kernel ("copy"), the NVLink exchange kernel through
the multicast address ("multimem"), the same kernel with peer loads and stores ("peer"), and the NCCL
all-reduce driver ("nccl").  Checked on every rank:
  * no barrier gave up, no library error;
  * within one driver all ranks end with bit-identical 16-bit weights (checksums are all-gathered);
  * multimem and peer agree with nccl on the CHANGE of the f32 master weights (this rank's shard
    of every layer) within 2 % of its largest entry (the three sum the ranks' 16-bit gradients in
    different orders and precisions; the 16-bit weights themselves move by at most a rounding step
    in a few steps, so they cannot show the difference);
  * the loss is the same to 1e-3 and decreases.
Rank 0 prints one JSON line with the verdict.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from maidenx_b200 import _lib  # noqa: E402
from maidenx_b200.mlp import make_mlp  # noqa: E402


def weights_of(m, lib, dim):
    out = []
    for l in range(m.layers):
        host = np.empty(dim * dim, dtype=np.uint16)
        assert lib.cuda_memcpy_d2h(host.ctypes.data, m.ptr("weight", l), host.nbytes) == 0
        out.append(host)
    return out


def master_shard_of(m, lib, dim, rank, world):
    """This rank's slice of every layer's f32 master weights (the DP engine holds only that slice)."""
    n = dim * dim // world
    out = []
    for l in range(m.layers):
        host = np.empty(n, dtype=np.float32)
        base = m.ptr("master_weight", l) + (0 if hasattr(m, "status") else rank * n * 4)
        assert lib.cuda_memcpy_d2h(host.ctypes.data, base, host.nbytes) == 0
        out.append(host)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dim", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=2048, help="global batch")
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--lr", type=float, default=0.05)
    args = ap.parse_args()
    rank, world, local_rank = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = _lib.load()
    local = args.batch // world
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    x_all = torch.randn(args.batch, args.dim, device="cuda", generator=g).bfloat16()
    g.manual_seed(5)
    y_all = torch.randn(args.batch, args.dim, device="cuda", generator=g).bfloat16()
    x = x_all[rank * local:(rank + 1) * local].contiguous()
    y = y_all[rank * local:(rank + 1) * local].contiguous()

    results, problems = {}, []
    for mode in ("multimem-exclusive", "copy", "multimem", "peer", "nccl"):
        m = make_mlp(args.layers, args.dim, local, "bf16", 6, torch, dist, world, exchange=mode)
        if m.exchange != mode:
            problems.append(f"{mode}: driver fell back to {m.exchange}")
        w0 = master_shard_of(m, lib, args.dim, rank, world)
        losses = []
        for _ in range(args.steps):
            m.train_step(x.data_ptr(), y.data_ptr(), args.lr, torch, dist, world)
            torch.cuda.synchronize()
            lt = torch.tensor([m.loss()], device="cuda")
            dist.all_reduce(lt)  # mean over ranks of the per-shard mean = loss of the global batch
            losses.append(float(lt.item()) / world)
        if hasattr(m, "status") and m.status() != 0:
            problems.append(f"{mode}: barrier gave up waiting for rank {m.status() - 1}")
        torch.cuda.synchronize()
        if lib.mx_last_error() != 0:
            problems.append(f"{mode}: library error {lib.mx_last_error()}")
        w = weights_of(m, lib, args.dim)
        sums = torch.tensor([int(a.astype(np.uint64).sum()) ^ int(np.bitwise_xor.reduce(a.astype(np.uint64) * np.arange(1, a.size + 1, dtype=np.uint64))) & 0x7FFFFFFFFFFF for a in w],
                            device="cuda", dtype=torch.int64)
        allsums = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(allsums, sums)
        if any(not torch.equal(allsums[0], s) for s in allsums):
            problems.append(f"{mode}: ranks hold different weights")
        w1 = master_shard_of(m, lib, args.dim, rank, world)
        results[mode] = {"delta": [a - b for a, b in zip(w1, w0)], "losses": losses}
        m.close()
        dist.barrier()
    for mode in ("multimem-exclusive", "copy", "multimem", "peer"):
        for l, (d, dn) in enumerate(zip(results[mode]["delta"], results["nccl"]["delta"])):
            scale = float(np.abs(dn).max())
            err = float(np.abs(d - dn).max())
            if not err <= 2e-2 * scale + 1e-12:
                problems.append(f"{mode}: layer {l} weight change differs from nccl by {err:.3e} (largest change {scale:.3e})")
        for a, b in zip(results[mode]["losses"], results["nccl"]["losses"]):
            if abs(a - b) > 1e-3 * abs(b):
                problems.append(f"{mode}: loss {a} vs nccl {b}")
    for mode, r in results.items():
        if not r["losses"][-1] < r["losses"][0]:
            problems.append(f"{mode}: loss did not decrease {r['losses']}")
    flag = torch.tensor([len(problems)], device="cuda")
    dist.all_reduce(flag)
    if rank == 0:
        print(json.dumps({"world": world, "dim": args.dim, "global_batch": args.batch, "steps": args.steps, "ok": int(flag.item()) == 0,
                          "losses": {k: [round(v, 6) for v in r["losses"]] for k, r in results.items()}, "problems_rank0": problems}))
    if problems:
        print(f"[rank {rank}] " + "; ".join(problems), file=sys.stderr)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
