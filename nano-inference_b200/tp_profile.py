"""Where a tensor-parallel decode step spends its time, read on the GPUs themselves.

    MINFER_PROFILE=1 python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        nano-inference_b200/tp_profile.py model.gguf [tokens] [cta]

Every rank loads its shard of the model, maps the peers' exchange blocks and runs the persistent kernel with the exchange
inside (one cooperative launch per GPU); with MINFER_PROFILE set the library launches the instrumented build, and rank 0
prints the per-token microseconds of one CTA (default: the first GEMV CTA) next to the device time of the run, taken as
the maximum over the ranks.  A profiler that replays kernels cannot be used here: the kernels of the ranks wait for one
another's data.  Works with N = 1 as well.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import __graft_entry__ as ge    # noqa: E402

SLOTS = {12: "waiting for other CTAs' / GPUs' words", 27: "norm: before the poll", 28: "norm: residual add", 23: "norm: sum of squares",
         24: "norm: barrier", 25: "norm: quantize", 26: "norm: barrier 2", 18: "tiles: loop and unit bookkeeping", 20: "tiles: ring wait",
         21: "tiles: arithmetic", 22: "tiles: issuing the next copy", 19: "fold + epilogues", 11: "lm_head rows + pick",
         0: "QKV stage", 1: "QKV tail", 3: "attention (this CTA)", 4: "O stage", 5: "O tail", 6: "gate/up stage", 7: "gate/up tail", 13: "step prologue"}


def main():
    path = sys.argv[1]
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 64
    if len(sys.argv) > 3:
        os.environ["MINFER_PROFILE_CTA"] = sys.argv[3]
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl")
    pkg, tpmod = ge.load_package(), ge.load_submodule("tp")
    ctx = pkg.Context(local)
    ctx.use_torch_stream()
    m = pkg.Model(ctx, path, 4096, tp_rank=rank, tp_world=world)
    dec = tpmod.TPDecoder(pkg, m, dist if world > 1 else None)
    if world > 1:
        dec.enable_peer_exchange()
    ids = [int(t) for t in np.random.default_rng(1).integers(0, m.config.n_vocab, 64)]
    out, _ = dec.decode_persistent(ids, 64, 0)
    warm, _ = dec.decode_persistent([out[-1]], 5, 64)
    profiled = bool(os.environ.get("MINFER_PROFILE"))
    before = m.state("profile", np.uint64, 32).copy() if profiled else None
    gen, ms = dec.decode_persistent([warm[-1]], n, 69)
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"{world} GPU(s), {n} tokens at positions 69..{68 + n}: {t.item() / n * 1e3:.1f} us/token (device time, max over ranks)", flush=True)
        if profiled:
            pr = (m.state("profile", np.uint64, 32) - before) / n / 1e3
            for k, name in SLOTS.items():
                print(f"  {name:40s} {pr[k]:8.1f} us/token")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
