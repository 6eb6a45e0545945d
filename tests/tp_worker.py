"""One rank of the tensor-parallel parity check (launched by tests/test_tp.py through
torch.distributed.run, one process per GPU).  Every rank decodes the same prompt with
the sharded model; rank 0 also decodes it with the unsharded model on its own GPU and
the token streams and the final-step state must be identical, bit for bit."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))

import numpy as np
import torch
import torch.distributed as dist

import __graft_entry__ as ge


def main():
    path, n_steps = sys.argv[1], int(sys.argv[2])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = ge.load_package()
    tpmod = ge.load_submodule("tp")
    ctx = pkg.Context(local)
    ctx.use_torch_stream()
    m = pkg.Model(ctx, path, n_steps + 2, tp_rank=rank, tp_world=world)
    dec = tpmod.TPDecoder(pkg, m, dist)
    V = m.config.n_vocab
    prompt = [int(t) for t in np.random.default_rng(3).integers(0, V, 6)]
    got = dec.decode(prompt, n_steps)
    dec.capture()                                # the same steps replayed as one CUDA graph per token
    got_graph = dec.decode(prompt, n_steps)
    dec.release()
    dec.enable_peer_exchange()                   # the library's own exchange kernel over peer memory instead of NCCL
    got_peer = dec.decode(prompt, n_steps)
    dec.capture()
    got_peer_graph = dec.decode(prompt, n_steps)
    dec.release()                                # before the process group goes away
    got_fused, _ = dec.decode_persistent(prompt, n_steps)   # one launch per GPU, the exchange inside the kernel
    h_tp = m.state("h_mid", np.float32, m.config.n_embd)
    ok = True
    if rank == 0:
        ref = pkg.Model(ctx, path, n_steps + 2)
        want, _ = ref.decode(prompt, n_steps, 0, None, pkg.DECODE_PER_PHASE)
        h_ref = ref.state("h_mid", np.float32, ref.config.n_embd)
        ok = got == want and got_graph == want and got_peer == want and got_peer_graph == want and got_fused == want and np.array_equal(h_tp, h_ref)
        print("TP_PARITY", "OK" if ok else f"MISMATCH got={got} want={want}", f"world={world} steps={n_steps}", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
