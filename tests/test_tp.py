"""Tensor parallelism: the host-side exchange logic on CPU ranks (gloo, world size 2),
the asynchronous launch path on one GPU, and - where the box has two or more GPUs -
bit-for-bit parity of the sharded decode against the unsharded one."""
import ctypes as C
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import gguf_util as gu

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def test_partition_covers_every_group_once(pkg):
    lib = pkg.load_library()
    import __graft_entry__ as ge
    tp = ge.load_submodule("tp")
    for groups in (1, 7, 36, 48, 64, 280, 4748):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                b, e = C.c_int(), C.c_int()
                lib.mi_tp_partition(groups, r, world, C.byref(b), C.byref(e))
                assert (b.value, e.value) == tp.partition(groups, r, world)
                seen += list(range(b.value, e.value))
            assert seen == list(range(groups))


_GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import __graft_entry__ as ge
tp = ge.load_submodule("tp")
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
rng = np.random.default_rng(5)
ok = True
# each buffer type the decode exchanges: fp32 vector, fp64 partial sums, [int8 | fp16] activations
for groups, per_group, dtype in ((64, 32, np.float32), (48, 96, np.float64), (280, 32, np.int8), (35, 8, np.float16)):
    full = (rng.standard_normal(groups * per_group) * 50).astype(dtype)
    b, e = tp.partition(groups, rank, world)
    mine = np.zeros_like(full)
    mine[b * per_group:e * per_group] = full[b * per_group:e * per_group]      # a rank writes only the rows it owns
    t = torch.from_numpy(mine.view(np.uint8).copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)                                   # reduced as raw bytes
    ok = ok and np.array_equal(t.numpy().view(dtype), full)
# greedy pick across ranks: largest value, lowest id on ties
vals = [(3.5, 900), (3.5, 17)]
mine = torch.tensor(np.array([vals[rank][0]], np.float32).view(np.uint8).tolist() + np.array([vals[rank][1]], np.int32).view(np.uint8).tolist(), dtype=torch.uint8)
gathered = [torch.zeros(8, dtype=torch.uint8) for _ in range(world)]
dist.all_gather(gathered, mine)
cands = [(float(g.numpy()[:4].view(np.float32)[0]), int(g.numpy()[4:].view(np.int32)[0])) for g in gathered]
best = max(cands, key=lambda c: (c[0], -c[1]))
ok = ok and best == (3.5, 17)
print("GLOO_TP", "OK" if ok else "FAIL", flush=True)
dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


def test_zero_padded_byte_allreduce_reproduces_the_full_buffers_gloo_world2(tmp_path):
    script = tmp_path / "gloo_worker.py"
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("GLOO_TP OK" in o for o in outs), outs


@pytest.mark.gpu
def test_async_launch_path_equals_blocking_decode_on_one_gpu(ctx, pkg, tmp_path):
    import __graft_entry__ as ge
    tp = ge.load_submodule("tp")
    p = gu.make_synthetic(tmp_path / "m.gguf", "tiny", seed=11, std=0.3, extra=["--bias-std", 0.3])
    toks = [5, 400, 33, 7]
    a = pkg.Model(ctx, p, 32)
    want, _ = a.decode(toks, 12, 0, None, pkg.DECODE_PERSISTENT)
    b = pkg.Model(ctx, p, 32)
    got = tp.TPDecoder(pkg, b).decode(toks, 12)
    assert got == want
    assert np.array_equal(a.state("h_mid", np.float32, 128), b.state("h_mid", np.float32, 128))


@pytest.mark.gpu
def test_sharded_decode_is_bit_identical_to_unsharded_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    p = gu.make_synthetic(tmp_path / "m.gguf", "tiny", seed=11, std=0.3, extra=["--bias-std", 0.3])
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "tp_worker.py"), str(p), "16"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "TP_PARITY OK" in r.stdout, r.stdout + r.stderr
