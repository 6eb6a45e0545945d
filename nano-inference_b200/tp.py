"""Tensor-parallel decode, one process per GPU: the host side of the exchange.

Each rank owns a contiguous range of the 32-row groups of the gate/up, down and lm_head
matrices (nine tenths of the bytes; QKV and O are computed in full by every rank, so
attention needs no exchange).  Two ways to run it:

  * decode_persistent(): one cooperative launch per GPU for the whole generation.  What a
    sharded phase produces leaves the kernel as tagged 8-byte words, stored into the local
    exchange block and, over NVLink, into every other GPU's (peer pointers from CUDA IPC
    handles, enable_peer_exchange()); consumers poll the words they need.  No collective,
    no barrier, no host in the loop.
  * step() / decode(): the phases through mi_decode_launch (asynchronous) with an exchange
    after each sharded phase - an NCCL all-reduce of the vector the phase wrote (entries a
    rank does not own are zero before the reduction, so the sum reproduces the single-GPU
    words bit for bit: the buffers are reduced as raw bytes, x + 0 never carries), or the
    library's own push kernel (mi_tp_exchange) - optionally captured into one CUDA graph
    per token.

The reference is single-GPU; this module has no counterpart in it.
"""
from __future__ import annotations


def partition(groups, rank, world):
    """Row-group range [begin, end) of `rank`; the same arithmetic as mi_tp_partition."""
    return groups * rank // world, groups * (rank + 1) // world


class TPDecoder:
    """Drives one rank of a tensor-parallel model.  `dist` is torch.distributed with an
    initialised process group (nccl on GPUs); world == 1 needs none."""

    def __init__(self, pkg, model, dist=None, group=None):
        import torch
        self.pkg, self.model, self.dist, self.group = pkg, model, dist, group
        self.world = model.tp_world
        self.L = model.config.n_layer
        self.torch = torch
        if self.world > 1:
            self.r_act = model.tp_region(pkg.TP_ACT)
            self.r_down = [model.tp_region(pkg.TP_PART_DOWN, l) for l in range(self.L)]
            self.r_best = model.tp_region(pkg.TP_BEST)
            self.gathered = torch.zeros(8 * self.world, dtype=torch.uint8, device="cuda")

        self.graph = None
        self.peer = False

    def enable_peer_exchange(self):
        """Exchange through peer memory (the library's own kernel over NVLink) instead of NCCL all-reduces: gathers every
        rank's CUDA IPC handles once (the only collective used), then every exchange is one small kernel."""
        import numpy as np
        torch, m = self.torch, self.model
        mine = torch.from_numpy(m.tp_ipc_handles()).cuda()
        allh = torch.zeros(192 * self.world, dtype=torch.uint8, device="cuda")
        self.dist.all_gather_into_tensor(allh, mine, group=self.group)
        m.tp_ipc_open(np.ascontiguousarray(allh.cpu().numpy()))
        self.dist.barrier(group=self.group)          # every rank has mapped every buffer before the first push
        self.peer = True

    def capture(self):
        """Capture one step - the phase launches and the all-reduces between them - into a CUDA graph that reads the
        position from device memory and advances it; decode() replays it per token.  One plain step runs first (it
        lets the library make its lazy allocations and NCCL open its channels); the KV cache entry it writes at the
        model's last position is never read before it is overwritten."""
        torch, m = self.torch, self.model
        m.set_pos(m.config.max_seq - 1)
        self.step(self.pkg.POS_DEVICE)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            m.ctx.use_torch_stream()
            with torch.cuda.graph(g, stream=side):
                self.step(self.pkg.POS_DEVICE)
                m.advance_pos(1)
        torch.cuda.current_stream().wait_stream(side)
        m.ctx.use_torch_stream()
        torch.cuda.synchronize()
        self.graph = g

    def release(self):
        """Drop the captured graph.  It holds NCCL work alive: the process group cannot be destroyed before it is gone
        (destroy_process_group waits forever otherwise)."""
        if self.graph is not None:
            import gc
            self.graph = None
            gc.collect()
            self.torch.cuda.synchronize()

    def _allreduce(self, t):
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)

    def step(self, pos):
        """One decode step at position pos from the model's current token; leaves the next token current."""
        m, L = self.model, self.L
        if self.world == 1:
            m.launch_fused(pos, 0, 5 * L + 1)
            return
        if self.peer:
            for l in range(L):
                m.launch_fused(pos, 5 * l, 5 * l + 4); m.tp_exchange(self.pkg.TP_ACT)
                m.launch(pos, 5 * l + 4, 5 * l + 5); m.tp_exchange(self.pkg.TP_PART_DOWN, l)
            m.launch(pos, 5 * L, 5 * L + 1)
            m.tp_exchange(self.pkg.TP_BEST)              # also picks the overall greedy token
            return
        for l in range(L):
            # QKV, attention and the O projection are computed in full by every rank; the two large projections
            # are sharded: one all-reduce after gate/up (the quantized activations), one after down (its partial sums)
            m.launch_fused(pos, 5 * l, 5 * l + 4); self._allreduce(self.r_act)       # one cooperative launch for the four phases
            m.launch(pos, 5 * l + 4, 5 * l + 5); self._allreduce(self.r_down[l])
        m.launch(pos, 5 * L, 5 * L + 1)
        self.dist.all_gather_into_tensor(self.gathered, self.r_best, group=self.group)
        m.tp_pick(self.gathered, self.world)

    def decode_persistent(self, in_tokens, n_steps, pos0=0):
        """All steps in ONE cooperative launch per GPU, the exchanges done inside the kernel over peer memory
        (enable_peer_exchange first; every rank makes the same call).  Returns (greedy tokens, device milliseconds)."""
        assert self.world == 1 or self.peer, "enable_peer_exchange() first"
        return self.model.decode(in_tokens, n_steps, pos0, None, self.pkg.DECODE_PERSISTENT)

    def decode(self, in_tokens, n_steps, pos0=0):
        """Like Model.decode: forced tokens first, then greedy; returns the greedy token after every step."""
        out = []
        if pos0 < 0 or pos0 + n_steps > self.model.config.max_seq:
            raise ValueError(f"positions {pos0}..{pos0 + n_steps - 1} exceed the KV cache of {self.model.config.max_seq}")
        if self.graph is not None:
            self.model.set_pos(pos0)
        for s in range(n_steps):
            if s < len(in_tokens):
                self.model.set_token(in_tokens[s])
            if self.graph is not None:
                self.graph.replay()
            else:
                self.step(pos0 + s)
            out.append(self.model.get_token()[0])
        return out
