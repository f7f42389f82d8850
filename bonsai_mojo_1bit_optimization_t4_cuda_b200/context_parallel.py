"""Context parallelism for ONE long sequence: the compressed region is split by context range
over the ranks of a ``torch.distributed`` group; every rank computes an unnormalised
``(24, 258)`` partial of its slice, the partials cross NVLink in one all-gather (24.8 KB per
rank), and every rank (or only the owner of the raw ring) finishes with one LSE merge + gate.

The reference has nothing distributed; what maps onto its kernel is that
``launch_khq_attn_fp16`` takes the absolute position of its first token (``start_pos``), so a
slice ``[lo, hi)`` of the compressed region is the call ``start_pos=lo, c_len=hi-lo`` on arrays
that hold only that slice's rows.

The one exchange step is ``all_gather`` (NCCL on GPUs, gloo in the CPU tests): an all-reduce
formulation would need two rounds (max, then rescaled sums) and is not better at this size.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

CHUNK = 128
H_Q, H_KV, D, PART = 24, 4, 256, 258


def partition_context(c_len: int, world: int, chunk: int = CHUNK) -> List[Tuple[int, int]]:
    """Contiguous token ranges, one per rank, cut on `chunk`-token boundaries (the compress
    granularity) and balanced to within one chunk.  Ranks past the data get empty ranges."""
    n_chunks = (c_len + chunk - 1) // chunk
    base, extra = divmod(n_chunks, world)
    out, lo = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        hi = min(c_len, lo + n * chunk)
        out.append((lo, hi))
        lo = hi
    return out


class ContextParallelDecode:
    """One rank's share of a context-parallel decode step.

    ``kv``: this rank's slice of the eight payload arrays (rows of tokens ``[lo, hi)`` only),
    ``tables``: the layer's fp16 tables, ``ring_k / ring_v``: the raw ring (only read on
    ``owner``).  ``ops`` is the launch backend (the package's ``CudaOps``).
    """

    def __init__(self, ops, group, kv: dict, tables: dict, lo: int, hi: int, alpha_k: float, alpha_v: float,
                 ring_k=None, ring_v=None, owner: int = 0, splits: int = 32, device="cuda"):
        self.ops, self.group = ops, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.kv, self.tables = kv, tables
        self.lo, self.hi = lo, hi
        self.alpha_k, self.alpha_v = alpha_k, alpha_v
        self.ring_k, self.ring_v, self.owner = ring_k, ring_v, owner
        self.splits = splits
        dev = torch.device(device)
        # slot-major partials: [rank][0 = compressed slice, 1 = raw window]
        self.mine = torch.zeros(2, H_Q, PART, dtype=torch.float32, device=dev)
        self.all = torch.zeros(self.world, 2, H_Q, PART, dtype=torch.float32, device=dev)
        self.scratch = torch.zeros(H_Q * max(splits, 1) * PART, dtype=torch.float32, device=dev)
        self.out = torch.zeros(H_Q * D, dtype=torch.float16, device=dev)
        self._neutral = torch.zeros(H_Q, PART, dtype=torch.float32, device=dev)
        self._neutral[:, D] = -1e20

    def split_count(self, n_tok: int) -> int:
        return int(min(max(n_tok // 8, 1), self.splits))

    def step(self, q_gate: torch.Tensor, win_start: int, win_len: int, scale: float = 1.0 / 16.0,
             rope_base: float = 1e7, broadcast_q: bool = True) -> torch.Tensor:
        """q_gate: (24*512,) fp16, valid on ``owner`` (broadcast to the others unless the caller
        already did).  Returns the gated output (24*256,) fp16, identical on every rank."""
        ops, kv, tb = self.ops, self.kv, self.tables
        if broadcast_q and self.world > 1:
            dist.broadcast(q_gate, src=dist.get_global_rank(self.group, self.owner), group=self.group)
        n = self.hi - self.lo
        if n > 0:
            ops.attn(q_gate, kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
                     kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], tb["cents_k"], tb["cents_v"], tb["vq"],
                     tb["rotor_k"], tb["rotor_v"], tb["d_k"], tb["d_v"], self.mine[0], self.scratch, H_Q, H_Q, 1, n,
                     n, H_Q // H_KV, scale, self.alpha_k, self.alpha_v, rope_base, self.lo, self.split_count(n))
        else:
            self.mine[0].copy_(self._neutral)
        if self.rank == self.owner and win_len > 0:
            ops.window_attn(q_gate, self.ring_k, self.ring_v, self.mine[1], win_start, win_len, 256, H_Q, H_KV, D,
                            scale)
        else:
            self.mine[1].copy_(self._neutral)
        if self.world > 1:
            dist.all_gather_into_tensor(self.all.view(-1), self.mine.view(-1), group=self.group)
        else:
            self.all.copy_(self.mine.unsqueeze(0))
        ops.merge_slots_gate(self.all, 2 * self.world, q_gate, self.out, H_Q, D)
        return self.out
