"""Context parallelism for ONE long sequence: the compressed region is split by context range
over the ranks of a ``torch.distributed`` group; every rank computes an unnormalised
``(24, 258)`` partial of its slice, the partials cross NVLink in one all-gather (24.8 KB per
rank), and every rank (or only the owner of the raw ring) finishes with one LSE merge + gate.

The reference has nothing distributed; what maps onto its kernel is that
``launch_khq_attn_fp16`` takes the absolute position of its first token (``start_pos``), so a
slice ``[lo, hi)`` of the compressed region is the call ``start_pos=lo, c_len=hi-lo`` on arrays
that hold only that slice's rows.

The one exchange step is either ``all_gather`` (NCCL on GPUs, gloo in the CPU tests; an all-reduce
formulation would need two rounds -- max, then rescaled sums -- and is not better at this size) or,
on GPUs, direct stores into the peers' slot buffers with a flag per producer, the merge kernel
waiting for the flags itself (``PeerExchange``): no collective launch on the step's critical path.
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


def partition_context_cyclic(c_len: int, world: int, chunk: int = CHUNK) -> List[List[int]]:
    """Chunk-cyclic partition: chunk c (tokens [c * chunk, (c + 1) * chunk)) goes to rank c mod world,
    so the chunks a growing context appends keep the ranks balanced to within one chunk.  Returns, per
    rank, its chunk indices in ascending order.  A rank's local arrays hold its chunks back to back;
    local token s then sits at absolute position rank * chunk + (s // chunk) * world * chunk + s % chunk,
    which is what ``launch_khq_attn_strided_fp16`` takes.  Only the last chunk of the context may be
    partial, and it is then the last local chunk of its rank."""
    n_chunks = (c_len + chunk - 1) // chunk
    return [list(range(r, n_chunks, world)) for r in range(world)]


def cyclic_local_tokens(c_len: int, world: int, rank: int, chunk: int = CHUNK) -> int:
    """How many of the c_len tokens a rank holds under the chunk-cyclic partition."""
    return sum(min(chunk, c_len - c * chunk) for c in partition_context_cyclic(c_len, world, chunk)[rank])


class PeerExchange:
    """Slot buffers and flags of a context-parallel group, mapped into every process with CUDA IPC
    (the library's ``khq_b200_peer_*`` helpers: plain ``cudaMalloc`` memory, opened by each peer on
    its own device, which also enables peer access; no multicast object is involved).

    Every rank owns one allocation: ``slots`` (2 parities x ``world * per_rank`` records of (24, 258)
    floats), ``flags`` (one 32-bit epoch word per producer) and a small check area.  ``publish``
    stores this rank's records into every peer's buffer and raises its flag there; ``merge`` waits
    (bounded) for all producers of the step and finishes with the LSE merge + gate.  Before any
    kernel touches a mapping the constructor proves it with blocking 4-byte runtime copies."""

    def __init__(self, ops, group, per_rank: int = 2, device="cuda"):
        import ctypes

        self.ops, self.group = ops, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.per_rank = per_rank
        dev = torch.device(device)
        lib = ops.lib
        self.n_slots = self.world * per_rank
        rec_bytes = H_Q * PART * 4
        self.flags_off = 2 * self.n_slots * rec_bytes              # multiple of 256 bytes (24768 = 96.75 * 256: rounded below)
        self.flags_off = (self.flags_off + 255) // 256 * 256
        # flags: word r = producer r's partials; word `world` = the owner's q_gate
        self.check_off = self.flags_off + 256 * ((4 * (self.world + 1) + 255) // 256)
        self.q_off = self.check_off + 256 * ((4 * self.world + 255) // 256)
        self.q_bytes = H_Q * 2 * D * 2                               # (24, 512) fp16, one per parity
        total = self.q_off + 2 * self.q_bytes
        with torch.cuda.device(dev):
            base = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            rc = lib.khq_b200_peer_alloc(total, ctypes.byref(base), handle)
            if rc != 0:
                raise RuntimeError(f"khq_b200_peer_alloc failed ({rc})")
            self.base = int(base.value)
            everyone = [None] * self.world
            dist.all_gather_object(everyone, bytes(handle.raw), group=group)
            self.peer_base = []
            for r, h in enumerate(everyone):
                if r == self.rank:
                    self.peer_base.append(self.base)
                    continue
                p = ctypes.c_void_p()
                rc = lib.khq_b200_peer_open(h, ctypes.byref(p))
                if rc != 0:
                    raise RuntimeError(f"khq_b200_peer_open of rank {r}'s buffer failed ({rc})")
                self.peer_base.append(int(p.value))
            # prove every mapping with runtime copies: write rank+1 into check[rank] of every peer ...
            for r in range(self.world):
                rc = lib.khq_b200_peer_poke(self.peer_base[r] + self.check_off + 4 * self.rank, self.rank + 1)
                if rc != 0:
                    raise RuntimeError(f"write through the mapping of rank {r}'s buffer failed ({rc})")
            dist.barrier(group=group)
            # ... and read back what the peers wrote here
            for r in range(self.world):
                v = ctypes.c_uint(0)
                rc = lib.khq_b200_peer_peek(self.base + self.check_off + 4 * r, ctypes.byref(v))
                if rc != 0 or v.value != r + 1:
                    raise RuntimeError(f"rank {r}'s write did not arrive here (code {rc}, value {v.value})")
        self.peer_bufs = torch.tensor(self.peer_base, dtype=torch.int64, device=dev)
        self.peer_slots = self.peer_bufs
        self.peer_flags = torch.tensor([b + self.flags_off for b in self.peer_base], dtype=torch.int64, device=dev)
        self.rec_bytes = rec_bytes
        self.epoch = 0
        dist.barrier(group=group)

    def begin_step(self) -> int:
        """Advance to the next epoch (once per step on every rank); returns the parity in use."""
        self.epoch += 1
        return self.epoch & 1

    def publish_q(self, q_gate: torch.Tensor) -> None:
        """On the owner of the query: store q_gate (24*512 fp16) into every rank's buffer."""
        par = self.epoch & 1
        self.ops.publish_bytes(q_gate, self.q_bytes, self.peer_bufs, self.q_off + par * self.q_bytes, self.peer_flags,
                               self.world, self.world, self.epoch)

    def wait_q(self, max_polls: int = 0) -> int:
        """Queue a wait for this step's q_gate on the stream; returns its device address here."""
        par = self.epoch & 1
        self.ops.wait_flag(self.base + self.flags_off + 4 * self.world, self.epoch, max_polls)
        return self.base + self.q_off + par * self.q_bytes

    def publish(self, records: torch.Tensor) -> None:
        """records: (per_rank, 24, 258) fp32 of this rank for the current step."""
        par = self.epoch & 1
        self.ops.publish_partials(records, self.per_rank, self.peer_slots, self.peer_flags, self.world, self.rank,
                                  self.rank * self.per_rank, par * self.n_slots, self.epoch)

    def merge(self, q_gate: torch.Tensor, out: torch.Tensor, max_polls: int = 0) -> None:
        par = self.epoch & 1
        self.ops.merge_slots_wait_gate(self.base + par * self.n_slots * self.rec_bytes, self.base + self.flags_off, self.world,
                                       self.epoch, self.n_slots, q_gate, out, H_Q, D, max_polls)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (after a barrier: nobody may still write)."""
        if getattr(self, "base", 0):
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            for r, p in enumerate(self.peer_base):
                if r != self.rank:
                    self.ops.lib.khq_b200_peer_close(p)
            dist.barrier(group=self.group)
            self.ops.lib.khq_b200_peer_free(self.base)
            self.base = 0


class PersistentSlice:
    """One rank's compressed slice (and, on the owner, the raw window) as ONE problem of the
    library's persistent batched decode kernel, ending in one unnormalised ``(24, 258)`` record
    (``launch_khq_decode_batched_partial_fp16``).  Against the split launches of the drop-in entry
    this fills every SM whatever the slice length (the host planner cuts one to three pieces per SM,
    raw-window pieces included), pays the per-CTA table set-up once and needs no second launch for
    the window.  CUDA only; the descriptor and the work items are re-sent only when the slice length
    or the window length changed."""

    def __init__(self, lib, kv: dict, tables: dict, alpha_k: float, alpha_v: float, ring_k, ring_v, start_pos: int,
                 pos_chunk: int = 0, pos_stride_chunks: int = 0, device="cuda", generation: int = -1):
        from .batched import SEQ_DESC, TABLES_DESC, WORK_ITEM
        from .lib import check, current_stream

        self.lib, self._check, self._stream = lib, check, current_stream
        self.generation = generation
        dev = torch.device(device)
        self._keep = (kv, tables, ring_k, ring_v)  # the descriptors hold raw addresses
        self.q = torch.zeros(H_Q * 2 * D, dtype=torch.float16, device=dev)
        t = np.zeros(1, TABLES_DESC)
        for name, key in (("cents_k", "cents_k"), ("cents_v", "cents_v"), ("vq", "vq"), ("k_rotor", "rotor_k"),
                          ("v_rotor", "rotor_v"), ("d_k", "d_k"), ("d_v", "d_v")):
            t[0][name] = tables[key].data_ptr()
        t[0]["alpha_k"], t[0]["alpha_v"] = alpha_k, alpha_v
        self.d_tables = torch.from_numpy(t.view(np.uint8).copy()).to(dev)
        self.h_desc = torch.zeros(SEQ_DESC.itemsize, dtype=torch.uint8).pin_memory()
        d = self.h_desc.numpy().view(SEQ_DESC)
        for k in ("k_payload", "v_payload", "v_shared_meta", "k_mask", "k_norms", "k_r_norms", "v_norms", "v_r_norms"):
            d[0][k] = kv[k].data_ptr()
        d[0]["q_gate"] = self.q.data_ptr()
        d[0]["ring_k"] = ring_k.data_ptr() if ring_k is not None else 0
        d[0]["ring_v"] = ring_v.data_ptr() if ring_v is not None else 0
        d[0]["start_pos"] = start_pos
        assert 0 <= pos_chunk < 65536 and pos_chunk % 2 == 0 and 0 <= pos_stride_chunks < 65536
        d[0]["pos_pack"] = (pos_chunk << 16) | pos_stride_chunks if pos_chunk else 0
        self.d_desc = torch.zeros(SEQ_DESC.itemsize, dtype=torch.uint8, device=dev)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.max_items = 16 * sms
        self.item_bytes = WORK_ITEM.itemsize
        self.h_items = torch.zeros(self.max_items * self.item_bytes, dtype=torch.uint8).pin_memory()
        self.d_items = torch.zeros(self.max_items * self.item_bytes, dtype=torch.uint8, device=dev)
        self.ws_bytes = int(lib.khq_b200_decode_workspace_bytes(self.max_items))
        self.workspace = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=dev)
        self._planned = None
        self._descs = {}
        self._sent = torch.cuda.Event()
        self.n_items = 0

    def launch(self, q_gate, n_tok: int, win_start: int, win_len: int, out_partial: torch.Tensor,
               scale: float, rope_base: float) -> None:
        """q_gate: (24*512,) fp16 tensor, or the device address of one (the peer exchange hands out the
        address of the query inside its own buffer).  out_partial: (24, 258) fp32.  n_tok + win_len must
        be positive."""
        from .batched import SEQ_DESC

        if isinstance(q_gate, int):
            q_ptr = q_gate
        else:
            self.q.copy_(q_gate.reshape(-1), non_blocking=True)
            q_ptr = self.q.data_ptr()
        if self._planned != (n_tok, win_start, win_len):
            self._sent.synchronize()  # the pinned buffers may still be the source of the last copies
            c = np.array([n_tok], np.int32)
            w = np.array([win_len], np.int32)
            first, cnt = np.zeros(1, np.int32), np.zeros(1, np.int32)
            n = self.lib.khq_b200_plan_decode(c.ctypes.data, w.ctypes.data, 1, 0, self.h_items.data_ptr(), self.max_items,
                                              first.ctypes.data, cnt.ctypes.data)
            if n <= 0 or n > self.max_items:
                raise RuntimeError(f"khq_b200_plan_decode returned {n} items (room for {self.max_items})")
            self.n_items = int(n)
            d = self.h_desc.numpy().view(SEQ_DESC)
            d[0]["c_len"], d[0]["win_start"], d[0]["win_len"] = n_tok, win_start, win_len
            d[0]["first_slot"], d[0]["n_slots"] = int(first[0]), int(cnt[0])
            nb = self.n_items * self.item_bytes
            self.d_items[:nb].copy_(self.h_items[:nb], non_blocking=True)
            self._sent.record(torch.cuda.current_stream())
            self._descs = {}
            self._planned = (n_tok, win_start, win_len)
        d_desc = self._descs.get(q_ptr)
        if d_desc is None:  # one device descriptor per query address (the exchange alternates between two)
            self._sent.synchronize()
            self.h_desc.numpy().view(SEQ_DESC)[0]["q_gate"] = q_ptr
            d_desc = torch.empty_like(self.d_desc)
            d_desc.copy_(self.h_desc, non_blocking=True)
            self._sent.record(torch.cuda.current_stream())
            self._descs[q_ptr] = d_desc
        self._check("launch_khq_decode_batched_partial_fp16", self.lib.launch_khq_decode_batched_partial_fp16(
            d_desc.data_ptr(), self.d_tables.data_ptr(), self.d_items.data_ptr(), 1, self.n_items,
            self.workspace.data_ptr(), self.ws_bytes, self.n_items, float(scale), float(rope_base), 256,
            int(self.generation), out_partial.data_ptr(), self._stream()))


class ContextParallelDecode:
    """One rank's share of a context-parallel decode step.

    ``kv``: this rank's slice of the eight payload arrays (rows of tokens ``[lo, hi)`` only),
    ``tables``: the layer's fp16 tables, ``ring_k / ring_v``: the raw ring (only read on
    ``owner``).  ``ops`` is the launch backend (the package's ``CudaOps``).
    """

    def __init__(self, ops, group, kv: dict, tables: dict, lo: int, hi: int, alpha_k: float, alpha_v: float,
                 ring_k=None, ring_v=None, owner: int = 0, splits: int = 32, device="cuda", exchange: str = "collective",
                 partition: str = "contiguous", engine: str = "splits"):
        """``exchange``: "collective" = one all-gather of the partials (NCCL / gloo), "peer" = every
        rank stores its partials into the peers' buffers over NVLink and the merge kernel waits for
        the flags (``PeerExchange``; CUDA only).  ``partition``: "contiguous" = ``kv`` holds the rows of
        tokens ``[lo, hi)``; "cyclic" = ``kv`` holds this rank's chunks of the chunk-cyclic partition
        back to back (``hi - lo`` local tokens; ``lo`` is ignored).  ``engine``: "splits" = the drop-in entries
        (``launch_khq_attn_fp16`` / ``_strided`` with ``splits`` splits, then the window launch); "persistent" =
        slice and window as one launch of the persistent batched kernel (``PersistentSlice``; CUDA only)."""
        self.ops, self.group = ops, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.kv, self.tables = kv, tables
        self.lo, self.hi = lo, hi
        self.alpha_k, self.alpha_v = alpha_k, alpha_v
        self.ring_k, self.ring_v, self.owner = ring_k, ring_v, owner
        self.splits = splits
        assert partition in ("contiguous", "cyclic")
        self.partition = partition
        dev = torch.device(device)
        # slot-major partials: [rank][0 = compressed slice, 1 = raw window]
        self.mine = torch.zeros(2, H_Q, PART, dtype=torch.float32, device=dev)
        self.all = torch.zeros(self.world, 2, H_Q, PART, dtype=torch.float32, device=dev)
        self.scratch = torch.zeros(H_Q * max(splits, 1) * PART, dtype=torch.float32, device=dev)
        self.out = torch.zeros(H_Q * D, dtype=torch.float16, device=dev)
        self._neutral = torch.zeros(H_Q, PART, dtype=torch.float32, device=dev)
        self._neutral[:, D] = -1e20
        assert exchange in ("collective", "peer")
        self.peer = PeerExchange(ops, group, per_rank=2, device=device) if exchange == "peer" and self.world > 1 else None
        # In peer mode a bounded wait that runs out (a slow or lost peer) only sets the library's
        # device status word; it is read back every `status_every` steps and at close().
        self.status_every = 64
        self._steps = 0
        assert engine in ("splits", "persistent")
        self.persistent = None
        if engine == "persistent":
            self.mine[1].copy_(self._neutral)
            mine_ring = self.rank == self.owner
            cyc = partition == "cyclic"
            self.persistent = PersistentSlice(ops.lib, kv, tables, alpha_k, alpha_v, ring_k if mine_ring else None,
                                              ring_v if mine_ring else None,
                                              start_pos=(self.rank * CHUNK if cyc else lo), pos_chunk=(CHUNK if cyc else 0),
                                              pos_stride_chunks=(self.world if cyc else 0), device=device)

    def check_status(self) -> None:
        """Read and clear the library's device status word (a blocking 4-byte copy) and raise if a
        bounded wait of the peer exchange ran out: the outputs since the last check may then have
        been merged from stale slots."""
        lib = getattr(self.ops, "lib", None)
        if lib is None or self.peer is None:
            return
        st = int(lib.khq_b200_device_status_clear())
        if st == 3:
            raise RuntimeError("context-parallel exchange: a wait for a peer's flag ran out (device status 3); "
                               "outputs since the last check are not trustworthy")
        if st < 0:
            raise RuntimeError(f"context-parallel exchange: reading the device status failed ({st})")

    def close(self) -> None:
        """Final status check, then release the peer mappings (collective call)."""
        try:
            self.check_status()
        finally:
            if self.peer is not None:
                self.peer.close()
                self.peer = None

    def split_count(self, n_tok: int) -> int:
        return int(min(max(n_tok // 8, 1), self.splits))

    def step(self, q_gate: torch.Tensor, win_start: int, win_len: int, scale: float = 1.0 / 16.0,
             rope_base: float = 1e7, broadcast_q: bool = True) -> torch.Tensor:
        """q_gate: (24*512,) fp16, valid on ``owner`` (broadcast to the others unless the caller
        already did).  Returns the gated output (24*256,) fp16, identical on every rank."""
        ops, kv, tb = self.ops, self.kv, self.tables
        if self.peer is not None:
            self.peer.begin_step()
            if broadcast_q:  # the owner's q_gate reaches the others through their buffers, no collective
                if self.rank == self.owner:
                    self.peer.publish_q(q_gate)
                q_gate = self.peer.wait_q()
        elif broadcast_q and self.world > 1:
            dist.broadcast(q_gate, src=dist.get_global_rank(self.group, self.owner), group=self.group)
        n = self.hi - self.lo
        if self.persistent is not None:
            wl = win_len if self.rank == self.owner else 0
            if n + wl > 0:
                self.persistent.launch(q_gate, n, win_start, wl, self.mine[0], scale, rope_base)
            else:
                self.mine[0].copy_(self._neutral)
            return self._exchange_and_merge(q_gate)  # mine[1] stays the neutral record it was initialised to
        if n > 0 and self.partition == "cyclic":
            ops.attn_strided(q_gate, kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
                             kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], tb["cents_k"], tb["cents_v"], tb["vq"],
                             tb["rotor_k"], tb["rotor_v"], tb["d_k"], tb["d_v"], self.mine[0], self.scratch, H_Q, H_Q, 1, n,
                             H_Q // H_KV, scale, self.alpha_k, self.alpha_v, rope_base, self.rank * CHUNK, self.split_count(n),
                             CHUNK, self.world * CHUNK)
        elif n > 0:
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
        return self._exchange_and_merge(q_gate)

    def _exchange_and_merge(self, q_gate: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        if self.peer is not None:
            self.peer.publish(self.mine)
            self.peer.merge(q_gate, self.out)
            self._steps += 1
            if self.status_every > 0 and self._steps % self.status_every == 0:
                self.check_status()
            return self.out
        if self.world > 1:
            dist.all_gather_into_tensor(self.all.view(-1), self.mine.view(-1), group=self.group)
        else:
            self.all.copy_(self.mine.unsqueeze(0))
        ops.merge_slots_gate(self.all, 2 * self.world, q_gate, self.out, H_Q, D)
        return self.out
