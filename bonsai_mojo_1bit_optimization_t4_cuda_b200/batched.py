"""Batched decode: descriptor tables for many (sequence, layer) KHQ states and one launch for all
of them.  The reference has no batch dimension (one sequence, one layer per call); this is the
host side of ``launch_khq_decode_batched_fp16``.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from . import lib as _lib
from .lib import check, current_stream

SEQ_DESC = np.dtype([
    ("q_gate", "<u8"), ("k_payload", "<u8"), ("v_payload", "<u8"), ("v_shared_meta", "<u8"),
    ("k_mask", "<u8"), ("k_norms", "<u8"), ("k_r_norms", "<u8"), ("v_norms", "<u8"), ("v_r_norms", "<u8"),
    ("ring_k", "<u8"), ("ring_v", "<u8"), ("out", "<u8"),
    ("table_id", "<i4"), ("c_len", "<i4"), ("start_pos", "<i4"), ("win_start", "<i4"), ("win_len", "<i4"),
    ("first_slot", "<i4"), ("n_slots", "<i4"), ("pos_pack", "<i4"),
])
TABLES_DESC = np.dtype([
    ("cents_k", "<u8"), ("cents_v", "<u8"), ("vq", "<u8"), ("k_rotor", "<u8"), ("v_rotor", "<u8"),
    ("d_k", "<u8"), ("d_v", "<u8"), ("alpha_k", "<f4"), ("alpha_v", "<f4"),
])
WORK_ITEM = np.dtype([("desc", "<i4"), ("kind", "<i4"), ("lo", "<i4"), ("hi", "<i4"), ("slot", "<i4"),
                      ("r0", "<i4"), ("r1", "<i4"), ("r2", "<i4")])
assert SEQ_DESC.itemsize == 128 and TABLES_DESC.itemsize == 64 and WORK_ITEM.itemsize == 32


def plan(c_len: np.ndarray, win_len: np.ndarray, tokens_per_item: int = 0):
    """Run the library's host planner.  Returns (items, first_slot, n_slots)."""
    lib = _lib.load()
    c_len = np.ascontiguousarray(c_len, np.int32)
    win_len = np.ascontiguousarray(win_len, np.int32)
    n = len(c_len)
    first = np.zeros(n, np.int32)
    cnt = np.zeros(n, np.int32)
    n_items = lib.khq_b200_plan_decode(c_len.ctypes.data, win_len.ctypes.data, n, int(tokens_per_item), 0, 0,
                                       first.ctypes.data, cnt.ctypes.data)
    if n_items < 0:
        raise _lib.KhqLaunchError("khq_b200_plan_decode", n_items)
    items = np.zeros(max(n_items, 1), WORK_ITEM)
    got = lib.khq_b200_plan_decode(c_len.ctypes.data, win_len.ctypes.data, n, int(tokens_per_item),
                                   items.ctypes.data, n_items, first.ctypes.data, cnt.ctypes.data)
    assert got == n_items
    return items[:n_items], first, cnt


class BatchedDecode:
    """Device-resident descriptors + workspace for a fixed set of problems.

    ``problems``: one dict per (sequence, layer) with the torch CUDA tensors ``q_gate, k_payload,
    v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms, v_r_norms, ring_k, ring_v, out``
    and the ints ``table_id, c_len, start_pos, win_start, win_len``.  Order them by ``table_id``.
    ``tables``: one dict per layer with ``cents_k, cents_v, vq, k_rotor, v_rotor, d_k, d_v`` (fp16
    CUDA tensors) and ``alpha_k, alpha_v``.
    """

    def __init__(self, problems: Sequence[dict], tables: Sequence[dict], tokens_per_item: int = 0,
                 ring_cap: int = 256, codebook_in_smem: int = -1):
        self.lib = _lib.load()
        self.n_desc = len(problems)
        self.ring_cap = ring_cap
        self.codebook_in_smem = codebook_in_smem
        self._keep = (problems, tables)  # the descriptors hold raw addresses of these tensors
        d = np.zeros(self.n_desc, SEQ_DESC)
        for i, p in enumerate(problems):
            for k in ("q_gate", "k_payload", "v_payload", "v_shared_meta", "k_mask", "k_norms", "k_r_norms",
                      "v_norms", "v_r_norms", "ring_k", "ring_v", "out"):
                d[k][i] = p[k].data_ptr()
                if d[k][i] % 16:
                    raise ValueError(f"problem {i}: {k} must be 16-byte aligned (bulk asynchronous copies)")
            for k in ("table_id", "c_len", "start_pos", "win_start", "win_len"):
                d[k][i] = int(p[k])
        items, first, cnt = plan(d["c_len"], d["win_len"], tokens_per_item)
        d["first_slot"], d["n_slots"] = first, cnt
        t = np.zeros(len(tables), TABLES_DESC)
        for i, tb in enumerate(tables):
            for k in ("cents_k", "cents_v", "vq", "k_rotor", "v_rotor", "d_k", "d_v"):
                t[k][i] = tb[k].data_ptr()
            t["alpha_k"][i], t["alpha_v"][i] = tb["alpha_k"], tb["alpha_v"]
        self.n_items = len(items)
        self.host_descs, self.host_items = d, items
        dev = problems[0]["q_gate"].device
        up = lambda a: torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).to(dev)
        self.descs, self.tables, self.items = up(d), up(t), up(items)
        self.ws_bytes = int(self.lib.khq_b200_decode_workspace_bytes(self.n_items))
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)

    @property
    def algorithmic_bytes(self) -> int:
        """H_kv * (220*c_len + 1024*win_len) summed over the problems."""
        d = self.host_descs
        return int(4 * (220 * d["c_len"].astype(np.int64) + 1024 * d["win_len"].astype(np.int64)).sum())

    def launch(self, scale: float = 1.0 / 16.0, rope_base: float = 1e7) -> None:
        rc = self.lib.launch_khq_decode_batched_fp16(
            self.descs.data_ptr(), self.tables.data_ptr(), self.items.data_ptr(), self.n_desc, self.n_items,
            self.workspace.data_ptr(), self.ws_bytes, self.n_items, float(scale), float(rope_base),
            int(self.ring_cap), int(self.codebook_in_smem), current_stream())
        check("launch_khq_decode_batched_fp16", rc)
