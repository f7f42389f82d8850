"""On-disk containers that sit either side of the KHQ attention path.

``kv_dump.bin`` (calibration input; written by ``khq_dump_flush``,
``src/models/qwen3_5/khq_dump.mojo:337-366``; layout comment ``:10-14``), little-endian:

    u32 magic 'KHQD' (0x4451484B) | u32 n_layers | u32 dim (= H_kv * head_dim = 1024)
    n_layers x (u32 layer_id | u32 n_tokens)
    per layer, in header order: K (n_tokens x dim f32) then V (n_tokens x dim f32)

K rows are post-head-RMSNorm, pre-RoPE; V rows come straight from the projection.

``attn_<layer>.bin`` (softmax scores for the attention-aware VQ loss; ``khq_dump.mojo:95-97``
layout, ``:249-317`` writer):

    u32 magic 'KHQA' (0x4151484B) | u32 H_q | u32 H_kv | u32 D
    per token: u32 n_valid (= pos + 1) | H_q x n_valid fp16 scores (one row per query head)

``khq_state.bin`` (checkpoint of the per-layer KHQ decode state; the reference keeps this state
only in device memory and cannot resume a sequence):

    u32 magic 'KHQS' (0x5351484B) | u32 version = 1 | u32 n_layers
    per layer: u32 layer_id | u32 H_q | u32 H_kv | u32 D | u32 cap | u32 boundary | u32 write_pos
               | ring_k, ring_v, ring_u  (256 x H_kv x D fp16 each)
               | for the boundary*H_kv compressed rows: k_mask (rows x 16 u32), k_payload (rows x 40),
                 k_norms, k_r_norms (rows fp16), v_payload (rows x 104), v_norms, v_r_norms (rows
                 fp16), v_shared_meta (rows x 4 bytes)
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np

KHQD_MAGIC = 0x4451484B
KHQA_MAGIC = 0x4151484B
KHQS_MAGIC = 0x5351484B
KHQS_VERSION = 1
KHQ_MAX_LAYERS = 64


# ------------------------------------------------------------------------------------ kv_dump.bin
def write_kv_dump(path, layers: Dict[int, Tuple[np.ndarray, np.ndarray]]) -> int:
    """Write ``{layer_id: (K, V)}`` with K, V of shape (n_tokens, dim); layers are stored in
    ascending id order and empty layers are skipped, as ``khq_dump_flush`` does.  Returns the
    number of layers written (0: no file is produced, ``khq_dump.mojo:351-353``)."""
    items = [(li, kv) for li, kv in sorted(layers.items()) if len(kv[0]) > 0]
    if not items:
        return 0
    dim = int(items[0][1][0].shape[1])
    with open(path, "wb") as f:
        f.write(struct.pack("<III", KHQD_MAGIC, len(items), dim))
        for li, (k, v) in items:
            if not 0 <= li < KHQ_MAX_LAYERS:
                raise ValueError(f"layer id {li} outside the {KHQ_MAX_LAYERS}-entry table")
            if k.shape != v.shape or k.shape[1] != dim:
                raise ValueError(f"layer {li}: K {k.shape} / V {v.shape} do not match dim {dim}")
            f.write(struct.pack("<II", li, k.shape[0]))
        for _, (k, v) in items:
            f.write(np.ascontiguousarray(k, dtype="<f4").tobytes())
            f.write(np.ascontiguousarray(v, dtype="<f4").tobytes())
    return len(items)


def read_kv_dump(path) -> Tuple[int, Dict[int, Tuple[np.ndarray, np.ndarray]]]:
    """Returns ``(dim, {layer_id: (K, V)})``; raises ValueError on a bad magic or a short file."""
    raw = Path(path).read_bytes()
    if len(raw) < 12:
        raise ValueError("kv_dump: shorter than its header")
    magic, n_layers, dim = struct.unpack_from("<III", raw, 0)
    if magic != KHQD_MAGIC:
        raise ValueError(f"kv_dump: bad magic 0x{magic:08X}")
    off = 12
    heads: List[Tuple[int, int]] = []
    for _ in range(n_layers):
        if off + 8 > len(raw):
            raise ValueError("kv_dump: truncated layer table")
        heads.append(struct.unpack_from("<II", raw, off))
        off += 8
    out: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}
    for li, n in heads:
        nb = n * dim * 4
        if off + 2 * nb > len(raw):
            raise ValueError(f"kv_dump: layer {li} data truncated")
        k = np.frombuffer(raw, dtype="<f4", count=n * dim, offset=off).reshape(n, dim).copy()
        v = np.frombuffer(raw, dtype="<f4", count=n * dim, offset=off + nb).reshape(n, dim).copy()
        out[li] = (k, v)
        off += 2 * nb
    return dim, out


class KvDumpCollector:
    """Host-side mirror of ``khq_dump_configure`` / ``khq_dump_kv`` / ``khq_dump_flush``
    (``khq_dump.mojo:27-86, 337-366``): collects one K (un-RoPE'd) and one V row per token and
    layer, at most ``max_tokens`` per layer, and writes ``<dir>/kv_dump.bin``."""

    def __init__(self, dir_path, max_tokens: int, kv_dim: int):
        self.dir = Path(dir_path)
        self.cap = int(max_tokens)
        self.dim = int(kv_dim)
        self.k: Dict[int, List[np.ndarray]] = {}
        self.v: Dict[int, List[np.ndarray]] = {}

    def dump_kv(self, layer_idx: int, k_row, v_row) -> bool:
        if layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return False
        rows = self.k.setdefault(layer_idx, [])
        if len(rows) >= self.cap:
            return False
        k = np.asarray(k_row, dtype=np.float16).reshape(self.dim).astype(np.float32)
        v = np.asarray(v_row, dtype=np.float16).reshape(self.dim).astype(np.float32)
        rows.append(k)
        self.v.setdefault(layer_idx, []).append(v)
        return True

    def flush(self) -> int:
        layers = {li: (np.stack(self.k[li]), np.stack(self.v[li])) for li in self.k if self.k[li]}
        n = write_kv_dump(self.dir / "kv_dump.bin", layers)
        self.k.clear()
        self.v.clear()
        return n


# ------------------------------------------------------------------------------------ attn_<L>.bin
def attn_scores(q_gate: np.ndarray, k_roll: np.ndarray, n_valid: int, H_q: int, H_kv: int, d: int,
                scale: float) -> np.ndarray:
    """softmax(q . K * scale) over rows 0..n_valid-1 per query head, fp32, as the dump writer
    computes it (``khq_dump.mojo:282-306``).  q_gate (H_q, 2d) interleaved, k_roll (>= n_valid,
    H_kv * d) RoPE'd keys.  Returns (H_q, n_valid) float32."""
    q = np.asarray(q_gate, dtype=np.float32).reshape(H_q, 2 * d)[:, :d]
    k = np.asarray(k_roll, dtype=np.float32)[:n_valid].reshape(n_valid, H_kv, d)
    n_rep = H_q // H_kv
    out = np.empty((H_q, n_valid), dtype=np.float32)
    for h in range(H_q):
        logits = (k[:, h // n_rep, :] @ q[h]).astype(np.float32) * np.float32(scale)
        e = np.exp(logits - logits.max(), dtype=np.float32)
        out[h] = e * (np.float32(1.0) / e.sum(dtype=np.float32))
    return out


class AttnDumpWriter:
    """Writes ``<dir>/attn_<layer>.bin`` record by record (one record per token)."""

    def __init__(self, dir_path, H_q: int, H_kv: int, d: int):
        self.dir = Path(dir_path)
        self.H_q, self.H_kv, self.D = int(H_q), int(H_kv), int(d)
        self.files: Dict[int, object] = {}

    def append(self, layer_idx: int, scores: np.ndarray) -> None:
        s = np.asarray(scores)
        if s.ndim != 2 or s.shape[0] != self.H_q:
            raise ValueError(f"scores {s.shape} are not (H_q={self.H_q}, n_valid)")
        f = self.files.get(layer_idx)
        if f is None:
            f = open(self.dir / f"attn_{layer_idx}.bin", "wb")
            f.write(struct.pack("<IIII", KHQA_MAGIC, self.H_q, self.H_kv, self.D))
            self.files[layer_idx] = f
        f.write(struct.pack("<I", s.shape[1]))
        f.write(np.ascontiguousarray(s, dtype="<f2").tobytes())  # round-to-nearest-even, as :98-118

    def close(self) -> None:
        for f in self.files.values():
            f.close()
        self.files.clear()


def read_attn_dump(path) -> Tuple[Tuple[int, int, int], List[np.ndarray]]:
    """Returns ``((H_q, H_kv, D), [scores of token 0 (H_q, 1), token 1 (H_q, 2), ...])``."""
    raw = Path(path).read_bytes()
    if len(raw) < 16:
        raise ValueError("attn dump: shorter than its header")
    magic, H_q, H_kv, D = struct.unpack_from("<IIII", raw, 0)
    if magic != KHQA_MAGIC:
        raise ValueError(f"attn dump: bad magic 0x{magic:08X}")
    off, recs = 16, []
    while off < len(raw):
        if off + 4 > len(raw):
            raise ValueError("attn dump: truncated record header")
        (n_valid,) = struct.unpack_from("<I", raw, off)
        off += 4
        nb = H_q * n_valid * 2
        if off + nb > len(raw):
            raise ValueError("attn dump: truncated record")
        recs.append(np.frombuffer(raw, dtype="<f2", count=H_q * n_valid, offset=off).reshape(H_q, n_valid).copy())
        off += nb
    return (H_q, H_kv, D), recs
