"""KHQ calibration tables: the ``khq_calib.bin`` container and its in-memory form.

File layout (little-endian), as written by ``src/khq/calib.mojo:323-329, 524-542`` and parsed by
``khq_init`` (``src/khq/runtime.mojo:312-375``):

    u32 magic 'KHQK' (0x4B51484B) | u32 version = 2 | u32 n_layers | u32 D = 256
    per layer:
      u32 layer_id | f32 ts_k | f32 alpha_k | f32 d_k[256] | f32 cents_k[4*256] | f32 rotor_k[64*16]
      | f32 ts_v | f32 alpha_v | f32 d_v[256] | f32 cents_v[4*256] | f32 rotor_v[64*16]
      | f32 vq[64*256*3]

Tables are fp32 in the file and fp16 on the device.  Rotor element R[p][k][c] sits at
p*16 + k*4 + c.  layer_id indexes a 64-entry table.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List

import numpy as np

KHQ_MAGIC = 0x4B51484B
KHQ_VERSION = 2
KHQ_MAX_LAYERS = 64
D = 256
NP = 64


@dataclass
class KhqLayerTables:
    """One attention layer's tables (fp32 host copies)."""

    layer_id: int
    ts_k: float
    alpha_k: float
    d_k: np.ndarray      # (256,)
    cents_k: np.ndarray  # (4, 256)
    rotor_k: np.ndarray  # (64, 16)
    ts_v: float
    alpha_v: float
    d_v: np.ndarray
    cents_v: np.ndarray
    rotor_v: np.ndarray
    vq: np.ndarray       # (64, 256, 3)

    def as_f16(self) -> Dict[str, np.ndarray]:
        """fp16 arrays in the layout the kernels read (what ``_upload_f16`` produces,
        ``src/khq/runtime.mojo:299-309``)."""
        return {
            "d_k": self.d_k.astype(np.float16).reshape(D),
            "cents_k": self.cents_k.astype(np.float16).reshape(4 * D),
            "rotor_k": self.rotor_k.astype(np.float16).reshape(NP * 16),
            "d_v": self.d_v.astype(np.float16).reshape(D),
            "cents_v": self.cents_v.astype(np.float16).reshape(4 * D),
            "rotor_v": self.rotor_v.astype(np.float16).reshape(NP * 16),
            "vq": self.vq.astype(np.float16).reshape(NP * 256 * 3),
        }


_LAYER_F32 = 2 + D + 4 * D + NP * 16  # ts, alpha, d, cents, rotor  (per K or V block)


def write_calib(path, layers: List[KhqLayerTables]) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<IIII", KHQ_MAGIC, KHQ_VERSION, len(layers), D))
        for L in layers:
            f.write(struct.pack("<I", L.layer_id))
            for ts, al, dv, ce, ro in ((L.ts_k, L.alpha_k, L.d_k, L.cents_k, L.rotor_k),
                                       (L.ts_v, L.alpha_v, L.d_v, L.cents_v, L.rotor_v)):
                f.write(struct.pack("<ff", ts, al))
                f.write(np.asarray(dv, np.float32).reshape(D).tobytes())
                f.write(np.asarray(ce, np.float32).reshape(4 * D).tobytes())
                f.write(np.asarray(ro, np.float32).reshape(NP * 16).tobytes())
            f.write(np.asarray(L.vq, np.float32).reshape(NP * 256 * 3).tobytes())


def read_calib(path) -> List[KhqLayerTables]:
    """Parse a calibration file; raises ValueError on the conditions ``khq_init`` rejects
    (bad magic, version != 2, layer_id outside 0..63) and on truncation."""
    buf = Path(path).read_bytes()
    if len(buf) < 16:
        raise ValueError("calibration file too short")
    magic, ver, n_lay, dim = struct.unpack_from("<IIII", buf, 0)
    if magic != KHQ_MAGIC:
        raise ValueError("bad magic: not a KHQK file")
    if ver != KHQ_VERSION:
        raise ValueError(f"unsupported version {ver}")
    if dim != D:
        raise ValueError(f"unsupported head_dim {dim}")
    off = 16
    out = []

    def take(n):
        nonlocal off
        if off + 4 * n > len(buf):
            raise ValueError("calibration file truncated")
        a = np.frombuffer(buf, dtype="<f4", count=n, offset=off).copy()
        off += 4 * n
        return a

    for _ in range(n_lay):
        if off + 4 > len(buf):
            raise ValueError("calibration file truncated")
        (layer_id,) = struct.unpack_from("<I", buf, off)
        off += 4
        if layer_id >= KHQ_MAX_LAYERS:
            raise ValueError(f"layer_id {layer_id} out of range")
        ts_k, al_k = take(2)
        d_k, c_k, r_k = take(D), take(4 * D).reshape(4, D), take(NP * 16).reshape(NP, 16)
        ts_v, al_v = take(2)
        d_v, c_v, r_v = take(D), take(4 * D).reshape(4, D), take(NP * 16).reshape(NP, 16)
        vq = take(NP * 256 * 3).reshape(NP, 256, 3)
        out.append(KhqLayerTables(int(layer_id), float(ts_k), float(al_k), d_k, c_k, r_k,
                                  float(ts_v), float(al_v), d_v, c_v, r_v, vq))
    return out
