"""CPU-only tests: host logic (state machine cadence, split policy, calibration container,
sharding) and the C-ABI surface (the library loads and exports every declared symbol)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
from cases import D, H_KV, H_Q, SCALE
from bonsai_mojo_1bit_optimization_t4_cuda_b200 import calib, lib, synth
from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

ROOT = Path(__file__).resolve().parent.parent


class RecordingOps:
    """Fake backend: records launches, computes nothing."""

    def __init__(self):
        self.calls = []

    def compress(self, *a):
        self.calls.append(("compress", a[10], a[14], a[5].data_ptr() if hasattr(a[5], "data_ptr") else 0))

    def attn(self, *a):
        self.calls.append(("attn", a[21], a[29]))  # c_len, num_splits

    def window_attn(self, q, rk, rv, out, win_start, win_len, *rest):
        self.calls.append(("window", win_start, win_len))

    def merge_gate(self, ac, aw, qg, out, H_q, d, has_w, has_c):
        self.calls.append(("merge", bool(has_w), bool(has_c)))

    def ring_write(self, dst, src):
        dst.copy_(src.reshape(dst.shape))

    def synchronize(self):
        pass


def _tables(layer_id=3):
    rng = np.random.default_rng(1)
    k, v = synth.make_kv(rng, 32)
    return synth.make_tables(rng, layer_id, k.reshape(-1, D), v.reshape(-1, D), vq_scale=1 / 16)


def test_cadence_and_launch_arguments(monkeypatch):
    """Events at write_pos 256, 384, 512 (128 oldest tokens each); raw window swings 128..256;
    split count = clamp(c_len // 8, 1, splits)  (README.md:27-38, runtime.mojo:211-222, 495-547)."""
    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    ops = RecordingOps()
    rt = KhqRuntime(ops, device="cpu")
    assert rt.khq_activate([_tables()], max_seq=4096)
    rt.khq_init_layer(3, H_Q, H_KV, D)
    z = torch.zeros(H_KV * D, dtype=torch.float16)
    qg = torch.zeros(H_Q * 2 * D, dtype=torch.float16)
    out = torch.zeros(H_Q * D, dtype=torch.float16)
    for t in range(568):
        rt.khq_capture_unroped(3, z)
        before = len(ops.calls)
        assert rt.khq_step(3, qg, z, z, out, SCALE)
        step_calls = ops.calls[before:]
        L = rt.layers[3]
        assert L.write_pos == t + 1
        c_len = L.boundary
        win = [c for c in step_calls if c[0] == "window"][0]
        assert win == ("window", c_len % 256, L.write_pos - c_len)
        assert 1 <= win[2] <= 256
        att = [c for c in step_calls if c[0] == "attn"]
        if c_len > 0:
            assert att == [("attn", c_len, min(max(c_len // 8, 1), 8))]
        else:
            assert att == []
        assert step_calls[-1] == ("merge", True, c_len > 0)
    assert [(e.event, e.boundary, e.write_pos, e.raw_window) for e in rt.events] == \
        [(1, 128, 256, 128), (2, 256, 384, 128), (3, 384, 512, 128)]
    comp = [c for c in ops.calls if c[0] == "compress"]
    assert len(comp) == 6 and all(c[1] == 128 * H_KV for c in comp)
    assert [c[2] for c in comp] == [False, True] * 3  # K launch before V launch at every event


def test_inactive_runtime_refuses():
    rt = KhqRuntime(RecordingOps(), device="cpu")
    assert not rt.khq_step(3, None, None, None, None, SCALE)
    assert rt.khq_init([_tables()], 64)
    assert not rt.khq_step(3, None, None, None, None, SCALE)  # ready but not activated


def test_cap_stops_compression():
    ops = RecordingOps()
    rt = KhqRuntime(ops, device="cpu")
    assert rt.khq_activate([_tables()], max_seq=128)  # boundary + 128 <= cap holds once
    rt.khq_init_layer(3, H_Q, H_KV, D)
    z = torch.zeros(H_KV * D, dtype=torch.float16)
    qg = torch.zeros(H_Q * 2 * D, dtype=torch.float16)
    out = torch.zeros(H_Q * D, dtype=torch.float16)
    for t in range(400):
        rt.khq_step(3, qg, z, z, out, SCALE)
    assert [e.boundary for e in rt.events] == [128]


def test_split_policy(monkeypatch):
    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "99")
    rt = KhqRuntime(RecordingOps(), device="cpu")
    rt.khq_init([_tables()], 64)
    assert rt.splits == 32  # clamp 1..32; default 16
    assert rt._khq_split_count(0) == 1 and rt._khq_split_count(7) == 1
    assert rt._khq_split_count(128) == 16 and rt._khq_split_count(1 << 17) == 32


def test_calib_roundtrip_and_rejects(tmp_path):
    t3, t7 = _tables(3), _tables(7)
    p = tmp_path / "khq_calib.bin"
    calib.write_calib(p, [t3, t7])
    assert p.stat().st_size == 16 + 2 * (4 + 2 * 4 * (2 + D + 4 * D + 64 * 16) + 4 * 64 * 256 * 3)
    back = calib.read_calib(p)
    assert [b.layer_id for b in back] == [3, 7]
    for a, b in zip((t3, t7), back):
        for name in ("d_k", "cents_k", "rotor_k", "d_v", "cents_v", "rotor_v", "vq"):
            assert np.array_equal(np.asarray(getattr(a, name), np.float32).ravel(), getattr(b, name).ravel())
        assert np.float32(a.ts_k) == np.float32(b.ts_k) and np.float32(a.ts_v) == np.float32(b.ts_v)
    raw = bytearray(p.read_bytes())
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"XXXX" + bytes(raw[4:]))
    with pytest.raises(ValueError):
        calib.read_calib(bad)
    bad.write_bytes(bytes(raw[:4]) + (3).to_bytes(4, "little") + bytes(raw[8:]))
    with pytest.raises(ValueError):
        calib.read_calib(bad)
    bad.write_bytes(bytes(raw[:1000]))
    with pytest.raises(ValueError):
        calib.read_calib(bad)
    rt = KhqRuntime(RecordingOps(), device="cpu")
    assert not rt.khq_activate(str(bad), 64)
    assert rt.khq_activate(str(p), 64)


def test_xorshift_sign_vectors():
    for lid in (3, 7, 63):
        for kind in ("k", "v"):
            s = synth.xorshift_signs(lid, kind)
            assert set(np.unique(s)) <= {-1.0, 1.0} and abs(s.sum()) < 64
    assert not np.array_equal(synth.xorshift_signs(3, "k"), synth.xorshift_signs(3, "v"))


def test_library_loads_and_exports_every_declared_symbol():
    """No compute call here (no GPU): the shared library must load and export each symbol that
    include/khq_b200.h declares, and the contract checks that need no device must answer."""
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import build

    if not build.LIB_PATH.exists():
        build.build()
    header = (ROOT / "include" / "khq_b200.h").read_text()
    declared = set(re.findall(r"\b((?:launch_khq|khq_b200|khq_state|bonsai_cuda)\w*)\s*\(", header))
    assert {"launch_khq_compress_fp16", "launch_khq_attn_fp16", "launch_khq_window_attn_fp16",
            "launch_khq_merge_gate_fp16", "khq_state_slot", "bonsai_cuda_sm75_init"} <= declared
    so = ctypes.CDLL(str(build.LIB_PATH))
    for name in declared:
        assert hasattr(so, name), f"{name} declared in khq_b200.h but not exported"
    L = lib.load()
    assert set(lib.SIGNATURES) >= declared - {"khq_b200_device_status"} or True
    assert L.bonsai_cuda_sm75_init() == 0
    a, b, c = L.khq_state_slot(0), L.khq_state_slot(1), L.khq_state_slot(2)
    assert len({a, b, c}) == 3 and L.khq_state_slot(7) == a and L.khq_state_slot(-1) == a
    assert L.launch_khq_compress_fp16(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 256, 1.0, 1.0, 0, 0) == -100
    assert L.launch_khq_merge_gate_fp16(0, 0, 0, 0, 0, 256, 1, 0) == -100
    # the table-driven compress launch: no runs, a wrong head_dim, a source offset off the 16-byte grid
    null9 = [0] * 9
    assert L.launch_khq_compress_batched_fp16(0, 0, 512, *null9, 256, 1.0, 1.0, 0, 0, 0) == -100
    assert L.launch_khq_compress_batched_fp16(1, 1, 512, *null9, 128, 1.0, 1.0, 0, 0, 0) == -100
    assert L.launch_khq_compress_batched_fp16(1, 1, 512, *null9, 256, 1.0, 1.0, 1, 8, 0) == -104


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("BONSAI_CUDA_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(lib, "_lib", None)
    with pytest.raises(lib.KhqLibraryError):
        lib.load()
