"""On-disk containers either side of the path: kv_dump.bin (KHQD), attn_<L>.bin (KHQA) and the
KHQ state checkpoint (KHQS)."""
import struct

import numpy as np
import pytest

from bonsai_mojo_1bit_optimization_t4_cuda_b200 import formats, synth
from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KHQ_RING, KhqRuntime


def test_kv_dump_round_trip_and_layout(tmp_path):
    rng = np.random.default_rng(1)
    layers = {7: (rng.standard_normal((5, 1024)).astype(np.float32), rng.standard_normal((5, 1024)).astype(np.float32)),
              3: (rng.standard_normal((2, 1024)).astype(np.float32), rng.standard_normal((2, 1024)).astype(np.float32)),
              9: (np.zeros((0, 1024), np.float32), np.zeros((0, 1024), np.float32))}
    p = tmp_path / "kv_dump.bin"
    assert formats.write_kv_dump(p, layers) == 2  # the empty layer is skipped
    raw = p.read_bytes()
    # header: magic, n_layers, dim, then (layer_id, n_tokens) in ascending layer order (khq_dump.mojo:355-366)
    assert struct.unpack_from("<IIIIIII", raw, 0) == (0x4451484B, 2, 1024, 3, 2, 7, 5)
    assert raw[:4] == b"KHQD"
    assert len(raw) == 12 + 16 + (2 + 5) * 2 * 1024 * 4
    # data: layer 3 K then V, then layer 7 K then V
    assert np.frombuffer(raw, "<f4", 1024, 28).tolist() == layers[3][0][0].tolist()
    dim, back = formats.read_kv_dump(p)
    assert dim == 1024 and sorted(back) == [3, 7]
    for li in (3, 7):
        assert np.array_equal(back[li][0], layers[li][0]) and np.array_equal(back[li][1], layers[li][1])


def test_kv_dump_collector_caps_tokens_and_rejects_bad_files(tmp_path):
    col = formats.KvDumpCollector(tmp_path, max_tokens=3, kv_dim=8)
    for t in range(5):
        ok = col.dump_kv(2, np.full(8, t, np.float16), np.full(8, -t, np.float16))
        assert ok == (t < 3)
    assert not col.dump_kv(64, np.zeros(8, np.float16), np.zeros(8, np.float16))
    assert col.flush() == 1
    dim, back = formats.read_kv_dump(tmp_path / "kv_dump.bin")
    assert dim == 8 and back[2][0].shape == (3, 8) and back[2][1][2, 0] == -2.0
    assert formats.KvDumpCollector(tmp_path / "none", 3, 8).flush() == 0  # nothing collected: no file
    bad = tmp_path / "bad.bin"
    bad.write_bytes(struct.pack("<III", 0x12345678, 1, 8))
    with pytest.raises(ValueError):
        formats.read_kv_dump(bad)
    bad.write_bytes((tmp_path / "kv_dump.bin").read_bytes()[:-4])
    with pytest.raises(ValueError):
        formats.read_kv_dump(bad)


def test_attn_dump_records(tmp_path):
    H_q, H_kv, d = 4, 2, 16
    rng = np.random.default_rng(2)
    kroll = rng.standard_normal((6, H_kv * d)).astype(np.float32)
    w = formats.AttnDumpWriter(tmp_path, H_q, H_kv, d)
    want = []
    for pos in range(6):
        qg = rng.standard_normal((H_q, 2 * d)).astype(np.float16)
        s = formats.attn_scores(qg, kroll, pos + 1, H_q, H_kv, d, 0.25)
        assert s.shape == (H_q, pos + 1) and np.allclose(s.sum(1), 1.0, atol=1e-6)
        # GQA: heads 0,1 read kv-head 0, heads 2,3 kv-head 1
        ref = np.exp((kroll[:pos + 1, d:2 * d] @ qg[2, :d].astype(np.float32)) * 0.25)
        assert np.allclose(s[2], ref / ref.sum(), rtol=1e-5)
        w.append(1, s)
        want.append(s.astype(np.float16))
    w.close()
    raw = (tmp_path / "attn_1.bin").read_bytes()
    assert struct.unpack_from("<IIII", raw, 0) == (0x4151484B, H_q, H_kv, d) and raw[:4] == b"KHQA"
    assert struct.unpack_from("<I", raw, 16)[0] == 1  # first record: n_valid = pos + 1 = 1
    assert len(raw) == 16 + sum(4 + H_q * (p + 1) * 2 for p in range(6))
    hdr, recs = formats.read_attn_dump(tmp_path / "attn_1.bin")
    assert hdr == (H_q, H_kv, d) and len(recs) == 6
    for a, b in zip(recs, want):
        assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        w.append(1, np.zeros((3, 2)))


def test_state_checkpoint_round_trip_on_cpu(tmp_path):
    """Save / load of the per-layer decode state; no compute call is involved, so the runtime can
    hold its tensors on the CPU here."""
    import torch

    rng = np.random.default_rng(5)
    sample = rng.standard_normal((64, 256)).astype(np.float16)
    tables = [synth.make_tables(rng, li, sample, sample) for li in (0, 3)]
    rt = KhqRuntime(ops=None, device="cpu")
    assert rt.khq_activate(tables, max_seq=512)
    g = torch.Generator().manual_seed(3)
    for li, (boundary, write_pos) in ((0, (256, 300)), (3, (0, 17))):
        rt.khq_init_layer(li, 24, 4, 256)
        L = rt.layers[li]
        for name, t in L.t.items():
            if name in ("dk", "ck", "rk", "dv", "cv", "rv", "vq"):
                continue
            t.view(torch.uint8).copy_(torch.randint(0, 256, t.view(torch.uint8).shape, generator=g, dtype=torch.uint8))
        L.boundary, L.write_pos = boundary, write_pos
    p = tmp_path / "khq_state.bin"
    assert rt.khq_save_state(p) == 2
    assert p.read_bytes()[:4] == b"KHQS"
    rt2 = KhqRuntime(ops=None, device="cpu")
    assert rt2.khq_activate(tables, max_seq=512)
    assert rt2.khq_load_state(p) == 2
    for li in (0, 3):
        A, B = rt.layers[li], rt2.layers[li]
        assert (A.boundary, A.write_pos, A.H_q, A.H_kv) == (B.boundary, B.write_pos, B.H_q, B.H_kv)
        rows = A.boundary * 4
        for r in ("ring_k", "ring_v", "ring_u"):
            assert torch.equal(A.t[r].view(torch.int16), B.t[r].view(torch.int16))
        for name, rb in KhqRuntime._STATE_ROW_ARRAYS:
            a, b = A.t[name].view(torch.uint8), B.t[name].view(torch.uint8)
            assert torch.equal(a[:rows * rb], b[:rows * rb]), name
            assert not b[rows * rb:].any()  # rows past the boundary are not part of the state
    # malformed files are refused
    raw = p.read_bytes()
    (tmp_path / "short.bin").write_bytes(raw[:-10])
    with pytest.raises(ValueError):
        KhqRuntime(ops=None, device="cpu").khq_load_state(p)  # tables not loaded
    rt3 = KhqRuntime(ops=None, device="cpu")
    rt3.khq_activate(tables, max_seq=512)
    with pytest.raises(ValueError):
        rt3.khq_load_state(tmp_path / "short.bin")
    rt4 = KhqRuntime(ops=None, device="cpu")
    rt4.khq_activate(tables, max_seq=128)  # smaller than the saved boundary
    with pytest.raises(ValueError):
        rt4.khq_load_state(p)
    assert KHQ_RING == 256
