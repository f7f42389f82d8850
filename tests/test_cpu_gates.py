"""The reference's deploy gates over the debug lines of this runtime (cadence and payload
contents, deploy_on_kaggle.sh:1826-1937), with the oracle as the compute backend."""
import numpy as np

import cases
from cases import D, H_KV, H_Q, SCALE
from bonsai_mojo_1bit_optimization_t4_cuda_b200 import formats, gates
from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime


def _run(oracle, monkeypatch, capsys, tmp_path, n_steps, layer_ids, shift=0):
    """Decode n_steps tokens on the layers with BONSAI_KHQ_DEBUG=1; the K rows handed to
    khq_capture_unroped are also collected into kv_dump.bin.  ``shift`` > 0 feeds the dump
    collector the K of a later token: a host that compresses the wrong tokens looks like this."""
    import torch

    monkeypatch.setenv("BONSAI_KHQ_DEBUG", "1")
    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "4")
    cs = {li: cases.make_case(cases.synth.seed_for(1, li), n_steps + shift, "calib", layer_id=li) for li in layer_ids}
    rt = KhqRuntime(oracle.OracleOps(), device="cpu")
    assert rt.khq_activate([cs[li]["tables"] for li in layer_ids], max_seq=1024)
    col = formats.KvDumpCollector(tmp_path, max_tokens=n_steps, kv_dim=H_KV * D)
    for li in layer_ids:
        rt.khq_init_layer(li, H_Q, H_KV, D)
    rng = np.random.default_rng(3)
    for t in range(n_steps):
        qg = torch.from_numpy(cases.synth.make_q_gate(rng, t))
        for li in layer_ids:
            c = cs[li]
            col.dump_kv(li, c["k_unroped"][t + shift], c["v"][t])
            rt.khq_capture_unroped(li, torch.from_numpy(c["k_unroped"][t]))
            out = torch.zeros(H_Q * D, dtype=torch.float16)
            assert rt.khq_step(li, qg, torch.from_numpy(c["k_roped"][t]), torch.from_numpy(c["v"][t]), out, SCALE)
    assert col.flush() == len(layer_ids)
    return capsys.readouterr().out


def test_cadence_and_payload_gates_pass(oracle, monkeypatch, capsys, tmp_path):
    log = _run(oracle, monkeypatch, capsys, tmp_path, 400, [3, 7])
    ev = gates.parse_compress_events(log)
    assert sorted(ev) == [3, 7]
    assert ev[3] == [(1, 128, 256, 128), (2, 256, 384, 128)]  # first at write_pos 256, then every 128
    assert gates.check_cadence(ev) == []
    recs = gates.parse_norm_lines(log)
    assert [(r.layer, r.boundary, r.n_rows) for r in recs] == [(3, 0, 512), (7, 0, 512), (3, 128, 512), (7, 128, 512)]
    _, dump = formats.read_kv_dump(tmp_path / "kv_dump.bin")
    res = gates.check_payload_norms(recs, dump, H_KV, D)
    assert res.failures == [] and res.events == 4
    assert res.err_aligned_max < 2e-3           # fp16 rounding of the stored norm
    assert res.err_shifted_mean > 50 * res.err_aligned_mean


def test_gates_catch_wrong_cadence_and_wrong_tokens(oracle, monkeypatch, capsys, tmp_path):
    # wrong tokens: the dump holds the K of tokens 128 later than the ones the runtime compressed
    log = _run(oracle, monkeypatch, capsys, tmp_path, 300, [3], shift=128)
    _, dump = formats.read_kv_dump(tmp_path / "kv_dump.bin")
    res = gates.check_payload_norms(gates.parse_norm_lines(log), dump, H_KV, D)
    assert any("off the ground truth" in f for f in res.failures)
    assert any("shifted" in f for f in res.failures)
    # cadence: a doctored log (second event one chunk late, layer 7 short of one event)
    good = gates.parse_compress_events(log)
    assert gates.check_cadence(good) == []
    bad = {3: [(1, 128, 256, 128), (2, 384, 512, 128)], 7: [(1, 128, 256, 128)]}
    fails = gates.check_cadence(bad)
    assert any("differ" in f for f in fails) and any("L3#2" in f for f in fails)
    assert gates.check_cadence({}) != [] and gates.check_payload_norms([], dump, H_KV, D).failures != []
