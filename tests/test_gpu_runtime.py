"""GPU test of the host state machine driving the CUDA library: the decode loop of a 56-token
prompt followed by decode steps, compared step by step with the same loop executed on the CPU
through the oracle backend (same seeded inputs, same code path above the launches)."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


def drive(rt, torch, device, case, n_steps, layer_ids, collect_at):
    outs = {}
    for li in layer_ids:
        rt.khq_init_layer(li, H_Q, H_KV, D)
    rng = np.random.default_rng(99)
    for t in range(n_steps):
        qg = torch.from_numpy(cases.synth.make_q_gate(rng, t)).to(device)
        for li in layer_ids:
            k_u = torch.from_numpy(case["k_unroped"][t]).to(device)
            k_r = torch.from_numpy(case["k_roped"][t]).to(device)
            v = torch.from_numpy(case["v"][t]).to(device)
            out = torch.zeros(H_Q * D, dtype=torch.float16, device=device)
            rt.khq_capture_unroped(li, k_u)
            assert rt.khq_step(li, qg, k_r, v, out, SCALE)
            if t in collect_at:
                outs[(li, t)] = out.float().cpu().numpy()
    return outs


def test_decode_loop_matches_oracle_backend(cuda_ops, oracle, monkeypatch):
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    n_steps = 56 + 340  # passes the events at write_pos 256 and 384
    case = cases.make_case(cases.synth.seed_for(1), n_steps, "calib", layer_id=3)
    tb7 = case["tables"]
    collect = {0, 55, 254, 255, 256, 300, 383, 384, 395}
    res = {}
    for name, ops, device in (("gpu", cuda_ops, "cuda"), ("cpu", oracle.OracleOps(), "cpu")):
        rt = KhqRuntime(ops, device=device)
        assert rt.khq_activate([tb7], max_seq=4096)
        res[name] = (drive(rt, torch, device, case, n_steps, [3], collect), rt)
    (g_out, g_rt), (c_out, c_rt) = res["gpu"], res["cpu"]
    assert [(e.boundary, e.write_pos, e.raw_window) for e in g_rt.events] == [(128, 256, 128), (256, 384, 128)]
    assert [(e.boundary, e.write_pos) for e in g_rt.events] == [(e.boundary, e.write_pos) for e in c_rt.events]
    # code words written by the two backends must be identical
    for key in ("kmask", "kpay", "knorm", "krn", "vpay", "vnorm", "vrn", "vsm"):
        a = g_rt.layers[3].t[key].cpu()
        b = c_rt.layers[3].t[key]
        n = 256 * H_KV * {"kmask": 16, "kpay": 40, "vpay": 104, "vsm": 4}.get(key, 1)
        assert torch.equal(a[:n].view(torch.uint8), b[:n].view(torch.uint8)), key
    for k in sorted(g_out):
        ok, mx, exc = cases.attention_close(g_out[k], c_out[k])
        assert ok, f"step {k}: max abs {mx:.3e} excess {exc:.3e}"


def test_decode_loop_with_fused_prestep(cuda_ops, oracle, monkeypatch):
    """Same loop, but q/k arrive un-normed and un-RoPE'd and go through khq_prestep (one launch
    for norm + capture + RoPE + ring appends) followed by khq_step(rings_written=True)."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    n_steps = 300
    case = cases.make_case(cases.synth.seed_for(1, 7), n_steps, "n01_idrot", layer_id=7)
    rng = np.random.default_rng(5)
    qw = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    q_raw = [(np.random.default_rng(100 + t).standard_normal((H_Q, 2 * D))).astype(np.float16) for t in range(n_steps)]
    collect = {0, 100, 255, 256, 299}
    res = {}
    for name, ops, device in (("gpu", cuda_ops, "cuda"), ("cpu", oracle.OracleOps(), "cpu")):
        rt = KhqRuntime(ops, device=device)
        assert rt.khq_activate([case["tables"]], max_seq=1024)
        rt.khq_init_layer(7, H_Q, H_KV, D)
        outs = {}
        for t in range(n_steps):
            qg = torch.from_numpy(q_raw[t].copy()).to(device).reshape(-1)
            k = torch.from_numpy(case["k_unroped"][t].copy()).to(device).reshape(-1)
            v = torch.from_numpy(case["v"][t].copy()).to(device).reshape(-1)
            out = torch.zeros(H_Q * D, dtype=torch.float16, device=device)
            assert rt.khq_prestep(7, qg, k, v, t, torch.from_numpy(qw).to(device), torch.from_numpy(kw).to(device))
            assert rt.khq_step(7, qg, k, v, out, SCALE, rings_written=True)
            if t in collect:
                outs[t] = out.float().cpu().numpy()
        res[name] = (outs, rt)
    (g_out, g_rt), (c_out, c_rt) = res["gpu"], res["cpu"]
    assert [e.boundary for e in g_rt.events] == [e.boundary for e in c_rt.events] == [128]
    for key in ("kmask", "kpay", "knorm", "krn", "vpay", "vnorm", "vrn", "vsm"):
        n = 128 * H_KV * {"kmask": 16, "kpay": 40, "vpay": 104, "vsm": 4}.get(key, 1)
        assert torch.equal(g_rt.layers[7].t[key].cpu()[:n].view(torch.uint8), c_rt.layers[7].t[key][:n].view(torch.uint8)), key
    for t in sorted(g_out):
        ok, mx, exc = cases.attention_close(g_out[t], c_out[t])
        assert ok, f"step {t}: max abs {mx:.3e} excess {exc:.3e}"
