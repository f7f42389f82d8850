"""GPU test of the host state machine driving the CUDA library: the decode loop of a 56-token
prompt followed by decode steps, compared step by step with the same loop executed on the CPU
through the oracle backend (same seeded inputs, same code path above the launches)."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


def drive(rt, torch, device, case, n_steps, layer_ids, collect_at, fused=False):
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
            if fused:
                assert rt.khq_step_fused(li, qg, k_u, k_r, v, out, SCALE)
            else:
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


@pytest.mark.parametrize("fused", [False, True])
def test_full_decode_loop_two_layers_three_events(cuda_ops, oracle, monkeypatch, fused):
    """The loop the reference's own measurement runs (README.md:27-47): a 56-token prompt plus 512
    decode steps, 8 splits, here over two attention layers with their own tables, through
    khq_step and through khq_step_fused.  Compression events must fire at tokens 256, 384 and 512
    on every layer, the code words of all 384 compressed tokens must be bit-identical to those the
    same state machine writes through the oracle backend, and the outputs at steps around every
    event and at the end must agree with it."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    n_steps = 56 + 512
    case = cases.make_case(cases.synth.seed_for(1, 3), n_steps, "calib", layer_id=3)
    other = cases.make_case(cases.synth.seed_for(1, 7), 64, "n01_idrot", layer_id=7)
    layers = [3, 7]
    collect = {0, 55, 56, 255, 256, 257, 383, 384, 511, 512, 567}
    res = {}
    for name, ops, device in (("gpu", cuda_ops, "cuda"), ("cpu", oracle.OracleOps(), "cpu")):
        rt = KhqRuntime(ops, device=device)
        assert rt.khq_activate([case["tables"], other["tables"]], max_seq=1024)
        res[name] = (drive(rt, torch, device, case, n_steps, layers, collect, fused=fused and name == "gpu"), rt)
    (g_out, g_rt), (c_out, c_rt) = res["gpu"], res["cpu"]
    want_events = [(li, b, w) for w, b in ((256, 128), (384, 256), (512, 384)) for li in layers]
    assert sorted((e.layer, e.boundary, e.write_pos) for e in g_rt.events) == sorted(want_events)
    assert sorted((e.layer, e.boundary, e.write_pos) for e in c_rt.events) == sorted(want_events)
    for li in layers:
        assert g_rt.layers[li].boundary == c_rt.layers[li].boundary == 384
        assert g_rt.layers[li].write_pos == c_rt.layers[li].write_pos == n_steps
        for key in ("kmask", "kpay", "knorm", "krn", "vpay", "vnorm", "vrn", "vsm"):
            n = 384 * H_KV * {"kmask": 16, "kpay": 40, "vpay": 104, "vsm": 4}.get(key, 1)
            a = g_rt.layers[li].t[key].cpu()[:n].view(torch.uint8)
            b = c_rt.layers[li].t[key][:n].view(torch.uint8)
            assert torch.equal(a, b), f"layer {li}: code words differ in {key}"
    assert len(g_out) == len(collect) * len(layers)
    for k in sorted(g_out):
        ok, mx, exc = cases.attention_close(g_out[k], c_out[k])
        assert ok, f"layer/step {k}: max abs {mx:.3e} excess {exc:.3e}"


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


@pytest.mark.parametrize("T", [300, 511, 640])
def test_prefill_leaves_the_per_token_state(cuda_ops, oracle, T, monkeypatch):
    """khq_prefill (one attention launch + two compress launches) must leave the KHQ state that T
    per-token khq_step calls leave: same boundary/write_pos, bit-identical code words, identical
    rings; then one more decode step on top of either state gives the same output."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    case = cases.make_case(8800 + T, T + 1, "calib", layer_id=3)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    ku, kr, v = dev(case["k_unroped"]), dev(case["k_roped"]), dev(case["v"])
    rng = np.random.default_rng(1)
    qg_all = dev(rng.standard_normal((T, H_Q, 2 * D)).astype(np.float16))
    # per-token path
    a = KhqRuntime(cuda_ops, device="cuda")
    assert a.khq_activate([case["tables"]], max_seq=1024)
    a.khq_init_layer(3, H_Q, H_KV, D)
    out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    for t in range(T):
        a.khq_capture_unroped(3, ku[t])
        assert a.khq_step(3, qg_all[t].reshape(-1), kr[t], v[t], out, SCALE)
    # prompt path
    b = KhqRuntime(cuda_ops, device="cuda")
    assert b.khq_activate([case["tables"]], max_seq=1024)
    b.khq_init_layer(3, H_Q, H_KV, D)
    out_p = torch.zeros(T, H_Q, D, dtype=torch.float16, device="cuda")
    assert b.khq_prefill(3, qg_all, ku[:T], kr[:T], v[:T], out_p, SCALE)
    La, Lb = a.layers[3], b.layers[3]
    assert (La.boundary, La.write_pos) == (Lb.boundary, Lb.write_pos)
    assert [(e.boundary, e.write_pos) for e in a.events] == [(e.boundary, e.write_pos) for e in b.events]
    rows = La.boundary * H_KV
    for key, w in (("kmask", 16), ("kpay", 40), ("knorm", 1), ("krn", 1), ("vpay", 104), ("vnorm", 1), ("vrn", 1), ("vsm", 4)):
        assert torch.equal(La.t[key][:rows * w].view(torch.uint8), Lb.t[key][:rows * w].view(torch.uint8)), key
    live = [(t % 256) for t in range(La.boundary, T)]
    for ring in ("ring_k", "ring_v", "ring_u"):
        assert torch.equal(La.t[ring].view(256, -1)[live], Lb.t[ring].view(256, -1)[live]), ring
    # prompt rows: exact causal attention == oracle
    ref = oracle.gqa_prefill(qg_all.cpu().numpy(), case["k_roped"][:T], case["v"][:T], T, H_Q, H_KV, D, SCALE)
    ok, mx, exc = cases.attention_close(out_p.float().cpu().numpy()[-5:], ref[-5:])
    assert ok, (mx, exc)
    # one more token on both states
    qn = dev(cases.synth.make_q_gate(rng, T)).reshape(-1)
    oa = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    ob = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    for rt, o in ((a, oa), (b, ob)):
        rt.khq_capture_unroped(3, ku[T])
        assert rt.khq_step(3, qn, kr[T], v[T], o, SCALE)
    torch.cuda.synchronize()
    assert torch.equal(oa, ob)


def test_checkpoint_resume_is_bit_identical(cuda_ops, tmp_path, monkeypatch):
    """Decode 300 steps, checkpoint the KHQ state, restore it into a fresh runtime and continue
    both for 120 more steps (across the compression event at write_pos 384): every output and every
    code word must be bit-identical -- the state file holds all that the path carries from step to
    step."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    n_a, n_b = 300, 120
    case = cases.make_case(cases.synth.seed_for(1, 11), n_a + n_b, "calib", layer_id=3)

    def step(rt, t):
        qg = torch.from_numpy(cases.synth.make_q_gate(np.random.default_rng(7000 + t), t)).cuda()
        out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
        rt.khq_capture_unroped(3, torch.from_numpy(case["k_unroped"][t]).cuda())
        assert rt.khq_step(3, qg, torch.from_numpy(case["k_roped"][t]).cuda(), torch.from_numpy(case["v"][t]).cuda(), out, SCALE)
        return out.cpu()

    rt = KhqRuntime(cuda_ops, device="cuda")
    assert rt.khq_activate([case["tables"]], max_seq=1024)
    rt.khq_init_layer(3, H_Q, H_KV, D)
    for t in range(n_a):
        step(rt, t)
    path = tmp_path / "khq_state.bin"
    assert rt.khq_save_state(path) == 1
    rt2 = KhqRuntime(cuda_ops, device="cuda")
    assert rt2.khq_activate([case["tables"]], max_seq=1024)
    assert rt2.khq_load_state(path) == 1
    assert (rt2.layers[3].boundary, rt2.layers[3].write_pos) == (rt.layers[3].boundary, rt.layers[3].write_pos) == (128, 300)
    for t in range(n_a, n_a + n_b):
        a, b = step(rt, t), step(rt2, t)
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), f"step {t}"
    assert rt.layers[3].boundary == rt2.layers[3].boundary == 256
    rows = 256 * H_KV
    for key, rb in KhqRuntime._STATE_ROW_ARRAYS:
        a, b = rt.layers[3].t[key].view(torch.uint8)[:rows * rb], rt2.layers[3].t[key].view(torch.uint8)[:rows * rb]
        assert torch.equal(a, b), key


def test_fused_step_matches_the_classic_sequence(cuda_ops, monkeypatch):
    """khq_step_fused (launch_khq_decode_step_fp16: appends + both regions + merge + gate in one
    call) against khq_capture_unroped + khq_step on the same inputs, 420 steps across three
    compression events: outputs within the attention bar (the merge is fused into the window kernel,
    so the last fp32 roundings differ), rings and code words bit-identical, same bookkeeping."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    monkeypatch.setenv("BONSAI_KHQ_SPLITS", "8")
    n = 420
    case = cases.make_case(cases.synth.seed_for(1, 21), n, "calib", layer_id=3)
    rts = []
    for _ in range(2):
        rt = KhqRuntime(cuda_ops, device="cuda")
        assert rt.khq_activate([case["tables"]], max_seq=1024)
        rt.khq_init_layer(3, H_Q, H_KV, D)
        rts.append(rt)
    classic, fused = rts
    worst = 0.0
    for t in range(n):
        qg = torch.from_numpy(cases.synth.make_q_gate(np.random.default_rng(9000 + t), t)).cuda()
        ku = torch.from_numpy(case["k_unroped"][t]).cuda()
        kr = torch.from_numpy(case["k_roped"][t]).cuda()
        v = torch.from_numpy(case["v"][t]).cuda()
        oa = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
        ob = torch.full((H_Q * D,), float("nan"), dtype=torch.float16, device="cuda")
        classic.khq_capture_unroped(3, ku)
        assert classic.khq_step(3, qg, kr, v, oa, SCALE)
        assert fused.khq_step_fused(3, qg, ku, kr, v, ob, SCALE)
        if t % 7 == 0 or t > 380:
            torch.cuda.synchronize()
            ok, mx, exc = cases.attention_close(ob.float().cpu().numpy(), oa.float().cpu().numpy())
            assert ok, f"step {t}: max abs {mx:.3e}, excess {exc:.3e}"
            worst = max(worst, mx)
    torch.cuda.synchronize()
    A, B = classic.layers[3], fused.layers[3]
    assert (A.boundary, A.write_pos) == (B.boundary, B.write_pos) == (256, n)
    assert [(e.boundary, e.write_pos) for e in classic.events] == [(e.boundary, e.write_pos) for e in fused.events]
    for key in ("ring_k", "ring_v", "ring_u", "kmask", "kpay", "knorm", "krn", "vpay", "vnorm", "vrn", "vsm"):
        assert torch.equal(A.t[key].view(torch.uint8), B.t[key].view(torch.uint8)), key
    assert cuda_ops.lib.khq_b200_device_status() == 0
    print(f"fused step: worst |difference| to the classic sequence {worst:.2e}")


def test_decode_step_error_codes(cuda_ops):
    fn = cuda_ops.lib.launch_khq_decode_step_fp16
    z = [0] * 25
    assert fn(*z, 0, 0, 1, 256, 1, 0.0625, 1.0, 1.0, 1e7, 0) == -100          # null pointers
    a = [16] * 25
    assert fn(*a, 0, 0, 0, 256, 1, 0.0625, 1.0, 1.0, 1e7, 0) == -100          # empty window
    assert fn(*a, 0, 0, 300, 256, 1, 0.0625, 1.0, 1.0, 1e7, 0) == -103        # window larger than the ring
    b = list(a)
    b[1] = 8
    assert fn(*b, 0, 0, 1, 256, 1, 0.0625, 1.0, 1.0, 1e7, 0) == -104          # misaligned token
