"""CPU-only tests of the oracle: self-consistency, the reference's own fixtures for the fp16-KV
attention and RoPE, and the golden vectors produced by the reference's CUDA kernels."""
from pathlib import Path

import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE
from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth

ROOT = Path(__file__).resolve().parent.parent
GOLD = ROOT / "tests" / "golden"


def test_fwht_involution():
    x = np.random.default_rng(0).standard_normal((3, D)).astype(np.float32)
    assert np.allclose(synth.fwht(synth.fwht(x)), 256.0 * x, rtol=1e-5, atol=1e-4)


def test_compress_contract(oracle):
    case = cases.make_case(11, 16, "calib")
    kv = cases.compress_with(oracle.compress, case, 16)
    assert kv["k_payload"].shape == (64, 40) and kv["v_payload"].shape == (64, 104)
    assert (kv["k_payload"][:, 36] == 2).all() and (kv["k_payload"][:, 37:] == 0).all()
    # stored norm is the fp16 of the row's L2 norm
    nrm = np.sqrt((case["k_unroped"].reshape(-1, D).astype(np.float64) ** 2).sum(1))
    assert np.allclose(kv["k_norms"].astype(np.float64), nrm, rtol=1e-3)
    # at most 50 outlier symbols per row, and the sign/residual fields beyond them are zero
    m = kv["k_mask"]
    n_out = np.array([sum(bin(int(w) & (int(w) >> 1) & 0x55555555).count("1") for w in row) for row in m])
    assert n_out.max() <= 50 and n_out.min() > 0
    assert oracle.compress(case["v"].reshape(-1, D), case["f16"]["d_v"], case["f16"]["rotor_v"],
                           case["f16"]["cents_v"], case["f16"]["vq"], 0, 1.95, 1.0, True)["rc"] == -100
    assert oracle.compress(case["v"].reshape(-1, D), case["f16"]["d_v"], case["f16"]["rotor_v"],
                           case["f16"]["cents_v"], case["f16"]["vq"], 4, 1.95, 1.0, True, d=128)["rc"] == -100


@pytest.mark.parametrize("variant", ["calib", "n01_idrot"])
def test_round_trip_error_is_bounded(oracle, variant):
    case = cases.make_case(12, 32, variant)
    f, tb = case["f16"], case["tables"]
    kv = cases.compress_with(oracle.compress, case, 32)
    ek, ev = [], []
    for r in range(0, 128, 5):
        kh = oracle.decode_k(kv["k_payload"][r], kv["k_mask"][r], kv["k_norms"][r], kv["k_r_norms"][r],
                             f["cents_k"], f["rotor_k"], f["d_k"], tb.alpha_k)
        x = case["k_unroped"].reshape(-1, D)[r].astype(np.float64)
        ek.append(np.linalg.norm(kh - x) / np.linalg.norm(x))
        vh = oracle.decode_v(kv["v_payload"][r], kv["v_norms"][r], kv["v_r_norms"][r],
                             float(kv["v_shared_meta"][r].view(np.float32)[0]), f["cents_v"], f["vq"],
                             f["rotor_v"], f["d_v"], tb.alpha_v)
        xv = case["v"].reshape(-1, D)[r].astype(np.float64)
        ev.append(np.linalg.norm(vh - xv) / np.linalg.norm(xv))
    assert np.mean(ek) < 0.4, np.mean(ek)          # 2-bit + outliers: ~0.28
    if variant == "calib":
        assert np.mean(ev) < 0.35, np.mean(ev)     # codebook at data scale: ~0.22


def _dense_two_region(oracle, case, kv, c_len, win_len):
    """softmax over [decoded compressed K/V ; raw window K/V] in float64, gate applied."""
    f, tb = case["f16"], case["tables"]
    freq = np.array([np.float32(1e7) ** np.float32(-2.0 * m / 64.0) for m in range(32)], np.float64)
    K = np.zeros((c_len + win_len, H_KV, D))
    V = np.zeros((c_len + win_len, H_KV, D))
    for s in range(c_len):
        for g in range(H_KV):
            r = s * H_KV + g
            kh = oracle.decode_k(kv["k_payload"][r], kv["k_mask"][r], kv["k_norms"][r], kv["k_r_norms"][r],
                                 f["cents_k"], f["rotor_k"], f["d_k"], tb.alpha_k)
            th = s * freq
            a, b = kh[:32].copy(), kh[32:64].copy()
            kh[:32], kh[32:64] = a * np.cos(th) - b * np.sin(th), a * np.sin(th) + b * np.cos(th)
            K[s, g] = kh
            V[s, g] = oracle.decode_v(kv["v_payload"][r], kv["v_norms"][r], kv["v_r_norms"][r],
                                      float(kv["v_shared_meta"][r].view(np.float32)[0]), f["cents_v"], f["vq"],
                                      f["rotor_v"], f["d_v"], tb.alpha_v)
    K[c_len:] = case["k_roped"][c_len:c_len + win_len]
    V[c_len:] = case["v"][c_len:c_len + win_len]
    qg = case["q_gate"].astype(np.float64)
    out = np.zeros((H_Q, D))
    for h in range(H_Q):
        g = h // 6
        s = (K[:, g] @ qg[h, :D]) * SCALE
        p = np.exp(s - s.max())
        out[h] = (p @ V[:, g]) / (p.sum() + 1e-8 * np.exp(-s.max()) * 0) * (1 / (1 + np.exp(-qg[h, D:])))
    return out


def test_two_region_merge_equals_one_softmax(oracle):
    c_len, win_len = 24, 9
    case = cases.make_case(13, c_len + win_len, "calib")
    kv = cases.compress_with(oracle.compress, case, c_len)
    ops = oracle.OracleOps()
    f, tb = case["f16"], case["tables"]
    ac = np.zeros((H_Q, 258), np.float32)
    ap = np.zeros((H_Q, 4, 258), np.float32)
    ops.attn(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
             kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"],
             f["rotor_v"], f["d_k"], f["d_v"], ac, ap, H_Q, H_Q, 1, c_len, c_len, 6, SCALE, tb.alpha_k, tb.alpha_v,
             1e7, 0, 4)
    ring_k = np.zeros((256, H_KV, D), np.float16)
    ring_v = np.zeros((256, H_KV, D), np.float16)
    ws = c_len % 256
    for s in range(win_len):
        ring_k[(ws + s) % 256] = case["k_roped"][c_len + s]
        ring_v[(ws + s) % 256] = case["v"][c_len + s]
    aw = np.zeros((H_Q, 258), np.float32)
    ops.window_attn(case["q_gate"], ring_k, ring_v, aw, ws, win_len, 256, H_Q, H_KV, D, SCALE)
    out = np.zeros((H_Q, D), np.float16)
    ops.merge_gate(ac, aw, case["q_gate"], out, H_Q, D, True, True)
    dense = _dense_two_region(oracle, case, kv, c_len, win_len)
    ok, mx, exc = cases.attention_close(out.astype(np.float64), dense)
    assert ok, (mx, exc)
    # split-K (4 splits) == single pass
    ac1 = np.zeros((H_Q, 258), np.float32)
    ops.attn(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
             kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"],
             f["rotor_v"], f["d_k"], f["d_v"], ac1, None, H_Q, H_Q, 1, c_len, c_len, 6, SCALE, tb.alpha_k,
             tb.alpha_v, 1e7, 0, 1)
    assert np.allclose(cases.normalised(ac), cases.normalised(ac1), rtol=1e-5, atol=1e-6)
    with pytest.raises(oracle.OracleLaunchError):  # splits > 1 without a partial buffer: -101
        ops.attn(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"],
                 kv["k_norms"], kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"],
                 f["vq"], f["rotor_k"], f["rotor_v"], f["d_k"], f["d_v"], ac1, None, H_Q, H_Q, 1, c_len, c_len, 6,
                 SCALE, tb.alpha_k, tb.alpha_v, 1e7, 0, 2)


# ---- the reference's own fixtures for the fp16-KV attention (tests/test_gqa_attention_gpu.mojo) ----
@pytest.mark.parametrize("H_q,H_kv,seq,max_seq", [(24, 4, 8, 16), (4, 2, 16, 16), (4, 2, 1, 16)])
def test_gqa_attention_on_reference_fixtures(oracle, H_q, H_kv, seq, max_seq):
    d = 256
    i = np.arange(H_q * 2 * d, dtype=np.int64)
    qg = (((i * 7919 + 1013) % 2000).astype(np.float32) * np.float32(0.001) - np.float32(1.0)).astype(np.float32)
    j = np.arange(max_seq * H_kv * d, dtype=np.int64)
    k = (((j * 6271 + 5003) % 2000).astype(np.float32) * np.float32(0.001) - np.float32(1.0)).astype(np.float32)
    v = (((j * 4931 + 7919) % 2000).astype(np.float32) * np.float32(0.002) - np.float32(2.0)).astype(np.float32)
    got = oracle.gqa_attention_f32(qg, k, v, seq, H_q, H_kv, d, 1.0 / np.sqrt(d))
    # independent float64 restatement of the test's FP64 reference, 1/(Z+1e-9) denominator included
    Q = qg.reshape(H_q, 2 * d).astype(np.float64)
    K = k.reshape(max_seq, H_kv, d).astype(np.float64)[:seq]
    V = v.reshape(max_seq, H_kv, d).astype(np.float64)[:seq]
    want = np.zeros((H_q, d))
    for h in range(H_q):
        g = h // (H_q // H_kv)
        s = K[:, g] @ Q[h, :d] / np.sqrt(d)
        e = np.exp(s - s.max())
        want[h] = (e / (e.sum() + 1e-9)) @ V[:, g] / (1 + np.exp(-Q[h, d:]))
    assert np.abs(got - want).max() / (np.abs(want).max() + 1e-12) <= 2e-3 * 1e-6  # same math, fp64


# ---- the reference's RoPE fixtures (tests/test_rope_gpu.mojo:132-160) ----
@pytest.mark.parametrize("heads,stride,pos", [(24, 512, 0), (24, 512, 1), (24, 512, 12345), (24, 512, 130000),
                                              (4, 256, 777), (4, 256, 262143)])
def test_rope_on_reference_fixtures(oracle, heads, stride, pos):
    total = heads * stride
    jx = np.arange(total, dtype=np.int64)
    x = (((jx * 7919 + 1013) % 2000).astype(np.float32) * np.float32(0.002) - np.float32(2.0)).astype(np.float16)
    got = oracle.partial_rope(x.copy(), heads, 256, 64, pos, 1e7, stride).reshape(heads, stride)
    x2 = x.reshape(heads, stride)
    want = x2.copy()
    want[:, :256] = synth.partial_rope(x2[:, :256], np.full((heads,), pos))
    assert np.abs(got[:, :64].astype(np.float32) - want[:, :64].astype(np.float32)).max() <= 0.05
    assert np.array_equal(got[:, 64:].view(np.uint16), x2[:, 64:].view(np.uint16))  # untouched region bitwise


def test_rope_small_case(oracle):
    # head_dim 8, rotary 4, pos 7, theta 1e4: pairs (0,2) and (1,3)
    x = np.array([1, 2, 3, 4, 5, 6, 7, 8], np.float16)
    got = oracle.partial_rope(x.copy(), 1, 8, 4, 7, 10000.0, 0).astype(np.float64)
    f = np.array([1.0, 10000.0 ** -0.5])
    c, s = np.cos(7 * f), np.sin(7 * f)
    want = np.array([1 * c[0] - 3 * s[0], 2 * c[1] - 4 * s[1], 1 * s[0] + 3 * c[0], 2 * s[1] + 4 * c[1], 5, 6, 7, 8])
    assert np.abs(got - want).max() < 5e-3


# ---- golden vectors produced by the reference's CUDA kernels on a B200 ----
def _golden(name):
    p = GOLD / name
    if not p.exists():
        pytest.skip(f"{name} not generated yet (tests/golden/make_golden_gpu.py)")
    return np.load(p)


@pytest.mark.parametrize("variant", list(cases.VARIANTS))
def test_oracle_compress_matches_reference_kernel_golden(oracle, variant):
    g = _golden(f"compress_{variant}.npz")
    rows = 96 * H_KV
    ck = oracle.compress(g["k_unroped"].reshape(-1, D), g["t_d_k"], g["t_rotor_k"], g["t_cents_k"], g["t_cents_k"],
                         rows, float(g["ts_k"]), float(g["alpha_k"]), False)
    cv = oracle.compress(g["v"].reshape(-1, D), g["t_d_v"], g["t_rotor_v"], g["t_cents_v"], g["t_vq"], rows,
                         float(g["ts_v"]), float(g["alpha_v"]), True)
    pairs = [("k_mask", ck["mask"]), ("k_payload", ck["payload"]), ("k_norms", ck["norms"]),
             ("k_r_norms", ck["r_norms"]), ("v_payload", cv["payload"]), ("v_norms", cv["norms"]),
             ("v_r_norms", cv["r_norms"]), ("v_shared_meta", cv["shared_meta"])]
    bad = {k: int((np.asarray(a).reshape(rows, -1).view(np.uint8) != g[k].reshape(rows, -1).view(np.uint8)).any(1).sum())
           for k, a in pairs}
    assert all(v == 0 for v in bad.values()), f"rows differing from the reference kernel: {bad} (ties {cv['near_ties']})"


@pytest.mark.parametrize("variant", list(cases.VARIANTS))
def test_oracle_decode_matches_reference_kernel_golden(oracle, variant):
    g = _golden(f"decode_{variant}.npz")
    kv = {k: g[k] for k in ("k_mask", "k_payload", "k_norms", "k_r_norms", "v_payload", "v_norms", "v_r_norms",
                            "v_shared_meta")}
    f = {k[2:]: g[k] for k in g.files if k.startswith("t_")}
    ops = oracle.OracleOps()
    ak, av = float(g["alpha_k"]), float(g["alpha_v"])
    for sp in (1, 8):
        ac = np.zeros((H_Q, 258), np.float32)
        ap = np.zeros((H_Q, sp, 258), np.float32)
        ops.attn(g["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
                 kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"],
                 f["rotor_v"], f["d_k"], f["d_v"], ac, ap, H_Q, H_Q, 1, 384, 384, 6, SCALE, ak, av, 1e7, 0, sp)
        ok, mx, exc = cases.attention_close(cases.normalised(ac), cases.normalised(g[f"attn_c_s{sp}"]))
        assert ok, (sp, mx, exc)
        lse_o = ac[:, D] + np.log(ac[:, D + 1])
        lse_g = g[f"attn_c_s{sp}"][:, D] + np.log(g[f"attn_c_s{sp}"][:, D + 1])
        assert np.abs(lse_o - lse_g).max() < 5e-3
    aw = np.zeros((H_Q, 258), np.float32)
    ops.window_attn(g["q_gate"], g["ring_k"], g["ring_v"], aw, 128, 128, 256, H_Q, H_KV, D, SCALE)
    ok, mx, exc = cases.attention_close(cases.normalised(aw), cases.normalised(g["attn_w"]))
    assert ok, (mx, exc)
    out = np.zeros((H_Q, D), np.float16)
    ops.merge_gate(ac, aw, g["q_gate"], out, H_Q, D, True, True)
    ok, mx, exc = cases.attention_close(out.astype(np.float32), g["out"].astype(np.float32))
    assert ok, (mx, exc)


def test_oracle_far_position_vs_reference_kernel_golden(oracle):
    """At position 1e5 the reference forms its RoPE angle in fp32 (ulp 0.0078 rad), the oracle in
    double; the two agree to the looser bound that rounding allows."""
    g = _golden("decode_farpos.npz")
    kv = {k: g[k] for k in ("k_mask", "k_payload", "k_norms", "k_r_norms", "v_payload", "v_norms", "v_r_norms",
                            "v_shared_meta")}
    f = {k[2:]: g[k] for k in g.files if k.startswith("t_")}
    got = oracle.attn_partial(g["q_gate"], kv, dict(cents_k=f["cents_k"], cents_v=f["cents_v"], vq=f["vq"],
                                                    rotor_k=f["rotor_k"], rotor_v=f["rotor_v"], d_k=f["d_k"],
                                                    d_v=f["d_v"]), H_Q, 6, SCALE, float(g["alpha_k"]),
                              float(g["alpha_v"]), 1e7, 100000, 0, 64)
    ok, mx, exc = cases.attention_close(cases.normalised(got), cases.normalised(g["attn_c_s1"]), atol=2e-2, rtol=5e-2)
    assert ok, (mx, exc)


def test_head_rmsnorm_matches_float64_formula(oracle):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((24, 512)) * 2).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    got = oracle.head_rmsnorm(x.copy(), 24, 256, 512, w, 1e-6)
    q = x[:, :256].astype(np.float64)
    want = q / np.sqrt((q * q).mean(1, keepdims=True) + 1e-6) * w
    assert np.abs(got[:, :256].astype(np.float64) - want).max() <= 2e-3 * np.abs(want).max()
    assert np.array_equal(got[:, 256:].view(np.uint16), x[:, 256:].view(np.uint16))  # gate half untouched
