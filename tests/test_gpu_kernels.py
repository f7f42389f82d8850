"""GPU parity tests: every kernel is called through the C ABI and checked against the CPU oracle
(and, where oracle/_ref was built, against the reference's own CUDA kernels on the same GPU).

Bars: KHQ code words bit-exact (exact-distance VQ ties counted and reported); attention
outputs within |err| <= 2e-3 + 1e-2*|ref| of the oracle.
"""
import ctypes
from pathlib import Path

import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF_SO = ROOT / "oracle" / "_ref" / "libbonsai_ref_sm100a.so"


def _torch():
    import torch

    return torch


def dev(a):
    torch = _torch()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_compress(ops, x, d_vec, rotor, cents, vq, rows, ts, alpha, is_v, poison=True):
    """The package's compress launch with the oracle's calling convention (numpy in/out)."""
    torch = _torch()
    pay = 104 if is_v else 40
    fill = 0xCD if poison else 0
    o_mask = torch.full((rows * 16,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    o_n = torch.zeros(rows, dtype=torch.float16, device="cuda")
    o_rn = torch.zeros(rows, dtype=torch.float16, device="cuda")
    o_pay = torch.full((rows * pay,), fill, dtype=torch.uint8, device="cuda")
    o_sm = torch.full((rows * 4,), fill, dtype=torch.uint8, device="cuda")
    t = [dev(a) for a in (x, d_vec, rotor, cents, vq)]
    ops.compress(*t, o_mask, o_n, o_rn, o_pay, o_sm, rows, D, ts, alpha, is_v)
    torch.cuda.synchronize()
    return dict(mask=o_mask.cpu().numpy().view(np.uint32).reshape(rows, 16), norms=o_n.cpu().numpy(),
                r_norms=o_rn.cpu().numpy(), payload=o_pay.cpu().numpy().reshape(rows, pay),
                shared_meta=o_sm.cpu().numpy().reshape(rows, 4), near_ties=0)


def _diff_rows(a, b):
    a = a.reshape(a.shape[0], -1)
    b = b.reshape(b.shape[0], -1)
    return np.nonzero((a.view(np.uint8) != b.view(np.uint8)).any(axis=1))[0]


# ------------------------------------------------------------------------------ compress
@pytest.mark.parametrize("variant", list(cases.VARIANTS))
@pytest.mark.parametrize("n_tok", [1, 96, 129])
def test_compress_bit_exact_vs_oracle(cuda_ops, oracle, variant, n_tok):
    case = cases.make_case(100 + n_tok, n_tok, variant)
    ref = cases.compress_with(oracle.compress, case, n_tok)
    got = cases.compress_with(lambda *a: gpu_compress(cuda_ops, *a), case, n_tok)
    bad = {}
    for key in ("k_mask", "k_payload", "k_norms", "k_r_norms", "v_payload", "v_norms", "v_r_norms",
                "v_shared_meta"):
        rows = _diff_rows(np.asarray(got[key]), np.asarray(ref[key]))
        if len(rows):
            bad[key] = rows[:8].tolist()
    # exact-distance VQ ties may legitimately resolve either way; report them
    print(f"compress {variant} n_tok={n_tok}: exact-distance VQ ties = {ref['near_ties']}")
    if ref["near_ties"] == 0:
        assert not bad, f"code words differ from the oracle in rows {bad}"
    else:
        assert set(bad) <= {"v_payload", "v_r_norms"}, bad


def test_compress_k_leaves_mask_alone_for_v_and_zeroes_meta(cuda_ops):
    case = cases.make_case(321, 8, "calib")
    tb, f = case["tables"], case["f16"]
    rows = 8 * H_KV
    k = gpu_compress(cuda_ops, case["k_unroped"].reshape(-1, D), f["d_k"], f["rotor_k"], f["cents_k"],
                     f["cents_k"], rows, tb.ts_k, tb.alpha_k, False)
    assert (k["shared_meta"] == 0).all()
    assert (k["payload"][:, 36] == 2).all() and (k["payload"][:, 37:] == 0).all()
    v = gpu_compress(cuda_ops, case["v"].reshape(-1, D), f["d_v"], f["rotor_v"], f["cents_v"], f["vq"], rows,
                     tb.ts_v, tb.alpha_v, True)
    assert (v["mask"] == 0x5A5A5A5A).all(), "the V launch must not write the K mask"


def test_compress_error_codes(cuda_ops):
    lib = cuda_ops.lib
    assert lib.launch_khq_compress_fp16(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 256, 1.0, 1.0, 0, 0) == -100
    assert lib.launch_khq_compress_fp16(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 128, 1.0, 1.0, 0, 0) == -100


@pytest.mark.skipif(not REF_SO.exists(), reason="reference library was not built")
@pytest.mark.parametrize("variant", list(cases.VARIANTS))
def test_compress_bit_exact_vs_reference_kernel(cuda_ops, oracle, variant):
    """Three-way: reference CUDA kernel == this library == CPU oracle, byte for byte."""
    from golden import make_golden_gpu as mg

    so = mg.load_ref()
    case = cases.make_case(555, 128, variant)
    ref = cases.compress_with(lambda *a: mg.ref_compress(so, *a), case, 128)
    got = cases.compress_with(lambda *a: gpu_compress(cuda_ops, *a), case, 128)
    ora = cases.compress_with(oracle.compress, case, 128)
    report = {}
    for key in ("k_mask", "k_payload", "k_norms", "k_r_norms", "v_payload", "v_norms", "v_r_norms",
                "v_shared_meta"):
        report[key] = (len(_diff_rows(np.asarray(got[key]), np.asarray(ref[key]))),
                       len(_diff_rows(np.asarray(ora[key]), np.asarray(ref[key]))))
    print(f"rows differing from the reference kernel (library, oracle) {variant}: {report}; "
          f"exact ties {ora['near_ties']}")
    assert all(v == (0, 0) for v in report.values()), report


# ------------------------------------------------------------------------------ compressed attention
def run_attn(ops, case, kv, c_len, splits, start_pos=0):
    torch = _torch()
    f, tb = case["f16"], case["tables"]
    arr = {k: dev(v) for k, v in kv.items() if k != "near_ties"}
    tab = {k: dev(v) for k, v in f.items()}
    q = dev(case["q_gate"])
    oa = torch.full((H_Q * 258,), float("nan"), dtype=torch.float32, device="cuda")
    op = torch.full((H_Q * max(splits, 1) * 258,), float("nan"), dtype=torch.float32, device="cuda")
    ops.attn(q, arr["k_payload"], arr["v_payload"], arr["v_shared_meta"], arr["k_mask"], arr["k_norms"],
             arr["k_r_norms"], arr["v_norms"], arr["v_r_norms"], tab["cents_k"], tab["cents_v"], tab["vq"],
             tab["rotor_k"], tab["rotor_v"], tab["d_k"], tab["d_v"], oa, op, H_Q, H_Q, 1, c_len, c_len, 6, SCALE,
             tb.alpha_k, tb.alpha_v, 1e7, start_pos, splits)
    torch.cuda.synchronize()
    return oa.cpu().numpy().reshape(H_Q, 258), op.cpu().numpy().reshape(H_Q, max(splits, 1), 258)


def check_partial(got, ref, what):
    """Unnormalised partials from different accumulation orders are compared through the
    order-independent quantities: acc/sum_exp and the log-sum-exp max + log(sum)."""
    ok, mx, exc = cases.attention_close(cases.normalised(got), cases.normalised(ref))
    lse_g = got[..., D] + np.log(np.maximum(got[..., D + 1], 1e-30))
    lse_r = ref[..., D] + np.log(np.maximum(ref[..., D + 1], 1e-30))
    lse_err = float(np.abs(lse_g - lse_r).max())
    assert ok, f"{what}: max abs err {mx:.3e}, worst excess over tolerance {exc:.3e}"
    assert lse_err < 5e-3, f"{what}: log-sum-exp differs by {lse_err:.3e}"
    return mx, lse_err


@pytest.mark.parametrize("variant", list(cases.VARIANTS))
@pytest.mark.parametrize("c_len,splits", [(1, 1), (7, 1), (8, 8), (127, 4), (128, 16), (129, 32), (384, 1),
                                          (384, 8), (50, 32), (1000, 3), (4096, 2), (2501, 1)])  # the last two take the tensor-core path
def test_attn_compressed_vs_oracle(cuda_ops, oracle, variant, c_len, splits):
    case = cases.make_case(900 + c_len, c_len + 1, variant)
    kv = cases.compress_with(oracle.compress, case, c_len)
    got, got_p = run_attn(cuda_ops, case, kv, c_len, splits)
    ref = np.zeros((H_Q, 258), np.float32)
    ref_p = np.zeros((H_Q, max(splits, 1), 258), np.float32)
    rc = oracle.attn_launch(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"],
                            kv["k_norms"], kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], case["f16"]["cents_k"],
                            case["f16"]["cents_v"], case["f16"]["vq"], case["f16"]["rotor_k"],
                            case["f16"]["rotor_v"], case["f16"]["d_k"], case["f16"]["d_v"], ref, ref_p, H_Q, H_Q,
                            c_len, 6, SCALE, case["tables"].alpha_k, case["tables"].alpha_v, 1e7, 0, splits)
    assert rc == 0
    mx, lse = check_partial(got, ref, f"{variant} c_len={c_len} splits={splits}")
    if splits > 1:
        # per-split partials sit in the reference's layout (query, split, 258); empty splits hold
        # (0, -1e20, 0)
        per = -(-c_len // splits)
        for sp in range(splits):
            lo = min(sp * per, c_len)
            hi = min(lo + per, c_len)
            if hi <= lo:
                assert (got_p[:, sp, :D] == 0).all() and (got_p[:, sp, D] == np.float32(-1e20)).all() \
                    and (got_p[:, sp, D + 1] == 0).all()
            else:
                check_partial(got_p[:, sp], ref_p[:, sp], f"split {sp}")
    print(f"attn {variant} c_len={c_len} splits={splits}: max|err|={mx:.2e} lse err={lse:.2e}")
    assert cuda_ops.lib.khq_b200_device_status() == 0


def test_attn_start_pos_far(cuda_ops, oracle):
    """Context-parallel style call: a slice of the compressed region at a large absolute position."""
    case = cases.make_case(4242, 65, "calib", q_pos=131072 + 64)
    kv = cases.compress_with(oracle.compress, case, 64)
    got, _ = run_attn(cuda_ops, case, kv, 64, 1, start_pos=131072)
    ref = oracle.attn_partial(case["q_gate"], kv, cases.tables_dict(case["f16"]), H_Q, 6, SCALE,
                              case["tables"].alpha_k, case["tables"].alpha_v, 1e7, 131072, 0, 64)
    check_partial(got, ref, "start_pos=131072")


def test_attn_error_codes(cuda_ops):
    lib = cuda_ops.lib
    z = [0] * 18
    assert lib.launch_khq_attn_fp16(*z, 0, 24, 1, 8, 8, 6, 0.0625, 1.0, 1.0, 1e7, 0, 1, 0) == -100
    assert lib.launch_khq_attn_fp16(*z, 24, 24, 1, 0, 0, 6, 0.0625, 1.0, 1.0, 1e7, 0, 1, 0) == -100
    assert lib.launch_khq_attn_fp16(*z, 24, 24, 1, 8, 8, 6, 0.0625, 1.0, 1.0, 1e7, 0, 4, 0) == -101
    assert lib.launch_khq_attn_fp16(*z, 8, 8, 1, 8, 8, 2, 0.0625, 1.0, 1.0, 1e7, 0, 1, 0) == -103


# ------------------------------------------------------------------------------ window + merge
def build_ring(case, first_tok, win_start, win_len):
    ring_k = np.zeros((256, H_KV, D), np.float16)
    ring_v = np.zeros((256, H_KV, D), np.float16)
    for s in range(win_len):
        slot = (win_start + s) % 256
        ring_k[slot] = case["k_roped"][first_tok + s]
        ring_v[slot] = case["v"][first_tok + s]
    return ring_k, ring_v


@pytest.mark.parametrize("win_start,win_len", [(0, 1), (128, 128), (0, 255), (128, 256), (200, 100), (7, 13)])
def test_window_attn_vs_oracle(cuda_ops, oracle, win_start, win_len):
    torch = _torch()
    case = cases.make_case(77 + win_len, win_len, "calib")
    ring_k, ring_v = build_ring(case, 0, win_start, win_len)
    q, rk, rv = dev(case["q_gate"]), dev(ring_k), dev(ring_v)
    out = torch.full((H_Q * 258,), float("nan"), dtype=torch.float32, device="cuda")
    cuda_ops.window_attn(q, rk, rv, out, win_start, win_len, 256, H_Q, H_KV, D, SCALE)
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(H_Q, 258)
    ref = np.zeros((H_Q, 258), np.float32)
    assert oracle.window_attn(case["q_gate"], ring_k, ring_v, ref, win_start, win_len, 256, H_Q, H_KV, D, SCALE) == 0
    check_partial(got, ref, f"window start={win_start} len={win_len}")


@pytest.mark.parametrize("has_w,has_c", [(1, 1), (0, 1), (1, 0)])
def test_merge_gate_vs_oracle(cuda_ops, oracle, has_w, has_c):
    torch = _torch()
    rng = np.random.default_rng(5)
    ac = rng.standard_normal((H_Q, 258)).astype(np.float32)
    aw = rng.standard_normal((H_Q, 258)).astype(np.float32)
    ac[:, D + 1] = np.abs(ac[:, D + 1]) + 1.0
    aw[:, D + 1] = np.abs(aw[:, D + 1]) + 1.0
    ac[:, D] *= 5
    aw[:, D] *= 5
    qg = rng.standard_normal((H_Q, 2 * D)).astype(np.float16)
    out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    cuda_ops.merge_gate(dev(ac), dev(aw), dev(qg), out, H_Q, D, has_w, has_c)
    torch.cuda.synchronize()
    ref = np.zeros((H_Q, D), np.float16)
    src_c = ac if has_c else aw
    assert oracle.merge_gate(src_c, aw, qg, ref, H_Q, D, 1 if (has_w and has_c) else 0) == 0
    ok, mx, exc = cases.attention_close(out.cpu().numpy().reshape(H_Q, D).astype(np.float32), ref.astype(np.float32))
    assert ok, (mx, exc)


def test_window_and_merge_error_codes(cuda_ops):
    lib = cuda_ops.lib
    assert lib.launch_khq_window_attn_fp16(0, 0, 0, 0, 0, 0, 256, 24, 4, 256, 0.0625, 0) == -100
    assert lib.launch_khq_window_attn_fp16(0, 0, 0, 0, 0, 4, 256, 0, 4, 256, 0.0625, 0) == -100
    assert lib.launch_khq_merge_gate_fp16(0, 0, 0, 0, 0, 256, 1, 0) == -100
    assert lib.launch_khq_merge_gate_fp16(0, 0, 0, 0, 24, 0, 1, 0) == -100


# ------------------------------------------------------------------------------ whole step vs golden
@pytest.mark.parametrize("variant", list(cases.VARIANTS))
def test_decode_step_vs_reference_golden(cuda_ops, variant):
    """Config-0 shaped step on the committed fixture: same payload bytes the reference kernel
    produced, final gated output compared with the reference kernel's."""
    torch = _torch()
    path = ROOT / "tests" / "golden" / f"decode_{variant}.npz"
    if not path.exists():
        pytest.skip("golden fixture not generated yet")
    g = np.load(path)
    f16 = {k[2:]: g[k] for k in g.files if k.startswith("t_")}
    kv = {k: g[k] for k in ("k_mask", "k_payload", "k_norms", "k_r_norms", "v_payload", "v_norms", "v_r_norms",
                            "v_shared_meta")}

    class TB:
        alpha_k, alpha_v = float(g["alpha_k"]), float(g["alpha_v"])

    case = dict(f16=f16, tables=TB, q_gate=g["q_gate"])
    for sp in (1, 8):
        got, _ = run_attn(cuda_ops, case, kv, 384, sp)
        check_partial(got, g[f"attn_c_s{sp}"], f"golden compressed splits={sp}")
    q, rk, rv = dev(g["q_gate"]), dev(g["ring_k"]), dev(g["ring_v"])
    ow = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
    cuda_ops.window_attn(q, rk, rv, ow, 128, 128, 256, H_Q, H_KV, D, SCALE)
    oc = dev(run_attn(cuda_ops, case, kv, 384, 8)[0])
    out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    cuda_ops.merge_gate(oc, ow, q, out, H_Q, D, True, True)
    torch.cuda.synchronize()
    ok, mx, exc = cases.attention_close(out.cpu().numpy().reshape(H_Q, D).astype(np.float32),
                                        g["out"].astype(np.float32))
    assert ok, f"final output vs reference kernel: max abs {mx:.3e} excess {exc:.3e}"


# ------------------------------------------------------------------------------ calibration: K-static
def test_cal_kstatic_vs_oracle_and_reference_kernel(cuda_ops, oracle):
    """launch_khq_cal_kstatic_fp32 against the oracle (a few ulp: the compiler chooses which product
    of the two-term sum it fuses) and, where oracle/_ref was built, bit for bit against op 2 of the
    reference's launch_cal_op."""
    import ctypes

    torch = _torch()
    rng = np.random.default_rng(33)
    k, _ = cases.synth.make_kv(rng, 200)
    rot = cases.synth.project(k.reshape(-1, D), cases.synth.xorshift_signs(7, "k"), cases.synth.random_rotors(rng))
    rows = rot.shape[0]
    d_rot = dev(rot)
    cents = torch.zeros(4 * D, dtype=torch.float32, device="cuda")
    ts = torch.zeros(1, dtype=torch.float32, device="cuda")
    sigma = torch.zeros(D, dtype=torch.float32, device="cuda")
    cuda_ops.cal_kstatic(d_rot, rows, cents, ts, sigma)
    torch.cuda.synchronize()
    o_cents, o_ts, o_sigma = oracle.cal_kstatic(rot)
    assert np.array_equal(sigma.cpu().numpy(), o_sigma)
    assert abs(float(ts[0]) - o_ts) <= 4e-7 * o_ts
    assert np.allclose(cents.cpu().numpy().reshape(4, D), o_cents, rtol=1e-6, atol=0)
    if REF_SO.exists():
        so = ctypes.CDLL(str(REF_SO))
        so.launch_cal_op.restype = ctypes.c_int
        so.launch_cal_op.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_float] * 2 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
        r_cents = torch.zeros(4 * D, dtype=torch.float32, device="cuda")
        r_ts = torch.zeros(1, dtype=torch.float32, device="cuda")
        rc = so.launch_cal_op(2, d_rot.data_ptr(), None, None, None, None, r_cents.data_ptr(), r_ts.data_ptr(), 0.0, 0.0, rows, 0, 0, 0, None)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(r_ts.view(torch.int32), ts.view(torch.int32))
        assert torch.equal(r_cents.view(torch.int32), cents.view(torch.int32))


def test_attn_strided_positions_vs_oracle(cuda_ops, oracle):
    """launch_khq_attn_strided_fp16: a slice that holds chunks 1, 4, 7, ... of a longer context (rank 1 of
    3 under the chunk-cyclic partition, the last chunk partial) against the oracle run chunk by chunk
    at the chunks' absolute positions; both kernel generations (few and many tokens per CTA)."""
    torch = _torch()
    for c_len, splits in ((1000, 4), (128 * 40 + 64, 2)):
        world, rank = 3, 1
        case = cases.make_case(5100 + c_len, c_len + 1, "calib")
        kv_full = cases.compress_with(oracle.compress, case, c_len)
        chunks = list(range(rank, (c_len + 127) // 128, world))
        idx = np.concatenate([np.arange(c * 128 * H_KV, min(c_len, (c + 1) * 128) * H_KV) for c in chunks])
        kv = {k: np.ascontiguousarray(v[idx]) for k, v in kv_full.items() if k != "near_ties"}
        n = len(idx) // H_KV
        f, tb = case["f16"], case["tables"]
        want = np.zeros((H_Q, 258), np.float32)
        oracle.OracleOps().attn_strided(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"],
                                        kv["k_norms"], kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"],
                                        f["vq"], f["rotor_k"], f["rotor_v"], f["d_k"], f["d_v"], want, None, H_Q, H_Q, 1, n, 6,
                                        SCALE, tb.alpha_k, tb.alpha_v, 1e7, rank * 128, 1, 128, world * 128)
        arr = {k: dev(v) for k, v in kv.items()}
        tab = {k: dev(v) for k, v in f.items()}
        oa = torch.full((H_Q * 258,), float("nan"), dtype=torch.float32, device="cuda")
        op = torch.full((H_Q * splits * 258,), float("nan"), dtype=torch.float32, device="cuda")
        cuda_ops.attn_strided(dev(case["q_gate"]), arr["k_payload"], arr["v_payload"], arr["v_shared_meta"], arr["k_mask"],
                              arr["k_norms"], arr["k_r_norms"], arr["v_norms"], arr["v_r_norms"], tab["cents_k"], tab["cents_v"],
                              tab["vq"], tab["rotor_k"], tab["rotor_v"], tab["d_k"], tab["d_v"], oa, op, H_Q, H_Q, 1, n, 6, SCALE,
                              tb.alpha_k, tb.alpha_v, 1e7, rank * 128, splits, 128, world * 128)
        torch.cuda.synchronize()
        check_partial(oa.cpu().numpy().reshape(H_Q, 258), want, f"strided c_len={c_len}")
    assert cuda_ops.lib.launch_khq_attn_strided_fp16(*([0] * 18), 24, 24, 1, 64, 6, 0.0625, 1.0, 1.0, 1e7, 0, 1, 127, 256, 0) == -103
    assert cuda_ops.lib.launch_khq_attn_strided_fp16(*([0] * 18), 24, 24, 1, 64, 6, 0.0625, 1.0, 1.0, 1e7, 0, 1, 128, 64, 0) == -103


def _merge_records(recs):
    """LSE merge of (n, 24, 258) unnormalised records into one (24, 258) record."""
    recs = np.asarray(recs, np.float64)
    M = recs[:, :, D].max(axis=0)
    w = np.exp(recs[:, :, D] - M[None])
    out = np.zeros((H_Q, 258))
    out[:, :D] = (recs[:, :, :D] * w[:, :, None]).sum(axis=0)
    out[:, D] = M
    out[:, D + 1] = (recs[:, :, D + 1] * w).sum(axis=0)
    return out.astype(np.float32)


@pytest.mark.parametrize("c_len,win_len,cyclic", [(1000, 0, True), (128 * 40 + 64, 200, True), (2500, 256, False), (0, 130, False)])
def test_persistent_slice_vs_oracle(cuda_ops, oracle, c_len, win_len, cyclic):
    """PersistentSlice (launch_khq_decode_batched_partial_fp16): the share of rank 1 of 3 of a context-parallel
    step -- its slice of the compressed region (chunk-cyclic or contiguous positions) and the raw window -- as
    one launch of the persistent kernel ending in one unnormalised record, against the oracle's records of the
    same slice and window merged on the host."""
    torch = _torch()
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.context_parallel import PersistentSlice, partition_context

    world, rank = 3, 1
    case = cases.make_case(5200 + c_len + win_len, c_len + win_len + 1, "calib")
    f, tb = case["f16"], case["tables"]
    tab = {k: dev(v) for k, v in f.items()}
    recs = []
    if c_len > 0:
        kv_full = cases.compress_with(oracle.compress, case, c_len)
        if cyclic:
            chunks = list(range(rank, (c_len + 127) // 128, world))
            idx = np.concatenate([np.arange(c * 128 * H_KV, min(c_len, (c + 1) * 128) * H_KV) for c in chunks])
            start_pos, chunk, stride = rank * 128, 128, world * 128
        else:
            lo, hi = partition_context(c_len, world)[rank]
            idx = np.arange(lo * H_KV, hi * H_KV)
            start_pos, chunk, stride = lo, 0, 0
        kv = {k: np.ascontiguousarray(v[idx]) for k, v in kv_full.items() if k != "near_ties"}
        n = len(idx) // H_KV
        want_c = np.zeros((H_Q, 258), np.float32)
        oracle.OracleOps().attn_strided(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"],
                                        kv["k_norms"], kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"],
                                        f["vq"], f["rotor_k"], f["rotor_v"], f["d_k"], f["d_v"], want_c, None, H_Q, H_Q, 1, n, 6,
                                        SCALE, tb.alpha_k, tb.alpha_v, 1e7, start_pos, 1, chunk if chunk else n + 2 - n % 2,
                                        stride if stride else n + 2 - n % 2)
        recs.append(want_c)
    else:
        # no compressed token on this rank: one dummy row keeps the arrays addressable
        kv = {k: np.zeros((H_KV,) + v.shape[1:], v.dtype) for k, v in cases.compress_with(oracle.compress, case, 1).items()
              if k != "near_ties"}
        n, start_pos, chunk, stride = 0, 0, 0, 0
    ring_k = np.zeros((256, H_KV, D), np.float16)
    ring_v = np.zeros((256, H_KV, D), np.float16)
    win_start = c_len % 256
    if win_len > 0:
        for s in range(win_len):
            ring_k[(win_start + s) % 256], ring_v[(win_start + s) % 256] = case["k_roped"][c_len + s], case["v"][c_len + s]
        want_w = np.zeros((H_Q, 258), np.float32)
        oracle.window_attn(case["q_gate"], ring_k, ring_v, want_w, win_start, win_len, 256, H_Q, H_KV, D, SCALE)
        recs.append(want_w)
    arr = {k: dev(v) for k, v in kv.items()}
    ps = PersistentSlice(cuda_ops.lib, arr, tab, tb.alpha_k, tb.alpha_v, dev(ring_k), dev(ring_v), start_pos=start_pos,
                         pos_chunk=chunk, pos_stride_chunks=(stride // chunk if chunk else 0))
    out = torch.full((H_Q, 258), float("nan"), dtype=torch.float32, device="cuda")
    q = dev(case["q_gate"])
    for _ in range(2):  # the second call reuses the plan
        ps.launch(q, n, win_start, win_len, out, SCALE, 1e7)
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_device_status() == 0
    check_partial(out.cpu().numpy(), _merge_records(recs), f"persistent slice c_len={c_len} win={win_len} cyclic={cyclic}")
