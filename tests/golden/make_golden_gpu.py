"""Generate the golden fixtures of tests/golden/ by running the REFERENCE's own CUDA kernels.

The reference project holds no golden vector for any KHQ kernel, and it has no CPU
implementation of them.  Its CUDA source compiles unmodified for sm_100a
(oracle/Makefile -> oracle/_ref/libbonsai_ref_sm100a.so), so this script runs that library on
a B200 on seeded inputs and stores inputs and outputs as compressed .npz files.  The CPU test
suite then checks the oracle against these files, which pins the oracle to the reference.

Needs a CUDA device and oracle/_ref/ (built where the reference checkout is mounted):

    python tests/golden/make_golden_gpu.py --out tests/golden

Fixtures:
  compress_<variant>.npz   K and V code words of 96 tokens x 4 kv-heads per table variant
  decode_<variant>.npz     config-0 shaped decode step: 384 compressed + 128 raw tokens;
                           compressed-region output at splits 1 and 8, window output, final
                           gated fp16 output
  decode_farpos.npz        64 compressed tokens at start_pos 100000 (RoPE at large positions)
"""
from __future__ import annotations

import argparse
import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import torch  # noqa: E402

from bonsai_mojo_1bit_optimization_t4_cuda_b200 import lib as khqlib  # noqa: E402
import cases  # noqa: E402

REF_SO = ROOT / "oracle" / "_ref" / "libbonsai_ref_sm100a.so"
H_Q, H_KV, D = 24, 4, 256


def load_ref():
    so = ctypes.CDLL(str(REF_SO))
    for name in ("launch_khq_compress_fp16", "launch_khq_attn_fp16", "launch_khq_window_attn_fp16",
                 "launch_khq_merge_gate_fp16"):
        res, args = khqlib.SIGNATURES[name]
        fn = getattr(so, name)
        fn.restype, fn.argtypes = res, args
    return so


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ref_compress(so, x, d_vec, rotor, cents, vq, rows, ts, alpha, is_v):
    pay = 104 if is_v else 40
    o_mask = torch.zeros(rows * 16, dtype=torch.int32, device="cuda")
    o_n = torch.zeros(rows, dtype=torch.float16, device="cuda")
    o_rn = torch.zeros(rows, dtype=torch.float16, device="cuda")
    o_pay = torch.zeros(rows * pay, dtype=torch.uint8, device="cuda")
    o_sm = torch.full((rows * 4,), 0xAB, dtype=torch.uint8, device="cuda")
    t = [dev(a) for a in (x, d_vec, rotor, cents, vq)]
    rc = so.launch_khq_compress_fp16(*[a.data_ptr() for a in t], o_mask.data_ptr(), o_n.data_ptr(),
                                     o_rn.data_ptr(), o_pay.data_ptr(), o_sm.data_ptr(), rows, D,
                                     float(ts), float(alpha), 1 if is_v else 0, 0)
    torch.cuda.synchronize()
    assert rc == 0, rc
    return dict(mask=o_mask.cpu().numpy().view(np.uint32).reshape(rows, 16), norms=o_n.cpu().numpy(),
                r_norms=o_rn.cpu().numpy(), payload=o_pay.cpu().numpy().reshape(rows, pay),
                shared_meta=o_sm.cpu().numpy().reshape(rows, 4), near_ties=0)


def ref_decode(so, case, kv, c_len, win_start, win_len, start_pos, splits_list):
    f, tb = case["f16"], case["tables"]
    q = dev(case["q_gate"])
    arr = {k: dev(v) for k, v in kv.items() if k != "near_ties"}
    tab = {k: dev(v) for k, v in f.items()}
    outs = {}
    for sp in splits_list:
        oa = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        op = torch.zeros(H_Q * max(sp, 1) * 258, dtype=torch.float32, device="cuda")
        rc = so.launch_khq_attn_fp16(
            q.data_ptr(), arr["k_payload"].data_ptr(), arr["v_payload"].data_ptr(),
            arr["v_shared_meta"].data_ptr(), arr["k_mask"].data_ptr(), arr["k_norms"].data_ptr(),
            arr["k_r_norms"].data_ptr(), arr["v_norms"].data_ptr(), arr["v_r_norms"].data_ptr(),
            tab["cents_k"].data_ptr(), tab["cents_v"].data_ptr(), tab["vq"].data_ptr(),
            tab["rotor_k"].data_ptr(), tab["rotor_v"].data_ptr(), tab["d_k"].data_ptr(),
            tab["d_v"].data_ptr(), oa.data_ptr(), op.data_ptr(), H_Q, H_Q, 1, c_len, c_len, 6,
            cases.SCALE, tb.alpha_k, tb.alpha_v, 1e7, start_pos, sp, 0)
        torch.cuda.synchronize()
        assert rc == 0, rc
        outs[f"attn_c_s{sp}"] = oa.cpu().numpy().reshape(H_Q, 258)
    if win_len > 0:
        ring_k = np.zeros((256, H_KV, D), np.float16)
        ring_v = np.zeros((256, H_KV, D), np.float16)
        for s in range(win_len):
            slot = (win_start + s) % 256
            ring_k[slot] = case["k_roped"][c_len + s]
            ring_v[slot] = case["v"][c_len + s]
        rk, rv = dev(ring_k), dev(ring_v)
        ow = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        rc = so.launch_khq_window_attn_fp16(q.data_ptr(), rk.data_ptr(), rv.data_ptr(), ow.data_ptr(),
                                            win_start, win_len, 256, H_Q, H_KV, D, cases.SCALE, 0)
        torch.cuda.synchronize()
        assert rc == 0, rc
        outs["attn_w"] = ow.cpu().numpy().reshape(H_Q, 258)
        outs["ring_k"], outs["ring_v"] = ring_k, ring_v
        oc = dev(outs[f"attn_c_s{splits_list[0]}"])
        out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
        rc = so.launch_khq_merge_gate_fp16(oc.data_ptr(), ow.data_ptr(), q.data_ptr(), out.data_ptr(), H_Q,
                                           D, 1, 0)
        torch.cuda.synchronize()
        assert rc == 0, rc
        outs["out"] = out.cpu().numpy().reshape(H_Q, D)
    return outs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden"))
    args = ap.parse_args()
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    so = load_ref()
    comp = lambda *a: ref_compress(so, *a)

    for vi, variant in enumerate(cases.VARIANTS):
        # ---- compress fixture: 96 tokens ------------------------------------------------------
        case = cases.make_case(7000 + vi, 96, variant)
        kv = cases.compress_with(comp, case, 96)
        np.savez_compressed(
            out_dir / f"compress_{variant}.npz", k_unroped=case["k_unroped"], v=case["v"],
            ts_k=np.float32(case["tables"].ts_k), alpha_k=np.float32(case["tables"].alpha_k),
            ts_v=np.float32(case["tables"].ts_v), alpha_v=np.float32(case["tables"].alpha_v),
            **{"t_" + k: v for k, v in case["f16"].items()}, **{k: v for k, v in kv.items() if k != "near_ties"})
        # ---- decode fixture: config-0 shape ----------------------------------------------------
        case = cases.make_case(7100 + vi, 512, variant)
        kv = cases.compress_with(comp, case, 384)
        outs = ref_decode(so, case, kv, 384, 128, 128, 0, [1, 8])
        np.savez_compressed(
            out_dir / f"decode_{variant}.npz", q_gate=case["q_gate"],
            alpha_k=np.float32(case["tables"].alpha_k), alpha_v=np.float32(case["tables"].alpha_v),
            **{"t_" + k: v for k, v in case["f16"].items()}, **{k: v for k, v in kv.items() if k != "near_ties"},
            **outs)
        print("wrote", variant)

    case = cases.make_case(7200, 64, "calib", q_pos=100063)
    kv = cases.compress_with(comp, case, 64)
    outs = ref_decode(so, case, kv, 64, 0, 0, 100000, [1])
    np.savez_compressed(out_dir / "decode_farpos.npz", q_gate=case["q_gate"],
                        alpha_k=np.float32(case["tables"].alpha_k), alpha_v=np.float32(case["tables"].alpha_v),
                        **{"t_" + k: v for k, v in case["f16"].items()},
                        **{k: v for k, v in kv.items() if k != "near_ties"}, **outs)
    print("wrote farpos")


if __name__ == "__main__":
    main()
