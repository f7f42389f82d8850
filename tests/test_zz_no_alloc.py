"""launch_khq_attn_static_fp16: the compressed-region attention for hosts that cannot allocate
the split-partial buffer (all device memory belongs to another runtime's pool, or a cudaMalloc,
which stalls the whole device, is not acceptable inside the decode loop).  The split partials
then live in a fixed array inside the library.  Checked here against launch_khq_attn_fp16 with a
caller-allocated partial buffer (same kernels, same split count: the two results must be
bit-identical) and against the CPU oracle, on two calls in a row that share the array.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

import cases
from cases import D, H_Q, SCALE

pytestmark = pytest.mark.gpu


def _args(case, kv, dev):
    f = case["f16"]
    arr = {k: dev(v) for k, v in kv.items() if k != "near_ties"}
    tab = {k: dev(v) for k, v in f.items()}
    q = dev(case["q_gate"])
    ptrs = [q, arr["k_payload"], arr["v_payload"], arr["v_shared_meta"], arr["k_mask"], arr["k_norms"],
            arr["k_r_norms"], arr["v_norms"], arr["v_r_norms"], tab["cents_k"], tab["cents_v"], tab["vq"],
            tab["rotor_k"], tab["rotor_v"], tab["d_k"], tab["d_v"]]
    return ptrs, (arr, tab, q)


def test_static_partials_match_caller_allocated_partials(cuda_ops, oracle):
    import torch

    lib = cuda_ops.lib
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first call's partials in the array
    for seed, c_len, splits in ((61, 384, 8), (62, 1000, 32)):
        case = cases.make_case(seed, c_len + 1, "calib")
        kv = cases.compress_with(oracle.compress, case, c_len)
        tb = case["tables"]
        ptrs, keep = _args(case, kv, dev)
        out_ref = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        part = torch.zeros(H_Q * splits * 258, dtype=torch.float32, device="cuda")
        rc = lib.launch_khq_attn_fp16(*[p.data_ptr() for p in ptrs], out_ref.data_ptr(), part.data_ptr(), H_Q, H_Q,
                                      1, c_len, c_len, 6, SCALE, tb.alpha_k, tb.alpha_v, 1e7, 0, splits, stream)
        assert rc == 0
        out_new = torch.full((H_Q * 258,), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.launch_khq_attn_static_fp16(*[p.data_ptr() for p in ptrs], out_new.data_ptr(), H_Q, H_Q, 1, c_len,
                                             6, SCALE, tb.alpha_k, tb.alpha_v, 1e7, 0, splits, stream)
        assert rc == 0
        torch.cuda.synchronize()
        # where the partials live changes nothing in the arithmetic
        assert torch.equal(out_new.view(torch.int32), out_ref.view(torch.int32)), f"c_len={c_len} splits={splits}"
        a = out_new.cpu().numpy().reshape(H_Q, 258)
        want = oracle.attn_partial(case["q_gate"], kv, cases.tables_dict(case["f16"]), H_Q, 6, SCALE, tb.alpha_k,
                                   tb.alpha_v, 1e7, 0, 0, c_len)
        ok, mx, exc = cases.attention_close(cases.normalised(a), cases.normalised(want))
        assert ok, f"c_len={c_len} splits={splits} vs oracle: max abs {mx:.3e}, excess {exc:.3e}"
        assert np.abs((a[:, D] + np.log(a[:, D + 1])) - (want[:, D] + np.log(want[:, D + 1]))).max() < 5e-3
        del keep


def test_static_entry_rejects_what_does_not_fit(cuda_ops):
    lib = cuda_ops.lib
    z = [0] * 17
    assert lib.launch_khq_attn_static_fp16(*z, 24, 24, 1, 64, 6, 0.0625, 1.0, 1.0, 1e7, 0, 33, 0) == -106
    assert lib.launch_khq_attn_static_fp16(*z, 48, 24, 2, 64, 6, 0.0625, 1.0, 1.0, 1e7, 0, 4, 0) == -106
    assert lib.launch_khq_attn_static_fp16(*z, 24, 24, 1, 0, 6, 0.0625, 1.0, 1.0, 1e7, 0, 4, 0) == -100
