"""Batched decode (one persistent launch for many sequence-layer problems) against the oracle."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


def oracle_step(oracle, case, kv, c_len, win_start, win_len, start_pos=0):
    ops = oracle.OracleOps()
    f, tb = case["f16"], case["tables"]
    ac = np.zeros((H_Q, 258), np.float32)
    aw = np.zeros((H_Q, 258), np.float32)
    if c_len > 0:
        ops.attn(case["q_gate"], kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"],
                 kv["k_r_norms"], kv["v_norms"], kv["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"],
                 f["rotor_v"], f["d_k"], f["d_v"], ac, None, H_Q, H_Q, 1, c_len, c_len, 6, SCALE, tb.alpha_k,
                 tb.alpha_v, 1e7, start_pos, 1)
    ring_k = np.zeros((256, H_KV, D), np.float16)
    ring_v = np.zeros((256, H_KV, D), np.float16)
    for s in range(win_len):
        ring_k[(win_start + s) % 256] = case["k_roped"][c_len + s]
        ring_v[(win_start + s) % 256] = case["v"][c_len + s]
    if win_len > 0:
        ops.window_attn(case["q_gate"], ring_k, ring_v, aw, win_start, win_len, 256, H_Q, H_KV, D, SCALE)
    out = np.zeros((H_Q, D), np.float16)
    ops.merge_gate(ac, aw, case["q_gate"], out, H_Q, D, win_len > 0, c_len > 0)
    return out, ring_k, ring_v


@pytest.mark.parametrize("codebook_in_smem", [1, 0, 2, 3, 4])  # 2 = mma.sync generation, 3 and 4 = tcgen05 generations
@pytest.mark.parametrize("tokens_per_item", [0, 48, 1000])
def test_batched_decode_vs_oracle(cuda_ops, oracle, codebook_in_smem, tokens_per_item):
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.batched import BatchedDecode

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    shapes = [  # (variant/layer, c_len, win_len)
        (0, 384, 128), (0, 0, 77), (0, 129, 1), (0, 1001, 256), (1, 640, 200), (1, 50, 0), (1, 2, 3)]
    variants = ["calib", "n01_idrot"]
    tables, problems, refs = [], [], []
    for li, variant in enumerate(variants):
        base = cases.make_case(3000 + li, 8, variant, layer_id=3 + 4 * li)
        tables.append(dict({k: dev(v) for k, v in [("cents_k", base["f16"]["cents_k"]), ("cents_v", base["f16"]["cents_v"]),
                                                   ("vq", base["f16"]["vq"]), ("k_rotor", base["f16"]["rotor_k"]),
                                                   ("v_rotor", base["f16"]["rotor_v"]), ("d_k", base["f16"]["d_k"]),
                                                   ("d_v", base["f16"]["d_v"])]},
                           alpha_k=base["tables"].alpha_k, alpha_v=base["tables"].alpha_v, _case=base))
    for pi, (li, c_len, win_len) in enumerate(shapes):
        case = cases.make_case(3100 + pi, c_len + win_len, variants[li], layer_id=3 + 4 * li)
        # share the layer's tables: recompress with the layer tables, not the case's own
        case["tables"], case["f16"] = tables[li]["_case"]["tables"], tables[li]["_case"]["f16"]
        kv = cases.compress_with(oracle.compress, case, c_len) if c_len > 0 else {
            "k_mask": np.zeros((4, 16), np.uint32), "k_payload": np.zeros((4, 40), np.uint8),
            "k_norms": np.zeros(4, np.float16), "k_r_norms": np.zeros(4, np.float16),
            "v_payload": np.zeros((4, 104), np.uint8), "v_norms": np.zeros(4, np.float16),
            "v_r_norms": np.zeros(4, np.float16), "v_shared_meta": np.zeros((4, 4), np.uint8)}
        win_start = c_len % 256
        ref, ring_k, ring_v = oracle_step(oracle, case, kv, c_len, win_start, win_len)
        refs.append(ref)
        p = {k: dev(v) for k, v in kv.items() if k != "near_ties"}
        p.update(q_gate=dev(case["q_gate"]), ring_k=dev(ring_k), ring_v=dev(ring_v),
                 out=torch.zeros(H_Q * D, dtype=torch.float16, device="cuda"),
                 table_id=li, c_len=c_len, start_pos=0, win_start=win_start, win_len=win_len)
        problems.append(p)
    bd = BatchedDecode(problems, tables, tokens_per_item=tokens_per_item, codebook_in_smem=codebook_in_smem)
    for _ in range(2):  # second launch reuses the workspace: the item counter must have been reset
        bd.launch(SCALE, 1e7)
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_device_status() == 0
    for pi, p in enumerate(problems):
        got = p["out"].float().cpu().numpy().reshape(H_Q, D)
        ok, mx, exc = cases.attention_close(got, refs[pi].astype(np.float32))
        assert ok, f"problem {pi} {shapes[pi]}: max abs {mx:.3e} excess {exc:.3e}"
    assert bd.algorithmic_bytes == sum(4 * (220 * c + 1024 * w) for _, c, w in shapes)


def test_batched_error_codes(cuda_ops):
    lib = cuda_ops.lib
    assert lib.launch_khq_decode_batched_fp16(0, 0, 0, 0, 0, 0, 0, 0, 0.0625, 1e7, 256, -1, 0) == -100
    assert lib.khq_b200_decode_workspace_bytes(2) == 256 + 2 * 24 * 258 * 4
    assert lib.khq_b200_plan_decode(0, 0, 1, 0, 0, 0, 0, 0) == -100
