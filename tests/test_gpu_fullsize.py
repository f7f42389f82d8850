"""Size-independent properties at the full sizes of the benchmark specification, where the CPU oracle is too slow to be
the checker: row independence of the compress kernel, context-split invariance of the
compressed-region attention (long context, configuration 2), causal-prefix invariance of the
prefill and agreement of its two independent kernels (configs[4]), and agreement of the batched
persistent kernel with the per-sequence drop-in launches on long sequences (configs[3])."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


def _tables(torch, seed=11):
    rng = np.random.default_rng(seed)
    sample = rng.standard_normal((256, D)).astype(np.float16)
    tb = cases.synth.make_tables(rng, 3, sample, sample)
    return tb, {k: torch.from_numpy(v).cuda() for k, v in tb.as_f16().items()}


def _compress_all(ops, torch, tb, tab, k, v, rows):
    kv = dict(k_mask=torch.zeros(rows * 16, dtype=torch.int32, device="cuda"),
              k_payload=torch.zeros(rows * 40, dtype=torch.uint8, device="cuda"),
              v_payload=torch.zeros(rows * 104, dtype=torch.uint8, device="cuda"),
              v_shared_meta=torch.zeros(rows * 4, dtype=torch.uint8, device="cuda"),
              k_norms=torch.zeros(rows, dtype=torch.float16, device="cuda"), k_r_norms=torch.zeros(rows, dtype=torch.float16, device="cuda"),
              v_norms=torch.zeros(rows, dtype=torch.float16, device="cuda"), v_r_norms=torch.zeros(rows, dtype=torch.float16, device="cuda"))
    ops.compress(k, tab["d_k"], tab["rotor_k"], tab["cents_k"], tab["cents_k"], kv["k_mask"], kv["k_norms"], kv["k_r_norms"],
                 kv["k_payload"], kv["v_shared_meta"], rows, D, tb.ts_k, tb.alpha_k, False)
    ops.compress(v, tab["d_v"], tab["rotor_v"], tab["cents_v"], tab["vq"], kv["k_mask"], kv["v_norms"], kv["v_r_norms"],
                 kv["v_payload"], kv["v_shared_meta"], rows, D, tb.ts_v, tb.alpha_v, True)
    return kv


def test_compress_rows_are_independent_at_prompt_size(cuda_ops):
    """32 256 rows x 4 kv heads (one prompt of configs[4]): the code words of any slice of rows are
    bit-identical to what a launch over that slice alone writes, and a second launch repeats the
    first bit for bit."""
    import torch

    tb, tab = _tables(torch)
    rows = 32256 * 4
    g = torch.Generator(device="cuda").manual_seed(5)
    k = torch.randn(rows, D, generator=g, device="cuda").half()
    v = torch.randn(rows, D, generator=g, device="cuda").half()
    full = _compress_all(cuda_ops, torch, tb, tab, k, v, rows)
    again = _compress_all(cuda_ops, torch, tb, tab, k, v, rows)
    torch.cuda.synchronize()
    for key in full:
        assert torch.equal(full[key].view(torch.uint8), again[key].view(torch.uint8)), key
    a, n = 51_200, 512  # one 128-token event somewhere in the middle
    part = _compress_all(cuda_ops, torch, tb, tab, k[a:a + n].contiguous(), v[a:a + n].contiguous(), n)
    per_row = dict(k_mask=64, k_payload=40, v_payload=104, v_shared_meta=4, k_norms=2, k_r_norms=2, v_norms=2, v_r_norms=2)
    for key, rb in per_row.items():
        whole = full[key].view(torch.uint8)[a * rb:(a + n) * rb]
        assert torch.equal(whole, part[key].view(torch.uint8)), key
    # every K row keeps at most 50 outliers (symbol 3) and every norm is finite
    sym = full["k_mask"].view(torch.uint8).cpu().numpy().reshape(rows, 64)
    n3 = sum((((sym >> s) & 3) == 3).sum(axis=1) for s in (0, 2, 4, 6))
    assert n3.max() <= 50
    assert torch.isfinite(full["k_norms"].float()).all() and torch.isfinite(full["v_norms"].float()).all()


def test_long_context_split_invariance(cuda_ops):
    """131 072 compressed tokens (configs[2]): the merged attention must not depend on how the
    context is cut -- 1, 8 or 32 splits in one launch, or four launches over context quarters
    (absolute start_pos) merged by the slot-merge kernel."""
    import torch

    tb, tab = _tables(torch, seed=12)
    c_len = 131072
    rows = c_len * H_KV
    g = torch.Generator(device="cuda").manual_seed(6)
    k = torch.randn(rows, D, generator=g, device="cuda").half()
    v = torch.randn(rows, D, generator=g, device="cuda").half()
    kv = _compress_all(cuda_ops, torch, tb, tab, k, v, rows)
    qg = torch.randn(H_Q * 2 * D, generator=g, device="cuda").half()

    def attn(lo, hi, splits):
        ac = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        ap = torch.zeros(H_Q * 32 * 258, dtype=torch.float32, device="cuda")
        r0 = lo * H_KV
        cuda_ops.attn(qg, kv["k_payload"][r0 * 40:], kv["v_payload"][r0 * 104:], kv["v_shared_meta"][r0 * 4:], kv["k_mask"][r0 * 16:],
                      kv["k_norms"][r0:], kv["k_r_norms"][r0:], kv["v_norms"][r0:], kv["v_r_norms"][r0:], tab["cents_k"],
                      tab["cents_v"], tab["vq"], tab["rotor_k"], tab["rotor_v"], tab["d_k"], tab["d_v"], ac, ap, H_Q, H_Q, 1,
                      hi - lo, hi - lo, 6, SCALE, tb.alpha_k, tb.alpha_v, 1e7, lo, splits)
        return ac

    def finish(partials, n_slots):
        out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
        cuda_ops.merge_slots_gate(partials, n_slots, qg, out, H_Q, D)
        torch.cuda.synchronize()
        return out.float().cpu().numpy()

    ref = finish(attn(0, c_len, 32), 1)
    assert np.isfinite(ref).all() and np.abs(ref).max() > 0
    for splits in (1, 8):
        got = finish(attn(0, c_len, splits), 1)
        ok, mx, exc = cases.attention_close(got, ref)
        assert ok, f"splits {splits}: max abs {mx:.3e}"
    q4 = c_len // 4
    parts = torch.cat([attn(i * q4, (i + 1) * q4, 8) for i in range(4)])
    got = finish(parts, 4)
    ok, mx, exc = cases.attention_close(got, ref)
    assert ok, f"context quarters: max abs {mx:.3e}"


def test_prefill_prefix_invariance_and_kernel_agreement_at_full_length(cuda_ops):
    """T = 8192 (configs[4]): the rows of a causal attention do not depend on what follows them,
    so the first 3000 rows must be bit-identical to the prefill of the 3000-token prefix (same tile
    schedule per row block); the tcgen05 kernel and the warp-level kernel, two independent
    implementations, must agree within the attention bar everywhere."""
    import torch

    B, T, T1 = 2, 8192, 3000
    g = torch.Generator(device="cuda").manual_seed(7)
    qg = torch.randn(B, T, H_Q, 2 * D, generator=g, device="cuda").half()
    k = (torch.randn(B, T, H_KV, D, generator=g, device="cuda") * 0.25).half()
    v = torch.randn(B, T, H_KV, D, generator=g, device="cuda").half()
    lib = cuda_ops.lib

    def run(which, qg_, k_, v_, t):
        out = torch.full((B, t, H_Q, D), float("nan"), dtype=torch.float16, device="cuda")
        assert lib.khq_b200_prefill_select(which) == 0
        try:
            cuda_ops.gqa_prefill(qg_, k_, v_, out, B, t, H_Q, H_KV, D, SCALE)
            torch.cuda.synchronize()
        finally:
            lib.khq_b200_prefill_select(0)
        assert lib.khq_b200_prefill_status() == 0
        return out

    full = run(0, qg, k, v, T)
    assert torch.isfinite(full.float()).all()
    pre = run(0, qg[:, :T1].contiguous(), k[:, :T1].contiguous(), v[:, :T1].contiguous(), T1)
    # whole 128-row blocks of the prefix see the same tiles in the same order in both launches
    nb = (T1 // 128) * 128
    assert torch.equal(full[:, :nb].view(torch.int16), pre[:, :nb].view(torch.int16))
    ok, mx, exc = cases.attention_close(pre[:, nb:].float().cpu().numpy(), full[:, nb:T1].float().cpu().numpy())
    assert ok, f"ragged last block: max abs {mx:.3e}"
    other = run(1, qg, k, v, T)
    ok, mx, exc = cases.attention_close(full.float().cpu().numpy(), other.float().cpu().numpy())
    assert ok, f"tcgen05 vs warp-level kernel: max abs {mx:.3e}, excess {exc:.3e}"


def test_batched_kernel_agrees_with_drop_in_launches_on_long_sequences(cuda_ops):
    """Six sequences with contexts up to 32 768 tokens (configs[3] range) through the batched
    persistent kernel, against the same sequences one by one through the drop-in launches
    (compressed attention + window attention + merge/gate), which are different kernels."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.engine import BatchEngine

    rng = np.random.default_rng(8)
    sample = rng.standard_normal((256, D)).astype(np.float16)
    tables = [cases.synth.make_tables(rng, li, sample, sample) for li in range(2)]
    c_len = np.array([32512, 4096, 16384, 128, 25600, 9984], dtype=np.int64)
    win = np.array([256, 128, 200, 255, 129, 256], dtype=np.int64)
    eng = BatchEngine(tables, c_len, win, device="cuda", codebook_in_smem=2)
    eng.fill_synthetic(99)
    torch.cuda.synchronize()
    ops = cuda_ops
    for layer in range(2):
        eng.attention_resident(layer)
        torch.cuda.synchronize()
        got = eng.out[layer].float().cpu().numpy().reshape(len(c_len), H_Q, D)
        tb, P = eng.tables[layer], eng.pay[layer]
        for s in range(len(c_len)):
            r0, cl, wl = int(eng.row_off[s]), int(c_len[s]), int(win[s])
            qg = eng.q_gate[layer][s]
            ac = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
            aw = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
            ap = torch.zeros(H_Q * 32 * 258, dtype=torch.float32, device="cuda")
            out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
            ops.attn(qg, P["k_payload"][r0 * 40:], P["v_payload"][r0 * 104:], P["v_shared_meta"][r0 * 4:], P["k_mask"][r0 * 16:],
                     P["k_norms"][r0:], P["k_r_norms"][r0:], P["v_norms"][r0:], P["v_r_norms"][r0:], tb["cents_k"], tb["cents_v"],
                     tb["vq"], tb["k_rotor"], tb["v_rotor"], tb["d_k"], tb["d_v"], ac, ap, H_Q, H_Q, 1, cl, cl, 6, SCALE,
                     tb["alpha_k"], tb["alpha_v"], 1e7, 0, 16)
            ops.window_attn(qg, eng.ring_k[layer][s].reshape(-1), eng.ring_v[layer][s].reshape(-1), aw, cl % 256, wl, 256,
                            H_Q, H_KV, D, SCALE)
            ops.merge_gate(ac, aw, qg, out, H_Q, D, True, True)
            torch.cuda.synchronize()
            ref = out.float().cpu().numpy().reshape(H_Q, D)
            ok, mx, exc = cases.attention_close(got[s], ref)
            assert ok, f"layer {layer} seq {s} (c_len {cl}): max abs {mx:.3e}, excess {exc:.3e}"
