"""The benchmark specification's full sizes.

First the comparisons against the CPU oracle (and, where ``oracle/_ref`` was built, against the
reference's own kernels recompiled for sm_100a): 131 072 compressed tokens + 256 raw ones through
the drop-in launches at 8 / 32 / 128 splits and through the batched kernels (configs[2]); a
batched launch holding a 32 640-token and a 4 096-token sequence (configs[3]); the T = 8192
prefill in fp16 and bf16 on a sample of query rows against the reference test's FP64 twin
(configs[4]).  Then size-independent properties: row independence of the compress kernel,
context-split invariance, causal-prefix invariance of the prefill and agreement of its two
independent kernels, agreement of the batched kernel with the drop-in launches."""
import sys
from pathlib import Path

import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF_SO = ROOT / "oracle" / "_ref" / "libbonsai_ref_sm100a.so"


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


def _synthetic_state(torch, cuda_ops, c_len, win_len, seed, layer_id=3, variant_kw=None):
    """c_len compressed + win_len raw tokens with the generator's distributions (per-channel
    lognormal scales, four x8 outlier channels per kv-head), drawn on the GPU, compressed by the
    library (whose code words are bit-identical to the oracle's, tests/test_gpu_kernels.py), and
    copied to the host for the oracle.  Returns (tables, device tables, device kv, host kv, q_gate,
    ring_k, ring_v) with the raw window RoPE'd at positions c_len.. and q at c_len + win_len - 1."""
    rng = np.random.default_rng(seed)
    sk, sv = cases.synth.channel_scales(rng), cases.synth.channel_scales(rng)
    g = torch.Generator(device="cuda").manual_seed(seed)
    n = c_len + win_len
    k = (torch.randn(n, H_KV, D, generator=g, device="cuda") * torch.from_numpy(sk).cuda()).half()
    v = (torch.randn(n, H_KV, D, generator=g, device="cuda") * torch.from_numpy(sv).cuda()).half()
    sample = slice(0, 512)
    tb = cases.synth.make_tables(rng, layer_id, k[sample].reshape(-1, D).cpu().numpy(), v[sample].reshape(-1, D).cpu().numpy(),
                                 **(variant_kw or dict(vq_scale=1.0 / 16.0)))
    tab = {key: torch.from_numpy(val).cuda() for key, val in tb.as_f16().items()}
    rows = c_len * H_KV
    kv = _compress_all(cuda_ops, torch, tb, tab, k[:c_len].reshape(rows, D).contiguous(), v[:c_len].reshape(rows, D).contiguous(), rows)
    torch.cuda.synchronize()
    host = {key: val.cpu().numpy() for key, val in kv.items()}
    host["k_mask"] = host["k_mask"].view(np.uint32)
    ring_k = np.zeros((256, H_KV, D), np.float16)
    ring_v = np.zeros((256, H_KV, D), np.float16)
    k_raw = k[c_len:].cpu().numpy()
    k_rot = cases.synth.partial_rope(k_raw, (c_len + np.arange(win_len))[:, None].repeat(H_KV, 1))
    for s_ in range(win_len):
        ring_k[(c_len + s_) % 256] = k_rot[s_]
        ring_v[(c_len + s_) % 256] = v[c_len + s_].cpu().numpy()
    q_gate = cases.synth.make_q_gate(rng, n - 1)
    return tb, tab, kv, host, q_gate, ring_k, ring_v


def _oracle_compressed(oracle, tb, host, q_gate, c_len, splits=1, start_pos=0):
    f = tb.as_f16()
    ref = np.zeros((H_Q, 258), np.float32)
    ref_p = np.zeros((H_Q, max(splits, 1), 258), np.float32)
    rc = oracle.attn_launch(q_gate, host["k_payload"], host["v_payload"], host["v_shared_meta"], host["k_mask"], host["k_norms"],
                            host["k_r_norms"], host["v_norms"], host["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"],
                            f["rotor_v"], f["d_k"], f["d_v"], ref, ref_p, H_Q, H_Q, c_len, 6, SCALE, tb.alpha_k, tb.alpha_v, 1e7,
                            start_pos, splits)
    assert rc == 0
    return ref


def _errs(got, ref):
    ok, mx, exc = cases.attention_close(cases.normalised(got), cases.normalised(ref))
    lse = float(np.abs((got[:, D] + np.log(np.maximum(got[:, D + 1], 1e-30))) - (ref[:, D] + np.log(np.maximum(ref[:, D + 1], 1e-30)))).max())
    return ok, mx, exc, lse


def test_long_context_vs_oracle_and_reference_kernel(cuda_ops, oracle):
    """configs[2]: 131 072 compressed tokens + 256 raw ones.  The drop-in launch at 8, 32 and 128
    splits (the launcher's choice of kernel generation differs with the tokens per CTA), the
    batched kernels of every generation, the raw window, and the final gated output, all against
    the CPU oracle; the reference's own kernel (32 splits) is compared with the same oracle result
    beside them when its recompiled library is present."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.batched import BatchedDecode

    c_len, win = 131072, 256
    tb, tab, kv, host, q_gate, ring_k, ring_v = _synthetic_state(torch, cuda_ops, c_len, win, seed=2026)
    ref = _oracle_compressed(oracle, tb, host, q_gate, c_len, splits=1)
    qg = torch.from_numpy(q_gate).cuda().reshape(-1)
    report = {}
    for splits in (8, 32, 128):
        ac = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        ap = torch.zeros(H_Q * splits * 258, dtype=torch.float32, device="cuda")
        cuda_ops.attn(qg, kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"], kv["k_r_norms"],
                      kv["v_norms"], kv["v_r_norms"], tab["cents_k"], tab["cents_v"], tab["vq"], tab["rotor_k"], tab["rotor_v"],
                      tab["d_k"], tab["d_v"], ac, ap, H_Q, H_Q, 1, c_len, c_len, 6, SCALE, tb.alpha_k, tb.alpha_v, 1e7, 0, splits)
        torch.cuda.synchronize()
        ok, mx, exc, lse = _errs(ac.cpu().numpy().reshape(H_Q, 258), ref)
        report[f"drop-in splits {splits}"] = (mx, lse)
        assert ok and lse < 5e-3, f"splits {splits}: max abs {mx:.3e} excess {exc:.3e} lse {lse:.3e}"
    # the window and the gated output of the whole step through the batched kernels
    aw = np.zeros((H_Q, 258), np.float32)
    oracle.window_attn(q_gate, ring_k, ring_v, aw, c_len % 256, win, 256, H_Q, H_KV, D, SCALE)
    want = np.zeros((H_Q, D), np.float16)
    oracle.merge_gate(ref, aw, q_gate, want, H_Q, D, 1)
    tables = [dict(cents_k=tab["cents_k"], cents_v=tab["cents_v"], vq=tab["vq"], k_rotor=tab["rotor_k"], v_rotor=tab["rotor_v"],
                   d_k=tab["d_k"], d_v=tab["d_v"], alpha_k=tb.alpha_k, alpha_v=tb.alpha_v)]
    for gen in (1, 2, 3, 4):
        prob = dict(kv)
        prob.update(q_gate=qg, ring_k=torch.from_numpy(ring_k).cuda().reshape(-1), ring_v=torch.from_numpy(ring_v).cuda().reshape(-1),
                    out=torch.zeros(H_Q * D, dtype=torch.float16, device="cuda"), table_id=0, c_len=c_len, start_pos=0,
                    win_start=c_len % 256, win_len=win)
        bd = BatchedDecode([prob], tables, codebook_in_smem=gen)
        bd.launch(SCALE, 1e7)
        torch.cuda.synchronize()
        assert cuda_ops.lib.khq_b200_device_status() == 0
        got = prob["out"].float().cpu().numpy().reshape(H_Q, D)
        ok, mx, exc = cases.attention_close(got, want.astype(np.float32))
        report[f"batched generation {gen}"] = (mx, None)
        assert ok, f"batched generation {gen}: max abs {mx:.3e} excess {exc:.3e}"
    if REF_SO.exists():
        import ctypes

        sys.path.insert(0, str(ROOT / "tests" / "golden"))
        import make_golden_gpu as mg

        so = mg.load_ref()
        ac = torch.zeros(H_Q * 258, dtype=torch.float32, device="cuda")
        ap = torch.zeros(H_Q * 32 * 258, dtype=torch.float32, device="cuda")
        args = [qg, kv["k_payload"], kv["v_payload"], kv["v_shared_meta"], kv["k_mask"], kv["k_norms"], kv["k_r_norms"], kv["v_norms"],
                kv["v_r_norms"], tab["cents_k"], tab["cents_v"], tab["vq"], tab["rotor_k"], tab["rotor_v"], tab["d_k"], tab["d_v"], ac, ap]
        rc = so.launch_khq_attn_fp16(*[ctypes.c_void_p(a.data_ptr()) for a in args], H_Q, H_Q, 1, c_len, c_len, 6, SCALE, tb.alpha_k,
                                     tb.alpha_v, 1e7, 0, 32, None)
        torch.cuda.synchronize()
        assert rc == 0
        ok, mx, exc, lse = _errs(ac.cpu().numpy().reshape(H_Q, 258), ref)
        report["reference kernel, 32 splits"] = (mx, lse)
        # the reference forms its RoPE angle in fp32, the oracle in double: at positions up to 131 071 the two
        # differ by more than the attention bar allows, so this one is reported, not asserted at that bar
        assert mx < 5e-2
    print("configs[2] vs oracle (max |err| of acc/sum, log-sum-exp err):", report)


def test_batched_long_and_short_sequence_vs_oracle(cuda_ops, oracle):
    """configs[3] range: one batched launch holding a 32 640-token sequence and a 4 096-token one
    (plus their raw windows), every kernel generation, against the CPU oracle."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.batched import BatchedDecode

    specs = [(32640, 128, 71), (4096, 256, 72)]
    states = [_synthetic_state(torch, cuda_ops, c, w, seed) for c, w, seed in specs]
    wants = []
    for (c, w, _), (tb, tab, kv, host, q_gate, ring_k, ring_v) in zip(specs, states):
        ref = _oracle_compressed(oracle, tb, host, q_gate, c)
        aw = np.zeros((H_Q, 258), np.float32)
        oracle.window_attn(q_gate, ring_k, ring_v, aw, c % 256, w, 256, H_Q, H_KV, D, SCALE)
        want = np.zeros((H_Q, D), np.float16)
        oracle.merge_gate(ref, aw, q_gate, want, H_Q, D, 1)
        wants.append(want.astype(np.float32))
    for gen in (1, 2, 3, 4):
        problems, tables = [], []
        for i, ((c, w, _), (tb, tab, kv, host, q_gate, ring_k, ring_v)) in enumerate(zip(specs, states)):
            tables.append(dict(cents_k=tab["cents_k"], cents_v=tab["cents_v"], vq=tab["vq"], k_rotor=tab["rotor_k"],
                               v_rotor=tab["rotor_v"], d_k=tab["d_k"], d_v=tab["d_v"], alpha_k=tb.alpha_k, alpha_v=tb.alpha_v))
            prob = dict(kv)
            prob.update(q_gate=torch.from_numpy(q_gate).cuda().reshape(-1), ring_k=torch.from_numpy(ring_k).cuda().reshape(-1),
                        ring_v=torch.from_numpy(ring_v).cuda().reshape(-1), out=torch.zeros(H_Q * D, dtype=torch.float16, device="cuda"),
                        table_id=i, c_len=c, start_pos=0, win_start=c % 256, win_len=w)
            problems.append(prob)
        bd = BatchedDecode(problems, tables, codebook_in_smem=gen)
        bd.launch(SCALE, 1e7)
        torch.cuda.synchronize()
        assert cuda_ops.lib.khq_b200_device_status() == 0
        for i, prob in enumerate(problems):
            got = prob["out"].float().cpu().numpy().reshape(H_Q, D)
            ok, mx, exc = cases.attention_close(got, wants[i])
            assert ok, f"generation {gen}, sequence {i} (c_len {specs[i][0]}): max abs {mx:.3e} excess {exc:.3e}"
            print(f"configs[3] generation {gen} c_len {specs[i][0]}: max|err| {mx:.2e}")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_prefill_full_length_vs_fp64_twin(cuda_ops, oracle, dtype):
    """configs[4]: T = 8192, both storage types, against the FP64 twin of the reference's own
    attention test (tests/test_gqa_attention_gpu.mojo:36-83) on 66 query rows (the first and last
    rows, both sides of the first tile edge, the rows next to the compressed/raw boundary of the
    prompt path and a random sample) for every head."""
    import torch

    T = 8192
    g = torch.Generator(device="cuda").manual_seed(17)
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    mk = lambda *shape, s=1.0: (torch.randn(*shape, generator=g, device="cuda") * s).to(tdt)
    qg, k, v = mk(1, T, H_Q, 2 * D), mk(1, T, H_KV, D, s=0.25), mk(1, T, H_KV, D)
    if dtype == "bf16":  # keep only values that fp16 (the oracle's storage type) holds exactly
        for t_ in (qg, k, v):
            t_.mul_((t_.half().to(tdt) == t_).to(tdt))
    out = torch.zeros(1, T, H_Q, D, dtype=tdt, device="cuda")
    if dtype == "fp16":
        cuda_ops.gqa_prefill(qg, k, v, out, 1, T, H_Q, H_KV, D, SCALE)
    else:
        from bonsai_mojo_1bit_optimization_t4_cuda_b200.lib import check, current_stream

        check("launch_khq_gqa_prefill_bf16", cuda_ops.lib.launch_khq_gqa_prefill_bf16(
            qg.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, T, H_Q, H_KV, D, SCALE, 0, 0, 0, current_stream()))
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_prefill_status() == 0
    rows = sorted({0, 1, 127, 128, 129, 8063, 8064, 8190, 8191} | set(np.random.default_rng(3).integers(0, T, 57).tolist()))
    kh = np.ascontiguousarray(k[0].float().cpu().numpy().reshape(T, H_KV * D))  # the twin takes fp32 arrays
    vh = np.ascontiguousarray(v[0].float().cpu().numpy().reshape(T, H_KV * D))
    worst = 0.0
    for r in rows:
        want = oracle.gqa_attention_f32(np.ascontiguousarray(qg[0, r].float().cpu().numpy()), kh, vh, r + 1, H_Q, H_KV, D, SCALE)
        got = out[0, r].float().cpu().numpy()
        if dtype == "fp16":
            ok, mx, exc = cases.attention_close(got, want)
        else:  # bf16 storage: 8 mantissa bits in P and in the output
            ok, mx, exc = cases.attention_close(got, want, atol=4e-3, rtol=2e-2)
        worst = max(worst, mx)
        assert ok, f"{dtype} row {r}: max abs {mx:.3e} excess {exc:.3e}"
    print(f"configs[4] {dtype} T=8192, {len(rows)} rows x 24 heads vs FP64: max|err| {worst:.2e}")


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


def test_compress_grouped_rows_ragged_tail_and_run_table(cuda_ops):
    """Large launches give a warp a group of rows (two K rows, four V rows: the in-order sums of the
    group run side by side, the V code search shares one codebook load).  A row count that is not
    a multiple of four (32 768 + 3 rows) and a table-driven launch of 65 runs of 512 rows (33 280
    rows, sources scattered) must write, row for row, what small launches (one row per warp) write."""
    import torch

    tb, tab = _tables(torch)
    rows = 32768 + 3
    g = torch.Generator(device="cuda").manual_seed(17)
    k = torch.randn(rows, D, generator=g, device="cuda").half()
    v = torch.randn(rows, D, generator=g, device="cuda").half()
    full = _compress_all(cuda_ops, torch, tb, tab, k, v, rows)
    per_row = dict(k_mask=64, k_payload=40, v_payload=104, v_shared_meta=4, k_norms=2, k_r_norms=2, v_norms=2, v_r_norms=2)
    for a, n in ((rows - 515, 515), (0, 509), (16384, 1024)):
        part = _compress_all(cuda_ops, torch, tb, tab, k[a:a + n].contiguous(), v[a:a + n].contiguous(), n)
        for key, rb in per_row.items():
            assert torch.equal(full[key].view(torch.uint8)[a * rb:(a + n) * rb], part[key].view(torch.uint8)), (key, a)

    # table-driven launch: run i reads 512 rows from a shuffled place in the source and writes rows
    # 512*perm2[i] ..; V sources sit at a fixed byte distance from the K sources
    lib = cuda_ops.lib
    n_seg, rps = 65, 512
    src = torch.randn(2, n_seg * rps, D, generator=g, device="cuda").half()  # [0] = K rows, [1] = V rows
    rng = np.random.default_rng(3)
    perm_src, perm_dst = rng.permutation(n_seg), rng.permutation(n_seg)
    segs = np.zeros((n_seg, 2), dtype=np.int64)
    for i in range(n_seg):
        segs[i, 0] = src[0].data_ptr() + int(perm_src[i]) * rps * D * 2
        segs[i, 1] = int(perm_dst[i]) * rps
    d_segs = torch.from_numpy(segs).cuda()
    total = n_seg * rps
    out = dict(k_mask=torch.zeros(total * 16, dtype=torch.int32, device="cuda"),
               k_payload=torch.zeros(total * 40, dtype=torch.uint8, device="cuda"),
               v_payload=torch.zeros(total * 104, dtype=torch.uint8, device="cuda"),
               v_shared_meta=torch.zeros(total * 4, dtype=torch.uint8, device="cuda"),
               k_norms=torch.zeros(total, dtype=torch.float16, device="cuda"), k_r_norms=torch.zeros(total, dtype=torch.float16, device="cuda"),
               v_norms=torch.zeros(total, dtype=torch.float16, device="cuda"), v_r_norms=torch.zeros(total, dtype=torch.float16, device="cuda"))
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.launch_khq_compress_batched_fp16(
        d_segs.data_ptr(), n_seg, rps, tab["d_k"].data_ptr(), tab["rotor_k"].data_ptr(), tab["cents_k"].data_ptr(),
        tab["cents_k"].data_ptr(), out["k_mask"].data_ptr(), out["k_norms"].data_ptr(), out["k_r_norms"].data_ptr(),
        out["k_payload"].data_ptr(), out["v_shared_meta"].data_ptr(), D, float(tb.ts_k), float(tb.alpha_k), 0, 0, st)
    assert rc == 0
    rc = lib.launch_khq_compress_batched_fp16(
        d_segs.data_ptr(), n_seg, rps, tab["d_v"].data_ptr(), tab["rotor_v"].data_ptr(), tab["cents_v"].data_ptr(),
        tab["vq"].data_ptr(), out["k_mask"].data_ptr(), out["v_norms"].data_ptr(), out["v_r_norms"].data_ptr(),
        out["v_payload"].data_ptr(), out["v_shared_meta"].data_ptr(), D, float(tb.ts_v), float(tb.alpha_v), 1,
        src[1].data_ptr() - src[0].data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    for i in (0, 7, 64):
        a, b = int(perm_src[i]) * rps, int(perm_dst[i]) * rps
        part = _compress_all(cuda_ops, torch, tb, tab, src[0, a:a + rps].contiguous(), src[1, a:a + rps].contiguous(), rps)
        for key, rb in per_row.items():
            assert torch.equal(out[key].view(torch.uint8)[b * rb:(b + rps) * rb], part[key].view(torch.uint8)), (key, i)


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
