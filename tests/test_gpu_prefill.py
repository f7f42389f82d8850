"""Causal GQA prefill attention (launch_khq_gqa_prefill_fp16) against the oracle."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


# tcgen05 / tensor-memory kernel (the default; also forced into each of its two work distributions)
# and the warp-level mma.sync kernel
KERNELS = ["tc5", "mma", "tc5-one-item-per-cta", "tc5-persistent"]


def _run(cuda_ops, qg, k, v, B, T, H_q=H_Q, H_kv=H_KV, kernel="tc5"):
    import torch

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = torch.full((B, T, H_q, D), float("nan"), dtype=torch.float16, device="cuda")
    assert cuda_ops.lib.khq_b200_prefill_select(1 if kernel == "mma" else 0) == 0
    assert cuda_ops.lib.khq_b200_prefill_tc5_items_per_cta({"tc5-one-item-per-cta": 1, "tc5-persistent": 1 << 20}.get(kernel, 0)) == 0
    try:
        cuda_ops.gqa_prefill(dev(qg), dev(k), dev(v), out, B, T, H_q, H_kv, D, SCALE)
        torch.cuda.synchronize()
    finally:
        cuda_ops.lib.khq_b200_prefill_select(0)
        cuda_ops.lib.khq_b200_prefill_tc5_items_per_cta(0)
    assert cuda_ops.lib.khq_b200_prefill_status() == 0
    return out.float().cpu().numpy()


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("T", [1, 64, 65, 128, 129, 200, 257, 321, 384, 1000])
def test_prefill_vs_oracle(cuda_ops, oracle, T, kernel):
    B = 2
    rng = np.random.default_rng(50 + T)
    qg = rng.standard_normal((B, T, H_Q, 2 * D)).astype(np.float16)
    sk, sv = cases.synth.channel_scales(rng), cases.synth.channel_scales(rng)
    k = np.stack([cases.synth.make_kv(rng, T, sk, sv)[0] for _ in range(B)])
    v = np.stack([cases.synth.make_kv(rng, T, sk, sv)[1] for _ in range(B)])
    k = (k.astype(np.float32) * 0.25).astype(np.float16)  # keep the scores in a softmax-friendly range
    got = _run(cuda_ops, qg, k, v, B, T, kernel=kernel)
    for b in range(B):
        ref = oracle.gqa_prefill(qg[b], k[b], v[b], T, H_Q, H_KV, D, SCALE)
        ok, mx, exc = cases.attention_close(got[b], ref)
        assert ok, f"T={T} batch {b}: max abs {mx:.3e}, excess {exc:.3e}"


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("H_q,H_kv,seq", [(24, 4, 8), (4, 2, 16), (4, 2, 1)])
def test_prefill_on_reference_fixture_fills(cuda_ops, oracle, H_q, H_kv, seq, kernel):
    """The reference's deterministic fills (tests/test_gqa_attention_gpu.mojo:105-109) and cases
    (:188-194): every prompt row carries the fixture query, so row seq-1 of the prefill is the
    reference test's single decode row over `seq` cache rows; bar 2e-3 of the largest output."""
    d = D
    i = np.arange(H_q * 2 * d, dtype=np.int64)
    qg1 = ((((i * 7919 + 1013) % 2000).astype(np.float32) * np.float32(0.001)) - np.float32(1.0)).astype(np.float16)
    j = np.arange(seq * H_kv * d, dtype=np.int64)
    k = ((((j * 6271 + 5003) % 2000).astype(np.float32) * np.float32(0.001)) - np.float32(1.0)).astype(np.float16)
    v = ((((j * 4931 + 7919) % 2000).astype(np.float32) * np.float32(0.002)) - np.float32(2.0)).astype(np.float16)
    qg = np.tile(qg1.reshape(1, 1, H_q, 2 * d), (1, seq, 1, 1))
    got = _run(cuda_ops, qg, k.reshape(1, seq, H_kv, d), v.reshape(1, seq, H_kv, d), 1, seq, H_q, H_kv,
               kernel=kernel)[0, seq - 1]
    want = oracle.gqa_attention_f32(qg1.astype(np.float32), k.astype(np.float32), v.astype(np.float32), seq, H_q, H_kv,
                                    d, 1.0 / np.sqrt(d))
    rel = np.abs(got - want).max() / (np.abs(want).max() + 1e-12)
    assert rel <= 2e-3, rel


def test_prefill_error_codes(cuda_ops):
    lib = cuda_ops.lib
    for fn in (lib.launch_khq_gqa_prefill_fp16, lib.launch_khq_gqa_prefill_tc5_fp16, lib.launch_khq_gqa_prefill_mma_fp16):
        assert fn(0, 0, 0, 0, 0, 8, 24, 4, 256, 0.0625, 0, 0, 0, 0) == -100
        assert fn(0, 0, 0, 0, 1, 8, 24, 4, 128, 0.0625, 0, 0, 0, 0) == -103
        assert fn(8, 0, 0, 0, 1, 8, 24, 4, 256, 0.0625, 0, 0, 0, 0) == -104
    assert lib.khq_b200_prefill_select(2) == -100
    assert lib.khq_b200_prefill_tc5_items_per_cta(-1) == -100


@pytest.mark.parametrize("mode", [1, 3, 1 << 20])
def test_prefill_tc5_against_the_warp_level_kernel_on_random_shapes(cuda_ops, mode):
    """Twelve random (batch, length) shapes per work distribution -- lengths around and off the
    128-row block size, several items per persistent CTA -- each launched three times back to back:
    the tcgen05 kernel must agree with the warp-level kernel (an independent implementation) and
    repeat itself bit for bit (its barriers carry no state from one item or launch to the next)."""
    import torch

    lib = cuda_ops.lib
    rng = np.random.default_rng(mode % 1000)
    try:
        for _ in range(12):
            B = int(rng.integers(1, 6))
            T = int(rng.choice([int(rng.integers(1, 140)), int(rng.integers(140, 1200)), 128 * int(rng.integers(1, 12)),
                                128 * int(rng.integers(1, 12)) + 1, int(rng.integers(1200, 2600))]))
            g = torch.Generator(device="cuda").manual_seed(int(rng.integers(1 << 30)))
            qg = torch.randn(B, T, H_Q, 2 * D, generator=g, device="cuda").half()
            k = (torch.randn(B, T, H_KV, D, generator=g, device="cuda") * 0.25).half()
            v = torch.randn(B, T, H_KV, D, generator=g, device="cuda").half()
            ref = torch.zeros(B, T, H_Q, D, dtype=torch.float16, device="cuda")
            assert lib.khq_b200_prefill_select(1) == 0
            cuda_ops.gqa_prefill(qg, k, v, ref, B, T, H_Q, H_KV, D, SCALE)
            assert lib.khq_b200_prefill_select(0) == 0 and lib.khq_b200_prefill_tc5_items_per_cta(mode) == 0
            outs = []
            for _rep in range(3):
                out = torch.full((B, T, H_Q, D), float("nan"), dtype=torch.float16, device="cuda")
                cuda_ops.gqa_prefill(qg, k, v, out, B, T, H_Q, H_KV, D, SCALE)
                outs.append(out)
            torch.cuda.synchronize()
            assert lib.khq_b200_prefill_status() == 0
            ok, mx, exc = cases.attention_close(outs[0].float().cpu().numpy(), ref.float().cpu().numpy())
            assert ok, f"B={B} T={T} mode={mode}: max abs {mx:.3e}, excess {exc:.3e}"
            for o in outs[1:]:
                assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16)), f"B={B} T={T} mode={mode}: not repeatable"
    finally:
        lib.khq_b200_prefill_select(0)
        lib.khq_b200_prefill_tc5_items_per_cta(0)


@pytest.mark.parametrize("mode", [0, 1, 1 << 20])
@pytest.mark.parametrize("T", [77, 128, 700])
def test_prefill_bf16_vs_torch_fp32(cuda_ops, T, mode):
    """bf16 tensors: the tcgen05 kernel with bf16 operands against a plain PyTorch fp32 reference of
    the same op on the same (bf16-rounded) inputs.  bf16 keeps 8 mantissa bits, so the bar is the
    storage type's: |err| <= 4e-3 + 2e-2*|ref| (probabilities and the output are rounded to bf16)."""
    import torch

    B = 2
    g = torch.Generator(device="cuda").manual_seed(300 + T)
    qg = torch.randn(B, T, H_Q, 2 * D, generator=g, device="cuda").bfloat16()
    k = (torch.randn(B, T, H_KV, D, generator=g, device="cuda") * 0.25).bfloat16()
    v = torch.randn(B, T, H_KV, D, generator=g, device="cuda").bfloat16()
    out = torch.full((B, T, H_Q, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    lib = cuda_ops.lib
    assert lib.khq_b200_prefill_tc5_items_per_cta(mode) == 0
    try:
        cuda_ops.gqa_prefill(qg, k, v, out, B, T, H_Q, H_KV, D, SCALE)
        torch.cuda.synchronize()
    finally:
        lib.khq_b200_prefill_tc5_items_per_cta(0)
    assert lib.khq_b200_prefill_status() == 0
    q = qg[..., :D].float().permute(0, 2, 1, 3)                       # (B, H_q, T, D)
    gate = qg[..., D:].float().permute(0, 2, 1, 3)
    kk = k.float().repeat_interleave(H_Q // H_KV, dim=2).permute(0, 2, 1, 3)
    vv = v.float().repeat_interleave(H_Q // H_KV, dim=2).permute(0, 2, 1, 3)
    s = (q @ kk.transpose(-1, -2)) * SCALE
    s = s.masked_fill(torch.ones(T, T, device="cuda", dtype=torch.bool).triu(1), float("-inf"))
    ref = (torch.softmax(s, dim=-1) @ vv) * torch.sigmoid(gate)
    ref = ref.permute(0, 2, 1, 3)
    err = (out.float() - ref).abs()
    lim = 4e-3 + 2e-2 * ref.abs()
    assert bool((err <= lim).all()), f"T={T}: max abs {err.max().item():.3e}, worst excess {(err - lim).max().item():.3e}"


@pytest.mark.parametrize("entry", ["launch_khq_gqa_prefill_tc5_fp16", "launch_khq_gqa_prefill_mma_fp16"])
def test_prefill_honours_batch_strides(cuda_ops, oracle, entry):
    """Batch strides larger than one prompt (each prompt sits in a max_seq-sized cache slab, as the
    reference's KV cache rows do): rows past T of a slab must be neither read into the result nor
    written."""
    import torch

    B, T, S = 3, 150, 256  # S = rows per slab
    rng = np.random.default_rng(77)
    qg = torch.from_numpy(rng.standard_normal((B, S, H_Q, 2 * D)).astype(np.float16)).cuda()
    k = torch.from_numpy((rng.standard_normal((B, S, H_KV, D)) * 0.25).astype(np.float16)).cuda()
    v = torch.from_numpy(rng.standard_normal((B, S, H_KV, D)).astype(np.float16)).cuda()
    k[:, T:] = float("nan")  # anything read from beyond the prompt would poison the output
    v[:, T:] = float("nan")
    out = torch.full((B, S, H_Q, D), -7.0, dtype=torch.float16, device="cuda")
    fn = getattr(cuda_ops.lib, entry)
    rc = fn(qg.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, T, H_Q, H_KV, D, SCALE, S * H_Q * 2 * D,
            S * H_KV * D, S * H_Q * D, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_prefill_status() == 0
    assert bool((out[:, T:] == -7.0).all()), "rows past the prompt were written"
    got = out[:, :T].float().cpu().numpy()
    assert np.isfinite(got).all()
    for b in range(B):
        ref = oracle.gqa_prefill(qg[b, :T].cpu().numpy(), k[b, :T].cpu().numpy(), v[b, :T].cpu().numpy(), T, H_Q, H_KV, D, SCALE)
        ok, mx, exc = cases.attention_close(got[b], ref)
        assert ok, f"{entry} batch {b}: max abs {mx:.3e}, excess {exc:.3e}"
