"""Fused pre-step (head RMSNorm + K capture + partial RoPE + ring appends) against the oracle,
with the bars of the reference's own RoPE test (tests/test_rope_gpu.mojo:96-110): rotated
elements within 0.05, everything else bit-identical."""
import numpy as np
import pytest

from cases import D, H_KV, H_Q

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pos", [0, 1, 777, 12345, 130000, 262143])
@pytest.mark.parametrize("has_norms", [True, False])
def test_prestep_vs_oracle(cuda_ops, oracle, pos, has_norms):
    import torch

    rng = np.random.default_rng(pos + 5)
    qg = (rng.standard_normal((H_Q, 2 * D)) * 2).astype(np.float16)
    k = (rng.standard_normal((H_KV, D)) * 3).astype(np.float16)
    v = rng.standard_normal((H_KV, D)).astype(np.float16)
    qw = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    t = dict(qg=dev(qg), k=dev(k), v=dev(v), qw=dev(qw), kw=dev(kw))
    rings = {n: torch.zeros(H_KV * D, dtype=torch.float16, device="cuda") for n in ("k", "v", "u")}
    cuda_ops.prestep(t["qg"], t["k"], t["v"], t["qw"], t["kw"], rings["k"], rings["v"], rings["u"], H_Q, H_KV, D, 64, pos,
                     1e7, 1e-6, has_norms)
    torch.cuda.synchronize()
    c = dict(qg=torch.from_numpy(qg.copy()), k=torch.from_numpy(k.copy()), v=torch.from_numpy(v.copy()))
    crings = {n: torch.zeros(H_KV * D, dtype=torch.float16) for n in ("k", "v", "u")}
    oracle.OracleOps().prestep(c["qg"], c["k"], c["v"], qw, kw, crings["k"], crings["v"], crings["u"], H_Q, H_KV, D, 64, pos,
                               1e7, 1e-6, has_norms)

    def same(a, b, rot_cols):
        a, b = a.cpu().numpy(), b.numpy()
        mask = np.zeros(a.shape, bool)
        mask[..., :64] = rot_cols
        assert np.array_equal(a[~mask].view(np.uint16), b[~mask].view(np.uint16)), "un-rotated elements must be bit-identical"
        assert np.abs(a[mask].astype(np.float32) - b[mask].astype(np.float32)).max(initial=0) <= 0.05

    same(t["qg"].view(H_Q, 2 * D), c["qg"].view(H_Q, 2 * D), True)
    same(t["k"].view(H_KV, D), c["k"].view(H_KV, D), True)
    same(rings["u"].view(H_KV, D), crings["u"].view(H_KV, D), False)  # captured before the rotation
    same(rings["k"].view(H_KV, D), crings["k"].view(H_KV, D), True)
    same(rings["v"].view(H_KV, D), crings["v"].view(H_KV, D), False)
    assert torch.equal(rings["k"].cpu(), t["k"].cpu().reshape(-1)) and torch.equal(rings["v"].cpu(), t["v"].cpu().reshape(-1))


def test_prestep_error_codes(cuda_ops):
    lib = cuda_ops.lib
    assert lib.launch_khq_prestep_fp16(0, 0, 0, 0, 0, 0, 0, 0, 24, 4, 256, 64, 0, 1e7, 1e-6, 1, 0) == -100
    assert lib.launch_khq_prestep_fp16(16, 16, 16, 0, 0, 0, 0, 0, 24, 4, 256, 128, 0, 1e7, 1e-6, 1, 0) == -103
    assert lib.launch_khq_prestep_fp16(16, 8, 16, 0, 0, 0, 0, 0, 24, 4, 256, 64, 0, 1e7, 1e-6, 1, 0) == -104
