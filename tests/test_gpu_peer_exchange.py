"""The peer-memory exchange of context-parallel partials (publish + wait-merge kernels).  The ranks
are emulated inside one process on one GPU: every "rank" owns a slot buffer and a flag array, the
publish launches of all ranks run one after the other on one stream, then every rank's merge runs
-- by then every flag is up, so no kernel ever waits on another launch of the same GPU."""
import numpy as np
import pytest

from cases import D, H_Q

pytestmark = pytest.mark.gpu
PART = 258


def _partials(torch, world, per_rank, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    p = torch.randn(world, per_rank, H_Q, PART, generator=g, device="cuda")
    p[..., D] = torch.randn(world, per_rank, H_Q, generator=g, device="cuda") * 3.0   # running maxima
    p[..., D + 1] = torch.rand(world, per_rank, H_Q, generator=g, device="cuda") * 50 + 1.0  # sums of exp
    p[1, 1, :, :D] = 0.0                                                              # a neutral slot
    p[1, 1, :, D] = -1e20
    p[1, 1, :, D + 1] = 0.0
    return p


@pytest.mark.parametrize("world", [2, 3, 8])
def test_publish_then_merge_equals_gathered_merge(cuda_ops, world):
    import torch

    per_rank, n_slots = 2, 2 * world
    slots = [torch.zeros(2, n_slots, H_Q, PART, dtype=torch.float32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    peer_slots = torch.tensor([s.data_ptr() for s in slots], dtype=torch.int64, device="cuda")
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device="cuda")
    qg = torch.randn(H_Q * 2 * D, device="cuda").half()
    assert cuda_ops.lib.khq_b200_device_status_clear() >= 0
    for epoch in (1, 2, 3):  # three steps: both parities, and a parity reused
        parts = _partials(torch, world, per_rank, 40 + epoch)
        par = epoch & 1
        for r in range(world):
            cuda_ops.publish_partials(parts[r].contiguous(), per_rank, peer_slots, peer_flags, world, r, r * per_rank,
                                      par * n_slots, epoch)
        want = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
        cuda_ops.merge_slots_gate(parts.reshape(n_slots, H_Q, PART).contiguous(), n_slots, qg, want, H_Q, D)
        for r in range(world):
            got = torch.full((H_Q * D,), float("nan"), dtype=torch.float16, device="cuda")
            cuda_ops.merge_slots_wait_gate(slots[r][par], flags[r], world, epoch, n_slots, qg, got, H_Q, D)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"rank {r} epoch {epoch}"
            assert flags[r].tolist() == [epoch] * world
    assert cuda_ops.lib.khq_b200_device_status() == 0


def test_publish_bytes_and_wait_flag(cuda_ops):
    """The owner's q_gate travels the same way: bytes into every buffer, then a flag word; the
    consumer queues a one-thread wait in front of the kernels that read it."""
    import torch

    world = 3
    bufs = [torch.zeros(65536, dtype=torch.uint8, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world + 1, dtype=torch.int32, device="cuda") for _ in range(world)]
    peer_bufs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device="cuda")
    qg = torch.randn(H_Q * 2 * D, device="cuda").half()
    assert cuda_ops.lib.khq_b200_device_status_clear() >= 0
    cuda_ops.publish_bytes(qg, qg.numel() * 2, peer_bufs, 4096, peer_flags, world, world, 7)
    for r in range(world):
        cuda_ops.wait_flag(flags[r][world:], 7)
        torch.cuda.synchronize()
        assert torch.equal(bufs[r][4096:4096 + qg.numel() * 2].view(torch.float16), qg)
        assert flags[r].tolist() == [0] * world + [7]
    assert cuda_ops.lib.khq_b200_device_status() == 0
    cuda_ops.wait_flag(flags[0][world:], 8, max_polls=1000)  # nothing publishes epoch 8
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_device_status_clear() == 3
    lib = cuda_ops.lib
    assert lib.launch_khq_publish_bytes(0, 16, 16, 0, 16, 0, 2, 1, 0) == -100
    assert lib.launch_khq_publish_bytes(16, 24, 16, 0, 16, 0, 2, 1, 0) == -104
    assert lib.launch_khq_wait_flag(0, 1, 0, 0) == -100


def test_wait_runs_out_and_reports(cuda_ops):
    """A producer that never publishes: the merge kernel gives up after its poll budget, records
    status 3 and returns; the context stays usable."""
    import torch

    world, n_slots = 2, 4
    slots = torch.zeros(n_slots, H_Q, PART, dtype=torch.float32, device="cuda")
    slots[..., D + 1] = 1.0
    flags = torch.tensor([5, 4], dtype=torch.int32, device="cuda")  # producer 1 is still at epoch 4
    qg = torch.zeros(H_Q * 2 * D, dtype=torch.float16, device="cuda")
    out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
    assert cuda_ops.lib.khq_b200_device_status_clear() >= 0
    cuda_ops.merge_slots_wait_gate(slots, flags, world, 5, n_slots, qg, out, H_Q, D, max_polls=2000)
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_device_status_clear() == 3
    assert cuda_ops.lib.khq_b200_device_status() == 0
    # an epoch that wrapped around 2^32 still compares as "reached"
    flags.copy_(torch.tensor([2, 1], dtype=torch.int32))
    cuda_ops.merge_slots_wait_gate(slots, flags, world, (1 << 32) - 3 + 4, n_slots, qg, out, H_Q, D, max_polls=2000)
    torch.cuda.synchronize()
    assert cuda_ops.lib.khq_b200_device_status_clear() == 0


def test_peer_exchange_error_codes(cuda_ops):
    lib = cuda_ops.lib
    assert lib.launch_khq_publish_partials_fp32(0, 2, 0, 0, 2, 0, 0, 0, 1, 0) == -100
    assert lib.launch_khq_publish_partials_fp32(16, 2, 16, 16, 2, 2, 0, 0, 1, 0) == -100   # rank outside the group
    assert lib.launch_khq_publish_partials_fp32(8, 2, 16, 16, 2, 0, 0, 0, 1, 0) == -104
    assert lib.launch_khq_merge_slots_wait_gate_fp16(16, 16, 2, 1, 0, 16, 16, 24, 256, 0, 0) == -100
    assert lib.launch_khq_merge_slots_wait_gate_fp16(16, 16, 2, 1, 4, 16, 16, 24, 128, 0, 0) == -103
