"""Context-parallel decode of one long sequence on 2 CPU ranks (gloo) with the oracle backend:
host logic of the N>1 path (partition, per-slice start_pos, all-gather, merge order)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from cases import D, H_KV, H_Q, SCALE
from bonsai_mojo_1bit_optimization_t4_cuda_b200.context_parallel import (ContextParallelDecode, cyclic_local_tokens, partition_context,
                                                                         partition_context_cyclic)


def test_partition_context():
    assert partition_context(131072, 8) == [(i * 16384, (i + 1) * 16384) for i in range(8)]
    p = partition_context(384, 2)
    assert p == [(0, 256), (256, 384)]
    p = partition_context(128, 4)
    assert p == [(0, 128), (128, 128), (128, 128), (128, 128)]
    p = partition_context(1000, 3)  # ragged tail: last chunk is short
    assert p[0][0] == 0 and p[-1][1] == 1000 and all(a[1] == b[0] for a, b in zip(p, p[1:]))
    assert all((lo % 128) == 0 for lo, _ in p)


def test_partition_context_cyclic():
    p = partition_context_cyclic(131072, 8)
    assert [len(x) for x in p] == [128] * 8 and p[3][:3] == [3, 11, 19]
    # a context that grows chunk by chunk stays balanced to within one chunk
    for c_len in (128, 1000, 1152, 4096 + 128):
        for world in (2, 3, 8):
            parts = partition_context_cyclic(c_len, world)
            assert sorted(c for x in parts for c in x) == list(range((c_len + 127) // 128))
            n = [len(x) for x in parts]
            assert max(n) - min(n) <= 1
            assert sum(cyclic_local_tokens(c_len, world, r) for r in range(world)) == c_len


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, c_len, win_len, q, partition="contiguous"):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    sys.path.insert(0, str(root / "tests"))
    os.environ["OMP_NUM_THREADS"] = "2"
    from oracle import khq_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        case = cases.make_case(4711, c_len + win_len, "calib")
        kv_full = cases.compress_with(O.compress, case, c_len)
        if partition == "cyclic":  # this rank's chunks back to back
            mine = partition_context_cyclic(c_len, world)[rank]
            idx = np.concatenate([np.arange(c * 128 * H_KV, min(c_len, (c + 1) * 128) * H_KV) for c in mine]) if mine else np.zeros(0, np.int64)
            lo, hi = 0, len(idx) // H_KV
            kv = {k: torch.from_numpy(np.ascontiguousarray(v[idx])) for k, v in kv_full.items() if k != "near_ties"}
        else:
            lo, hi = partition_context(c_len, world)[rank]
            rows = slice(lo * H_KV, hi * H_KV)
            kv = {k: torch.from_numpy(np.ascontiguousarray(v[rows])) for k, v in kv_full.items() if k != "near_ties"}
        tb = {k: torch.from_numpy(v) for k, v in cases.tables_dict(case["f16"]).items()}
        ring_k = np.zeros((256, H_KV, D), np.float16)
        ring_v = np.zeros((256, H_KV, D), np.float16)
        ws = c_len % 256
        for s in range(win_len):
            ring_k[(ws + s) % 256] = case["k_roped"][c_len + s]
            ring_v[(ws + s) % 256] = case["v"][c_len + s]
        owner = world - 1
        cp = ContextParallelDecode(O.OracleOps(), dist.group.WORLD, kv, tb, lo, hi, case["tables"].alpha_k,
                                   case["tables"].alpha_v, torch.from_numpy(ring_k), torch.from_numpy(ring_v),
                                   owner=owner, splits=4, device="cpu", partition=partition)
        qg = torch.from_numpy(case["q_gate"].copy()).reshape(-1)
        if rank != owner:
            qg.zero_()  # only the owner has this step's query: the broadcast must deliver it
        out = cp.step(qg, ws, win_len, SCALE).float().numpy().reshape(H_Q, D)
        if rank == 0:
            # single-rank answer through the same oracle
            ops = O.OracleOps()
            f, t = case["f16"], case["tables"]
            ac = np.zeros((H_Q, 258), np.float32)
            aw = np.zeros((H_Q, 258), np.float32)
            ops.attn(case["q_gate"], kv_full["k_payload"], kv_full["v_payload"], kv_full["v_shared_meta"],
                     kv_full["k_mask"], kv_full["k_norms"], kv_full["k_r_norms"], kv_full["v_norms"],
                     kv_full["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"], f["rotor_v"], f["d_k"],
                     f["d_v"], ac, None, H_Q, H_Q, 1, c_len, c_len, 6, SCALE, t.alpha_k, t.alpha_v, 1e7, 0, 1)
            ops.window_attn(case["q_gate"], ring_k, ring_v, aw, ws, win_len, 256, H_Q, H_KV, D, SCALE)
            ref = np.zeros((H_Q, D), np.float16)
            ops.merge_gate(ac, aw, case["q_gate"], ref, H_Q, D, True, True)
            ok, mx, exc = cases.attention_close(out, ref.astype(np.float32))
            q.put(("ok" if ok else "bad", mx, exc))
        # every rank must hold the same answer
        t_out = torch.from_numpy(out.copy())
        gathered = [torch.zeros_like(t_out) for _ in range(world)]
        dist.all_gather(gathered, t_out)
        assert all(torch.equal(gathered[0], g) for g in gathered)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,c_len,win_len,partition", [(2, 384, 128, "contiguous"), (2, 128, 77, "contiguous"),
                                                            (3, 1000, 1, "contiguous"), (2, 640, 128, "cyclic"), (3, 1000, 5, "cyclic")])
def test_context_parallel_matches_single_rank(world, c_len, win_len, partition):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, c_len, win_len, q, partition)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    status, mx, exc = q.get(timeout=5)
    assert status == "ok", (mx, exc)
