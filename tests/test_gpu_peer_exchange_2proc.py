"""The peer-store exchange across two real processes on two GPUs (CUDA IPC buffers, flags over
NVLink) against the NCCL all-gather path: same bits.  Skipped on a box with fewer than two GPUs.
NVLS is switched off in NCCL and the library's own exchange uses plain peer stores (no multimem), so a
rank that died would not leave the other GPU with a bound multicast object."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    sys.path.insert(0, str(root / "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch
    import torch.distributed as dist

    import cases
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.context_parallel import ContextParallelDecode, partition_context
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps
    from oracle import khq_oracle as O

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = False
    try:
        c_len, win_len = 1024, 100
        case = cases.make_case(4712, c_len + win_len, "calib")
        kv_full = cases.compress_with(O.compress, case, c_len)
        lo, hi = partition_context(c_len, world)[rank]
        rows = slice(lo * 4, hi * 4)
        kv = {k: torch.from_numpy(np.ascontiguousarray(v[rows])).to(dev) for k, v in kv_full.items() if k != "near_ties"}
        tb = {k: torch.from_numpy(v).to(dev) for k, v in cases.tables_dict(case["f16"]).items()}
        ring_k = np.zeros((256, 4, 256), np.float16)
        ring_v = np.zeros((256, 4, 256), np.float16)
        ws = c_len % 256
        for s in range(win_len):
            ring_k[(ws + s) % 256], ring_v[(ws + s) % 256] = case["k_roped"][c_len + s], case["v"][c_len + s]
        owner = world - 1
        ops = CudaOps()
        outs = {}
        for exchange in ("peer", "collective"):
            cp = ContextParallelDecode(ops, dist.group.WORLD, kv, tb, lo, hi, case["tables"].alpha_k, case["tables"].alpha_v,
                                       torch.from_numpy(ring_k).to(dev).reshape(-1), torch.from_numpy(ring_v).to(dev).reshape(-1),
                                       owner=owner, splits=8, device=dev, exchange=exchange)
            cp.status_every = 1
            res = []
            for step in range(3):  # three steps: both slot parities and a reused one
                qg = torch.from_numpy(case["q_gate"].copy()).to(dev).reshape(-1)
                if rank != owner:
                    qg.zero_()  # only the owner has the query: the exchange must deliver it
                res.append(cp.step(qg, ws, win_len, cases.SCALE).clone())
            torch.cuda.synchronize()
            cp.close()
            outs[exchange] = res
        ok = all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for a, b in zip(outs["peer"], outs["collective"]))
        ok = ok and all(torch.equal(outs["peer"][0], r) for r in outs["peer"][1:])
        if rank == 0:
            # and the answer is the single-GPU one
            f, t = case["f16"], case["tables"]
            oo = O.OracleOps()
            ac, aw = np.zeros((24, 258), np.float32), np.zeros((24, 258), np.float32)
            oo.attn(case["q_gate"], kv_full["k_payload"], kv_full["v_payload"], kv_full["v_shared_meta"], kv_full["k_mask"],
                    kv_full["k_norms"], kv_full["k_r_norms"], kv_full["v_norms"], kv_full["v_r_norms"], f["cents_k"], f["cents_v"],
                    f["vq"], f["rotor_k"], f["rotor_v"], f["d_k"], f["d_v"], ac, None, 24, 24, 1, c_len, c_len, 6, cases.SCALE,
                    t.alpha_k, t.alpha_v, 1e7, 0, 1)
            oo.window_attn(case["q_gate"], ring_k, ring_v, aw, ws, win_len, 256, 24, 4, 256, cases.SCALE)
            ref = np.zeros((24, 256), np.float16)
            oo.merge_gate(ac, aw, case["q_gate"], ref, 24, 256, True, True)
            good, mx, exc = cases.attention_close(outs["peer"][0].float().cpu().numpy().reshape(24, 256), ref.astype(np.float32))
            ok = ok and good
    finally:
        q.put((rank, bool(ok)))
        dist.destroy_process_group()


def test_peer_exchange_across_two_processes_matches_all_gather():
    import torch
    import torch.multiprocessing as mp

    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    got = dict(q.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}, got
