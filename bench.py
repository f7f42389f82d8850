#!/usr/bin/env python
"""Benchmark of the KHQ decode-attention path on B200.

Default workload (the benchmark specification's configuration 3): batched decode of 256 independent sequences with contexts
uniform in [4096, 32768] (compressed prefix + raw window of 128..256 tokens), 16 attention layers,
H_q 24 / H_kv 4 / head_dim 256, fp16 payloads, fp32 accumulate.  A "step" generates one token for
every sequence: per layer one batched launch over all sequences.  Seeded synthetic state (the
reference measures on real weights, which are not available): see the package's ``engine.py``.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value``: tokens/s with all state resident in HBM.  ``e2e``: the same
step through ``BatchEngine.decode_step`` with this step's q/K/V coming from pinned host memory
and the outputs copied back.  ``roofline``: algorithmic payload bytes of one layer launch divided
by that launch's CUDA-event duration, against the measured copy bandwidth.  ``cpu_baseline``: the
CPU port of the reference math (oracle/) on a bounded sample of the same workload.
With N>1 (torchrun, one rank per GPU) every rank owns its own 256 sequences: sharding is by
sequence with no collective, so scaling is weak by construction.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

METRIC = "KHQ batched decode attention throughput (16 attention layers)"
UNIT = "tok/s"
N_LAYERS = 16
LAYER_IDS = [4 * i + 3 for i in range(N_LAYERS)]  # Bonsai-27B's full-attention layers


# dram bytes per algorithmic byte of the batched decode kernel, from one ncu capture of an
# 8-sequence launch (117.0 MB read + 0.4 MB written for 116 604 928 algorithmic bytes); the ratio
# does not depend on the number of rows
NCU_TRAFFIC_RATIO = 1.0034


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=256, help="sequences per GPU")
    ap.add_argument("--ctx-min", type=int, default=4096)
    ap.add_argument("--ctx-max", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--cpu-sample-mult", type=int, default=4, help="CPU sample = mult x host threads sequences")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--prefill-batch", type=int, default=4, help="prompts per GPU (--workload prefill)")
    ap.add_argument("--prefill-len", type=int, default=8192, help="prompt length (--workload prefill)")
    ap.add_argument("--prefill-dtype", default="fp16", choices=["fp16", "bf16"], help="storage type of the prefill tensors")
    ap.add_argument("--prefill-kernel", default="tc5", choices=["tc5", "mma"],
                    help="tc5: tcgen05 / tensor-memory kernel; mma: warp-level mma.sync kernel")
    ap.add_argument("--workload", default="batched", choices=["batched", "long", "prefill", "compress", "single", "loop"],
                    help="batched = configuration 3 of the benchmark specification (default); long = configuration 2, one 131072-token sequence "
                         "split by context range over the ranks")
    ap.add_argument("--long-ctx", type=int, default=131072)
    ap.add_argument("--splits", type=int, default=32)
    ap.add_argument("--exchange", default="peer", choices=["peer", "collective"],
                    help="--workload long on N>1 GPUs: partials stored into the peers' buffers over NVLink (peer) or "
                         "one NCCL all-gather (collective)")
    ap.add_argument("--partition", default="contiguous", choices=["contiguous", "cyclic"],
                    help="--workload long / long_context: contiguous context ranges, or 128-token chunks dealt cyclically")
    ap.add_argument("--tokens-per-item", type=int, default=0,
                    help="largest work item of the batched decode in tokens (0: the library's planner chooses)")
    ap.add_argument("--cp-engine", default="persistent", choices=["persistent", "splits"],
                    help="--workload long / long_context: each rank's slice and the raw window as one launch of the persistent "
                         "batched kernel, or the drop-in split launches (--splits) plus the window launch")
    ap.add_argument("--kernel", default="auto", choices=["auto", "cuda-core", "mma", "tc5", "tc5w"],
                    help="generation of the batched decode kernel")
    return ap.parse_args()


def workload(args, rank: int):
    """Per-rank contexts: total ctx ~ U{ctx_min..ctx_max}, window ~ U{128..256}, compressed length
    = 128 * floor((ctx - window) / 128)."""
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth

    rng = np.random.default_rng(synth.seed_for(3, 0, rank))
    ctx = rng.integers(args.ctx_min, args.ctx_max + 1, size=args.seqs)
    win = rng.integers(128, 257, size=args.seqs)
    c_len = 128 * ((ctx - win) // 128)
    # whatever is left over stays raw; at most 255 tokens, the largest window the attention ever sees (at 256 the
    # state machine compresses the 128 oldest before it attends)
    win = np.minimum(ctx - c_len, 255)
    return c_len.astype(np.int64), win.astype(np.int64)


def make_tables(n_layers: int):
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth

    out = []
    for li in range(n_layers):
        rng = np.random.default_rng(synth.seed_for(3, LAYER_IDS[li % N_LAYERS]))
        k, v = synth.make_kv(rng, 128)
        # identity K rotor: what the reference's calibration writes (src/khq/calib.mojo:386-390)
        out.append(synth.make_tables(rng, LAYER_IDS[li % N_LAYERS], k.reshape(-1, 256), v.reshape(-1, 256),
                                     vq_scale=1.0 / 16.0, k_rotor_identity=True))
    return out


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for nm, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU port of the reference math on a bounded sample (test infrastructure used as a baseline only)
# ------------------------------------------------------------------------------------------------
def random_payload(rng, n_tok: int):
    """Valid KHQ code words drawn directly (the decode cost does not depend on their values):
    symbols with the Gaussian cell probabilities of the 0.47/1.60 sigma thresholds, at most 50
    outliers per row, random residual nibbles / signs / VQ fields, plausible fp16 norms."""
    rows = n_tok * 4
    lut = np.repeat(np.arange(4, dtype=np.uint32), [93, 67, 68, 28])  # 0.36 / 0.26 / 0.27 / 0.11
    sym = lut[rng.integers(0, 256, size=(rows, 256), dtype=np.uint8)]
    over = (np.cumsum(sym == 3, axis=1) > 50) & (sym == 3)
    sym[over] = 2
    sh = (2 * (np.arange(256) % 16)).astype(np.uint32)
    mask = np.zeros((rows, 16), np.uint32)
    for w in range(16):
        mask[:, w] = (sym[:, 16 * w:16 * w + 16] << sh[:16]).sum(axis=1, dtype=np.uint32)
    kp = rng.integers(0, 256, size=(rows, 40), dtype=np.uint8)
    kp[:, 0:4] = np.frombuffer(np.uint32(1000).tobytes(), np.uint8)
    kp[:, 36] = 2
    kp[:, 37:] = 0
    vp = rng.integers(0, 256, size=(rows, 104), dtype=np.uint8)
    f16 = lambda lo, hi: rng.uniform(lo, hi, size=rows).astype(np.float16)
    return dict(k_mask=mask, k_payload=kp, v_payload=vp, k_norms=f16(10, 40), k_r_norms=f16(0.01, 0.1),
                v_norms=f16(10, 40), v_r_norms=f16(0.5, 1.5),
                v_shared_meta=np.ascontiguousarray(rng.uniform(0.01, 0.1, size=rows).astype(np.float32)).view(np.uint8).reshape(rows, 4))


class CpuSample:
    """n_seqs sequences of the workload's context distribution, ONE layer, decoded through the
    oracle (compressed region + window + merge + gate): one sequence per host thread."""

    def __init__(self, args, threads: int):
        # one oracle call spreads over the 4 kv-heads with OpenMP; sequences run on a thread pool
        # set, not defaulted: torchrun exports OMP_NUM_THREADS=1 to its workers
        os.environ["OMP_NUM_THREADS"] = "4"
        from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth
        from oracle import khq_oracle as O

        O.build()
        self.O, self.ops, self.threads, self.args = O, O.OracleOps(), threads, args
        self.pool = max(1, threads // 4)
        n_seqs = min(args.seqs, 64, max(2, args.cpu_sample_mult * self.pool))
        c_len, win = workload(args, 0)
        self.tb = make_tables(1)[0]
        self.f = self.tb.as_f16()
        rng = np.random.default_rng(synth.seed_for(3, 3, 999))
        self.probs = []
        bases = [random_payload(rng, int(c_len[:n_seqs].max())) for _ in range(min(4, n_seqs))]
        for i in range(n_seqs):
            cl, wl = int(c_len[i]), int(win[i])
            p = {k: v[:cl * 4] for k, v in bases[i % len(bases)].items()}
            p.update(ring_k=rng.standard_normal((256, 4, 256)).astype(np.float16),
                     ring_v=rng.standard_normal((256, 4, 256)).astype(np.float16), cl=cl, wl=wl, ws=cl % 256,
                     q=synth.make_q_gate(rng, cl + wl - 1))
            self.probs.append(p)
        self.n_seqs = n_seqs
        self.ctx = (c_len[:n_seqs] + win[:n_seqs])

    def _one(self, p):
        f, tb, ops = self.f, self.tb, self.ops
        ac = np.zeros((24, 258), np.float32)
        aw = np.zeros((24, 258), np.float32)
        out = np.zeros((24, 256), np.float16)
        ops.attn(p["q"], p["k_payload"], p["v_payload"], p["v_shared_meta"], p["k_mask"], p["k_norms"], p["k_r_norms"],
                 p["v_norms"], p["v_r_norms"], f["cents_k"], f["cents_v"], f["vq"], f["rotor_k"], f["rotor_v"],
                 f["d_k"], f["d_v"], ac, None, 24, 24, 1, p["cl"], p["cl"], 6, 1 / 16, tb.alpha_k, tb.alpha_v, 1e7, 0, 1)
        ops.window_attn(p["q"], p["ring_k"], p["ring_v"], aw, p["ws"], p["wl"], 256, 24, 4, 256, 1 / 16)
        ops.merge_gate(ac, aw, p["q"], out, 24, 256, True, True)
        return out

    def time_once(self) -> float:
        from concurrent.futures import ThreadPoolExecutor

        t0 = time.perf_counter()
        with ThreadPoolExecutor(self.pool) as ex:
            list(ex.map(self._one, self.probs))
        return time.perf_counter() - t0

    def result(self, dt: float):
        # n_seqs sequences advanced by one LAYER in dt; one token needs `layers` layer steps
        tok_s = self.n_seqs / (dt * self.args.layers)
        return {"value": tok_s, "unit": UNIT, "cores": self.threads, "kind": "port",
                "sample": f"{self.n_seqs} sequences (ctx {int(self.ctx.min())}..{int(self.ctx.max())}) x 1 layer in "
                          f"{dt:.2f} s on {self.threads} host threads, scaled to {self.args.layers} layers; "
                          "code words drawn at random (decode cost is value-independent)"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    t_all = time.perf_counter()
    cores = os.cpu_count() or 1
    smp = CpuSample(args, cores)
    for _ in range(min(args.warmup, 1)):
        smp.time_once()
    reps = max(1, min(args.steps, 5))
    dt = float(np.mean([smp.time_once() for _ in range(reps)]))
    base = smp.result(dt)
    v = base["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * args.seqs / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, world), "cpu_baseline": base,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU KHQ kernel: this is the CPU port of its math (oracle/) on the host cores; "
                "timed repetitions of the bounded sample: %d" % reps,
        "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line), flush=True)


def config_dict(args, world):
    return {"workload": "BASELINE configs[3]: batched decode, %d sequences per GPU, ctx U[%d,%d] = KHQ-compressed "
                        "prefix + raw window 128..256, %d attention layers, H_q 24 / H_kv 4 / d 256" %
                        (args.seqs, args.ctx_min, args.ctx_max, args.layers),
            "sequences_per_gpu": args.seqs, "layers": args.layers, "sharding": "by sequence, no collective",
            "l2": "inputs larger than L2: every layer launch streams GBs of payload against a 126 MB L2",
            "world": world}


# ------------------------------------------------------------------------------------------------
def long_measure(args, rank, world, dev, steps, warm):
    """Configuration 2 of the benchmark specification on an initialised process group: one sequence, --long-ctx compressed
    tokens + 256 raw ring tokens, one layer, the compressed region partitioned by context range over the
    ranks; per step every rank computes its (24, 258) partial, the partials are exchanged (peer stores
    with flags, or one NCCL all-gather), every rank merges + gates.  Returns microseconds per layer-step
    (max over ranks) and what was checked."""
    import torch
    import torch.distributed as dist

    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import lib as khqlib
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.context_parallel import (ContextParallelDecode, cyclic_local_tokens,
                                                                             partition_context)
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps

    ops = CudaOps()
    tb = make_tables(1)[0]
    f = tb.as_f16()
    tab = {k: torch.from_numpy(v).to(dev) for k, v in dict(cents_k=f["cents_k"], cents_v=f["cents_v"], vq=f["vq"],
                                                            rotor_k=f["rotor_k"], rotor_v=f["rotor_v"], d_k=f["d_k"],
                                                            d_v=f["d_v"]).items()}
    if args.partition == "cyclic":
        lo, hi = 0, cyclic_local_tokens(args.long_ctx, world, rank)
    else:
        lo, hi = partition_context(args.long_ctx, world)[rank]
    n = hi - lo
    rows = max(n, 1) * 4
    g = torch.Generator(device=dev).manual_seed(20260914 + 2000 + rank)
    kv = dict(k_mask=torch.zeros(rows * 16, dtype=torch.int32, device=dev),
              k_payload=torch.zeros(rows * 40, dtype=torch.uint8, device=dev),
              v_payload=torch.zeros(rows * 104, dtype=torch.uint8, device=dev),
              v_shared_meta=torch.zeros(rows * 4, dtype=torch.uint8, device=dev),
              k_norms=torch.zeros(rows, dtype=torch.float16, device=dev), k_r_norms=torch.zeros(rows, dtype=torch.float16, device=dev),
              v_norms=torch.zeros(rows, dtype=torch.float16, device=dev), v_r_norms=torch.zeros(rows, dtype=torch.float16, device=dev))
    if n > 0:
        k = torch.randn(n, 4, 256, generator=g, device=dev).half()
        v = torch.randn(n, 4, 256, generator=g, device=dev).half()
        ops.compress(k, tab["d_k"], tab["rotor_k"], tab["cents_k"], tab["cents_k"], kv["k_mask"], kv["k_norms"], kv["k_r_norms"],
                     kv["k_payload"], kv["v_shared_meta"], n * 4, 256, tb.ts_k, tb.alpha_k, False)
        ops.compress(v, tab["d_v"], tab["rotor_v"], tab["cents_v"], tab["vq"], kv["k_mask"], kv["v_norms"], kv["v_r_norms"],
                     kv["v_payload"], kv["v_shared_meta"], n * 4, 256, tb.ts_v, tb.alpha_v, True)
        del k, v
    ring_k = torch.randn(256 * 1024, generator=g, device=dev).half()
    ring_v = torch.randn(256 * 1024, generator=g, device=dev).half()
    owner = world - 1
    exchange = args.exchange if world > 1 else "collective"
    cp = ContextParallelDecode(ops, dist.group.WORLD, kv, tab, lo, hi, tb.alpha_k, tb.alpha_v, ring_k, ring_v, owner=owner,
                               splits=args.splits, device=dev, exchange=exchange, partition=args.partition, engine=args.cp_engine)
    checked = []
    qg0 = torch.randn(24 * 512, generator=g, device=dev).half()
    if world > 1 and exchange == "peer":
        # the two exchanges must give the same answer
        ref = ContextParallelDecode(ops, dist.group.WORLD, kv, tab, lo, hi, tb.alpha_k, tb.alpha_v, ring_k, ring_v, owner=owner,
                                    splits=args.splits, device=dev, exchange="collective", partition=args.partition,
                                    engine=args.cp_engine)
        a = cp.step(qg0.clone(), args.long_ctx % 256, 256).clone()
        b = ref.step(qg0.clone(), args.long_ctx % 256, 256).clone()
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), "peer exchange differs from the all-gather"
        checked.append("peer-store exchange bit-identical to the NCCL all-gather path on one step")
    if args.cp_engine == "persistent":
        # ... and so must the two ways of computing a rank's share (different cuts, different merge order: to rounding)
        ref = ContextParallelDecode(ops, dist.group.WORLD, kv, tab, lo, hi, tb.alpha_k, tb.alpha_v, ring_k, ring_v, owner=owner,
                                    splits=args.splits, device=dev, exchange="collective", partition=args.partition, engine="splits")
        a = cp.step(qg0.clone(), args.long_ctx % 256, 256).float().clone()
        b = ref.step(qg0.clone(), args.long_ctx % 256, 256).float().clone()
        torch.cuda.synchronize()
        err = float((a - b).abs().max())
        assert err < 2e-3 and bool(torch.isfinite(a).all()), f"persistent slice differs from the split launches: {err}"
        checked.append("persistent-kernel share equal to the drop-in split launches on one step (max |diff| %.1e)" % err)
    checked = "; ".join(checked) if checked else None
    qg = torch.randn(24 * 512, generator=g, device=dev).half()
    win_start, win_len = args.long_ctx % 256, 256
    for _ in range(warm):
        cp.step(qg, win_start, win_len)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        cp.step(qg, win_start, win_len)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t[0]) * 1e3 / steps
    status = khqlib.load().khq_b200_device_status()
    cp.close()
    b_alg = 4 * (220 * args.long_ctx + 1024 * win_len)
    return {"us_per_layer_step": us, "algorithmic_bytes_per_step": b_alg, "achieved_gbs": b_alg / (us * 1e-6) / 1e9,
            "exchange": ("peer stores over NVLink, the merge kernel waits for the producers' flags" if exchange == "peer" and world > 1
                         else "one NCCL all-gather of the (24, 258) partials" if world > 1 else "none (one rank)"),
            "partition": ("128-token chunks dealt cyclically (chunk c on rank c mod N)" if args.partition == "cyclic"
                          else "contiguous context ranges cut on 128-token chunks"), "tokens": args.long_ctx, "raw_tokens": win_len,
            "splits": args.splits, "steps": steps, "warmup": warm, "checked": checked, "device_status": status,
            "engine": ("one launch of the persistent batched kernel per rank (slice + raw window), planner-cut"
                       if args.cp_engine == "persistent" else "drop-in split launches + window launch"),
            "gpu_launches_per_step": (3 if args.cp_engine == "persistent" else 5) + (1 if world > 1 and exchange == "peer" else 0)}


def run_long(args, rank, world, local_rank):
    """--workload long: configuration 2 alone (see long_measure)."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), init_method=None if world > 1 or
                            "MASTER_ADDR" in os.environ else "tcp://127.0.0.1:29533", rank=rank, world_size=world)
    dev = torch.device("cuda", local_rank)
    r = long_measure(args, rank, world, dev, args.steps, max(args.warmup, 3))
    if rank == 0:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        us = r["us_per_layer_step"]
        print(json.dumps({
            "metric": "KHQ long-context decode attention latency", "value": us, "unit": "us/layer-step", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BASELINE configs[2]: one sequence, %d compressed + %d raw tokens, 1 layer, %s, "
                                   "context-partitioned over %d GPU(s), partials: %s"
                                   % (args.long_ctx, r["raw_tokens"], r["engine"], world, r["exchange"]),
                       "l2": "payload 115 MB per step, larger than L2 only in aggregate at 1 GPU"},
            "roofline": {"bound": "hbm", "achieved": r["achieved_gbs"], "peak": peak * world, "unit": "GB/s",
                         "frac": r["achieved_gbs"] / (peak * world), "traffic": None,
                         "algorithmic_bytes_per_step": r["algorithmic_bytes_per_step"]},
            "gpu_launches": r["gpu_launches_per_step"] * args.steps, "device_status": r["device_status"],
            "checked": r["checked"]}), flush=True)
    dist.destroy_process_group()


def prefill_measure(args, dev, steps, warm, local_rank, sample_clocks=True):
    """Causal GQA prefill attention + sigmoid gate of --prefill-batch prompts of --prefill-len tokens on this GPU:
    milliseconds per launch (CUDA events, a 256 MB buffer rewritten between launches), TFLOP/s of the causal-attention
    flops 4 * d * H_q * T(T+1)/2 per prompt, and the clocks seen."""
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import lib as khqlib
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps

    ops = CudaOps()
    lib = khqlib.load()
    assert lib.khq_b200_prefill_select(0 if args.prefill_kernel == "tc5" else 1) == 0
    B, T = args.prefill_batch, args.prefill_len
    g = torch.Generator(device=dev).manual_seed(20260914 + 3000 + local_rank)
    dt = torch.bfloat16 if args.prefill_dtype == "bf16" else torch.float16
    assert not (args.prefill_dtype == "bf16" and args.prefill_kernel == "mma"), "the warp-level kernel is fp16 only"
    qg = torch.randn(B, T, 24, 512, generator=g, device=dev).to(dt)
    k = (torch.randn(B, T, 4, 256, generator=g, device=dev) * 0.25).to(dt)
    v = torch.randn(B, T, 4, 256, generator=g, device=dev).to(dt)
    out = torch.zeros(B, T, 24, 256, device=dev, dtype=dt)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    def launch():
        if dt == torch.float16:
            ops.gqa_prefill(qg, k, v, out, B, T, 24, 4, 256, 1.0 / 16.0)
        else:
            khqlib.check("launch_khq_gqa_prefill_bf16", lib.launch_khq_gqa_prefill_bf16(
                qg.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, T, 24, 4, 256, 1.0 / 16.0, qg.stride(0), k.stride(0),
                out.stride(0), khqlib.current_stream()))

    for _ in range(warm):
        launch()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if sample_clocks:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in evs:
        flush.fill_(1)
        e0.record()
        launch()
        e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sample_clocks else None
    ms = sum(e0.elapsed_time(e1) for e0, e1 in evs) / steps
    status = lib.khq_b200_prefill_status()
    flops = 4.0 * 256 * 24 * (T * (T + 1) / 2.0) * B
    return {"ms": ms, "flops": flops, "tflops": flops / (ms * 1e-3) / 1e12, "clocks": clocks, "status": status, "B": B, "T": T,
            "dtype": "bf16" if dt == torch.bfloat16 else "f16", "steps": steps, "warmup": warm}


def run_prefill(args, rank, world, local_rank):
    """--workload prefill: prompts sharded by prompt over the ranks, no collective.  Value: prompt tokens
    per second through one attention layer; roofline: causal-attention FLOPs against the measured dense
    bf16 GEMM burst peak."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warm = max(args.warmup, 3)
    if world > 1:
        dist.barrier()
    r = prefill_measure(args, dev, args.steps, warm, local_rank, sample_clocks=(rank == 0))
    t = torch.tensor([r["ms"]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    B, T = r["B"], r["T"]
    if rank == 0:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks.get("bf16_tflops", 1590.0))
        ach = r["flops"] / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "causal GQA prefill attention throughput", "value": B * T * world / (ms * 1e-3), "unit": "prompt tok/s/layer",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "%s operands, f32 accumulate" % r["dtype"],
            "data": "synthetic",
            "config": {"workload": "causal GQA prefill attention + gate, %d prompts x %d tokens per GPU, H_q 24 / H_kv 4 / "
                                   "d 256, kernel %s" % (B, T, args.prefill_kernel),
                       "l2": "a 256 MB buffer is rewritten between timed launches", "world": world},
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                         # dram bytes of an ncu capture of 1 prompt x 8192 tokens (235.1 MB read + 73.8 MB written, the
                         # tensors themselves: K/V tiles are re-read from L2), scaled by the tensor bytes of this run
                         "traffic": 309.0e6 * (B * T) / 8192.0 if args.prefill_kernel == "tc5" else None,
                         "algorithmic_flops_per_launch": r["flops"],
                         "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst)" if peaks else "fallback"},
            "gpu_launches": args.steps, "clocks": r["clocks"], "device_status": r["status"]}), flush=True)
    if world > 1:
        dist.destroy_process_group()


class _RefKernelOps:
    """The launch interface of the package's CudaOps over the REFERENCE's own kernels, recompiled
    unmodified for sm_100a (oracle/_ref/, a baseline leg like the CPU one): lets the same host state
    machine drive them.  Ring writes are plain copies, as the reference's are."""

    name = "reference-kernels"

    def __init__(self, so):
        self.so = so

    @staticmethod
    def _p(t):
        return 0 if t is None else (t if isinstance(t, int) else t.data_ptr())

    def compress(self, x, d_vec, rotor, centroids, vq_centroids, out_mask, out_norms, out_r_norms, out_payload,
                 out_shared_meta, n, d, ts, alpha, is_v):
        P = self._p
        rc = self.so.launch_khq_compress_fp16(P(x), P(d_vec), P(rotor), P(centroids), P(vq_centroids), P(out_mask), P(out_norms),
                                              P(out_r_norms), P(out_payload), P(out_shared_meta), int(n), int(d), float(ts),
                                              float(alpha), 1 if is_v else 0, None)
        assert rc == 0, rc

    def attn(self, q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms, v_r_norms, centroids_k,
             centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k, d_vec_v, out_attn, out_partial, num_queries, num_heads, L_q,
             c_len, stride_s, n_rep, scale, alpha_k, alpha_v, rope_base, start_pos, num_splits):
        P = self._p
        rc = self.so.launch_khq_attn_fp16(P(q), P(k_payload), P(v_payload), P(v_shared_meta), P(k_mask), P(k_norms), P(k_r_norms),
                                          P(v_norms), P(v_r_norms), P(centroids_k), P(centroids_v), P(vq_centroids), P(k_rotor),
                                          P(v_rotor), P(d_vec_k), P(d_vec_v), P(out_attn), P(out_partial), int(num_queries),
                                          int(num_heads), int(L_q), int(c_len), int(stride_s), int(n_rep), float(scale),
                                          float(alpha_k), float(alpha_v), float(rope_base), int(start_pos), int(num_splits), None)
        assert rc == 0, rc

    def window_attn(self, q, ring_k, ring_v, out_attn, win_start, win_len, ring_cap, H_q, H_kv, d, scale):
        P = self._p
        rc = self.so.launch_khq_window_attn_fp16(P(q), P(ring_k), P(ring_v), P(out_attn), int(win_start), int(win_len), int(ring_cap),
                                                 int(H_q), int(H_kv), int(d), float(scale), None)
        assert rc == 0, rc

    def merge_gate(self, attn_c, attn_w, q_gate, out, H_q, d, has_w, has_c):
        P = self._p
        src_c = attn_c if has_c else attn_w
        rc = self.so.launch_khq_merge_gate_fp16(P(src_c), P(attn_w), P(q_gate), P(out), int(H_q), int(d),
                                                1 if (has_w and has_c) else 0, None)
        assert rc == 0, rc

    def ring_write(self, dst_row, src):
        dst_row.copy_(src.reshape(dst_row.shape))

    def synchronize(self):
        import torch

        torch.cuda.synchronize()


def loop_measure(args, dev, n_layers, with_reference_kernels=True):
    """Configuration 1 of the benchmark specification, the loop the reference's own measurement runs (README.md:27-47): a
    56-token prompt + 512 decode steps over `n_layers` attention layers, 8 splits, compression events
    at tokens 256, 384 and 512 on every layer, all inside the timed region.  This library: the prompt
    through khq_prefill (one prefill launch + appends), the decode steps through khq_step_fused.  The
    like-for-like leg drives the reference's kernels (recompiled for sm_100a) through the same state
    machine the way the reference does: 568 per-token khq_step calls.  Inputs are seeded stand-ins (no
    weights here): per step and layer a fresh q_gate / K / V row."""
    import ctypes

    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import lib as khqlib
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    os.environ["BONSAI_KHQ_SPLITS"] = "8"
    prompt, decode = 56, 512
    n_tok = prompt + decode
    tables = make_tables(n_layers)
    ids = [t.layer_id for t in tables]
    g = torch.Generator(device=dev).manual_seed(20260914 + 1000)
    rng = np.random.default_rng(synth.seed_for(1))
    sk = torch.from_numpy(synth.channel_scales(rng)).to(dev)
    sv = torch.from_numpy(synth.channel_scales(rng)).to(dev)
    # one set of rows per token, shared by the layers (each layer has its own tables and state)
    q_all = torch.randn(n_tok, 24 * 512, generator=g, device=dev).half()
    ku_all = (torch.randn(n_tok, 4, 256, generator=g, device=dev) * sk).half().reshape(n_tok, 1024)
    v_all = (torch.randn(n_tok, 4, 256, generator=g, device=dev) * sv).half().reshape(n_tok, 1024)
    kr_all = torch.from_numpy(synth.partial_rope(ku_all.reshape(n_tok, 4, 256).cpu().numpy(),
                                                 np.arange(n_tok)[:, None].repeat(4, 1))).to(dev).reshape(n_tok, 1024)
    out = torch.zeros(24 * 256, dtype=torch.float16, device=dev)
    out_p = torch.zeros(prompt * 24 * 256, dtype=torch.float16, device=dev)

    def run(ops, fused):
        rt = KhqRuntime(ops, device=dev)
        assert rt.khq_activate(tables, max_seq=1024)
        for li in ids:
            rt.khq_init_layer(li, 24, 4, 256)
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        t0 = 0
        if fused:
            for li in ids:
                assert rt.khq_prefill(li, q_all[:prompt].view(prompt, 24, 512), ku_all[:prompt].view(prompt, 4, 256),
                                      kr_all[:prompt].view(prompt, 4, 256), v_all[:prompt].view(prompt, 4, 256),
                                      out_p.view(prompt, 24, 256), 1.0 / 16.0)
            t0 = prompt
        e[1].record()
        for t in range(t0, n_tok):
            for li in ids:
                if fused:
                    assert rt.khq_step_fused(li, q_all[t], ku_all[t], kr_all[t], v_all[t], out, 1.0 / 16.0)
                else:
                    rt.khq_capture_unroped(li, ku_all[t])
                    assert rt.khq_step(li, q_all[t], kr_all[t], v_all[t], out, 1.0 / 16.0)
        e[2].record()
        torch.cuda.synchronize()
        ev = sorted((x.write_pos, x.boundary) for x in rt.events if x.layer == ids[0])
        assert ev == [(256, 128), (384, 256), (512, 384)], ev
        assert all(rt.layers[li].boundary == 384 and rt.layers[li].write_pos == n_tok for li in ids)
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), out.float().cpu().numpy().copy()

    ours_ops = CudaOps()
    run(ours_ops, True)  # warm-up pass (kernel attributes, caches, allocator)
    ms_prompt, ms_decode, o_ours = run(ours_ops, True)
    res = {"layers": n_layers, "prompt_tokens": prompt, "decode_steps": decode, "splits": 8, "events_per_layer": 3,
           "ours": {"prompt_ms": ms_prompt, "decode_ms": ms_decode,
                    "us_per_layer_step": 1e3 * ms_decode / (decode * n_layers),
                    "tok_s": decode / (ms_decode * 1e-3), "path": "khq_prefill (tcgen05 prefill + appends) then khq_step_fused"},
           "reference_t4_published": {"khq_overhead_us_per_layer_step": 176.0, "source": "the reference's README.md:44-47 (Tesla T4)"},
           "device_status": khqlib.load().khq_b200_device_status()}
    ref_path = ROOT / "oracle" / "_ref" / "libbonsai_ref_sm100a.so"
    if with_reference_kernels and ref_path.exists():
        so = ctypes.CDLL(str(ref_path))
        for name in ("launch_khq_compress_fp16", "launch_khq_attn_fp16", "launch_khq_window_attn_fp16", "launch_khq_merge_gate_fp16"):
            fn = getattr(so, name)
            fn.restype, fn.argtypes = khqlib.SIGNATURES[name]
        _, ms_ref, o_ref = run(_RefKernelOps(so), False)
        res["reference_kernels_sm100a"] = {"loop_ms": ms_ref, "us_per_layer_step": 1e3 * ms_ref / (n_tok * n_layers),
                                           "tok_s": n_tok / (ms_ref * 1e-3),
                                           "path": "568 per-token khq_step calls over the reference's own kernels recompiled for sm_100a",
                                           "final_output_max_abs_diff_vs_ours": float(np.abs(o_ref - o_ours).max())}
    return res


def run_loop(args, rank, world, local_rank):
    """--workload loop: configuration 1 (see loop_measure).  Replicas only: one sequence does not shard;
    every rank runs the same loop and rank 0 prints."""
    import torch

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sampler = ClockSampler(local_rank)
    sampler.start()
    r = loop_measure(args, dev, args.layers)
    clocks = sampler.stop()
    if rank != 0:
        return
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("hbm_gbs", 6650.0))
    # bytes a decode layer-step reads at the end of the loop (384 compressed + 184 raw tokens): the loop is
    # launch- and latency-bound at this size, the fraction says how far from the bytes it runs
    b_alg = 4 * (220 * 384 + 1024 * 184)
    us = r["ours"]["us_per_layer_step"]
    line = {"metric": "KHQ decode loop latency (56-token prompt + 512 steps)", "value": us, "unit": "us/layer-step", "n_gpus": world,
            "steps": 512, "warmup": 1, "ms_per_step": us * r["layers"] / 1e3, "higher_is_better": False, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BASELINE configs[1]: %d attention layers, batch 1, 56-token prompt + 512 decode steps, splits 8, "
                                   "compression events at tokens 256/384/512 inside the timed region" % r["layers"],
                       "l2": "working set under 1 MB per layer: L2-resident by nature"},
            "roofline": {"bound": "hbm", "achieved": b_alg / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": b_alg / (us * 1e-6) / 1e9 / peak, "traffic": None, "algorithmic_bytes_per_step": b_alg},
            "loop": r, "gpu_launches": 512 * r["layers"] * 2, "clocks": clocks}
    if not args.no_extras:
        try:
            line["cpu_baseline"] = cpu_loop_baseline(min(r["layers"], 1))
        except Exception as e:  # the checker is optional equipment of the box
            line["cpu_baseline"] = {"error": repr(e)}
    print(json.dumps(line), flush=True)


def cpu_loop_baseline(n_layers):
    """The same loop through the CPU port of the reference math (oracle/): one layer, all 568
    per-token khq_step calls with their three compression events."""
    import torch

    threads = min(os.cpu_count() or 1, 16)
    os.environ["OMP_NUM_THREADS"] = str(threads)
    os.environ["BONSAI_KHQ_SPLITS"] = "8"
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime
    from oracle import khq_oracle as O

    O.build()
    tables = make_tables(1)
    li = tables[0].layer_id
    rt = KhqRuntime(O.OracleOps(), device="cpu")
    assert rt.khq_activate(tables, max_seq=1024)
    rt.khq_init_layer(li, 24, 4, 256)
    rng = np.random.default_rng(synth.seed_for(1))
    n_tok = 568
    k_u, v = synth.make_kv(rng, n_tok)
    k_r = synth.partial_rope(k_u, np.arange(n_tok)[:, None].repeat(4, 1))
    qs = [torch.from_numpy(synth.make_q_gate(rng, t)).reshape(-1) for t in range(n_tok)]
    out = torch.zeros(24 * 256, dtype=torch.float16)
    t0 = time.perf_counter()
    for t in range(n_tok):
        rt.khq_capture_unroped(li, torch.from_numpy(k_u[t]).reshape(-1))
        assert rt.khq_step(li, qs[t], torch.from_numpy(k_r[t]).reshape(-1), torch.from_numpy(v[t]).reshape(-1), out, 1.0 / 16.0)
    wall = time.perf_counter() - t0
    assert rt.layers[li].boundary == 384
    return {"value": 1e6 * wall / n_tok, "unit": "us/layer-step", "cores": threads, "kind": "port",
            "sample": "1 layer, all 568 per-token steps with their 3 compression events through the CPU port in %.1f s "
                      "(OpenMP over kv-heads, %d threads offered)" % (wall, threads)}


def run_single(args, rank, world, local_rank):
    """Configuration 0 of the benchmark specification: one decode-attention layer-step of one sequence through the drop-in
    launches (compressed attention, splits 1 + window attention + merge/gate), context 512 = 384
    compressed + 128 raw tokens.  Value: microseconds per layer-step (plain launches; CUDA-graph
    replay beside it).  When the reference's own kernels, recompiled for sm_100a, are present
    (oracle/_ref/, a baseline leg like the CPU one), the same three launches are timed through that
    library.  Replicas only: every rank runs the same step."""
    import ctypes

    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import lib as khqlib
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ops = CudaOps()
    tb = make_tables(1)[0]
    tab = {k: torch.from_numpy(v).to(dev) for k, v in tb.as_f16().items()}
    c_len, win_len, win_start = 384, 128, 384 % 256
    rows = c_len * 4
    g = torch.Generator(device=dev).manual_seed(20260914 + rank)
    kv = dict(k_mask=torch.zeros(rows * 16, dtype=torch.int32, device=dev), k_payload=torch.zeros(rows * 40, dtype=torch.uint8, device=dev),
              v_payload=torch.zeros(rows * 104, dtype=torch.uint8, device=dev), v_shared_meta=torch.zeros(rows * 4, dtype=torch.uint8, device=dev),
              k_norms=torch.zeros(rows, dtype=torch.float16, device=dev), k_r_norms=torch.zeros(rows, dtype=torch.float16, device=dev),
              v_norms=torch.zeros(rows, dtype=torch.float16, device=dev), v_r_norms=torch.zeros(rows, dtype=torch.float16, device=dev))
    k = torch.randn(c_len, 4, 256, generator=g, device=dev).half()
    v = torch.randn(c_len, 4, 256, generator=g, device=dev).half()
    ops.compress(k, tab["d_k"], tab["rotor_k"], tab["cents_k"], tab["cents_k"], kv["k_mask"], kv["k_norms"], kv["k_r_norms"],
                 kv["k_payload"], kv["v_shared_meta"], rows, 256, tb.ts_k, tb.alpha_k, False)
    ops.compress(v, tab["d_v"], tab["rotor_v"], tab["cents_v"], tab["vq"], kv["k_mask"], kv["v_norms"], kv["v_r_norms"],
                 kv["v_payload"], kv["v_shared_meta"], rows, 256, tb.ts_v, tb.alpha_v, True)
    ring_k = torch.randn(256 * 1024, generator=g, device=dev).half()
    ring_v = torch.randn(256 * 1024, generator=g, device=dev).half()
    qg = torch.randn(24 * 512, generator=g, device=dev).half()
    ac = torch.zeros(24 * 258, dtype=torch.float32, device=dev)
    aw = torch.zeros(24 * 258, dtype=torch.float32, device=dev)
    ap = torch.zeros(24 * 32 * 258, dtype=torch.float32, device=dev)
    out = torch.zeros(24 * 256, dtype=torch.float16, device=dev)

    def step_with(lib_handle, stream):
        P = lambda t: t.data_ptr()
        rc = lib_handle.launch_khq_attn_fp16(
            P(qg), P(kv["k_payload"]), P(kv["v_payload"]), P(kv["v_shared_meta"]), P(kv["k_mask"]), P(kv["k_norms"]),
            P(kv["k_r_norms"]), P(kv["v_norms"]), P(kv["v_r_norms"]), P(tab["cents_k"]), P(tab["cents_v"]), P(tab["vq"]),
            P(tab["rotor_k"]), P(tab["rotor_v"]), P(tab["d_k"]), P(tab["d_v"]), P(ac), P(ap), 24, 24, 1, c_len, c_len, 6,
            1.0 / 16.0, tb.alpha_k, tb.alpha_v, 1e7, 0, 1, stream)
        rc |= lib_handle.launch_khq_window_attn_fp16(P(qg), P(ring_k), P(ring_v), P(aw), win_start, win_len, 256, 24, 4, 256,
                                                     1.0 / 16.0, stream)
        rc |= lib_handle.launch_khq_merge_gate_fp16(P(ac), P(aw), P(qg), P(out), 24, 256, 1, stream)
        assert rc == 0, rc

    def timed(fn, n):
        for _ in range(max(args.warmup, 3) * 10):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    n_it = max(args.steps, 10) * 20
    ours = khqlib.load()
    cur = lambda: torch.cuda.current_stream().cuda_stream
    sampler = ClockSampler(local_rank)
    sampler.start()
    us_plain = timed(lambda: step_with(ours, cur()), n_it)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step_with(ours, side.cuda_stream)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=side):
        step_with(ours, side.cuda_stream)
    us_graph = timed(graph.replay, n_it)
    # the same step through the single-call entry (ring appends + both regions + merge + gate)
    kr = torch.randn(1024, generator=g, device=dev).half()
    vn = torch.randn(1024, generator=g, device=dev).half()
    ku = torch.randn(1024, generator=g, device=dev).half()
    ring_u = torch.zeros(256 * 1024, dtype=torch.float16, device=dev)
    tabs = dict(cents_k=tab["cents_k"], cents_v=tab["cents_v"], vq=tab["vq"], rotor_k=tab["rotor_k"], rotor_v=tab["rotor_v"],
                d_k=tab["d_k"], d_v=tab["d_v"])

    def fused_step():
        ops.decode_step(qg, kr, vn, ku, ring_k, ring_v, ring_u, kv, tabs, ac, ap, out, c_len, win_start, win_len, 256, 1,
                        1.0 / 16.0, tb.alpha_k, tb.alpha_v, 1e7)

    us_fused = timed(fused_step, n_it)
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fused_step()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph2, stream=side):
        fused_step()
    us_fused_graph = timed(graph2.replay, n_it)
    # the same state as ONE problem of the batched entry (planner-cut persistent launch + merge and gate): what a serving
    # host calls; output checked against the three launches
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.batched import BatchedDecode

    prob = dict(kv)
    out_b = torch.zeros(24 * 256, dtype=torch.float16, device=dev)
    prob.update(q_gate=qg, ring_k=ring_k, ring_v=ring_v, out=out_b, table_id=0, c_len=c_len, start_pos=0, win_start=win_start,
                win_len=win_len)
    tabs_b = [dict(cents_k=tab["cents_k"], cents_v=tab["cents_v"], vq=tab["vq"], k_rotor=tab["rotor_k"], v_rotor=tab["rotor_v"],
                   d_k=tab["d_k"], d_v=tab["d_v"], alpha_k=tb.alpha_k, alpha_v=tb.alpha_v)]
    bd = BatchedDecode([prob], tabs_b)
    step_with(ours, 0)
    bd.launch(1.0 / 16.0, 1e7)
    torch.cuda.synchronize()
    batched_diff = float((out_b.float() - out.float()).abs().max())
    assert batched_diff < 2e-3, f"batched entry differs from the three launches: {batched_diff}"
    us_batched = timed(lambda: bd.launch(1.0 / 16.0, 1e7), n_it)
    ref_us = None
    ref_path = ROOT / "oracle" / "_ref" / "libbonsai_ref_sm100a.so"
    if ref_path.exists():
        so = ctypes.CDLL(str(ref_path))
        for name in ("launch_khq_attn_fp16", "launch_khq_window_attn_fp16", "launch_khq_merge_gate_fp16"):
            fn = getattr(so, name)
            fn.restype, fn.argtypes = khqlib.SIGNATURES[name]
        ref_us = timed(lambda: step_with(so, 0), max(n_it // 10, 20))
    clocks = sampler.stop()
    if rank == 0:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        b_alg = 4 * (220 * c_len + 1024 * win_len)
        ach = b_alg / (us_graph * 1e-6) / 1e9
        print(json.dumps({
            "metric": "KHQ decode attention latency", "value": us_plain, "unit": "us/layer-step", "n_gpus": world,
            "steps": n_it, "warmup": max(args.warmup, 3) * 10, "ms_per_step": us_plain / 1e3, "higher_is_better": False,
            "scaling": "replicas only", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BASELINE configs[0]: one sequence, 384 compressed + 128 raw tokens, 1 layer, splits 1, "
                                   "three drop-in launches per step", "l2": "862 KB working set: L2-resident by nature (a "
                       "latency case, not a bandwidth one)"},
            "graph_replay_us": us_graph, "fused_entry_us": us_fused, "fused_entry_graph_replay_us": us_fused_graph,
            "batched_entry_us": us_batched, "batched_entry_items": int(bd.n_items), "batched_entry_max_abs_diff": batched_diff,
            "reference_kernels_sm100a_us": ref_us,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_bytes_per_step": b_alg, "note": "launch-latency bound at this size"},
            "gpu_launches": 3 * n_it, "clocks": clocks, "device_status": ours.khq_b200_device_status()}), flush=True)


def run_compress(args, rank, world, local_rank):
    """KHQ compression of a prompt prefix (configuration 4 of the benchmark specification: --prefill-batch prompts of
    --prefill-len tokens per GPU, rows 0..T-129 of every prompt, K launch + V launch per prompt)
    and of one 128-token event (512 rows).  Value: rows per second; roofline: algorithmic bytes
    N x (512 + 512 + 220) against the measured HBM copy bandwidth."""
    import torch
    import torch.distributed as dist

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ops = CudaOps()
    tb = make_tables(1)[0]
    f = tb.as_f16()
    tab = {k: torch.from_numpy(v).to(dev) for k, v in f.items()}
    B, T = args.prefill_batch, args.prefill_len
    n_tok = (T // 128 - 1) * 128  # every full chunk but the last stays raw
    rows = n_tok * 4
    g = torch.Generator(device=dev).manual_seed(20260914 + 4000 + rank)
    ks = [torch.randn(rows, 256, generator=g, device=dev).half() for _ in range(B)]
    vs = [torch.randn(rows, 256, generator=g, device=dev).half() for _ in range(B)]
    out = dict(mask=torch.zeros(rows * 16, dtype=torch.int32, device=dev), kpay=torch.zeros(rows * 40, dtype=torch.uint8, device=dev),
               vpay=torch.zeros(rows * 104, dtype=torch.uint8, device=dev), sm=torch.zeros(rows * 4, dtype=torch.uint8, device=dev),
               kn=torch.zeros(rows, dtype=torch.float16, device=dev), krn=torch.zeros(rows, dtype=torch.float16, device=dev),
               vn=torch.zeros(rows, dtype=torch.float16, device=dev), vrn=torch.zeros(rows, dtype=torch.float16, device=dev))

    def one(k, v, n):
        ops.compress(k, tab["d_k"], tab["rotor_k"], tab["cents_k"], tab["cents_k"], out["mask"], out["kn"], out["krn"],
                     out["kpay"], out["sm"], n, 256, tb.ts_k, tb.alpha_k, False)
        ops.compress(v, tab["d_v"], tab["rotor_v"], tab["cents_v"], tab["vq"], out["mask"], out["vn"], out["vrn"],
                     out["vpay"], out["sm"], n, 256, tb.ts_v, tb.alpha_v, True)

    def timed(fn, reps):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_prompt = timed(lambda: [one(ks[b], vs[b], rows) for b in range(B)], args.steps)
    ms_event = timed(lambda: one(ks[0], vs[0], 512), max(args.steps, 50))
    clocks = sampler.stop()
    if rank == 0:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks.get("hbm_gbs", 6650.0))
        b_alg = B * rows * (512 + 512 + 220)
        ach = b_alg / (ms_prompt * 1e-3) / 1e9
        print(json.dumps({
            "metric": "KHQ compression throughput", "value": B * rows * world / (ms_prompt * 1e-3), "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_prompt,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BASELINE configs[4] compression: %d prompts x %d tokens per GPU, %d rows of 256 per "
                                   "prompt (K launch + V launch each)" % (B, T, rows),
                       "l2": "%.0f MB of fp16 rows per step, larger than the 126 MB L2" % (2 * B * rows * 512 / 1e6), "world": world},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "algorithmic_bytes_per_step": b_alg},
            "event_512_rows_us": ms_event * 1e3, "gpu_launches": 2 * B * args.steps, "clocks": clocks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "long":
        run_long(args, rank, world, local_rank)
        return
    if args.workload == "prefill":
        run_prefill(args, rank, world, local_rank)
        return
    if args.workload == "compress":
        run_compress(args, rank, world, local_rank)
        return
    if args.workload == "single":
        run_single(args, rank, world, local_rank)
        return
    if args.workload == "loop":
        run_loop(args, rank, world, local_rank)
        return

    import torch
    import torch.distributed as dist

    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import sharding
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.engine import BatchEngine

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    gen = {"auto": -1, "cuda-core": 1, "mma": 2, "tc5": 3, "tc5w": 4}[args.kernel]
    tables = make_tables(args.layers)
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(eng, steps, warm, seed, clocks_on_rank0):
        """Resident attention (per-launch events) and the end-to-end decode step of `eng`; both timings are
        the max over the ranks.  Returns (ms_resident_total, launch_ms, ms_e2e_total, clocks, bytes_layer)."""
        bytes_layer = eng.algorithmic_bytes_per_layer

        def resident_step(evs=None):
            for l in range(eng.L):
                if evs is not None:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                eng.attention_resident(l)
                if evs is not None:
                    b.record(stream)
                    evs.append((a, b))

        for _ in range(warm):
            resident_step()
        sampler = ClockSampler(local_rank)
        barrier()
        if clocks_on_rank0 and rank == 0:
            sampler.start()
        evs = []
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in range(steps):
            resident_step(evs)
        s1.record(stream)
        barrier()
        ms_total = s0.elapsed_time(s1)
        launch_ms = [a.elapsed_time(b) for a, b in evs]
        # end to end: host buffers in, every sequence one token on (append, events, attention), host buffers out
        g = torch.Generator().manual_seed(seed)
        for t in (eng.h_q, eng.h_k, eng.h_v):
            t.copy_(torch.randn(t.shape, generator=g).half())
        for _ in range(warm):
            eng.decode_step()
            stream.synchronize()
        barrier()
        ev0 = eng.events_fired
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            out = eng.decode_step()
            stream.synchronize()  # the host consumes this step's outputs before the next token
            _ = float(out[0, 0, 0])
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        clocks = sampler.stop() if (clocks_on_rank0 and rank == 0) else None
        t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), launch_ms, float(t[1]), clocks, bytes_layer, eng.events_fired - ev0

    # ---- headline: args.seqs sequences on every GPU (weak scaling), no collective -------------------
    c_len, win = workload(args, rank)
    t_setup = time.perf_counter()
    eng = BatchEngine(tables, c_len, win, device=f"cuda:{local_rank}", codebook_in_smem=gen, grow_tokens=256,
                      tokens_per_item=args.tokens_per_item)
    eng.fill_synthetic(20260914 + 1000 * 3 + rank)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup
    ms_total, launch_ms, ms_e2e, clocks, bytes_layer, n_events = measure(eng, args.steps, args.warmup, 7 + rank, True)
    status = eng.lib.khq_b200_device_status()
    h2d, d2h, n_items = eng.h2d_bytes_per_step, eng.d2h_bytes_per_step, eng.n_items
    del eng
    torch.cuda.empty_cache()

    extras = {}
    if world > 1 and not args.no_extras:
        # ---- configs[3] as written: args.seqs sequences IN TOTAL, dealt to the GPUs by greedy bin-packing ----
        gc, gw = workload(args, 0)  # every rank draws the same global workload
        cost = sharding.algorithmic_bytes(gc, gw)
        parts = sharding.partition_sequences(cost, world)
        mine = parts[rank]
        eng2 = BatchEngine(tables, gc[mine], gw[mine], device=f"cuda:{local_rank}", codebook_in_smem=gen, grow_tokens=256)
        eng2.fill_synthetic(20260914 + 5000 + rank)
        torch.cuda.synchronize()
        st_steps = max(3, min(args.steps, 10))
        ms_t, _, ms_e, _, _, _ = measure(eng2, st_steps, max(args.warmup, 3), 11 + rank, False)
        loads = [int(cost[p].sum()) for p in parts]
        extras["strong"] = {
            "workload": "BASELINE configs[3] as written: %d sequences in total over %d GPUs, greedy bin-packing on algorithmic "
                        "bytes, no collective" % (args.seqs, world),
            "value": args.seqs / (ms_t / st_steps / 1e3), "unit": UNIT, "ms_per_step": ms_t / st_steps,
            "e2e": {"value": args.seqs / (ms_e / st_steps / 1e3), "unit": UNIT, "ms_per_step": ms_e / st_steps},
            "sequences_per_rank": [int(len(p)) for p in parts], "algorithmic_bytes_per_layer_per_rank": loads,
            "imbalance_max_over_mean": sharding.imbalance(cost, parts), "steps": st_steps, "scaling": "strong"}
        del eng2
        torch.cuda.empty_cache()
        # ---- configs[2]: one long sequence split by context range, partials merged over NVLink ------------
        extras["long_context"] = long_measure(args, rank, world, dev, max(args.steps, 20), 5)
    if world == 1 and not args.no_extras and rank == 0:
        try:
            r = prefill_measure(args, dev, 3, 3, local_rank, sample_clocks=True)
            peaks_ = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
            pk = float(peaks_.get("bf16_tflops", 1590.0))
            extras["prefill"] = {"workload": "BASELINE configs[4] attention: %d prompts x %d tokens, causal GQA + gate, tcgen05 kernel"
                                             % (r["B"], r["T"]), "ms": r["ms"], "tflops": r["tflops"], "peak_tflops": pk,
                                 "frac": r["tflops"] / pk, "peak_source": "MEASURED_PEAKS.json bf16_tflops (burst)" if peaks_ else "fallback",
                                 "clocks": r["clocks"], "steps": r["steps"], "warmup": r["warmup"], "device_status": r["status"],
                                 "l2": "a 256 MB buffer is rewritten between timed launches"}
        except Exception as e:
            extras["prefill"] = {"error": repr(e)}
        torch.cuda.empty_cache()
        try:
            extras["decode_loop"] = loop_measure(args, dev, args.layers)
        except Exception as e:
            extras["decode_loop"] = {"error": repr(e)}

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
        ms_step = ms_total / args.steps
        value = args.seqs * world / (ms_step / 1e3)
        e2e_val = args.seqs * world / (ms_e2e / args.steps / 1e3)
        avg_launch_ms = float(np.mean(launch_ms))
        achieved = bytes_layer / (avg_launch_ms / 1e3) / 1e9
        kname = {"cuda-core": "khq_decode_batched_kernel", "mma": "khq_decode_batched_mma_kernel",
                 "tc5": "khq_decode_batched_tc5_kernel", "tc5w": "khq_decode_batched_tc5w_kernel", "auto": "khq_decode_batched_mma_kernel"}[args.kernel]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(args, world),
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps,
                    "covers": "per sequence and layer: pinned-host copies of q_gate/K/V, batched pre-step (norm, K capture, RoPE, "
                              "ring appends), batched compression of the sequences whose window reached 256 (%d events in the "
                              "timed steps), re-planned batched attention, copy of the gated output to pinned host memory" % n_events},
            "gpu_launches": 2 * len(launch_ms),
            "gpu_launches_e2e_per_step": "per layer: 1 pre-step + 2 compress (steps with events) + 2 attention; + 1 descriptor update",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                         "frac": achieved / peak_gbs, "traffic": NCU_TRAFFIC_RATIO * bytes_layer,
                         "traffic_source": "ncu dram__bytes_read+write of an 8-sequence x 1-layer launch (117.0 MB for "
                                           "116.6 MB algorithmic), scaled by payload rows: nothing is re-read",
                         "peak_source": peak_src,
                         "kernel": "%s (+ its merge kernel and a 256 B memset, inside the same events)" % kname,
                         "algorithmic_bytes_per_launch": bytes_layer, "avg_launch_ms": avg_launch_ms},
            "payload_gb_per_layer_launch": bytes_layer / 1e9, "work_items_per_launch": n_items,
            "us_per_layer_step_per_sequence": 1e3 * avg_launch_ms / args.seqs,
            "clocks": clocks, "device_status": status, "setup_s": setup_s,
        }
        line.update(extras)
        if not args.no_extras and world == 1:
            try:
                smp = CpuSample(args, os.cpu_count() or 1)
                line["cpu_baseline"] = smp.result(smp.time_once())
            except Exception as e:  # the checker is optional equipment of the box
                line["cpu_baseline"] = {"error": repr(e)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
