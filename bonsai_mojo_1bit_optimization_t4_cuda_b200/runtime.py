"""Host state machine of the KHQ runtime -- a Python restatement of ``src/khq/runtime.mojo``.

Same names, same arguments, same bookkeeping as the reference:

* ``KhqLayer`` (``runtime.mojo:77-152``): per-layer tables, three 256-slot rings (K RoPE'd, V,
  K un-RoPE'd), SoA payload buffers with row = token*H_kv + kv_head, ``boundary``/``write_pos``.
* ``khq_init`` (``:312-392``), ``khq_init_layer`` (``:395-429``), ``khq_capture_unroped``
  (``:432-451``), ``khq_step`` (``:454-613``), ``_khq_split_count`` (``:211-222``).

The compute backend is injected (``ops``): the shipped backend is ``ops.CudaOps`` (the CUDA
library through its C ABI); nothing here computes on the host.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from .calib import KhqLayerTables, read_calib

KHQ_MAX_LAYERS = 64
KHQ_RING = 256
KHQ_WATERMARK = 256
KHQ_CHUNK = 128
KHQ_MAX_SPLITS = 32
KHQ_MIN_TOKENS_PER_SPLIT = 8
ROPE_BASE = 10000000.0

# profiling phases (BONSAI_KHQ_PROF=1), runtime.mojo:46-53
KHQ_P_RING, KHQ_P_CK, KHQ_P_CV, KHQ_P_ATTN, KHQ_P_WIN, KHQ_P_MERGE = range(6)
KHQ_PHASE_NAMES = ["ring-write", "compress-K", "compress-V", "attn-compressed", "attn-window", "merge+gate"]


def _env_int(name: str, fallback: int) -> int:
    v = os.environ.get(name)
    if not v:
        return fallback
    try:
        return int(v)
    except ValueError:
        return fallback


class KhqLayer:
    """KHQ state of one attention layer (all tensors live on the runtime's device)."""

    def __init__(self):
        self.ready = False
        self.has_tables = False
        self.ts_k, self.alpha_k, self.ts_v, self.alpha_v = 1.0, 1.0, 1.95, 1.0
        self.H_q = self.H_kv = 0
        self.D = 256
        self.cap = 0
        self.boundary = 0
        self.write_pos = 0
        # tables: h_dk h_ck h_rk h_dv h_cv h_rv h_vq; rings: h_ring_k h_ring_v h_ring_u;
        # payload: h_kmask h_kpay h_knorm h_krn h_vpay h_vnorm h_vrn h_vsm; scratch: h_ac h_aw h_ap
        self.t: Dict[str, torch.Tensor] = {}

    def __getattr__(self, name):  # h_xxx accessors, as the reference's fields are named
        t = self.__dict__.get("t")
        if t is not None and name.startswith("h_") and name[2:] in t:
            return t[name[2:]]
        raise AttributeError(name)


@dataclass
class KhqCompressEvent:
    layer: int
    event: int       # boundary // 128 after the event
    boundary: int
    write_pos: int
    raw_window: int


class KhqRuntime:
    """Module state of the reference (``KhqGlobals``) plus its free functions as methods."""

    def __init__(self, ops, device="cuda"):
        self.ops = ops
        self.device = torch.device(device)
        self.layers: List[KhqLayer] = [KhqLayer() for _ in range(KHQ_MAX_LAYERS)]
        self.n_layers = 0
        self.active = False
        self.ready = False
        self.splits = 1
        self.prof = False
        self.debug = False
        self.prof_ns = [0.0] * 6
        self.events: List[KhqCompressEvent] = []

    # ------------------------------------------------------------------ khq_init / activate
    def khq_init(self, tables, max_seq: int) -> bool:
        """``tables``: path of a khq_calib.bin or a list of ``KhqLayerTables``.  Idempotent."""
        if self.ready:
            return True
        if isinstance(tables, (str, os.PathLike)):
            try:
                tables = read_calib(tables)
            except (OSError, ValueError) as e:
                print(">> [KHQ] file centroid tidak valid:", e)
                return False
        for tb in tables:
            if tb.layer_id < 0 or tb.layer_id >= KHQ_MAX_LAYERS:
                return False
            L = self.layers[tb.layer_id]
            L.ts_k, L.alpha_k, L.ts_v, L.alpha_v = tb.ts_k, tb.alpha_k, tb.ts_v, tb.alpha_v
            f16 = tb.as_f16()
            for key, name in (("d_k", "dk"), ("cents_k", "ck"), ("rotor_k", "rk"), ("d_v", "dv"),
                              ("cents_v", "cv"), ("rotor_v", "rv"), ("vq", "vq")):
                L.t[name] = torch.from_numpy(f16[key]).to(self.device)
            L.cap = max_seq
            L.ready = False
            L.has_tables = True
        self.n_layers = len(tables)
        self.ready = True
        self.splits = min(max(_env_int("BONSAI_KHQ_SPLITS", 16), 1), KHQ_MAX_SPLITS)
        self.prof = os.environ.get("BONSAI_KHQ_PROF", "")[:1] == "1"
        self.debug = os.environ.get("BONSAI_KHQ_DEBUG", "")[:1] == "1"
        return True

    def khq_activate(self, tables, max_seq: int) -> bool:
        if not self.khq_init(tables, max_seq):
            return False
        self.active = True
        return True

    def khq_active(self) -> bool:
        return self.active

    # ------------------------------------------------------------------ khq_init_layer
    def khq_init_layer(self, layer_idx: int, H_q: int, H_kv: int, d: int) -> None:
        if layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return
        L = self.layers[layer_idx]
        if L.ready:
            return
        kv = H_kv * d
        L.H_q, L.H_kv, L.D = H_q, H_kv, d
        L.boundary = 0
        L.write_pos = 0
        dev = self.device
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        for r in ("ring_k", "ring_v", "ring_u"):
            L.t[r] = z(KHQ_RING * kv, torch.float16)
        rows = L.cap * H_kv  # row = token*H_kv + head
        L.t["kmask"] = z(rows * 16, torch.int32)
        L.t["kpay"] = z(rows * 40, torch.uint8)
        L.t["knorm"] = z(rows, torch.float16)
        L.t["krn"] = z(rows, torch.float16)
        L.t["vpay"] = z(rows * 104, torch.uint8)
        L.t["vnorm"] = z(rows, torch.float16)
        L.t["vrn"] = z(rows, torch.float16)
        L.t["vsm"] = z(rows * 4, torch.uint8)
        L.t["ac"] = z(H_q * (d + 2), torch.float32)
        L.t["aw"] = z(H_q * (d + 2), torch.float32)
        L.t["ap"] = z(H_q * KHQ_MAX_SPLITS * (d + 2), torch.float32)
        L.ready = True

    # ------------------------------------------------------------------ split policy
    def _khq_split_count(self, c_len: int) -> int:
        if self.splits <= 1 or c_len <= 0:
            return 1
        eff = max(c_len // KHQ_MIN_TOKENS_PER_SPLIT, 1)
        return min(eff, self.splits)

    # ------------------------------------------------------------------ khq_capture_unroped
    def khq_capture_unroped(self, layer_idx: int, k_dev: torch.Tensor) -> None:
        """Copy the post-norm PRE-RoPE K of the current token into its ring slot; called before
        RoPE and before ``khq_step`` (``write_pos`` has not advanced yet)."""
        if not self.active or not self.ready or layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return
        L = self.layers[layer_idx]
        if not L.ready:
            return
        kv = L.H_kv * L.D
        slot = L.write_pos % KHQ_RING
        self.ops.ring_write(L.t["ring_u"][slot * kv:(slot + 1) * kv], k_dev)

    # ------------------------------------------------------------------ fused pre-step (addition)
    def khq_prestep(self, layer_idx: int, q_gate_dev, k_dev, v_dev, pos: int, q_norm_w=None, k_norm_w=None,
                    has_norms: bool = True, rms_eps: float = 1e-6, rope_theta: float = ROPE_BASE,
                    rotary_dim: int = 64) -> bool:
        """One launch for what the reference does in five before ``khq_step``
        (``attention.mojo:329-353`` + ``khq_capture_unroped`` + the ring append of ``khq_step``):
        q/k head RMSNorm, K un-RoPE'd -> ring_u, partial RoPE of q and k, K RoPE'd and V -> rings.
        Follow it with ``khq_step(..., rings_written=True)``."""
        if not self.active or not self.ready or layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return False
        L = self.layers[layer_idx]
        if not L.ready:
            return False
        kv = L.H_kv * L.D
        slot = L.write_pos % KHQ_RING
        T = L.t
        self.ops.prestep(q_gate_dev, k_dev, v_dev, q_norm_w, k_norm_w, T["ring_k"][slot * kv:(slot + 1) * kv],
                         T["ring_v"][slot * kv:(slot + 1) * kv], T["ring_u"][slot * kv:(slot + 1) * kv], L.H_q, L.H_kv,
                         L.D, rotary_dim, pos, rope_theta, rms_eps, has_norms)
        return True

    # ------------------------------------------------------------------ khq_step
    def _tick(self):
        if self.prof:
            self.ops.synchronize()
            import time
            return time.monotonic_ns()
        return 0

    def _tock(self, phase, t0):
        if self.prof:
            self.ops.synchronize()
            import time
            self.prof_ns[phase] += time.monotonic_ns() - t0

    def khq_step(self, layer_idx: int, q_gate_dev, k_roped_dev, v_dev, out_dev, scale: float,
                 rings_written: bool = False) -> bool:
        """One KHQ attention step of one layer.  False = the KHQ path is not active/ready
        (the caller then raises, as ``attention.mojo:359-365`` does)."""
        if not self.active or not self.ready or layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return False
        L = self.layers[layer_idx]
        if not L.ready:
            return False
        ops, T = self.ops, L.t
        H_q, H_kv, d = L.H_q, L.H_kv, L.D
        kv = H_kv * d
        slot = L.write_pos % KHQ_RING

        # 1. ring append: K RoPE'd + V (K un-RoPE'd was written by khq_capture_unroped)
        t0 = self._tick()
        if not rings_written:  # khq_prestep already appended this token
            ops.ring_write(T["ring_k"][slot * kv:(slot + 1) * kv], k_roped_dev)
            ops.ring_write(T["ring_v"][slot * kv:(slot + 1) * kv], v_dev)
        self._tock(KHQ_P_RING, t0)
        L.write_pos += 1

        # 2. compression event: watermark 256 -> compress the 128 oldest tokens, which are
        #    contiguous in the ring because boundary is a multiple of 128
        window = L.write_pos - L.boundary
        if window >= KHQ_WATERMARK and L.boundary + KHQ_CHUNK <= L.cap:
            s0 = L.boundary % KHQ_RING
            nrows = KHQ_CHUNK * H_kv
            r0 = L.boundary * H_kv
            uptr = T["ring_u"][s0 * kv:]
            vptr = T["ring_v"][s0 * kv:]
            t0 = self._tick()
            # K first: it zeroes the shared meta rows that the V launch then fills
            ops.compress(uptr, T["dk"], T["rk"], T["ck"], T["ck"], T["kmask"][r0 * 16:],
                         T["knorm"][r0:], T["krn"][r0:], T["kpay"][r0 * 40:], T["vsm"][r0 * 4:],
                         nrows, d, L.ts_k, L.alpha_k, False)
            self._tock(KHQ_P_CK, t0)
            t0 = self._tick()
            ops.compress(vptr, T["dv"], T["rv"], T["cv"], T["vq"], T["kmask"][r0 * 16:],
                         T["vnorm"][r0:], T["vrn"][r0:], T["vpay"][r0 * 104:], T["vsm"][r0 * 4:],
                         nrows, d, L.ts_v, L.alpha_v, True)
            self._tock(KHQ_P_CV, t0)
            if self.debug:
                bits = T["knorm"][r0:r0 + nrows].view(torch.int16).cpu().numpy().astype(np.uint16)
                print(">> [KHQ-NORM]", layer_idx, L.boundary, nrows, " ".join(str(int(b)) for b in bits))
            L.boundary += KHQ_CHUNK
            ev = KhqCompressEvent(layer_idx, L.boundary // KHQ_CHUNK, L.boundary, L.write_pos,
                                  L.write_pos - L.boundary)
            self.events.append(ev)
            if self.debug:
                print(">> [KHQ-COMPRESS] layer", layer_idx, "event#", ev.event, "boundary", ev.boundary,
                      "write_pos", ev.write_pos, "raw_window", ev.raw_window)

        # 3. attention over both regions; q is read from the interleaved [H_q, 2d] buffer
        c_len = L.boundary
        has_c = c_len > 0
        win_len = L.write_pos - c_len
        has_w = win_len > 0
        if not (has_c or has_w):
            return False
        if has_c:
            n_rep = H_q // H_kv
            n_sp = self._khq_split_count(c_len)
            t0 = self._tick()
            ops.attn(q_gate_dev, T["kpay"], T["vpay"], T["vsm"], T["kmask"], T["knorm"], T["krn"],
                     T["vnorm"], T["vrn"], T["ck"], T["cv"], T["vq"], T["rk"], T["rv"], T["dk"],
                     T["dv"], T["ac"], T["ap"], H_q, H_q, 1, c_len, c_len, n_rep, scale, L.alpha_k,
                     L.alpha_v, ROPE_BASE, 0, n_sp)
            self._tock(KHQ_P_ATTN, t0)
        if has_w:
            win_start = c_len % KHQ_RING
            t0 = self._tick()
            ops.window_attn(q_gate_dev, T["ring_k"], T["ring_v"], T["aw"], win_start, win_len,
                            KHQ_RING, H_q, H_kv, d, scale)
            self._tock(KHQ_P_WIN, t0)

        # 4. merge + sigmoid gate
        t0 = self._tick()
        ops.merge_gate(T["ac"], T["aw"], q_gate_dev, out_dev, H_q, d, has_w, has_c)
        self._tock(KHQ_P_MERGE, t0)
        return True

    # ------------------------------------------------------------------ fused step (addition)
    def khq_step_fused(self, layer_idx: int, q_gate_dev, k_unroped_dev, k_roped_dev, v_dev, out_dev, scale: float) -> bool:
        """``khq_capture_unroped`` + ``khq_step`` of one token through ``launch_khq_decode_step_fp16``:
        the three ring appends, both attention regions, the merge and the gate in two or three
        launches (and one host call) instead of seven.  A step on which a compression event is due
        takes the classic sequence (the event sits between the append and the attention), and so does
        a step whose window would exceed the ring (compressed capacity exhausted: the reference keeps
        stepping with window > 256, ``README.md:259``, and so does ``khq_step``).  The state afterwards
        is the one the classic calls leave."""
        if not self.active or not self.ready or layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return False
        L = self.layers[layer_idx]
        if not L.ready:
            return False
        window_after = L.write_pos + 1 - L.boundary
        event_due = window_after >= KHQ_WATERMARK and L.boundary + KHQ_CHUNK <= L.cap
        if event_due or window_after > KHQ_RING or not hasattr(self.ops, "decode_step"):
            self.khq_capture_unroped(layer_idx, k_unroped_dev)
            return self.khq_step(layer_idx, q_gate_dev, k_roped_dev, v_dev, out_dev, scale)
        T = L.t
        c_len = L.boundary
        kv = dict(k_payload=T["kpay"], v_payload=T["vpay"], v_shared_meta=T["vsm"], k_mask=T["kmask"], k_norms=T["knorm"],
                  k_r_norms=T["krn"], v_norms=T["vnorm"], v_r_norms=T["vrn"])
        tab = dict(cents_k=T["ck"], cents_v=T["cv"], vq=T["vq"], rotor_k=T["rk"], rotor_v=T["rv"], d_k=T["dk"], d_v=T["dv"])
        t0 = self._tick()
        self.ops.decode_step(q_gate_dev, k_roped_dev, v_dev, k_unroped_dev, T["ring_k"], T["ring_v"], T["ring_u"], kv, tab,
                             T["ac"], T["ap"], out_dev, c_len, c_len % KHQ_RING, window_after, KHQ_RING,
                             self._khq_split_count(c_len) if c_len > 0 else 1, scale, L.alpha_k, L.alpha_v, ROPE_BASE)
        self._tock(KHQ_P_ATTN, t0)
        L.write_pos += 1
        return True

    # ------------------------------------------------------------------ prompt prefill (addition)
    def khq_prefill(self, layer_idx: int, q_gate_dev, k_unroped_dev, k_roped_dev, v_dev, out_dev, scale: float) -> bool:
        """Whole-prompt path for one layer: causal GQA attention of all T prompt rows at once
        (``ops.gqa_prefill``; the reference loops its decode kernel over the prompt,
        ``src/models/qwen3_5/layer.mojo:630-641``), then the KHQ state that the per-token path would
        have left behind: every full 128-token chunk except the last one is compressed (K from the
        un-RoPE'd rows, V as is), the remaining 128..255 newest tokens sit in the rings at slots
        ``token % 256``, ``boundary``/``write_pos`` are advanced accordingly.

        q_gate (T, H_q, 2d), k_unroped / k_roped (T, H_kv, d), v (T, H_kv, d), out (T, H_q, d): fp16.
        The code words are bit-identical to the per-token path's (same inputs to the same compress
        launches); the attention outputs of prompt rows are exact fp16-KV attention, whereas the
        per-token path attends older tokens through their lossy decompression.
        Only valid on a fresh layer (write_pos == 0)."""
        if not self.active or not self.ready or layer_idx < 0 or layer_idx >= KHQ_MAX_LAYERS:
            return False
        L = self.layers[layer_idx]
        if not L.ready or L.write_pos != 0:
            return False
        ops, Tn = self.ops, L.t
        H_q, H_kv, d = L.H_q, L.H_kv, L.D
        kv = H_kv * d
        T = int(k_roped_dev.shape[0])
        # the prompt length comes from the leading dimension: refuse tensors whose sizes do not agree
        # with it before any kernel is given their addresses
        want = {"q_gate": T * H_q * 2 * d, "k_unroped": T * kv, "k_roped": T * kv, "v": T * kv, "out": T * H_q * d}
        have = {"q_gate": q_gate_dev.numel(), "k_unroped": k_unroped_dev.numel(), "k_roped": k_roped_dev.numel(),
                "v": v_dev.numel(), "out": out_dev.numel()}
        if T <= 0 or any(have[k] != want[k] for k in want):
            raise ValueError(f"khq_prefill: tensors do not hold T={T} rows of (H_q={H_q}, H_kv={H_kv}, d={d}): {have} vs {want}")
        ops.gqa_prefill(q_gate_dev, k_roped_dev, v_dev, out_dev, 1, T, H_q, H_kv, d, scale)
        # the per-token path compresses chunk c when write_pos reaches 128*(c+2), capped by `cap`
        n_chunks = 0
        while (n_chunks + 2) * KHQ_CHUNK <= T and (n_chunks + 1) * KHQ_CHUNK <= L.cap:
            n_chunks += 1
        if n_chunks > 0:
            rows = n_chunks * KHQ_CHUNK * H_kv
            ku = k_unroped_dev.reshape(-1)
            vv = v_dev.reshape(-1)
            ops.compress(ku, Tn["dk"], Tn["rk"], Tn["ck"], Tn["ck"], Tn["kmask"], Tn["knorm"], Tn["krn"], Tn["kpay"],
                         Tn["vsm"], rows, d, L.ts_k, L.alpha_k, False)
            ops.compress(vv, Tn["dv"], Tn["rv"], Tn["cv"], Tn["vq"], Tn["kmask"], Tn["vnorm"], Tn["vrn"], Tn["vpay"],
                         Tn["vsm"], rows, d, L.ts_v, L.alpha_v, True)
        L.boundary = n_chunks * KHQ_CHUNK
        L.write_pos = T
        # newest min(T, 256) tokens into the rings at slot = token % 256
        first = max(0, T - KHQ_RING)
        for name, src in (("ring_k", k_roped_dev), ("ring_v", v_dev), ("ring_u", k_unroped_dev)):
            ring = Tn[name].view(KHQ_RING, kv)
            s2 = src.reshape(T, kv)
            a = first % KHQ_RING
            n = T - first
            head = min(n, KHQ_RING - a)
            ring[a:a + head].copy_(s2[first:first + head])
            if n > head:
                ring[0:n - head].copy_(s2[first + head:T])
        for c in range(n_chunks):
            self.events.append(KhqCompressEvent(layer_idx, c + 1, (c + 1) * KHQ_CHUNK, (c + 2) * KHQ_CHUNK, KHQ_CHUNK))
        return True

    # ------------------------------------------------------------------ khq_prof_report
    def khq_prof_report(self, n_tokens: int) -> Optional[str]:
        if not self.prof or n_tokens <= 0:
            return None
        total = sum(self.prof_ns)
        lines = [">> [KHQ-PROF] per token (ms), %d tokens" % n_tokens]
        for name, ns in zip(KHQ_PHASE_NAMES, self.prof_ns):
            lines.append(">> [KHQ-PROF]   %-16s %8.4f" % (name, ns / 1e6 / n_tokens))
        lines.append(">> [KHQ-PROF]   %-16s %8.4f" % ("total", total / 1e6 / n_tokens))
        return "\n".join(lines)

    # ------------------------------------------------------------------ checkpoint / resume (addition)
    _STATE_ROW_ARRAYS = (("kmask", 16 * 4), ("kpay", 40), ("knorm", 2), ("krn", 2), ("vpay", 104), ("vnorm", 2),
                         ("vrn", 2), ("vsm", 4))

    def khq_save_state(self, path) -> int:
        """Write the decode state of every initialised layer (rings, the compressed rows up to
        ``boundary``, ``boundary`` / ``write_pos``) to a ``khq_state.bin`` container
        (``formats`` module docstring).  The reference keeps this state in device memory only and
        cannot resume a sequence.  Tables are not stored: they come from khq_calib.bin.  Returns
        the number of layers written."""
        import struct

        from .formats import KHQS_MAGIC, KHQS_VERSION

        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        ids = [i for i, L in enumerate(self.layers) if L.ready]
        with open(path, "wb") as f:
            f.write(struct.pack("<III", KHQS_MAGIC, KHQS_VERSION, len(ids)))
            for i in ids:
                L = self.layers[i]
                f.write(struct.pack("<IIIIIII", i, L.H_q, L.H_kv, L.D, L.cap, L.boundary, L.write_pos))
                for r in ("ring_k", "ring_v", "ring_u"):
                    f.write(L.t[r].cpu().numpy().tobytes())
                rows = L.boundary * L.H_kv
                for name, row_bytes in self._STATE_ROW_ARRAYS:
                    flat = L.t[name].view(torch.uint8)
                    f.write(flat[:rows * row_bytes].cpu().numpy().tobytes())
        return len(ids)

    def khq_load_state(self, path) -> int:
        """Restore what ``khq_save_state`` wrote into this runtime (tables must already be loaded
        with ``khq_init`` / ``khq_activate`` and ``max_seq`` must be at least the saved boundary).
        Layers are initialised on demand.  Raises ValueError on a malformed file or a shape that
        does not fit; returns the number of layers restored."""
        import struct

        from .formats import KHQS_MAGIC, KHQS_VERSION

        raw = open(path, "rb").read()
        if len(raw) < 12:
            raise ValueError("khq_state: shorter than its header")
        magic, version, n = struct.unpack_from("<III", raw, 0)
        if magic != KHQS_MAGIC or version != KHQS_VERSION:
            raise ValueError(f"khq_state: bad magic/version 0x{magic:08X}/{version}")
        if not self.ready:
            raise ValueError("khq_state: load the calibration tables first (khq_init)")
        off = 12
        for _ in range(n):
            if off + 28 > len(raw):
                raise ValueError("khq_state: truncated layer header")
            i, H_q, H_kv, D, cap, boundary, write_pos = struct.unpack_from("<IIIIIII", raw, off)
            off += 28
            if i >= KHQ_MAX_LAYERS or not self.layers[i].has_tables:
                raise ValueError(f"khq_state: layer {i} has no tables in this runtime")
            L = self.layers[i]
            # the only shape the library's kernels serve; checked before anything is allocated from it
            if (H_q, H_kv, D) != (24, 4, 256):
                raise ValueError(f"khq_state: layer {i}: unsupported shape H_q={H_q} H_kv={H_kv} D={D}")
            if cap > L.cap:
                raise ValueError(f"khq_state: layer {i}: saved capacity {cap} exceeds this runtime's {L.cap}")
            if boundary > L.cap or boundary % KHQ_CHUNK != 0 or write_pos < boundary or write_pos - boundary > KHQ_RING:
                raise ValueError(f"khq_state: layer {i}: boundary {boundary} / write_pos {write_pos} do not fit cap {L.cap}")
            self.khq_init_layer(i, H_q, H_kv, D)
            if (L.H_q, L.H_kv, L.D) != (H_q, H_kv, D):
                raise ValueError(f"khq_state: layer {i} shape differs from the initialised layer")
            ring_bytes = KHQ_RING * H_kv * D * 2
            rows = boundary * H_kv
            need = 3 * ring_bytes + sum(rows * rb for _, rb in self._STATE_ROW_ARRAYS)
            if off + need > len(raw):
                raise ValueError(f"khq_state: layer {i} data truncated")
            for r in ("ring_k", "ring_v", "ring_u"):
                src = torch.frombuffer(bytearray(raw[off:off + ring_bytes]), dtype=torch.float16)
                L.t[r].copy_(src.to(self.device))
                off += ring_bytes
            for name, row_bytes in self._STATE_ROW_ARRAYS:
                nb = rows * row_bytes
                if nb:
                    src = torch.frombuffer(bytearray(raw[off:off + nb]), dtype=torch.uint8)
                    L.t[name].view(torch.uint8)[:nb].copy_(src.to(self.device))
                off += nb
            L.boundary, L.write_pos = boundary, write_pos
        return n
