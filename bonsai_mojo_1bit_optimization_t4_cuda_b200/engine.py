"""Batched KHQ decode engine: B independent sequences x L attention layers resident on one GPU.

This is the public entry a serving host calls once per generated token: hand it this step's
projections for every sequence (host buffers), get the gated attention outputs back (host
buffers).  Sequences are independent, so they shard across GPUs by sequence with no collective
(one engine per rank).

Per step and sequence the engine does what the reference's ``khq_step`` does for its single
sequence (``src/khq/runtime.mojo:454-613``): the new token goes to ring slot ``write_pos % 256``
and ``write_pos`` advances; when the raw window has reached 256 tokens (and the compressed
capacity allows) the 128 oldest tokens are compressed and ``boundary`` moves on by 128; the
attention then runs over ``c_len = boundary`` compressed tokens and the ``write_pos - boundary``
raw ones.  Per layer that is one launch for the q/k head norms, K capture, RoPE and the three
ring appends of ALL sequences (``launch_khq_prestep_batched_fp16``), one K and one V compress
launch over the sequences whose event is due (``launch_khq_compress_batched_fp16``), and one
batched attention launch (``launch_khq_decode_batched_fp16``); the work items are re-planned
on the host every step and the step-dependent descriptor fields of every layer are rewritten by
one small launch (``launch_khq_update_descs``).

State layout: one contiguous device buffer per payload array and per layer, each sequence's
slice sized for its capacity and starting on a 128-row boundary.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from . import lib as _lib
from .batched import SEQ_DESC, TABLES_DESC, WORK_ITEM
from .calib import KhqLayerTables
from .lib import check, current_stream
from .synth import H_KV, H_Q

D = 256
RING = 256
CHUNK = 128
WATERMARK = 256
KV = H_KV * D  # halfs per token row group
ROTARY_DIM = 64
SEQ_DYN = np.dtype([("c_len", "<i4"), ("start_pos", "<i4"), ("win_start", "<i4"), ("win_len", "<i4"),
                    ("first_slot", "<i4"), ("n_slots", "<i4"), ("r0", "<i4"), ("r1", "<i4")])
COMPRESS_SEG = np.dtype([("x", "<u8"), ("row0", "<i8")])
assert SEQ_DYN.itemsize == 32 and COMPRESS_SEG.itemsize == 16


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class BatchEngine:
    def __init__(self, tables: Sequence[KhqLayerTables], c_len: Sequence[int], win_len: Sequence[int],
                 device="cuda", tokens_per_item: int = 0, codebook_in_smem: int = -1, grow_tokens: int = 1024,
                 norm_weights: Optional[Sequence] = None, rope_theta: float = 1e7, rms_eps: float = 1e-6):
        """``c_len`` / ``win_len``: compressed and raw tokens each sequence starts with (``c_len`` a
        multiple of 128, as the state machine leaves it).  ``grow_tokens``: compressed capacity kept
        free behind every sequence's initial prefix.  ``norm_weights``: per layer ``(q_w, k_w)`` fp32
        (256,) arrays for the head RMS norms, or None for the unweighted norm."""
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.L = len(tables)
        self.B = len(c_len)
        self.boundary = np.asarray(c_len, np.int64).copy()
        self.write_pos = self.boundary + np.asarray(win_len, np.int64)
        assert (self.boundary % CHUNK == 0).all(), "compressed prefixes are whole 128-token chunks"
        assert ((self.write_pos - self.boundary) <= RING).all() and (np.asarray(win_len) >= 0).all()
        self.cap = self.boundary + _align(max(int(grow_tokens), 0), CHUNK)
        self.codebook_in_smem = codebook_in_smem
        self.rope_theta, self.rms_eps = float(rope_theta), float(rms_eps)
        self.host_tables = list(tables)
        dev = self.device
        z = lambda n, dt: torch.zeros(max(int(n), 1), dtype=dt, device=dev)
        # ---- tables ------------------------------------------------------------------------
        self.tables = []
        for tb in tables:
            f = tb.as_f16()
            self.tables.append(dict(
                cents_k=torch.from_numpy(f["cents_k"]).to(dev), cents_v=torch.from_numpy(f["cents_v"]).to(dev),
                vq=torch.from_numpy(f["vq"]).to(dev), k_rotor=torch.from_numpy(f["rotor_k"]).to(dev),
                v_rotor=torch.from_numpy(f["rotor_v"]).to(dev), d_k=torch.from_numpy(f["d_k"]).to(dev),
                d_v=torch.from_numpy(f["d_v"]).to(dev), alpha_k=tb.alpha_k, alpha_v=tb.alpha_v,
                ts_k=tb.ts_k, ts_v=tb.ts_v))
        t = np.zeros(self.L, TABLES_DESC)
        for i, tb in enumerate(self.tables):
            for k in ("cents_k", "cents_v", "vq", "k_rotor", "v_rotor", "d_k", "d_v"):
                t[k][i] = tb[k].data_ptr()
            t["alpha_k"][i], t["alpha_v"][i] = tb["alpha_k"], tb["alpha_v"]
        self.d_tables = torch.from_numpy(t.view(np.uint8).reshape(-1).copy()).to(dev)
        self.norm_w = None
        if norm_weights is not None:
            self.norm_w = [(torch.as_tensor(np.asarray(q, np.float32)).to(dev), torch.as_tensor(np.asarray(k, np.float32)).to(dev))
                           for q, k in norm_weights]
        # ---- payload arrays: per layer one buffer per array, sequences at aligned row offsets --
        rows = self.cap * H_KV
        self.row_off = np.zeros(self.B + 1, np.int64)  # in rows, multiples of 128 rows
        for i in range(self.B):
            self.row_off[i + 1] = self.row_off[i] + _align(int(rows[i]), 128)
        R = int(self.row_off[-1])
        self.pay = [dict(k_mask=z(R * 16, torch.int32), k_payload=z(R * 40, torch.uint8),
                         v_payload=z(R * 104, torch.uint8), v_shared_meta=z(R * 4, torch.uint8),
                         k_norms=z(R, torch.float16), k_r_norms=z(R, torch.float16),
                         v_norms=z(R, torch.float16), v_r_norms=z(R, torch.float16)) for _ in range(self.L)]
        ring = lambda: z(self.B * RING * KV, torch.float16).view(self.B, RING, KV)
        self.ring_k = [ring() for _ in range(self.L)]
        self.ring_v = [ring() for _ in range(self.L)]
        self.ring_u = [ring() for _ in range(self.L)]
        self.q_gate = [z(self.B * H_Q * 2 * D, torch.float16).view(self.B, H_Q * 2 * D) for _ in range(self.L)]
        self.out = [z(self.B * H_Q * D, torch.float16).view(self.B, H_Q * D) for _ in range(self.L)]
        # two parities of the K / V input rows: the copy stream fills one while the pre-step reads the other
        self.d_k = [z(self.B * KV, torch.float16).view(self.B, KV) for _ in range(2)]
        self.d_v = [z(self.B * KV, torch.float16).view(self.B, KV) for _ in range(2)]
        self._copy_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        # ---- descriptors: layer-major, pointers fixed, the step-dependent ints rewritten per step
        d = np.zeros(self.L * self.B, SEQ_DESC)
        for l in range(self.L):
            P = self.pay[l]
            for i in range(self.B):
                r0 = int(self.row_off[i])
                e = d[l * self.B + i]
                e["q_gate"], e["out"] = self.q_gate[l][i].data_ptr(), self.out[l][i].data_ptr()
                e["ring_k"], e["ring_v"] = self.ring_k[l][i].data_ptr(), self.ring_v[l][i].data_ptr()
                e["k_mask"], e["k_payload"] = P["k_mask"][r0 * 16:].data_ptr(), P["k_payload"][r0 * 40:].data_ptr()
                e["v_payload"], e["v_shared_meta"] = P["v_payload"][r0 * 104:].data_ptr(), P["v_shared_meta"][r0 * 4:].data_ptr()
                e["k_norms"], e["k_r_norms"] = P["k_norms"][r0:].data_ptr(), P["k_r_norms"][r0:].data_ptr()
                e["v_norms"], e["v_r_norms"] = P["v_norms"][r0:].data_ptr(), P["v_r_norms"][r0:].data_ptr()
                e["table_id"] = l
        self.d_descs = torch.from_numpy(d.view(np.uint8).reshape(-1).copy()).to(dev)
        # ---- planning ----------------------------------------------------------------------
        # tokens_per_item <= 0: the library's planner chooses (it is handed 0 every step); the size it would start
        # from only bounds the buffers here
        self.tokens_per_item_arg = int(tokens_per_item) if tokens_per_item > 0 else 0
        if tokens_per_item <= 0:
            sms = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
            tokens_per_item = int(min(max(int(self.cap.sum()) // (2 * sms), 96), 8192))
        self.tokens_per_item = (tokens_per_item + 95) // 96 * 96
        # the planner shrinks the last items of a launch (down to 48 tokens), or cuts one to three pieces per
        # SM: room for either on top of the full-size items
        sms_plan = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
        tail_items = int(4 * sms_plan * (1.0 + np.log(self.tokens_per_item / 48.0))) + 16
        self.max_items = int(sum((int(c) + self.tokens_per_item - 1) // self.tokens_per_item + 2 for c in self.cap)) + tail_items
        self.ws_bytes = int(self.lib.khq_b200_decode_workspace_bytes(self.max_items))
        self.workspace = z(self.ws_bytes, torch.uint8)
        self.d_items = z(self.max_items * WORK_ITEM.itemsize, torch.uint8)
        self.d_dyn = z(self.B * SEQ_DYN.itemsize, torch.uint8)
        self.d_slots = z(self.B, torch.int32)
        self.d_pos = z(self.B, torch.int32)
        self.d_segs = z(self.L * self.B * COMPRESS_SEG.itemsize, torch.uint8)
        # ---- pinned host staging: two parities of the control block, one set of data buffers ----
        cuda = dev.type == "cuda"
        pin = lambda *shape, dt=torch.float16: (torch.zeros(*shape, dtype=dt).pin_memory() if cuda else torch.zeros(*shape, dtype=dt))
        self.h_q = pin(self.L, self.B, H_Q * 2 * D)
        self.h_k = pin(self.L, self.B, KV)
        self.h_v = pin(self.L, self.B, KV)
        self.h_out = pin(self.L, self.B, H_Q * D)
        self._ctl = [dict(items=pin(self.max_items * WORK_ITEM.itemsize, dt=torch.uint8), dyn=pin(self.B * SEQ_DYN.itemsize, dt=torch.uint8),
                          slots=pin(self.B, dt=torch.int32), pos=pin(self.B, dt=torch.int32),
                          segs=pin(self.L * self.B * COMPRESS_SEG.itemsize, dt=torch.uint8),
                          done=(torch.cuda.Event() if cuda else None)) for _ in range(2)]
        self._step = 0
        self.n_items = 0
        self.events_fired = 0
        self._plan_and_upload(self._ctl[0])

    # ---------------------------------------------------------------------------------- sizes
    @property
    def c_len(self) -> np.ndarray:
        return self.boundary

    @property
    def win_len(self) -> np.ndarray:
        return self.write_pos - self.boundary

    @property
    def win_start(self) -> np.ndarray:
        return self.boundary % RING

    @property
    def algorithmic_bytes_per_layer(self) -> int:
        return int(H_KV * (220 * self.boundary + 1024 * (self.write_pos - self.boundary)).sum())

    @property
    def h2d_bytes_per_step(self) -> int:
        """Projections of one step for every layer and sequence plus the step's control block
        (work items, per-sequence state, ring slots, positions)."""
        return self.L * self.B * (H_Q * 2 * D + 2 * KV) * 2 + self.n_items * WORK_ITEM.itemsize + self.B * (SEQ_DYN.itemsize + 8)

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.L * self.B * H_Q * D * 2

    # ---------------------------------------------------------------------------------- planning
    def _plan_and_upload(self, ctl) -> None:
        """Cut the current compressed prefixes and windows into work items (host planner of the
        library), and send items + per-sequence state to the device; one launch then rewrites the
        step-dependent fields of all L x B descriptors."""
        c = np.ascontiguousarray(self.boundary, np.int32)
        w = np.ascontiguousarray(self.write_pos - self.boundary, np.int32)
        first = np.zeros(self.B, np.int32)
        cnt = np.zeros(self.B, np.int32)
        items = ctl["items"].numpy().view(WORK_ITEM)
        n = self.lib.khq_b200_plan_decode(c.ctypes.data, w.ctypes.data, self.B, self.tokens_per_item_arg, items.ctypes.data,
                                          self.max_items, first.ctypes.data, cnt.ctypes.data)
        if n < 0 or n > self.max_items:
            raise _lib.KhqLaunchError("khq_b200_plan_decode", n)
        self.n_items = int(n)
        dyn = ctl["dyn"].numpy().view(SEQ_DYN)
        dyn["c_len"], dyn["start_pos"], dyn["win_start"], dyn["win_len"] = c, 0, (self.boundary % RING).astype(np.int32), w
        dyn["first_slot"], dyn["n_slots"] = first, cnt
        nb = self.n_items * WORK_ITEM.itemsize
        self.d_items[:nb].copy_(ctl["items"][:nb], non_blocking=True)
        self.d_dyn.copy_(ctl["dyn"], non_blocking=True)
        if self.device.type == "cuda":
            check("launch_khq_update_descs", self.lib.launch_khq_update_descs(self.d_descs.data_ptr(), self.d_dyn.data_ptr(), self.B,
                                                                              self.L, current_stream()))

    # ---------------------------------------------------------------------------------- loading
    def compress_into(self, layer: int, seq: int, k_unroped: torch.Tensor, v: torch.Tensor, tok0: int = 0) -> None:
        """Compress tokens [tok0, tok0+n) of one sequence-layer from fp16 (n, 4, 256) device tensors
        (two launch_khq_compress_fp16 calls, K then V)."""
        n = k_unroped.shape[0]
        rows = n * H_KV
        tb, P = self.tables[layer], self.pay[layer]
        r0 = int(self.row_off[seq]) + tok0 * H_KV
        st = current_stream()
        rc = self.lib.launch_khq_compress_fp16(
            k_unroped.data_ptr(), tb["d_k"].data_ptr(), tb["k_rotor"].data_ptr(), tb["cents_k"].data_ptr(),
            tb["cents_k"].data_ptr(), P["k_mask"][r0 * 16:].data_ptr(), P["k_norms"][r0:].data_ptr(),
            P["k_r_norms"][r0:].data_ptr(), P["k_payload"][r0 * 40:].data_ptr(), P["v_shared_meta"][r0 * 4:].data_ptr(),
            rows, D, float(tb["ts_k"]), float(tb["alpha_k"]), 0, st)
        check("launch_khq_compress_fp16", rc)
        rc = self.lib.launch_khq_compress_fp16(
            v.data_ptr(), tb["d_v"].data_ptr(), tb["v_rotor"].data_ptr(), tb["cents_v"].data_ptr(),
            tb["vq"].data_ptr(), P["k_mask"][r0 * 16:].data_ptr(), P["v_norms"][r0:].data_ptr(),
            P["v_r_norms"][r0:].data_ptr(), P["v_payload"][r0 * 104:].data_ptr(), P["v_shared_meta"][r0 * 4:].data_ptr(),
            rows, D, float(tb["ts_v"]), float(tb["alpha_v"]), 1, st)
        check("launch_khq_compress_fp16", rc)

    def load_window(self, layer: int, seq: int, k_roped: torch.Tensor, v: torch.Tensor, k_unroped: Optional[torch.Tensor] = None) -> None:
        """Place the sequence's raw tokens (fp16 (win_len, 4, 256)) into the ring slots of its window."""
        ws, wl = int(self.boundary[seq] % RING), int(self.write_pos[seq] - self.boundary[seq])
        slots = (ws + torch.arange(wl, device=self.device)) % RING
        self.ring_k[layer][seq, slots] = k_roped.reshape(wl, KV)
        self.ring_v[layer][seq, slots] = v.reshape(wl, KV)
        self.ring_u[layer][seq, slots] = (k_unroped if k_unroped is not None else k_roped).reshape(wl, KV)

    def fill_synthetic(self, seed: int, chunk_tokens: int = 16384) -> None:
        """Seeded synthetic state: per layer and kv-head channel scales exp(0.5 N(0,1)) with four x8
        outlier channels; K/V ~ N(0, s_c); compressed with the library's own compress kernel."""
        g = torch.Generator(device=self.device)
        for l in range(self.L):
            g.manual_seed(seed + 17 * l)
            sc = torch.exp(0.5 * torch.randn(2, H_KV, D, generator=g, device=self.device))
            for h in range(H_KV):
                for kv in range(2):
                    idx = torch.randperm(D, generator=g, device=self.device)[:4]
                    sc[kv, h, idx] *= 8.0
            for i in range(self.B):
                n = int(self.boundary[i])
                for t0 in range(0, n, chunk_tokens):
                    m = min(chunk_tokens, n - t0)
                    k = (torch.randn(m, H_KV, D, generator=g, device=self.device) * sc[0]).half()
                    v = (torch.randn(m, H_KV, D, generator=g, device=self.device) * sc[1]).half()
                    self.compress_into(l, i, k, v, t0)
                wl = int(self.write_pos[i] - self.boundary[i])
                if wl:
                    k = (torch.randn(wl, H_KV, D, generator=g, device=self.device) * sc[0]).half()
                    v = (torch.randn(wl, H_KV, D, generator=g, device=self.device) * sc[1]).half()
                    self.load_window(l, i, k, v)
            self.q_gate[l].copy_(torch.randn(self.B, H_Q * 2 * D, generator=g, device=self.device).half())

    # ---------------------------------------------------------------------------------- stepping
    def attention_resident(self, layer: int, scale: float = 1.0 / 16.0) -> None:
        """The hot path alone: one batched attention launch for `layer` over the current state,
        inputs already in HBM."""
        rc = self.lib.launch_khq_decode_batched_fp16(
            self.d_descs.data_ptr() + layer * self.B * SEQ_DESC.itemsize, self.d_tables.data_ptr(), self.d_items.data_ptr(),
            self.B, self.n_items, self.workspace.data_ptr(), self.ws_bytes, self.n_items, float(scale), self.rope_theta, RING,
            int(self.codebook_in_smem), current_stream())
        check("launch_khq_decode_batched_fp16", rc)

    def decode_step(self, scale: float = 1.0 / 16.0) -> torch.Tensor:
        """End-to-end token step from HOST buffers.  ``h_q`` (L, B, 24*512: query and gate halves, the
        query not yet normed or rotated), ``h_k`` and ``h_v`` (L, B, 4*256) hold this step's projections
        in pinned host memory.  Every sequence advances by one token: append, compression event if
        due, attention.  The gated outputs land in ``h_out`` (returned; valid once the stream has
        synchronised)."""
        ctl = self._ctl[self._step & 1]
        if ctl["done"] is not None:
            ctl["done"].synchronize()  # the copies that last read this parity's host block have finished
        self._step += 1
        # ---- host state machine (src/khq/runtime.mojo:486-553, for every sequence) -----------------
        slots = (self.write_pos % RING).astype(np.int32)
        pos = self.write_pos.astype(np.int32)
        self.write_pos += 1
        window = self.write_pos - self.boundary
        due = np.nonzero((window >= WATERMARK) & (self.boundary + CHUNK <= self.cap))[0]
        if (window[np.setdiff1d(np.arange(self.B), due)] > RING).any():
            raise RuntimeError("a sequence's compressed capacity is exhausted (raise grow_tokens)")
        ctl["slots"].numpy()[:] = slots
        ctl["pos"].numpy()[:] = pos
        n_ev = len(due)
        if n_ev:
            segs = ctl["segs"].numpy().view(COMPRESS_SEG).reshape(self.L, self.B)
            for l in range(self.L):
                base_u, base_v = self.ring_u[l].data_ptr(), self.ring_v[l].data_ptr()
                s0 = (self.boundary[due] % RING)
                off = (due * RING + s0) * KV * 2
                segs["x"][l, :n_ev] = base_u + off
                segs["row0"][l, :n_ev] = self.row_off[due] + self.boundary[due] * H_KV
            # the V launch reads ring_v at the same offsets: keep the byte distance per layer
            self._v_minus_u = [self.ring_v[l].data_ptr() - self.ring_u[l].data_ptr() for l in range(self.L)]
        self.boundary[due] += CHUNK
        self.events_fired += n_ev
        st = current_stream()
        self.d_slots.copy_(ctl["slots"], non_blocking=True)
        self.d_pos.copy_(ctl["pos"], non_blocking=True)
        if n_ev:
            self.d_segs.copy_(ctl["segs"], non_blocking=True)
        self._plan_and_upload(ctl)
        if ctl["done"] is not None:
            ctl["done"].record()
        seg_bytes = self.B * COMPRESS_SEG.itemsize
        # Host <-> device copies run on their own stream, one layer ahead of (inputs) and behind (outputs) the
        # kernels: layer l's inputs land while layer l - 1 computes.  Events order the two streams.
        main, cs = torch.cuda.current_stream(), self._copy_stream
        cs.wait_stream(main)  # everything queued so far (the previous step's reads of q_gate / d_k / d_v, the control block)
        in_ready, k_free = [None] * self.L, [None] * self.L

        def stage_inputs(l):
            with torch.cuda.stream(cs):
                if l >= 2:
                    cs.wait_event(k_free[l - 2])  # the pre-step of layer l - 2 has consumed this parity of d_k / d_v
                self.q_gate[l].copy_(self.h_q[l], non_blocking=True)
                self.d_k[l & 1].copy_(self.h_k[l], non_blocking=True)
                self.d_v[l & 1].copy_(self.h_v[l], non_blocking=True)
                in_ready[l] = cs.record_event()

        stage_inputs(0)
        for l in range(self.L):
            if l + 1 < self.L:
                stage_inputs(l + 1)
            main.wait_event(in_ready[l])
            d_k, d_v = self.d_k[l & 1], self.d_v[l & 1]
            qw, kw = self.norm_w[l] if self.norm_w is not None else (None, None)
            rc = self.lib.launch_khq_prestep_batched_fp16(
                self.q_gate[l].data_ptr(), d_k.data_ptr(), d_v.data_ptr(), _lib.ptr(qw), _lib.ptr(kw),
                self.ring_k[l].data_ptr(), self.ring_v[l].data_ptr(), self.ring_u[l].data_ptr(), RING * KV, self.d_slots.data_ptr(),
                self.d_pos.data_ptr(), self.B, H_Q, H_KV, D, ROTARY_DIM, self.rope_theta, self.rms_eps, 1 if qw is not None else 0, st)
            check("launch_khq_prestep_batched_fp16", rc)
            k_free[l] = main.record_event()
            if n_ev:
                tb, P = self.tables[l], self.pay[l]
                seg_ptr = self.d_segs.data_ptr() + l * seg_bytes
                rc = self.lib.launch_khq_compress_batched_fp16(
                    seg_ptr, n_ev, CHUNK * H_KV, tb["d_k"].data_ptr(), tb["k_rotor"].data_ptr(), tb["cents_k"].data_ptr(),
                    tb["cents_k"].data_ptr(), P["k_mask"].data_ptr(), P["k_norms"].data_ptr(), P["k_r_norms"].data_ptr(),
                    P["k_payload"].data_ptr(), P["v_shared_meta"].data_ptr(), D, float(tb["ts_k"]), float(tb["alpha_k"]), 0, 0, st)
                check("launch_khq_compress_batched_fp16", rc)
                rc = self.lib.launch_khq_compress_batched_fp16(
                    seg_ptr, n_ev, CHUNK * H_KV, tb["d_v"].data_ptr(), tb["v_rotor"].data_ptr(), tb["cents_v"].data_ptr(),
                    tb["vq"].data_ptr(), P["k_mask"].data_ptr(), P["v_norms"].data_ptr(), P["v_r_norms"].data_ptr(),
                    P["v_payload"].data_ptr(), P["v_shared_meta"].data_ptr(), D, float(tb["ts_v"]), float(tb["alpha_v"]), 1,
                    self._v_minus_u[l], st)
                check("launch_khq_compress_batched_fp16", rc)
            self.attention_resident(l, scale)
            done_l = main.record_event()
            with torch.cuda.stream(cs):
                cs.wait_event(done_l)
                self.h_out[l].copy_(self.out[l], non_blocking=True)
        main.wait_stream(cs)  # the caller synchronises the current stream before it reads h_out
        return self.h_out
