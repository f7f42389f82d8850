"""ctypes front end of the CPU oracle (oracle/khq_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
may import this module; the shipped package never does.  ``OracleOps`` offers the same launch
interface as the package's ``ops.CudaOps`` but executes every launch on the host through the
oracle, so the host state machine can be driven end to end on CPU tensors and compared with the
GPU run step by step.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_uint16, c_uint32, c_void_p
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = _DIR / "libkhq_oracle.so"
_lib = None

D = 256
PART = D + 2


def build(force: bool = False) -> Path:
    """Compile the C restatement (and, when the reference checkout is present, the reference's
    own CUDA source for sm_100a into oracle/_ref/)."""
    src = _DIR / "khq_oracle.c"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "libkhq_oracle.so"], check=True, capture_output=True)
    ref_root = _reference_root()
    if ref_root:
        subprocess.run(["make", "-C", str(_DIR), "ref", "REF_ROOT=" + ref_root], check=False, capture_output=True)
    return _LIB


def _reference_root() -> str:
    """Where the reference checkout lies, if anywhere: $KHQ_REF_ROOT, else the ``reference_path``
    the repository's BASELINE.json records.  Empty when neither names an existing directory."""
    import json
    import os

    cand = os.environ.get("KHQ_REF_ROOT", "")
    if not cand:
        try:
            cand = json.loads((_DIR.parent / "BASELINE.json").read_text()).get("reference_path", "")
        except (OSError, ValueError):
            cand = ""
    return cand if cand and Path(cand).is_dir() else ""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB))
        _lib.khq_oracle_h2f.restype = c_float
        _lib.khq_oracle_h2f.argtypes = [c_uint16]
        _lib.khq_oracle_f2h.restype = c_uint16
        _lib.khq_oracle_f2h.argtypes = [c_float]
    return _lib


def _p(a):
    """Host address of a numpy array / CPU torch tensor / None."""
    if a is None:
        return c_void_p(0)
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return c_void_p(a.ctypes.data)
    return c_void_p(a.data_ptr())  # CPU torch tensor (possibly a view)


# ---------------------------------------------------------------------------- compress
def compress(x, d_vec, rotor, cents, vq, n, ts, alpha, is_v, d=D):
    """Returns dict(mask, norms, r_norms, payload, shared_meta, near_ties, rc).  Inputs are fp16
    numpy arrays (viewed as uint16 bit patterns)."""
    lib = load()
    n_alloc = max(n, 0)
    out = {
        "mask": np.zeros((n_alloc, 16), np.uint32),
        "norms": np.zeros(n_alloc, np.float16),
        "r_norms": np.zeros(n_alloc, np.float16),
        "payload": np.zeros((n_alloc, 104 if is_v else 40), np.uint8),
        "shared_meta": np.zeros((n_alloc, 4), np.uint8),
    }
    ties = c_uint32(0)
    rc = lib.khq_oracle_compress(_p(x), _p(d_vec), _p(rotor), _p(cents), _p(vq), _p(out["mask"]),
                                 _p(out["norms"]), _p(out["r_norms"]), _p(out["payload"]),
                                 _p(out["shared_meta"]), c_int(n), c_int(d), c_float(ts), c_float(alpha),
                                 c_int(1 if is_v else 0), ctypes.byref(ties))
    out["near_ties"] = ties.value
    out["rc"] = rc
    return out


def compress_into(x, d_vec, rotor, cents, vq, out_mask, out_norms, out_r_norms, out_payload,
                  out_shared_meta, n, d, ts, alpha, is_v) -> int:
    lib = load()
    return lib.khq_oracle_compress(_p(x), _p(d_vec), _p(rotor), _p(cents), _p(vq), _p(out_mask),
                                   _p(out_norms), _p(out_r_norms), _p(out_payload), _p(out_shared_meta),
                                   c_int(n), c_int(d), c_float(ts), c_float(alpha),
                                   c_int(1 if is_v else 0), None)


# ---------------------------------------------------------------------------- decode rows
def decode_k(payload_row, mask_row, norm, r_norm, cents, rotor, d_vec, alpha_k):
    lib = load()
    out = np.zeros(D, np.float64)
    lib.khq_oracle_decode_k(_p(payload_row), _p(mask_row), c_uint16(int(np.float16(norm).view(np.uint16))),
                            c_uint16(int(np.float16(r_norm).view(np.uint16))), _p(cents), _p(rotor),
                            _p(d_vec), c_float(alpha_k), _p(out))
    return out


def decode_v(payload_row, norm, energy, sm_scale, cents_v, vq, rotor_v, d_vec_v, alpha_v):
    lib = load()
    out = np.zeros(D, np.float64)
    lib.khq_oracle_decode_v(_p(payload_row), c_uint16(int(np.float16(norm).view(np.uint16))),
                            c_uint16(int(np.float16(energy).view(np.uint16))), c_float(sm_scale),
                            _p(cents_v), _p(vq), _p(rotor_v), _p(d_vec_v), c_float(alpha_v), _p(out))
    return out


# ---------------------------------------------------------------------------- attention
def attn_launch(q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms, v_r_norms,
                cents_k, cents_v, vq, k_rotor, v_rotor, d_k, d_v, out_attn, out_partial, num_queries,
                num_heads, c_len, n_rep, scale, alpha_k, alpha_v, rope_base, start_pos, num_splits) -> int:
    lib = load()
    return lib.khq_oracle_attn_launch(
        _p(q), _p(k_payload), _p(v_payload), _p(v_shared_meta), _p(k_mask), _p(k_norms), _p(k_r_norms),
        _p(v_norms), _p(v_r_norms), _p(cents_k), _p(cents_v), _p(vq), _p(k_rotor), _p(v_rotor), _p(d_k),
        _p(d_v), _p(out_attn), _p(out_partial), c_int(num_queries), c_int(num_heads), c_int(c_len),
        c_int(n_rep), c_float(scale), c_float(alpha_k), c_float(alpha_v), c_float(rope_base),
        c_int(start_pos), c_int(num_splits))


def attn_partial(q, kv, tables, num_heads, n_rep, scale, alpha_k, alpha_v, rope_base, start_pos, s_lo, s_hi):
    """kv: dict with k_payload.. arrays; tables: dict cents_k.. ; returns (num_heads, 258) fp32."""
    lib = load()
    out = np.zeros((num_heads, PART), np.float32)
    lib.khq_oracle_attn_partial(
        _p(q), _p(kv["k_payload"]), _p(kv["v_payload"]), _p(kv["v_shared_meta"]), _p(kv["k_mask"]),
        _p(kv["k_norms"]), _p(kv["k_r_norms"]), _p(kv["v_norms"]), _p(kv["v_r_norms"]), _p(tables["cents_k"]),
        _p(tables["cents_v"]), _p(tables["vq"]), _p(tables["rotor_k"]), _p(tables["rotor_v"]), _p(tables["d_k"]),
        _p(tables["d_v"]), _p(out), c_int(num_heads), c_int(n_rep), c_float(scale), c_float(alpha_k),
        c_float(alpha_v), c_float(rope_base), c_int(start_pos), c_int(s_lo), c_int(s_hi))
    return out


def attn_reduce(partial, nq, splits):
    lib = load()
    out = np.zeros((nq, PART), np.float32)
    lib.khq_oracle_attn_reduce(_p(partial), _p(out), c_int(nq), c_int(splits))
    return out


def window_attn(q, ring_k, ring_v, out, win_start, win_len, ring_cap, H_q, H_kv, d, scale) -> int:
    lib = load()
    return lib.khq_oracle_window_attn(_p(q), _p(ring_k), _p(ring_v), _p(out), c_int(win_start),
                                      c_int(win_len), c_int(ring_cap), c_int(H_q), c_int(H_kv), c_int(d),
                                      c_float(scale))


def merge_gate(attn_c, attn_w, q_gate, out, H_q, d, has_w) -> int:
    lib = load()
    return lib.khq_oracle_merge_gate(_p(attn_c), _p(attn_w), _p(q_gate), _p(out), c_int(H_q), c_int(d),
                                     c_int(has_w))


def gqa_attention_f32(q_gate, k_cache, v_cache, seq_len, H_q, H_kv, d, scale):
    lib = load()
    out = np.zeros((H_q, d), np.float64)
    lib.khq_oracle_gqa_attention_f32(_p(q_gate), _p(k_cache), _p(v_cache), _p(out), c_int(seq_len),
                                     c_int(H_q), c_int(H_kv), c_int(d), c_double(scale))
    return out


def gqa_prefill(q_gate, k, v, T, H_q, H_kv, d, scale):
    lib = load()
    out = np.zeros((T, H_q, d), np.float32)
    lib.khq_oracle_gqa_prefill(_p(q_gate), _p(k), _p(v), _p(out), c_int(T), c_int(H_q), c_int(H_kv),
                               c_int(d), c_float(scale))
    return out


def partial_rope(vec, num_heads, head_dim, rotary_dim, pos, theta, stride):
    """In place on a fp16 numpy array."""
    lib = load()
    lib.khq_oracle_partial_rope(_p(vec), c_int(num_heads), c_int(head_dim), c_int(rotary_dim), c_int(pos),
                                c_float(theta), c_int(stride))
    return vec


def head_rmsnorm(x, num_heads, head_dim, stride, weight, eps):
    """In place on a fp16 numpy array / CPU tensor."""
    lib = load()
    lib.khq_oracle_head_rmsnorm(_p(x), c_int(num_heads), c_int(head_dim), c_int(stride), _p(weight), c_float(eps))
    return x


def cal_kstatic(rot):
    """K-static fit of a projected sample (rows, 256) fp32 -> (cents (4, 256), ts, sigma (256,))."""
    lib = load()
    rot = np.ascontiguousarray(rot, np.float32)
    cents = np.zeros((4, 256), np.float32)
    ts = np.zeros(1, np.float32)
    sigma = np.zeros(256, np.float32)
    lib.khq_oracle_cal_kstatic(_p(rot), c_int(rot.shape[0]), _p(cents), _p(ts), _p(sigma))
    return cents, float(ts[0]), sigma


# ---------------------------------------------------------------------------- launch backend
class OracleLaunchError(RuntimeError):
    def __init__(self, name, code):
        super().__init__(f"{name} returned {code}")
        self.code = code


class OracleOps:
    """Drop-in for the package's CudaOps on CPU torch tensors: every launch runs in the oracle."""

    name = "oracle"

    def compress(self, x, d_vec, rotor, centroids, vq_centroids, out_mask, out_norms, out_r_norms,
                 out_payload, out_shared_meta, n, d, ts, alpha, is_v):
        rc = compress_into(x, d_vec, rotor, centroids, vq_centroids, out_mask, out_norms, out_r_norms,
                           out_payload, out_shared_meta, n, d, ts, alpha, is_v)
        if rc:
            raise OracleLaunchError("compress", rc)

    def attn(self, q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms,
             v_r_norms, centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k, d_vec_v,
             out_attn, out_partial, num_queries, num_heads, L_q, c_len, stride_s, n_rep, scale,
             alpha_k, alpha_v, rope_base, start_pos, num_splits):
        assert L_q == 1
        rc = attn_launch(q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms,
                         v_r_norms, centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k,
                         d_vec_v, out_attn, out_partial, num_queries, num_heads, c_len, n_rep, scale,
                         alpha_k, alpha_v, rope_base, start_pos, num_splits)
        if rc:
            raise OracleLaunchError("attn", rc)

    def attn_strided(self, q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms, v_norms,
                     v_r_norms, centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k, d_vec_v,
                     out_attn, out_partial, num_queries, num_heads, L_q, c_len, n_rep, scale, alpha_k, alpha_v,
                     rope_base, start_pos, num_splits, pos_chunk, pos_stride):
        """A slice whose local chunk j sits at absolute position start_pos + j * pos_stride: one oracle
        call per chunk at that position, then the oracle's own split reduce over the chunks."""
        assert L_q == 1
        np_ = lambda a: a if isinstance(a, np.ndarray) else a.numpy()
        arrs = {"k_payload": (np_(k_payload), 40), "v_payload": (np_(v_payload), 104), "v_shared_meta": (np_(v_shared_meta), 4),
                "k_mask": (np_(k_mask), 16), "k_norms": (np_(k_norms), 1), "k_r_norms": (np_(k_r_norms), 1),
                "v_norms": (np_(v_norms), 1), "v_r_norms": (np_(v_r_norms), 1)}
        n_chunks = (c_len + pos_chunk - 1) // pos_chunk
        parts = np.zeros((num_heads, n_chunks, PART), np.float32)
        for j in range(n_chunks):
            t0, t1 = j * pos_chunk, min(c_len, (j + 1) * pos_chunk)
            sl = {k: np.ascontiguousarray(a.reshape(-1)[t0 * 4 * w:t1 * 4 * w]) for k, (a, w) in arrs.items()}
            one = np.zeros((num_heads, PART), np.float32)
            rc = attn_launch(q, sl["k_payload"], sl["v_payload"], sl["v_shared_meta"], sl["k_mask"], sl["k_norms"], sl["k_r_norms"],
                             sl["v_norms"], sl["v_r_norms"], centroids_k, centroids_v, vq_centroids, k_rotor, v_rotor, d_vec_k,
                             d_vec_v, one, None, num_queries, num_heads, t1 - t0, n_rep, scale, alpha_k, alpha_v, rope_base,
                             start_pos + j * pos_stride, 1)
            if rc:
                raise OracleLaunchError("attn_strided", rc)
            parts[:, j] = one
        merged = attn_reduce(parts, num_heads, n_chunks)
        dst = out_attn if isinstance(out_attn, np.ndarray) else out_attn.numpy()
        dst.reshape(num_heads, PART)[:] = merged

    def window_attn(self, q, ring_k, ring_v, out_attn, win_start, win_len, ring_cap, H_q, H_kv, d, scale):
        rc = window_attn(q, ring_k, ring_v, out_attn, win_start, win_len, ring_cap, H_q, H_kv, d, scale)
        if rc:
            raise OracleLaunchError("window_attn", rc)

    def merge_gate(self, attn_c, attn_w, q_gate, out, H_q, d, has_w, has_c):
        src_c = attn_c if has_c else attn_w
        rc = merge_gate(src_c, attn_w, q_gate, out, H_q, d, 1 if (has_w and has_c) else 0)
        if rc:
            raise OracleLaunchError("merge_gate", rc)

    def merge_slots_gate(self, partials, n_slots, q_gate, out, H_q, d):
        """(n_slots, H_q, 258) slot-major partials -> LSE merge -> gate -> fp16 (reduce + merge_gate)."""
        import torch

        p = partials if isinstance(partials, np.ndarray) else partials.numpy()
        p = np.ascontiguousarray(p.reshape(n_slots, H_q, PART).transpose(1, 0, 2))
        merged = attn_reduce(p, H_q, n_slots)
        rc = merge_gate(merged, merged, q_gate, out, H_q, d, 0)
        if rc:
            raise OracleLaunchError("merge_slots_gate", rc)

    def gqa_prefill(self, q_gate, k, v, out, batch, T, H_q, H_kv, d, scale):
        import torch

        for b in range(batch):
            o = gqa_prefill(q_gate.reshape(batch, -1)[b].numpy(), k.reshape(batch, -1)[b].numpy(),
                            v.reshape(batch, -1)[b].numpy(), T, H_q, H_kv, d, scale)
            out.reshape(batch, -1)[b].copy_(torch.from_numpy(o.reshape(-1)).to(out.dtype))

    def prestep(self, q_gate, k, v, q_norm_w, k_norm_w, ring_k_slot, ring_v_slot, ring_u_slot, H_q, H_kv, d,
                rotary_dim, pos, rope_theta, rms_eps, has_norms):
        """q/k head RMSNorm, K capture, partial RoPE, ring appends (CPU torch tensors, in place)."""
        # the norm always runs; has_norms == 0 only drops the learned weight (src/ops.mojo:1397-1411)
        head_rmsnorm(q_gate, H_q, d, 2 * d, q_norm_w if has_norms else None, rms_eps)
        head_rmsnorm(k, H_kv, d, d, k_norm_w if has_norms else None, rms_eps)
        if ring_u_slot is not None:
            ring_u_slot.copy_(k.reshape(ring_u_slot.shape))
        lib = load()
        lib.khq_oracle_partial_rope(_p(q_gate), c_int(H_q), c_int(d), c_int(rotary_dim), c_int(pos),
                                    c_float(rope_theta), c_int(2 * d))
        lib.khq_oracle_partial_rope(_p(k), c_int(H_kv), c_int(d), c_int(rotary_dim), c_int(pos),
                                    c_float(rope_theta), c_int(d))
        if ring_k_slot is not None:
            ring_k_slot.copy_(k.reshape(ring_k_slot.shape))
        if ring_v_slot is not None:
            ring_v_slot.copy_(v.reshape(ring_v_slot.shape))

    def ring_write(self, dst_row, src):
        dst_row.copy_(src.reshape(dst_row.shape))

    def synchronize(self):
        pass
