"""Seeded synthetic inputs with Bonsai-27B's attention shapes and value distributions.

The reference measures on a real prompt through real weights; neither is available, so every
test and benchmark here draws from one generator:

* per kv-head and channel a scale ``s_c = exp(0.5*N(0,1))``, four outlier channels per kv-head
  multiplied by 8, drawn independently for K and V;
* ``K_unroped[t,h,c] = s_c*N(0,1)``, ``V[t,h,c] = s'_c*N(0,1)``, stored as fp16;
* raw-ring K is the un-RoPE'd K rotated at its absolute position with the reference's fp32
  half-split RoPE (``src/kernels/elementwise_sm75.mojo:1023-1061``);
* ``q_gate`` (24, 512): query part N(0,1) rotated at the query position, gate part N(0,1);
* calibration tables in the ``khq_calib.bin`` layout: the reference's xorshift +-1 sign vectors
  (``src/khq/calib.mojo:137-143, 197-203``), random orthogonal 4x4 rotors (or identity, which is
  what the reference's calibration leaves for K, ``src/khq/calib.mojo:386-390``), K centroids
  from the K-static formula (``src/csrc/qmv_sm75_kernel.cu:2645-2680``), V dim-3 centroids
  -+0.7979*sigma, and an N(0,1) 256x3 VQ codebook per patch.
"""
from __future__ import annotations

import numpy as np

from .calib import D, NP, KhqLayerTables

H_Q, H_KV, N_REP = 24, 4, 6
ROTARY_DIM = 64
ROPE_THETA = 1e7
SEED_BASE = 20260914


def seed_for(config: int, layer: int = 0, seq: int = 0) -> int:
    return SEED_BASE + 1000 * config + 17 * layer + seq


def xorshift_signs(layer_id: int, kind: str) -> np.ndarray:
    """The reference's +-1 sign vectors: xorshift32 seeded per layer, one draw per dim."""
    if kind == "k":
        s = (layer_id * 2654435761 + 12345) & 0xFFFFFFFF
    else:
        s = (layer_id * 40503 + 987654321) & 0xFFFFFFFF
    out = np.empty(D, np.float32)
    for i in range(D):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = 1.0 if (s & 1) else -1.0
    return out


def channel_scales(rng: np.random.Generator) -> np.ndarray:
    """(H_KV, D) per-channel standard deviations with four x8 outlier channels per head."""
    s = np.exp(0.5 * rng.standard_normal((H_KV, D))).astype(np.float32)
    for h in range(H_KV):
        s[h, rng.choice(D, size=4, replace=False)] *= 8.0
    return s


def make_kv(rng: np.random.Generator, n_tok: int, scales_k=None, scales_v=None):
    """K (un-RoPE'd) and V, fp16 (n_tok, H_KV, D)."""
    if scales_k is None:
        scales_k = channel_scales(rng)
    if scales_v is None:
        scales_v = channel_scales(rng)
    k = (rng.standard_normal((n_tok, H_KV, D)).astype(np.float32) * scales_k).astype(np.float16)
    v = (rng.standard_normal((n_tok, H_KV, D)).astype(np.float32) * scales_v).astype(np.float16)
    return k, v


def rope_freqs_raw() -> np.ndarray:
    """freq_i = exp(log(theta) * (-2i/64)) in fp32 -- the raw-K / query RoPE of the reference."""
    i = np.arange(ROTARY_DIM // 2, dtype=np.float32)
    ex = -(2.0 * i) / np.float32(ROTARY_DIM)
    return np.exp(np.log(np.float32(ROPE_THETA)) * ex).astype(np.float32)


def partial_rope(x: np.ndarray, pos) -> np.ndarray:
    """Half-split RoPE on dims (i, i+32), i<32, of the last axis; fp32 angle pos*freq.
    ``x``: (..., D) fp16; ``pos``: scalar or array broadcastable to x.shape[:-1]."""
    xf = x.astype(np.float32)
    freq = rope_freqs_raw()
    ang = (np.asarray(pos, np.float32)[..., None] * freq).astype(np.float32)
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    half = ROTARY_DIM // 2
    x0, x1 = xf[..., :half].copy(), xf[..., half:ROTARY_DIM].copy()
    out = xf.copy()
    out[..., :half] = x0 * c - x1 * s
    out[..., half:ROTARY_DIM] = x0 * s + x1 * c
    return out.astype(np.float16)


def make_q_gate(rng: np.random.Generator, pos: int) -> np.ndarray:
    """(H_Q, 2*D) fp16: RoPE'd query at [0,D), gate logits at [D,2D)."""
    q = rng.standard_normal((H_Q, D)).astype(np.float32).astype(np.float16)
    q = partial_rope(q, np.full((H_Q,), pos))
    g = rng.standard_normal((H_Q, D)).astype(np.float32).astype(np.float16)
    return np.concatenate([q, g], axis=1)


def random_rotors(rng: np.random.Generator) -> np.ndarray:
    """(64, 16): 64 random orthogonal 4x4 matrices (QR of N(0,1)), element [k][c] at k*4+c."""
    out = np.empty((NP, 16), np.float32)
    for p in range(NP):
        qm, r = np.linalg.qr(rng.standard_normal((4, 4)))
        qm = qm * np.sign(np.diag(r))
        out[p] = qm.astype(np.float32).reshape(16)
    return out


def fwht(x: np.ndarray) -> np.ndarray:
    """Unnormalised natural-order FWHT over the last axis (length 256)."""
    y = x.astype(np.float32).copy()
    n = y.shape[-1]
    h = 1
    while h < n:
        y = y.reshape(y.shape[:-1] + (n // (2 * h), 2, h))
        a, b = y[..., 0, :].copy(), y[..., 1, :].copy()
        y[..., 0, :], y[..., 1, :] = a + b, a - b
        y = y.reshape(y.shape[:-3] + (n,))
        h *= 2
    return y


def project(x: np.ndarray, d_vec: np.ndarray, rotor: np.ndarray) -> np.ndarray:
    """rows (N, D) -> the projected domain the code words live in: rotor(FWHT(x*d/|x|))/16."""
    xf = x.astype(np.float32)
    nrm = np.sqrt((xf * xf).sum(-1, keepdims=True) + 1e-8)
    r = fwht(xf * d_vec / (nrm + 1e-8))
    r = r.reshape(-1, NP, 4)
    R = rotor.reshape(NP, 4, 4)  # [p][k][c]
    rot = np.einsum("npk,pkc->npc", r, R).reshape(-1, D)
    return (rot * np.float32(0.0625)).astype(np.float32)


def make_tables(rng: np.random.Generator, layer_id: int, k_sample: np.ndarray, v_sample: np.ndarray,
                vq_scale: float = 1.0, k_rotor_identity: bool = False,
                adaptive_mult: bool = False) -> KhqLayerTables:
    """Synthetic calibration tables for one layer.

    ``k_sample`` / ``v_sample``: (N, D) fp16 rows the per-dim sigmas are measured on.
    ``adaptive_mult``: store unscaled K centroids (ts_k = 1) so that the per-row base multiplier
    of the compress kernel lands inside its accepted range 0.1..10 and is actually exercised;
    with the K-static formula it is always clamped to 1.
    """
    d_k, d_v = xorshift_signs(layer_id, "k"), xorshift_signs(layer_id, "v")
    rotor_k = np.tile(np.eye(4, dtype=np.float32).reshape(16), (NP, 1)) if k_rotor_identity else random_rotors(rng)
    rotor_v = random_rotors(rng)
    sig_k = project(k_sample, d_k, rotor_k).std(axis=0).astype(np.float32)
    sig_v = project(v_sample, d_v, rotor_v).std(axis=0).astype(np.float32)
    if adaptive_mult:
        ts_k = np.float32(1.0)
    else:
        psum = 0.528756 * (0.9350 * sig_k) ** 2 + 0.464545 * sig_k ** 2
        ts_k = np.float32(16.0 / np.sqrt(psum.sum()))
    cb = (0.9350 * sig_k * ts_k).astype(np.float32)
    cents_k = np.stack([np.zeros(D, np.float32), -cb, cb, cb])
    cv = (0.7979 * sig_v).astype(np.float32)
    cents_v = np.stack([-cv, cv, np.zeros(D, np.float32), np.zeros(D, np.float32)])
    vq = (rng.standard_normal((NP, 256, 3)) * vq_scale).astype(np.float32)
    return KhqLayerTables(layer_id, float(ts_k), 1.0, d_k, cents_k, rotor_k, 1.95, 1.0, d_v,
                          cents_v, rotor_v, vq)
