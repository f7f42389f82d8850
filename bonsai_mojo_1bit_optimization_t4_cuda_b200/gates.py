"""The reference's deploy-time checks of the KHQ path, restated over this runtime's debug lines.

The reference runs its decode with ``BONSAI_KHQ_DEBUG=1`` and greps two instrument lines out of
the log (``src/khq/runtime.mojo:530-552``; checks in ``deploy_on_kaggle.sh:1826-1937``):

    >> [KHQ-COMPRESS] layer <L> event# <k> boundary <b> write_pos <wp> raw_window <raw>
    >> [KHQ-NORM] <L> <boundary before the event> <n_rows> <fp16 bit pattern of every K norm>

* cadence gate (``:1826-1853``): per layer event k has boundary 128*k and leaves a raw window of
  128 tokens, and every layer sees the same number of events (first event at write_pos 256, then
  one every 128 tokens);
* payload-content gate (``:1855-1933``): the K norms of the rows just compressed are a fingerprint
  of WHICH tokens were compressed -- they must match the norms of the same tokens in
  ``kv_dump.bin`` (mean relative error <= 1e-2 per event) and match them at least five times
  better than the norms of the tokens 128 positions earlier or later.

The two model-level gates of the same script (top-1 logit and greedy-token prefix against the
uncompressed baseline, ``:1796-1824``) need the model weights and stay with the reference.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

_COMPRESS_RE = re.compile(r"\[KHQ-COMPRESS\] layer (\d+) event# (\d+) boundary (\d+) write_pos (\d+) raw_window (\d+)")
_NORM_RE = re.compile(r"\[KHQ-NORM\] (\d+) (\d+) (\d+) ([0-9 ]+)")


def parse_compress_events(log_text: str) -> Dict[int, List[Tuple[int, int, int, int]]]:
    """``{layer: [(event number, boundary, write_pos, raw_window), ...]}`` in log order."""
    ev: Dict[int, List[Tuple[int, int, int, int]]] = {}
    for m in _COMPRESS_RE.finditer(log_text):
        lay, num, bnd, wp, raw = (int(x) for x in m.groups())
        ev.setdefault(lay, []).append((num, bnd, wp, raw))
    return ev


def check_cadence(events: Dict[int, List[Tuple[int, int, int, int]]]) -> List[str]:
    """Failures of the cadence gate (empty list = pass)."""
    if not events:
        return ["no KHQ-COMPRESS line: cadence not measured"]
    fails = []
    counts = sorted({len(v) for v in events.values()})
    if len(counts) != 1:
        fails.append(f"events per layer differ: {counts}")
    off = []
    for lay, lst in sorted(events.items()):
        for k, (num, bnd, wp, raw) in enumerate(lst, 1):
            if num != k or bnd != 128 * k or raw != 128:
                off.append(f"L{lay}#{k}:b{bnd}/raw{raw}")
    if off:
        fails.append("cadence pattern off: " + "; ".join(off[:4]))
    return fails


@dataclass
class NormRecord:
    layer: int
    boundary: int   # first token of the rows just compressed
    n_rows: int
    bits: np.ndarray  # uint16 fp16 patterns, row = token*H_kv + head


def parse_norm_lines(log_text: str) -> List[NormRecord]:
    out = []
    for m in _NORM_RE.finditer(log_text):
        bits = np.array([int(x) for x in m.group(4).split()], dtype=np.uint16)
        out.append(NormRecord(int(m.group(1)), int(m.group(2)), int(m.group(3)), bits))
    return out


@dataclass
class PayloadGateResult:
    failures: List[str]
    events: int
    err_aligned_max: Optional[float]
    err_aligned_mean: Optional[float]
    err_shifted_mean: Optional[float]


def check_payload_norms(records: List[NormRecord], kv_dump_layers: Dict[int, Tuple[np.ndarray, np.ndarray]],
                        H_kv: int, head_dim: int) -> PayloadGateResult:
    """Payload-content gate.  ``kv_dump_layers``: what ``formats.read_kv_dump`` returns (K rows
    un-RoPE'd, (n_tokens, H_kv*head_dim) fp32)."""
    fails: List[str] = []
    if not records:
        return PayloadGateResult(["no KHQ-NORM line: payload contents not verified"], 0, None, None, None)
    cache: Dict[int, np.ndarray] = {}
    results = []
    for rec in records:
        if len(rec.bits) != rec.n_rows:
            fails.append(f"L{rec.layer} B{rec.boundary}: {len(rec.bits)} norms != {rec.n_rows} rows")
            continue
        if rec.layer not in kv_dump_layers:
            fails.append(f"L{rec.layer}: not in the dump")
            continue
        if rec.layer not in cache:
            k = kv_dump_layers[rec.layer][0]
            cache[rec.layer] = np.sqrt((k.reshape(k.shape[0], H_kv, head_dim).astype(np.float64) ** 2).sum(axis=2))
        g = cache[rec.layer]
        nt = g.shape[0]
        got = rec.bits.view(np.float16).astype(np.float64)
        idx = np.arange(rec.n_rows)
        tok, head = rec.boundary + idx // H_kv, idx % H_kv

        def err(tokens):
            ok = (tokens >= 0) & (tokens < nt)
            if not ok.any():
                return None
            a, b = g[tokens[ok], head[ok]], got[ok]
            return float(np.mean(np.abs(a - b) / (np.abs(a) + 1e-6)))

        results.append((err(tok), err(tok + 128), err(tok - 128)))
    e0 = np.array([r[0] for r in results if r[0] is not None])
    alt = np.array([x for r in results for x in r[1:] if x is not None])
    if e0.size and e0.max() > 1e-2:
        fails.append(f"payload norms off the ground truth (max rel-err {e0.max():.3e})")
    if e0.size and alt.size and alt.mean() < 5 * e0.mean():
        fails.append("the right alignment matches no better than a shifted one: wrong tokens compressed?")
    return PayloadGateResult(fails, len(results), float(e0.max()) if e0.size else None,
                             float(e0.mean()) if e0.size else None, float(alt.mean()) if alt.size else None)
