"""khq_b200_plan_decode: the host planner of the batched decode (pure host code in the CUDA
library, so it runs without a GPU).  Every problem's compressed tokens must be tiled exactly once by
items that start on even tokens (16-byte aligned rows of every payload array), slots must be
contiguous per problem, an explicit tokens_per_item bounds every piece, and the plan must keep the
tail of the launch short (list scheduling on 148 workers, the way the CTAs pull items)."""
import heapq

import numpy as np
import pytest

from bonsai_mojo_1bit_optimization_t4_cuda_b200 import batched


def _check_cover(items, first, cnt, c_len, win_len):
    # slots: problem by problem, the window's first; array order: all windows, then the pieces in problem order
    assert sorted(items["slot"]) == list(range(len(items)))
    n_win = int((items["kind"] == 1).sum())
    assert np.all(items["kind"][:n_win] == 1) and np.all(items["kind"][n_win:] == 0)
    assert np.all(np.diff(items["desc"][:n_win]) >= 0) and np.all(np.diff(items["desc"][n_win:]) >= 0)
    pos = 0
    for i, (cl, wl) in enumerate(zip(c_len, win_len)):
        assert first[i] == pos
        mine = items[items["desc"] == i]
        assert len(mine) == cnt[i] and sorted(mine["slot"]) == list(range(pos, pos + cnt[i]))
        comp = mine[mine["kind"] == 0]
        lo = 0
        for it in comp:
            assert it["lo"] == lo and it["lo"] % 2 == 0 and it["hi"] > it["lo"]
            lo = it["hi"]
        assert lo == max(cl, 0)
        win = mine[mine["kind"] == 1]
        assert (len(win) > 0) == (wl > 0)
        lo = 0
        for j, it in enumerate(win):  # window pieces tile [0, wl) and own the problem's first slots
            assert it["lo"] == lo and it["hi"] > it["lo"] and it["slot"] == pos + j
            lo = it["hi"]
        assert lo == max(wl, 0)
        pos += cnt[i]
    assert pos == len(items)


def _makespan(items, workers=148):
    free = [0.0] * workers
    heapq.heapify(free)
    for it in items:
        n = float(it["hi"] - it["lo"])
        heapq.heappush(free, heapq.heappop(free) + (3.0 * n if it["kind"] else n))
    return max(free)


@pytest.mark.parametrize("tokens_per_item", [0, 48, 96, 1000, 2048])
def test_plan_tiles_every_problem_exactly(tokens_per_item):
    rng = np.random.default_rng(5)
    c_len = np.concatenate([[0, 1, 2, 95, 96, 97, 143, 144, 131072], 128 * rng.integers(1, 256, size=40)]).astype(np.int32)
    win_len = rng.integers(0, 257, size=len(c_len)).astype(np.int32)
    win_len[0] = 0  # a problem with nothing at all: empty slot range
    items, first, cnt = batched.plan(c_len, win_len, tokens_per_item)
    _check_cover(items, first, cnt, c_len, win_len)
    if tokens_per_item > 0:
        cap = (tokens_per_item + 95) // 96 * 96
        comp = items[items["kind"] == 0]
        assert (comp["hi"] - comp["lo"]).max() <= cap + cap // 2


@pytest.mark.parametrize("c_len", [[131072], [65536], [16384], [384]])
def test_one_sequence_is_cut_into_one_balanced_wave(c_len):
    items, _, _ = batched.plan(np.array(c_len, np.int32), np.array([0], np.int32), 0)
    size = (items["hi"] - items["lo"]).astype(np.int64)
    assert size.sum() == c_len[0] and len(items) <= 148
    ideal = max(c_len[0] / 148.0, 24.0)
    assert size.max() <= ideal + 2


def test_many_sequences_end_with_small_items():
    rng = np.random.default_rng(6)
    c_len = (128 * rng.integers(30, 256, size=256)).astype(np.int32)
    win_len = rng.integers(128, 256, size=256).astype(np.int32)
    items, first, cnt = batched.plan(c_len, win_len, 0)
    _check_cover(items, first, cnt, c_len, win_len)
    comp = items[items["kind"] == 0]
    size = (comp["hi"] - comp["lo"]).astype(np.int64)
    assert size[: len(size) // 4].max() == 8256 and size[-20:].max() <= 144
    ideal = (float(c_len.sum()) + 3.0 * float(win_len.sum())) / 148.0
    assert _makespan(items) <= 1.01 * ideal


def test_small_launch_cuts_the_raw_window_too():
    # one sequence of 16 384 + 128 tokens: a raw token costs three compressed ones, so the window is cut into
    # pieces of about a third of a compressed piece and everything fits one wave of 148 items
    c_len, win_len = np.array([16384], np.int32), np.array([128], np.int32)
    items, first, cnt = batched.plan(c_len, win_len, 0)
    _check_cover(items, first, cnt, c_len, win_len)
    assert len(items) <= 148
    win = items[items["kind"] == 1]
    comp = items[items["kind"] == 0]
    assert len(win) >= 3 and (win["hi"] - win["lo"]).max() * 3 <= (comp["hi"] - comp["lo"]).max() + 24
