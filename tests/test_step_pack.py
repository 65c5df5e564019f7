"""What a step checks before it launches anything, and the integers it hands to the kernels
(no GPU: the packing is plain host code)."""
from __future__ import annotations

import numpy as np
import pytest

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200.engine.step import StepError, check_entries, pack_step
from longbow_quarrel_b200.kernels.attention import PREFILL_LISTS, step_needs


def _part(flat, info, name):
    o, n = info["layout"][name]
    return flat[o:o + n]


def test_errors_are_found_before_a_launch():
    check_entries([(0, [1, 2]), (3, [5])], None, 10)
    check_entries([(0, [1, 2]), (3, [5])], [[0, 1], []], 10)
    with pytest.raises(StepError, match="at least one"):
        check_entries([], None, 10)
    with pytest.raises(StepError, match="twice"):
        check_entries([(2, [1]), (2, [3])], None, 10)
    with pytest.raises(StepError, match="no tokens"):
        check_entries([(0, [1]), (1, [])], None, 10)
    with pytest.raises(StepError, match=r"token 10 at place 1 of sequence 0"):
        check_entries([(0, [1, 10])], None, 10)
    with pytest.raises(StepError, match="outside the vocabulary"):
        check_entries([(0, [-1])], None, 10)
    with pytest.raises(StepError, match="one list for each"):
        check_entries([(0, [1]), (1, [2])], [[0]], 10)
    with pytest.raises(StepError, match="wanted place 2 of sequence 1"):
        check_entries([(0, [1]), (1, [2, 3])], [[0], [2]], 10)


def test_positions_follow_each_sequences_own_past():
    entries = [(4, [7, 8, 9]), (1, [5]), (6, [3, 3, 3, 3, 3])]
    past = [0, 70, 129]
    flat, info = pack_step(entries, [[0, 2], [], [4]], past)
    assert flat.dtype == np.int32
    assert info["B"] == 3 and info["T"] == 9 and info["max_new"] == 5 and info["max_kv"] == 134
    assert _part(flat, info, "tokens").tolist() == [7, 8, 9, 5, 3, 3, 3, 3, 3]
    assert _part(flat, info, "tok_seq").tolist() == [0, 0, 0, 1, 2, 2, 2, 2, 2]
    assert _part(flat, info, "tok_pos").tolist() == [0, 1, 2, 70, 129, 130, 131, 132, 133]
    assert _part(flat, info, "slots").tolist() == [4, 1, 6]
    assert _part(flat, info, "kv_len").tolist() == [3, 71, 134]
    assert _part(flat, info, "cu_rows").tolist() == [0, 3, 4, 9]
    assert _part(flat, info, "want_rows").tolist() == [0, 2, 8]            # in the order of the entries and of want
    for name, (offset, _) in info["layout"].items():
        assert offset % 4 == 0, name                                      # every part starts on a 16-byte boundary


def test_without_want_the_last_row_of_every_sequence_is_asked_for():
    flat, info = pack_step([(0, [1, 2, 3]), (1, [4])], None, [0, 5])
    assert _part(flat, info, "want_rows").tolist() == [2, 3]
    flat, info = pack_step([(0, [1, 2, 3])], [[]], [0])
    assert len(_part(flat, info, "want_rows")) == 0


@pytest.mark.parametrize("name,size", [("query_blocks64", 64), ("query_blocks128", 128)])
def test_query_blocks_cover_every_row_once_longest_first(name, size):
    """The work lists of the prompt attention kernels are no business of the step function: the attention
    part names them (`step_needs`) and the step function packs what it is given."""
    rng = np.random.default_rng(3)
    new = [1, 64, 65, 200, 128, 129, 17]
    past = [0, 0, 100, 3, 64, 0, 700]
    entries = [(b, rng.integers(0, 50, n).tolist()) for b, n in enumerate(new)]
    flat, info = pack_step(entries, None, past, {name: PREFILL_LISTS[name]})
    assert info["extra"] == [name]
    seq, row, rows, pos = _part(flat, info, name).reshape(4, -1)
    tok_seq, tok_pos = _part(flat, info, "tok_seq"), _part(flat, info, "tok_pos")
    covered = np.zeros(sum(new), dtype=int)
    for s, r, n, p in zip(seq, row, rows, pos):
        assert 1 <= n <= size
        covered[r:r + n] += 1
        assert (tok_seq[r:r + n] == s).all()                               # a block stays inside one sequence
        assert tok_pos[r:r + n].tolist() == list(range(p, p + n))          # and its rows are consecutive positions
        assert (p - past[s]) % size == 0                                   # blocks start at multiples of the size
    assert (covered == 1).all()
    assert list(pos) == sorted(pos, reverse=True)                          # the blocks with the most keys come first
    assert len(seq) == sum(-(-n // size) for n in new)


def test_parts_name_the_step_arrays_they_need():
    import torch
    assert list(step_needs(torch.bfloat16, 128)) == ["query_blocks128"]
    assert list(step_needs(torch.bfloat16, 96)) == ["query_blocks64"]
    assert step_needs(torch.bfloat16, 40) == {} and step_needs(torch.float32, 128) == {}
    # a step of one token per sequence has no prompt work: the list is empty, whatever the batch
    flat, info = pack_step([(0, [1]), (1, [2])], None, [5, 9], step_needs(torch.bfloat16, 128))
    assert len(_part(flat, info, "query_blocks128")) == 0
    # any part may add integers of its own; a name of the step context itself is refused
    flat, info = pack_step([(0, [1, 2]), (1, [2])], None, [5, 9], {"twice_past": lambda st: [2 * p for p in st.past]})
    assert _part(flat, info, "twice_past").tolist() == [10, 18]
    with pytest.raises(StepError, match="named 'tokens'"):
        pack_step([(0, [1])], None, [0], {"tokens": lambda st: [0]})


def _check_decode_work(positions, window, teams):
    """Every key tile of every token lies in exactly one segment, the parts of a token are numbered in
    order, every team has at most one segment and the longest come first.  Returns the segments' lengths."""
    from longbow_quarrel_b200.kernels.attention import cut_decode_work, decode_work_size, MAX_SPLITS, MIN_PART_TILES
    work = cut_decode_work(positions, window, teams)
    assert work.dtype == np.int32 and len(work) == decode_work_size(len(positions), teams)
    offsets, n = work[:teams + 1], int(work[teams])
    assert offsets.tolist() == [min(i, n) for i in range(teams + 1)] and len(positions) <= n <= teams
    segments = work[teams + 1:].reshape(-1, 5)[:n]
    pos = np.asarray(positions)
    first = np.where((window > 0) & (pos >= window), pos - window + 1, 0) // 16
    tiles = pos // 16 + 1 - first
    seen = {b: [] for b in range(len(pos))}
    for tok, lo, hi, part, parts in segments.tolist():
        seen[tok].append((lo, hi, part, parts))
    for b, segs in seen.items():
        segs.sort()
        assert segs[0][0] == 0 and segs[-1][1] == tiles[b] and len(segs) <= MAX_SPLITS, (b, segs)
        for i, (lo, hi, part, parts) in enumerate(segs):
            assert lo < hi and part == i and parts == len(segs) and (i == 0 or segs[i - 1][1] == lo), (b, segs)
            assert parts == 1 or hi - lo >= MIN_PART_TILES, (b, segs)
    lengths = (segments[:, 2] - segments[:, 1]).tolist()
    assert lengths == sorted(lengths, reverse=True)
    return lengths


def test_decode_work_covers_every_tile_once():
    rng = np.random.default_rng(5)
    for _ in range(1500):
        B = int(rng.integers(1, 80))
        teams = B + int(rng.integers(0, 150))
        window = int(rng.choice([0, 0, 7, 64, 1000]))
        _check_decode_work(rng.integers(0, int(rng.choice([5, 60, 700, 9000])), size=B), window, teams)
    _check_decode_work([0], 0, 1)
    assert len(_check_decode_work([100000], 0, 148)) == 32       # one token has no more parts than the merge takes
    with pytest.raises(ValueError, match="at least as many teams"):
        _check_decode_work([5, 6, 7], 0, 2)


def test_decode_work_gives_long_sequences_more_parts():
    # unequal sequences (7 ... 250 tiles) and 18 teams: the longest part is far shorter than half the
    # longest sequence, which the same two slices for everyone would leave
    lengths = _check_decode_work([int(2048 * (0.05 + 1.9 * i / 7)) for i in range(8)], 0, 18)
    assert len(lengths) == 18 and lengths[0] <= 76, lengths
    # equal sequences: the same number of slices each, as many as fit
    assert _check_decode_work([2047] * 8, 0, 18) == [64] * 16
    assert _check_decode_work([1199] * 16, 0, 18) == [75] * 16
    # short sequences are not cut at all
    assert _check_decode_work([40] * 8, 0, 18) == [3] * 8
    # one sequence alone is shared by all teams
    lengths = _check_decode_work([4095], 0, 18)
    assert len(lengths) == 18 and lengths[0] - lengths[-1] <= 1, lengths
    # more tokens than teams that run at a time: one part each, the longest first
    assert _check_decode_work([16 * i for i in range(64)], 0, 64) == list(range(64, 0, -1))


def test_attention_asks_for_decode_work_by_its_head_counts():
    import torch
    from longbow_quarrel_b200.kernels.attention import decode_work_name
    needs = step_needs(torch.bfloat16, 128, 32, 8, None, "cpu")
    assert list(needs) == ["query_blocks128", decode_work_name(32, 8, None)]
    assert list(step_needs(torch.float32, 128, 32, 8, None, "cpu")) == []
    assert list(step_needs(torch.bfloat16, 40, 8, 8, None, "cpu")) == []
    # in a step with prompts the decode list is empty
    flat, info = pack_step([(0, [1, 2]), (1, [2])], None, [5, 9], {"w": needs[decode_work_name(32, 8, None)]})
    assert len(_part(flat, info, "w")) == 0
