"""Row layout and accept rule of batched speculative verification (host mirror of
crates/peregrine-model/src/model.rs:383-406 and 4028-4116), no GPU."""
import numpy as np
import pytest

from peregrine_b200.speculative import accept_run, draft_rows, verify_drafts


def test_rows_are_laid_out_sequence_by_sequence():
    rows = draft_rows([7, 9, 4], [[1, 2], [], [5, 6, 8]], [10, 3, 0])
    assert rows.tokens.tolist() == [7, 1, 2, 9, 4, 5, 6, 8]
    assert rows.owner.tolist() == [0, 0, 0, 1, 2, 2, 2, 2]
    assert rows.positions.tolist() == [10, 11, 12, 3, 0, 1, 2, 3]
    assert rows.first_row.tolist() == [0, 3, 4]
    with pytest.raises(ValueError):
        draft_rows([1, 2], [[3]], [0, 0])


def test_accept_rule_is_greedy_identity():
    # row k predicts the token after draft k - 1: row 0 judges the first draft
    assert accept_run([5, 6, 7], [5, 6]) == (2, 7)    # all accepted: the pick after the last draft
    assert accept_run([5, 9, 7], [5, 6]) == (1, 9)    # second draft wrong: the model's own pick replaces it
    assert accept_run([4, 9, 7], [5, 6]) == (0, 4)    # first draft wrong
    assert accept_run([3], []) == (0, 3)              # nothing drafted: plain greedy
    assert accept_run([5], [5, 6]) == (1, 0)          # a missing row ends the run (next falls back to 0)
    assert accept_run([], []) == (0, 0)


def test_verify_uses_one_forward_for_all_sequences():
    calls = []
    succ = {1: 2, 2: 3, 3: 4, 4: 5, 5: 6, 6: 7, 7: 8, 8: 9, 9: 1}   # the "model": next token by table

    def forward_rows(tokens):
        calls.append(np.asarray(tokens).tolist())
        return np.asarray([succ[int(t)] for t in tokens])

    out = verify_drafts(forward_rows, [1, 5], [[2, 3, 9], [6, 6]], [0, 0])
    assert len(calls) == 1 and calls[0] == [1, 2, 3, 9, 5, 6, 6]
    assert out[0].tokens == [1, 2, 3] and out[0].accepted == 2 and out[0].next == 4
    assert out[1].tokens == [5, 6] and out[1].accepted == 1 and out[1].next == 7
