"""Row plumbing of batched speculative verification around the MoE path: B sequences that each
speculate gamma tokens deep are B * (1 + gamma) rows of ONE forward, so they share one set of expert
reads (crates/peregrine-model/src/model.rs:4028-4116), and a draft is kept only where it equals the
model's own greedy pick, so the emitted stream is exactly what token-by-token greedy decoding
produces (``accept_run``, model.rs:383-406).

The decode stack of this package has no attention, so a row's logits depend on its token alone and
the positions only travel with the rows (they are what a KV cache would be indexed by)."""
from __future__ import annotations

from typing import Callable, List, NamedTuple, Sequence

import numpy as np


class DraftRows(NamedTuple):
    tokens: np.ndarray     # int32 [rows]: per sequence its confirmed token, then its drafts
    owner: np.ndarray      # int32 [rows]: sequence of each row
    positions: np.ndarray  # int64 [rows]: position of each row in its sequence
    first_row: np.ndarray  # int32 [B]: first row of each sequence


def draft_rows(next_of: Sequence[int], drafts: Sequence[Sequence[int]], pos_of: Sequence[int]) -> DraftRows:
    """Row layout of one verification forward: sequence ``s`` owns ``1 + len(drafts[s])`` consecutive
    rows ``[next_of[s], drafts[s]...]`` at positions ``pos_of[s], pos_of[s] + 1, ...``
    (model.rs:4058-4086, including its length check)."""
    b = len(next_of)
    if len(drafts) != b or len(pos_of) != b:
        raise ValueError(f"verify_drafts_batched: {b} tokens but {len(drafts)} drafts / {len(pos_of)} positions")
    tokens, owner, positions, first_row = [], [], [], []
    for s in range(b):
        first_row.append(len(tokens))
        tokens.append(int(next_of[s]))
        owner.append(s)
        positions.append(int(pos_of[s]))
        for j, t in enumerate(drafts[s]):
            tokens.append(int(t))
            owner.append(s)
            positions.append(int(pos_of[s]) + 1 + j)
    return DraftRows(np.asarray(tokens, np.int32), np.asarray(owner, np.int32), np.asarray(positions, np.int64),
                     np.asarray(first_row, np.int32))


def accept_run(row_argmax: Sequence[int], drafts: Sequence[int]) -> tuple[int, int]:
    """The greedy-identity rule on the greedy picks of a sequence's rows (model.rs:394-406 applies
    ``argmax`` to the logits rows; the device stack returns the picks): row ``k`` predicts the token
    after draft ``k - 1``, so row 0 judges the first draft.  Returns how many drafts were accepted and
    the model's pick at the first rejected position (the next round's token, already paid for).  A
    missing row ends the run; with no row at all the next token is 0, as in the reference."""
    k = 0
    while k < len(drafts):
        if k >= len(row_argmax) or int(row_argmax[k]) != int(drafts[k]):
            break
        k += 1
    nxt = int(row_argmax[k]) if k < len(row_argmax) else 0
    return k, nxt


class Verified(NamedTuple):
    tokens: List[int]  # confirmed this round: next_of[s] and the accepted drafts
    next: int          # the model's pick after them
    accepted: int


def verify_drafts(forward_rows: Callable[[np.ndarray], np.ndarray], next_of: Sequence[int],
                  drafts: Sequence[Sequence[int]], pos_of: Sequence[int]) -> List[Verified]:
    """One forward over all sequences' rows, then the accept rule per sequence
    (model.rs:4052-4116).  ``forward_rows(tokens[int32 rows]) -> greedy picks [rows]``."""
    rows = draft_rows(next_of, drafts, pos_of)
    picks = np.asarray(forward_rows(rows.tokens), np.int64)
    if picks.shape[0] != rows.tokens.shape[0]:
        raise ValueError("verify_drafts: the forward returned a different number of rows")
    out = []
    for s in range(len(next_of)):
        base, g = int(rows.first_row[s]), len(drafts[s])
        k, nxt = accept_run(picks[base:base + g + 1], drafts[s])
        out.append(Verified([int(next_of[s])] + [int(t) for t in drafts[s][:k]], nxt, k))
    return out


def stack_forward_rows(stack) -> Callable[[np.ndarray], np.ndarray]:
    """``forward_rows`` over a ``DeviceStack``: the rows are one decode step of the resident stack,
    padded to its batch (the padding rows are computed and dropped)."""

    def run(tokens: np.ndarray) -> np.ndarray:
        tokens = np.asarray(tokens, np.int32)
        if tokens.shape[0] > stack.batch:
            raise ValueError("verify_drafts: more rows than the stack's batch")
        ids0 = np.zeros(stack.batch, np.int32)
        ids0[: tokens.shape[0]] = tokens
        return stack.decode(ids0, 1)[0][: tokens.shape[0]]

    return run
