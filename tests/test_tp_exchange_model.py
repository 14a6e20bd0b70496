"""Model of the tensor-parallel stack's exchange protocol (awq_b200_ffn_stack_decode_tp_bf16), on the CPU.

Every rank, for exchange e = 0, 1, ... (one per layer, counted across launches): stores its words
`tag = e + 1` into slot `e & 1` of every rank's receive area, then waits until its own slot holds tag
e + 1 from every rank, adds them up and goes on.  Stores travel for an arbitrary time.  The model
runs random schedules and checks the two properties the kernel relies on: nobody waits for ever, and
a word is never overwritten before its receiver has consumed it (two slots are enough)."""
import random

import pytest


def run(n_ranks, n_exchanges, seed, n_slots=2):
    rng = random.Random(seed)
    recv = [[[0] * n_ranks for _ in range(n_slots)] for _ in range(n_ranks)]   # recv[dst][slot][src] = tag
    consumed = [[[0] * n_ranks for _ in range(n_slots)] for _ in range(n_ranks)]  # highest tag dst has added up
    in_flight = []                    # (dst, slot, src, tag) stores that have been issued but not yet landed
    pushed = [0] * n_ranks            # exchanges this rank has stored
    reduced = [0] * n_ranks           # exchanges this rank has added up
    steps = 0
    while min(reduced) < n_exchanges:
        steps += 1
        assert steps < 200000, "no progress: the protocol deadlocked"
        moves = []
        for r in range(n_ranks):
            if pushed[r] == reduced[r] and pushed[r] < n_exchanges:
                moves.append(("push", r))          # the down phase of the next layer can end
            elif pushed[r] > reduced[r]:
                e = reduced[r]
                if all(recv[r][e % n_slots][s] == e + 1 for s in range(n_ranks)):
                    moves.append(("reduce", r))
        if in_flight:
            moves.append(("land", None))
        kind, r = rng.choice(moves)
        if kind == "push":
            e = pushed[r]
            for dst in range(n_ranks):
                in_flight.append((dst, e % n_slots, r, e + 1))
            pushed[r] += 1
        elif kind == "land":
            dst, slot, src, tag = in_flight.pop(rng.randrange(len(in_flight)))
            # the word this store replaces must have been consumed by its receiver
            assert recv[dst][slot][src] == consumed[dst][slot][src], (dst, slot, src, tag, recv[dst][slot][src])
            assert tag > recv[dst][slot][src]
            recv[dst][slot][src] = tag
        else:
            e = reduced[r]
            for s in range(n_ranks):
                consumed[r][e % n_slots][s] = e + 1
            reduced[r] += 1
    return steps


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_two_slots_are_enough_and_nobody_waits_for_ever(n_ranks):
    for seed in range(40):
        run(n_ranks, n_exchanges=7 if seed % 2 else 12, seed=seed)


def test_one_slot_would_lose_words():
    """The check has teeth: with a single slot a fast rank overwrites what a slow one has not read."""
    with pytest.raises(AssertionError):
        for seed in range(200):
            run(4, n_exchanges=6, seed=seed, n_slots=1)
