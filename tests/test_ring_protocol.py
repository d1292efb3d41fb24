"""CPU: the page rings of the streaming decode kernels, stepped through under random interleavings.

A model of the synchronisation in richengine_b200/csrc/decode_attention.cu and nothing else: one producer, twelve
consumer warps (4 KV heads x 3 page residues), mbarriers with parity waits, the per-head barrier at a lane change,
the barrier of all consumers before a CTA's last segment is folded in the ring. The scheduler picks a random
runnable actor at every step, consumer warps are split into two halves that read and release independently (every
lane of a warp arrives on its own), copies land in random order, and heads drift apart freely between lane changes.

What is asserted, for lane segments whose lengths are not multiples of three (the mapping of residues to units shifts):
  * a consumer that passes its wait on a stage reads exactly the unit it meant to read (no wait passes two phases
    early or late: a parity cannot tell completions two apart, the protocol must never let it matter);
  * a stage is never refilled while a reader of its previous fill has not released it, and every release counted
    towards a refill is a release of THAT fill;
  * no barrier gets more arrivals than its phase takes;
  * when the consumers meet to fold the last segment, nothing is in flight and nothing is left to issue;
  * no deadlock.
The int4 / one-byte kernels: one completion barrier and one release barrier (128 arrivals) per stage, 6 or 3 stages.
The bf16 kernel: (page, head) units, one completion barrier per consumer warp, release barriers of 32 arrivals that
only the producer waits on, 6 stages.
"""
import random

import pytest

HEADS, RESIDUES, HALVES = 4, 3, 2


class Barrier:
    """An mbarrier: `count` arrivals complete a phase; wait(parity) passes when the phase of that parity is done."""

    def __init__(self, count):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self, n=1):
        self.arrived += n
        assert self.arrived <= self.count, "more arrivals than the phase takes"
        if self.arrived == self.count:
            self.arrived = 0
            self.completed += 1

    def passes(self, parity):
        return (self.completed & 1) != parity


def page_ring(segments, stages, seed):
    """int4 / int8 / fp8 kernels: unit = page, read by the warp (head, residue) of each head."""
    rnd = random.Random(seed)
    total = sum(segments)
    full = [Barrier(1) for _ in range(stages)]
    empty = [Barrier(HEADS * HALVES) for _ in range(stages)]  # one arrival per half-warp here, 32 lanes each there
    content = [None] * stages      # unit whose bytes the stage holds (None while a copy is landing)
    readers = [0] * stages         # half-warps between their wait and their release
    released_of = [None] * stages  # the unit the arrivals of the current empty phase belong to
    issued, in_flight = 0, []
    # consumer programs: per (head, residue, half) the list of (segment index, unit)
    programs = {}
    before = 0
    bounds = []
    for index, length in enumerate(segments):
        bounds.append((before, before + length))
        before += length
    for head in range(HEADS):
        for residue in range(RESIDUES):
            for half in range(HALVES):
                program = []
                for index, (begin, end) in enumerate(bounds):
                    program.append(("lane", index))
                    program += [("page", unit) for unit in range(begin + residue, end, RESIDUES)]
                    program.append(("flush", index))
                programs[(head, residue, half)] = program
    position = {key: 0 for key in programs}
    reading = {key: None for key in programs}
    at_lane = {head: {} for head in range(HEADS)}   # head -> segment index -> halves that arrived
    at_fold = set()
    steps = 0
    while any(position[k] < len(programs[k]) for k in programs) or issued < total or in_flight:
        steps += 1
        assert steps < 400 * (total + 8) * len(programs), "deadlock"
        kind = rnd.choice("pllcccccccc")
        if kind == "p" and issued < total:
            slot, round_ = issued % stages, issued // stages
            if empty[slot].passes((round_ & 1) ^ 1):
                assert empty[slot].completed == round_, ("producer passed a release wait of another round", issued)
                assert readers[slot] == 0, ("refill under a reader", issued)
                content[slot] = None
                in_flight.append(issued)
                issued += 1
        elif kind == "l" and in_flight:
            unit = in_flight.pop(rnd.randrange(len(in_flight)))
            content[unit % stages] = unit
            full[unit % stages].arrive()
        elif kind == "c":
            key = rnd.choice(list(programs))
            head, residue, half = key
            if reading[key] is not None:  # done reading: fence, then this half's lanes arrive on the release barrier
                unit = reading[key]
                slot = unit % stages
                assert content[slot] == unit, ("stage changed under a reader", key, unit)
                assert released_of[slot] in (None, unit), ("release counted towards another fill", key, unit)
                released_of[slot] = unit
                readers[slot] -= 1
                empty[slot].arrive()
                if empty[slot].arrived == 0:
                    released_of[slot] = None
                reading[key] = None
                position[key] += 1
                continue
            if position[key] >= len(programs[key]):
                continue
            what, value = programs[key][position[key]]
            if what == "lane":  # the head's three warps meet before the query fragments are replaced
                waiting = at_lane[head].setdefault(value, set())
                waiting.add((residue, half))
                if len(waiting) == RESIDUES * HALVES:
                    for r, h in waiting:
                        position[(head, r, h)] += 1
                    at_lane[head][value] = set()
            elif what == "page":
                slot, round_ = value % stages, value // stages
                if full[slot].passes(round_ & 1):
                    assert full[slot].completed == round_ + 1, ("consumer passed a wait of another fill", key, value)
                    assert content[slot] == value, ("consumer reads another unit's bytes", key, value, content[slot])
                    readers[slot] += 1
                    reading[key] = value
            else:  # flush; the last segment's flush meets every consumer first and then writes into the ring
                if value + 1 < len(segments):
                    position[key] += 1
                    continue
                at_fold.add(key)
                if len(at_fold) == len(programs):
                    assert issued == total and not in_flight, "fold while pages are in flight"
                    assert all(r == 0 for r in readers), "fold under a reader"
                    for k in programs:
                        position[k] += 1
    return True


def unit_ring(segments, seed, stages=6):
    """bf16 kernel: unit = (page ordinal, head), one consumer warp per unit, the ordinal's residue picks the warp."""
    rnd = random.Random(seed)
    empty = [Barrier(1) for _ in range(stages)]
    warp_full = [Barrier(1) for _ in range(HEADS * RESIDUES)]
    content = [None] * stages
    units = [(ordinal, head) for ordinal in range(sum(segments)) for head in range(HEADS)]
    programs = {w: [] for w in range(HEADS * RESIDUES)}
    before = 0
    for length in segments:
        for w in programs:
            residue = w >> 2
            first = (residue + RESIDUES - before % RESIDUES) % RESIDUES
            programs[w] += [before + page for page in range(first, length, RESIDUES)]
        before += length
    position = {w: 0 for w in programs}
    issued, in_flight, steps = 0, [], 0
    while issued < len(units) or in_flight or any(position[w] < len(programs[w]) for w in programs):
        steps += 1
        assert steps < 10 ** 6, "deadlock"
        kind = rnd.choice("plcccc")
        if kind == "p" and issued < len(units):
            slot, round_ = issued % stages, issued // stages
            if empty[slot].passes((round_ & 1) ^ 1):
                assert empty[slot].completed == round_, ("producer passed a release wait of another round", issued)
                content[slot] = None
                in_flight.append(issued)
                issued += 1
        elif kind == "l" and in_flight:
            unit = in_flight.pop(rnd.randrange(len(in_flight)))
            ordinal, head = units[unit]
            content[unit % stages] = unit
            warp_full[head + HEADS * (ordinal % RESIDUES)].arrive()
        elif kind == "c":
            w = rnd.randrange(HEADS * RESIDUES)
            if position[w] < len(programs[w]):
                ordinal = programs[w][position[w]]
                if warp_full[w].passes((ordinal // RESIDUES) & 1):
                    unit = ordinal * HEADS + (w & 3)
                    assert warp_full[w].completed == ordinal // RESIDUES + 1, ("consumer passed a wait of another unit", w, ordinal)
                    assert content[unit % stages] == unit, ("consumer reads another unit's bytes", w, ordinal)
                    empty[unit % stages].arrive()
                    position[w] += 1
    return True


def mixes(seed):
    rnd = random.Random(seed)
    return [rnd.choice([1, 1, 2, 3, 4, 5, 7, 20, 23]) for _ in range(rnd.randint(1, 6))]


@pytest.mark.parametrize("stages", [6, 3])
def test_page_ring_under_random_interleavings(stages):
    for seed in range(120):
        assert page_ring(mixes(seed), stages, seed)
    # the mixes that exposed the missing proxy fence on the GPU (in pages): a lane change after a long lane
    for segments in ([47, 47], [22, 2, 47, 2], [94, 94, 94]):
        for seed in range(10):
            assert page_ring(segments, stages, 1000 + seed)


def test_unit_ring_under_random_interleavings():
    for seed in range(200):
        assert unit_ring(mixes(seed), seed)


def test_the_model_catches_a_release_that_runs_ahead():
    """The model is not vacuous: let ONE half-warp release a stage before it has read it (what a warp-elected arrive
    ahead of a slower lane amounts to) and the refill lands under a reader."""
    def broken(segments, stages, seed):
        rnd = random.Random(seed)
        total = sum(segments)
        full = [Barrier(1) for _ in range(stages)]
        empty = [Barrier(2) for _ in range(stages)]
        content, readers = [None] * stages, [0] * stages
        issued, in_flight = 0, []
        position = {0: 0, 1: 0}   # two halves of one warp reading every unit; half 0 releases for both, early
        reading = {0: None, 1: None}
        steps = 0
        while issued < total or in_flight or any(position[h] < total for h in position) or any(v is not None for v in reading.values()):
            steps += 1
            if steps > 200000:
                return "deadlock"
            kind = rnd.choice("plcc")
            if kind == "p" and issued < total:
                slot, round_ = issued % stages, issued // stages
                if empty[slot].passes((round_ & 1) ^ 1):
                    if readers[slot]:
                        return "refill under a reader"
                    content[slot] = None
                    in_flight.append(issued)
                    issued += 1
            elif kind == "l" and in_flight:
                unit = in_flight.pop(rnd.randrange(len(in_flight)))
                content[unit % stages] = unit
                full[unit % stages].arrive()
            elif kind == "c":
                half = rnd.randrange(2)
                if reading[half] is not None:
                    readers[reading[half] % stages] -= 1
                    reading[half] = None
                    position[half] += 1
                elif position[half] < total:
                    unit = position[half]
                    slot = unit % stages
                    if full[slot].passes((unit // stages) & 1) and content[slot] == unit:
                        readers[slot] += 1
                        reading[half] = unit
                        if half == 0:
                            empty[slot].arrive(2)  # the elected lane arrives for the whole warp as soon as IT has passed the wait
        return "clean"
    outcomes = {broken([40], 3, seed) for seed in range(60)}
    assert "refill under a reader" in outcomes
