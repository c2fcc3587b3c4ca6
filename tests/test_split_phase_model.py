"""The split-phase exchange's host bookkeeping (P2PCombiner.begin_split / end_split: sequence numbers, ring
slots, parity of the partials) driven against a small model of what the serving warp does with the values
it is handed (appy_split_service in csrc/templates/t_flat.cuh): launch k+1 folds launch k's partials and
stores the rank's total into slot (k mod 8) of every rank's mailbox; launch k+2 collects launch k from its
own mailbox, waiting for words whose tag is not k yet.  Ranks advance in random order, as far apart as the
waits allow.  Checked for up to 8 ranks: no rank ever waits for a word that cannot come (no deadlock), no
word is overwritten before its reader has taken it, and every cell ends with the world's total.  CPU only:
the model replaces the kernel, the bookkeeping is the real one."""
import random

import pytest

from appy_b200.backends.cuda_sm100 import multi_gpu as mg


class Rank:
    def __init__(self, rank, world):
        self.rank, self.world = rank, world
        c = mg.P2PCombiner.__new__(mg.P2PCombiner)           # bookkeeping only: no device context
        c.rank, c.world = rank, world
        c._seq, c.pending, c.to_fold, c.to_collect, c.split_count = 0, [], None, None, 0
        self.comb = c
        self.mailbox = {}            # (slot, source rank) -> (sequence tag, value)
        self.unread = set()          # (slot, source rank) written and not yet collected
        self.partials = {}           # address -> value this rank's launch left there
        self.cell = 0                # the shared scalar (an integer, so that sums are exact)
        self.launched = 0
        self.collected = 0


def service(ranks, me, pend):
    """What warp 0 of the last CTA does at the start of a kernel; False if it would have to wait."""
    c, f = pend.coll, pend.fold
    if c.seq:                        # the wait comes last in the kernel, but nothing before it depends on it
        for src in range(me.world):
            tag_val = me.mailbox.get((c.slot, src))
            if tag_val is None or tag_val[0] != c.seq:
                return False
    if f.seq:
        total = me.partials[f.partials]
        for r in ranks:
            key = (f.slot, me.rank)
            assert key not in r.unread, f"rank {me.rank} overwrites slot {f.slot} of rank {r.rank} unread"
            r.mailbox[key] = (f.seq, total)
            r.unread.add(key)
    if c.seq:
        me.cell += sum(me.mailbox[(c.slot, src)][1] for src in range(me.world))
        for src in range(me.world):
            me.unread.discard((c.slot, src))
        me.collected += 1
    return True


def try_launch(ranks, me, value, flush=False):
    """One split-phase launch of rank `me` (or one flush step): bookkeeping, then the model of the kernel."""
    comb = me.comb
    pend = mg.Pending2()
    if flush:
        comb._fill(pend.fold, comb.to_fold)
        comb._fill(pend.coll, comb.to_collect)
        if not service(ranks, me, pend):
            return False
        comb.to_collect, comb.to_fold = comb.to_fold, None
        return True
    saved = (comb.to_fold, comb.to_collect, comb.split_count, comb._seq)
    mine = comb.begin_split(pend, 1 << 20, 64)
    if not service(ranks, me, pend):
        comb.to_fold, comb.to_collect, comb.split_count, comb._seq = saved      # the kernel is still waiting
        return False
    seq = comb.next_seq()
    me.partials[mine] = value                         # the CTAs' partials, here already folded into one number
    comb.end_split(seq, 64, mine, [(0x1000, 0, 3)])   # one int64 cell, operator +
    me.launched += 1
    return True


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_ring_slots_and_sequence_numbers_hold_for_any_interleaving(world):
    rng = random.Random(100 + world)
    for trial in range(20):
        ranks = [Rank(r, world) for r in range(world)]
        launches = rng.choice([1, 2, 3, 9, 17, 40])
        values = [[rng.randrange(1000) for _ in range(launches)] for _ in range(world)]
        flushed = [0] * world
        stuck = 0
        while any(r.launched < launches or flushed[r.rank] < 2 for r in ranks):
            r = rng.choice(ranks)
            if r.launched < launches:
                ok = try_launch(ranks, r, values[r.rank][r.launched])
            elif flushed[r.rank] < 2:
                ok = try_launch(ranks, r, 0, flush=True)
                flushed[r.rank] += ok
            else:
                continue
            stuck = 0 if ok else stuck + 1
            assert stuck < 1000 * world, "every rank is waiting: deadlock"
        want = sum(sum(v) for v in values)
        for r in ranks:
            assert r.cell == want and r.collected == launches
            assert r.comb.to_fold is None and r.comb.to_collect is None
