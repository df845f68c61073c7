"""CPU model of the exchange protocol of ``csrc/peer_reduce.cu``: two slots per source rank,
monotonically growing per-rank flags, a device-side step counter per rank.

Every rank is a little state machine (write contribution -> publish -> wait for all flags ->
read all contributions -> advance); a seeded scheduler interleaves the ranks' micro-operations in
arbitrary order, in the pull form (contribution in the owner's buffer, read remotely), the push
form (contribution written into every rank's buffer, read locally) and a mix of both.  The
property checked is the one the kernels rely on: whenever a rank reads slot (step & 1, src) it
holds src's contribution of exactly that step -- i.e. two slots are enough and no rank can
overwrite data a slower peer still has to read."""
import random

import pytest


class Rank:
    def __init__(self, r, world):
        self.r, self.world = r, world
        self.step = 0
        self.flags = [0] * world                          # flags[src] = steps src has published, as seen here
        self.slots = [[None] * world for _ in range(2)]   # slots[parity][src] = (src, step) tag
        self.pc = 0                                       # 0 write, 1 publish, 2 wait, 3.. read src, then advance
        self.read_src = 0


def run(world, steps, seed, mode):
    rng = random.Random(seed)
    ranks = [Rank(r, world) for r in range(world)]
    push_of_step = [rng.random() < 0.5 if mode == "mixed" else mode == "push" for _ in range(steps)]
    reads = 0
    while any(k.step < steps for k in ranks):
        k = rng.choice([k for k in ranks if k.step < steps])
        s, par = k.step, k.step & 1
        push = push_of_step[s]
        if k.pc == 0:                                     # write the contribution of step s
            targets = ranks if push else [k]
            for t in targets:
                t.slots[par][k.r] = (k.r, s)
            k.pc = 1
        elif k.pc == 1:                                   # publish s + 1 into every rank's flag array
            for t in ranks:
                assert t.flags[k.r] <= s + 1
                t.flags[k.r] = s + 1
            k.pc = 2
        elif k.pc == 2:                                   # wait (a poll that may fail and be retried later)
            if all(f >= s + 1 for f in k.flags):
                k.pc, k.read_src = 3, 0
        elif k.pc == 3:                                   # read one source's slot
            src = k.read_src
            holder = k if push else ranks[src]
            assert holder.slots[par][src] == (src, s), (k.r, s, src, holder.slots[par][src], mode)
            reads += 1
            k.read_src += 1
            if k.read_src == world:
                k.pc = 4
        else:                                             # advance
            k.step, k.pc = s + 1, 0
    return reads


@pytest.mark.parametrize("mode", ["pull", "push", "mixed"])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_two_slots_suffice_under_any_interleaving(world, mode):
    for seed in range(40):
        assert run(world, steps=12, seed=seed, mode=mode) == world * world * 12


def test_a_single_slot_would_not_suffice():
    """The model is sharp enough to see the bug the second slot prevents."""
    class OneSlot(Rank):
        pass

    def run_one_slot(seed):
        rng = random.Random(seed)
        world, steps = 2, 6
        ranks = [Rank(r, world) for r in range(world)]
        while any(k.step < steps for k in ranks):
            k = rng.choice([k for k in ranks if k.step < steps])
            s = k.step
            if k.pc == 0:
                k.slots[0][k.r] = (k.r, s)                # always parity 0
                k.pc = 1
            elif k.pc == 1:
                for t in ranks:
                    t.flags[k.r] = s + 1
                k.pc = 2
            elif k.pc == 2:
                if all(f >= s + 1 for f in k.flags):
                    k.pc, k.read_src = 3, 0
            elif k.pc == 3:
                src = k.read_src
                if ranks[src].slots[0][src] != (src, s):
                    return True                           # stale or overwritten data observed
                k.read_src += 1
                if k.read_src == world:
                    k.pc = 4
            else:
                k.step, k.pc = s + 1, 0
        return False

    assert any(run_one_slot(seed) for seed in range(200))
