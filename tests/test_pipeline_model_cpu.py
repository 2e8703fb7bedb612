"""A small executable model of the shared-memory ring of the forward / data-gradient convolution kernel
(helium_b200/csrc/conv_sm100.cuh: one producer thread, two MMA-issuing threads, `full` / `empty` mbarriers per
slot), run under many random interleavings.

Why it exists.  An mbarrier parity wait does not name a phase; it only says "the latest phase of this parity has
completed".  A waiter that observes every phase of a barrier in order is safe.  One that skips a phase is not: if it
comes back for phase L + 1 while phase L is still open, the completed phase L - 1 (same parity) lets it through.
The first two-issuer version of the kernel let each issuing thread wait only for the groups it multiplies; with
loads of different groups completing in any order that happened about once in 10^4 launches on the GPU, and the ring
stopped (the bounded waits then gave up).  The model below reproduces the failure for that protocol and shows none
for the one the kernel uses now: both threads wait for every group, only the MMAs are divided, and a slot goes back
to the producer when BOTH threads have let go of it.

Modelled: barrier phases and parity waits, transaction-style completion of loads in any order, commits that arrive
some time after the MMAs were issued (in order per thread), the per-tile assignment of groups to threads.  Not
modelled: the accumulator barriers between issuers and epilogue (every waiter there observes every phase)."""
import random

import pytest


class Barrier:
    def __init__(self, count=1):
        self.phase = 0          # index of the phase that is currently open
        self.count = count      # arrivals that complete a phase
        self.pending = count

    def passed(self, parity):   # mbarrier.try_wait.parity
        return (self.phase & 1) != parity

    def complete(self):         # one arrival (or the last byte of a transaction)
        self.pending -= 1
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count


SKIP, OBSERVE, OBSERVE_AND_RELEASE = "skip", "observe", "observe and release"


def run(groups_per_tile, n_tiles, slots, protocol, seed, max_events=200000):
    """Returns None when all groups were multiplied on the right data, else a description of what went wrong.

    protocol SKIP: a thread waits only for the groups it multiplies.  OBSERVE: it waits for every group.
    OBSERVE_AND_RELEASE: it waits for every group and the slot is handed back to the producer by BOTH threads (the
    one that multiplied it when its MMAs have retired, the other one right after its wait), so neither thread can
    fall a whole lap behind the barrier it has to observe next."""
    rng = random.Random(seed)
    wait_for_every_group = protocol != SKIP
    full = [Barrier() for _ in range(slots)]
    empty = [Barrier(2 if protocol == OBSERVE_AND_RELEASE else 1) for _ in range(slots)]
    smem = [None] * slots                    # which group's tiles a slot holds
    total = groups_per_tile * n_tiles
    owner = lambda g: (g % groups_per_tile) & 1       # the group's index inside its tile decides (g_idx & 1)
    prod = 0                                 # next group the producer fills
    prod_armed = False                       # waited for `empty`, loads not yet issued
    loads = []                               # groups whose loads are in flight
    pos = [0, 0]                             # next group each issuing thread looks at
    commits = [[], []]                       # per thread: groups whose MMAs are issued but not yet retired (in order)
    done = 0
    for _ in range(max_events):
        if done == total:
            return None
        actions = []
        if prod < total:
            slot, lap = prod % slots, prod // slots
            if prod_armed or empty[slot].passed((lap & 1) ^ 1):
                actions.append(("issue_load",))
        for g in loads:
            actions.append(("load_lands", g))
        for i in (0, 1):
            if pos[i] < total:
                g = pos[i]
                slot, lap = g % slots, g // slots
                if owner(g) != i and not wait_for_every_group:
                    actions.append(("skip", i))
                elif full[slot].passed(lap & 1):
                    actions.append(("consume" if owner(g) == i else "observe", i))
            if commits[i]:
                actions.append(("retire", i))
        if not actions:
            return f"deadlock: producer at group {prod}, issuers at {pos}, {done}/{total} groups done"
        a = rng.choice(actions)
        if a[0] == "issue_load":
            loads.append(prod)
            prod += 1
            prod_armed = False
        elif a[0] == "load_lands":
            g = a[1]
            loads.remove(g)
            smem[g % slots] = g
            full[g % slots].complete()
        elif a[0] in ("skip", "observe"):
            if a[0] == "observe" and protocol == OBSERVE_AND_RELEASE:
                empty[pos[a[1]] % slots].complete()
            pos[a[1]] += 1
        elif a[0] == "consume":
            i = a[1]
            g = pos[i]
            if smem[g % slots] != g:
                return f"issuer {i} multiplied slot {g % slots} holding group {smem[g % slots]} instead of {g}"
            commits[i].append(g)
            pos[i] += 1
        else:
            i = a[1]
            g = commits[i].pop(0)
            if smem[g % slots] != g:
                return f"slot {g % slots} was overwritten while issuer {i} still read group {g}"
            empty[g % slots].complete()
            done += 1
    return "no progress within the event limit"


# (groups per tile, ring slots): 3 x 3 layers with 64 / 128 / 256 channels at 128 columns (3 slots of two k-blocks)
# and at 64 columns (4 slots); tiles of one group exercise the thread that has nothing to multiply
SHAPES = [(5, 3), (9, 3), (18, 3), (5, 4), (9, 4), (2, 3), (1, 3), (3, 4)]


@pytest.mark.parametrize("groups_per_tile,slots", SHAPES)
def test_the_kernels_protocol_never_reads_stale_tiles_and_never_stops(groups_per_tile, slots):
    for seed in range(300):
        assert run(groups_per_tile, 6, slots, OBSERVE_AND_RELEASE, seed) is None, seed


def test_skipping_the_other_threads_phases_goes_wrong():
    """The protocol the kernel had first: some interleaving lets a thread through a phase early."""
    failures = [run(9, 6, 3, SKIP, seed) for seed in range(300)]
    failures = [f for f in failures if f is not None]
    assert failures, "the model no longer shows the hazard it was written for"
    assert any("instead of" in f or "deadlock" in f or "overwritten" in f for f in failures)


def test_observing_without_releasing_can_still_fall_a_lap_behind():
    """Waiting for every group is not enough under an arbitrary scheduler: a thread that does not hold the slot
    back can be overtaken by a whole lap of the barrier it still has to observe (on the GPU that needs one thread to
    stall for well over a thousand cycles while the other runs on; it was never seen, and it is excluded by
    construction once both threads release the slot)."""
    failures = [run(5, 6, 3, OBSERVE, seed) for seed in range(300)]
    assert any(f is not None for f in failures)


def run_shared_stages(n_issuers, stages, n_stages_total, seed, max_events=200000):
    """The filter-gradient kernel's ring (conv_sm100.cuh, conv_wgrad_kernel): every stage holds one tap tile per
    issuing thread, every thread waits for every stage, multiplies its taps and commits; `empty` takes one arrival
    per thread.  Same modelling as above."""
    rng = random.Random(seed)
    full = [Barrier() for _ in range(stages)]
    empty = [Barrier(n_issuers) for _ in range(stages)]
    smem = [None] * stages
    prod, loads, done = 0, [], 0
    pos = [0] * n_issuers
    commits = [[] for _ in range(n_issuers)]
    for _ in range(max_events):
        if done == n_stages_total * n_issuers:
            return None
        actions = []
        if prod < n_stages_total and empty[prod % stages].passed(((prod // stages) & 1) ^ 1):
            actions.append(("issue_load",))
        actions += [("load_lands", k) for k in loads]
        for i in range(n_issuers):
            if pos[i] < n_stages_total and full[pos[i] % stages].passed((pos[i] // stages) & 1):
                actions.append(("consume", i))
            if commits[i]:
                actions.append(("retire", i))
        if not actions:
            return f"deadlock: producer at {prod}, issuers at {pos}"
        a = rng.choice(actions)
        if a[0] == "issue_load":
            loads.append(prod)
            prod += 1
        elif a[0] == "load_lands":
            loads.remove(a[1])
            smem[a[1] % stages] = a[1]
            full[a[1] % stages].complete()
        elif a[0] == "consume":
            i = a[1]
            if smem[pos[i] % stages] != pos[i]:
                return f"issuer {i} multiplied stage {pos[i] % stages} holding {smem[pos[i] % stages]} instead of {pos[i]}"
            commits[i].append(pos[i])
            pos[i] += 1
        else:
            i = a[1]
            k = commits[i].pop(0)
            if smem[k % stages] != k:
                return f"stage {k % stages} was overwritten while issuer {i} still read {k}"
            empty[k % stages].complete()
            done += 1
    return "no progress within the event limit"


@pytest.mark.parametrize("n_issuers,stages", [(3, 3), (3, 5), (3, 6), (1, 6)])
def test_the_filter_gradient_ring_is_safe(n_issuers, stages):
    for seed in range(200):
        assert run_shared_stages(n_issuers, stages, 40, seed) is None, seed
