"""Host-side model of the cross-GPU barrier protocol of ``csrc/comm.cuh`` (``barrier_all_ranks``).

The device code cannot be run under a race detector, so its state machine is checked here: every thread of
the protocol becomes an agent that executes the same three memory operations per barrier, and a scheduler
explores their interleavings (all of them for small worlds, random ones for eight ranks). The memory
model is the one the kernel relies on: single-word stores and loads of a flag are atomic and the stores of
one agent become visible in program order (release / acquire on the flag).

Per barrier ``k``, thread ``p`` of rank ``r`` (one CTA per rank, ``world`` signalling threads):

  A  store 1 to rank ``p``'s flag ``[set(k)][r]``          (one-way signal, no read-back)
  B  poll own flag ``[set(k)][p]`` until it reads 1
  C  store 0 to own flag ``[set(k)][p]``
  -- CTA barrier: no thread of rank ``r`` starts barrier ``k + 1`` before all finished ``k``

Checked: no deadlock; a signal never lands on a flag that still holds an unconsumed signal; a clear never
erases the signal of a later barrier; a rank leaves barrier ``k`` only after every peer arrived at it; all
flags are zero at the end when the number of barriers is even (the pads are reusable by the next kernel or
by a CUDA-graph replay). With a single flag set instead of two alternating ones the same exploration must
find the lost-signal interleaving - the reason the kernel alternates sets.
"""
import random
from collections import deque

import pytest


class Violation(Exception):
    pass


def _initial(world, barriers):
    # agent (r, p): [barrier index, phase]; phase 0 = before A, 1 = before B, 2 = before C, 3 = waiting at the CTA barrier
    agents = tuple((0, 0) for _ in range(world * world))
    flags = tuple(None for _ in range(world * 2 * world))       # [rank][set][peer] -> barrier tag or None
    return agents, flags


def _fidx(world, rank, s, peer):
    return (rank * 2 + s) * world + peer


def _set_map(barriers, sets):
    """Flag set used by barrier ``k``. ``sets``: 1 (a single set), 2 (alternating, one kernel), or a list of
    barrier counts per kernel launch - every launch restarts its own count at set 0, like the device code."""
    if isinstance(sets, (list, tuple)):
        m = [j % 2 for n in sets for j in range(n)]
        assert len(m) == barriers
        return tuple(m)
    return tuple((k % 2) if sets == 2 else 0 for k in range(barriers))


def _steps(state, world, barriers, sets):
    """Yield every successor state of ``state`` (one agent performing its next operation)."""
    setmap = _set_map(barriers, sets)
    agents, flags = state
    for a, (k, ph) in enumerate(agents):
        if k >= barriers:
            continue
        r, p = divmod(a, world)
        s = setmap[k]
        if ph == 0:                                            # A: signal peer p
            i = _fidx(world, p, s, r)
            if flags[i] is not None:
                raise Violation(f"rank {r} signals barrier {k} into rank {p}'s flag that still holds barrier {flags[i]}")
            nf = flags[:i] + (k,) + flags[i + 1:]
            yield agents[:a] + ((k, 1),) + agents[a + 1:], nf
        elif ph == 1:                                          # B: poll own flag
            i = _fidx(world, r, s, p)
            if flags[i] is None:
                continue                                       # spins
            if flags[i] != k:
                raise Violation(f"rank {r} barrier {k} consumed the signal of barrier {flags[i]} from rank {p}")
            # the peer's arrival at barrier k is implied by the tag: it stored it in its phase A of barrier k
            yield agents[:a] + ((k, 2),) + agents[a + 1:], flags
        elif ph == 2:                                          # C: clear own flag
            i = _fidx(world, r, s, p)
            if flags[i] != k:
                raise Violation(f"rank {r} clears barrier {k} but the flag holds {flags[i]}")
            nf = flags[:i] + (None,) + flags[i + 1:]
            yield agents[:a] + ((k, 3),) + agents[a + 1:], nf
        else:                                                  # CTA barrier of rank r
            mine = agents[r * world:(r + 1) * world]
            if all(x == (k, 3) for x in mine):
                na = agents[:r * world] + tuple((k + 1, 0) for _ in range(world)) + agents[(r + 1) * world:]
                yield na, flags


def _done(state, barriers):
    return all(k >= barriers for k, _ in state[0])


def explore_all(world, barriers, sets=2):
    """Breadth-first over every reachable state. Returns the number of states; raises Violation."""
    start = _initial(world, barriers)
    seen, queue = {start}, deque([start])
    finals = 0
    while queue:
        st = queue.popleft()
        succ = list(_steps(st, world, barriers, sets))
        if not succ:
            if not _done(st, barriers):
                raise Violation(f"deadlock: {st}")
            finals += 1
            assert all(f is None for f in st[1]), "flags must be zero after the last barrier"
        for n in succ:
            if n not in seen:
                seen.add(n)
                queue.append(n)
    assert finals >= 1
    return len(seen)


def random_walks(world, barriers, sets, walks, seed):
    rng = random.Random(seed)
    for _ in range(walks):
        st = _initial(world, barriers)
        # a biased scheduler: one rank runs far ahead of the others most of the time
        fast = rng.randrange(world)
        while True:
            succ = list(_steps(st, world, barriers, sets))
            if not succ:
                if not _done(st, barriers):
                    raise Violation("deadlock")
                assert all(f is None for f in st[1])
                break
            ahead = [n for n in succ if any(n[0][fast * world + p] != st[0][fast * world + p] for p in range(world))]
            st = rng.choice(ahead) if ahead and rng.random() < 0.8 else rng.choice(succ)


def test_two_alternating_sets_are_safe_in_every_interleaving():
    assert explore_all(world=2, barriers=4) > 1000
    assert explore_all(world=2, barriers=2) > 100


def test_eight_ranks_random_interleavings():
    random_walks(world=8, barriers=4, sets=2, walks=30, seed=1)
    random_walks(world=4, barriers=6, sets=2, walks=60, seed=2)
    random_walks(world=3, barriers=2, sets=2, walks=200, seed=3)


def test_kernels_must_run_an_even_number_of_barriers():
    """Every launch starts on set 0. Two launches of two barriers each are safe back to back; launches with an
    odd count put two consecutive barriers on the same set, which is the single-set hazard again."""
    assert explore_all(world=2, barriers=4, sets=[2, 2]) > 1000
    with pytest.raises(Violation, match="still holds"):
        explore_all(world=2, barriers=2, sets=[1, 1])
    with pytest.raises(Violation):
        explore_all(world=2, barriers=4, sets=[3, 1])


def test_a_single_flag_set_loses_a_signal():
    """Negative control: without the alternation a fast rank's next signal lands on a flag its peer has not
    consumed yet; the exploration must find that interleaving."""
    with pytest.raises(Violation, match="still holds"):
        explore_all(world=2, barriers=2, sets=1)
    with pytest.raises(Violation):
        random_walks(world=4, barriers=4, sets=1, walks=200, seed=4)
