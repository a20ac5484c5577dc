"""The ring protocol of the TMA / tensor-core kernels (csrc/gemm_tc.cu and its relatives), checked as a model on
the CPU: every interleaving of the four actors on a small ring.

    producer     requests slice i into stage i % S once the stage's `empty` barrier shows that the products of
                 slice i - S are done (no wait for the first S slices); the parity it waits on starts at 1 and flips
                 at every wrap of the ring
    copy engine  lands the requested slices in any order; a landed slice completes one phase of its stage's
                 `full` barrier
    issuer       waits for slice i's stage on `full` (parity (i / S) & 1) and issues its products; optionally it asks
                 about the NEXT stage at the same moment and skips the next wait after a yes
    tensor pipe  finishes issued slices in order; a finished slice completes one phase of its stage's `empty` barrier

A barrier is modelled as its number of completed phases, and a wait on parity P succeeds iff the barrier's current
phase has the other parity (`mbarrier.try_wait.parity` / `test_wait.parity`).  Checked: no slice's products are issued
before its data has landed, and nothing ever waits for ever.  (The kernels' arithmetic for stage and parity is
restated here, not imported: a change there has to be made here too, and then checked again.)"""

from collections import deque

import pytest


def _ok(completed: int, parity: int) -> bool:
    return (completed & 1) != parity


def _explore(S: int, T: int, ask_ahead: bool):
    """Breadth-first over all reachable states; returns (states visited, first problem found or None)."""
    start = (0, (), (0,) * S, (0,) * S, 0, 0, (), frozenset())
    seen, queue = {start}, deque([start])
    while queue:
        p_it, flying, full, empty, i_it, ready, issued, landed = st = queue.popleft()
        nxt = []
        if p_it < T:  # producer
            s, parity = p_it % S, ((p_it // S) & 1) ^ 1
            if p_it < S or _ok(empty[s], parity):
                nxt.append((p_it + 1, flying + (p_it,), full, empty, i_it, ready, issued, landed))
        for k, sl in enumerate(flying):  # copy engine
            f = list(full)
            f[sl % S] += 1
            nxt.append((p_it, flying[:k] + flying[k + 1:], tuple(f), empty, i_it, ready, issued, landed | {sl}))
        if i_it < T:  # issuer
            s, parity = i_it % S, (i_it // S) & 1
            if ready or _ok(full[s], parity):
                if i_it not in landed:
                    return len(seen), f"slice {i_it} issued before its data landed"
                yes = 0
                if ask_ahead:
                    s1, parity1 = (i_it + 1) % S, ((i_it + 1) // S) & 1
                    yes = 1 if _ok(full[s1], parity1) else 0
                nxt.append((p_it, flying, full, empty, i_it + 1, yes, issued + (i_it,), landed))
        if issued:  # tensor pipe
            e = list(empty)
            e[issued[0] % S] += 1
            nxt.append((p_it, flying, full, tuple(e), i_it, ready, issued[1:], landed))
        if not nxt and (p_it < T or i_it < T):
            return len(seen), f"nothing can move at producer {p_it}, issuer {i_it}"
        for n in nxt:
            if n not in seen:
                seen.add(n)
                queue.append(n)
    return len(seen), None


@pytest.mark.parametrize("S, T", [(2, 7), (3, 10), (4, 11), (5, 12)])
@pytest.mark.parametrize("ask_ahead", [False, True])
def test_ring_of_stages_never_issues_early_and_never_stalls(S, T, ask_ahead):
    states, problem = _explore(S, T, ask_ahead)
    assert problem is None, problem
    assert states > T * S


def test_the_model_sees_a_wrong_parity():
    """The checker itself: an issuer that waits on the producer's parity convention is caught."""
    S, T = 3, 8
    # the same exploration with the issuer's parity flipped
    start = (0, (), (0,) * S, 0, frozenset())
    seen, queue, problem = {start}, deque([start]), None
    while queue and problem is None:
        p_it, flying, full, i_it, landed = queue.popleft()
        nxt = []
        if p_it < min(T, S):
            nxt.append((p_it + 1, flying + (p_it,), full, i_it, landed))
        for k, sl in enumerate(flying):
            f = list(full)
            f[sl % S] += 1
            nxt.append((p_it, flying[:k] + flying[k + 1:], tuple(f), i_it, landed | {sl}))
        if i_it < S and _ok(full[i_it % S], ((i_it // S) & 1) ^ 1):  # wrong: succeeds on a fresh barrier
            if i_it not in landed:
                problem = f"slice {i_it} issued before its data landed"
            nxt.append((p_it, flying, full, i_it + 1, landed))
        for n in nxt:
            if n not in seen:
                seen.add(n)
                queue.append(n)
    assert problem is not None
