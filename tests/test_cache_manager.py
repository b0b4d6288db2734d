"""The cache manager: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; pages are used again."""
import numpy as np
import pytest

from alofa_b200.cache import CacheManager, GroupSpec
from alofa_b200.errors import AlofaError


def holders(cm, live, group):
    seen = []
    for slot in live:
        seen += [int(p) for p in cm.block_table(slot, group) if p >= 0]
    return seen


def check_books(cm, live):
    assert cm.defects() == 0
    for g, spec in enumerate(cm.groups):
        held = holders(cm, live, g)
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + cm.free_pages(g) == spec.num_pages, "a page was lost"


def test_first_allocations_are_in_order_and_reuse_is_lifo():
    cm = CacheManager([GroupSpec(16, 8)], max_requests=4, max_tokens=128)
    a = cm.admit(1)
    cm.reserve(a, 33)
    assert list(cm.block_table(a, 0)) == [0, 1, 2]
    b = cm.admit(2)
    cm.reserve(b, 16)
    assert list(cm.block_table(b, 0)) == [3]
    cm.release(a)
    c = cm.admit(3)
    assert c == a  # the lowest free state slot
    cm.reserve(c, 40)
    assert list(cm.block_table(c, 0)) == [2, 1, 0]  # last freed, first used again: tables need not ascend
    check_books(cm, [b, c])


def test_reserve_is_all_or_nothing_and_refusals_are_named():
    cm = CacheManager([GroupSpec(16, 4), GroupSpec(16, 2, window=16)], max_requests=2, max_tokens=256)
    a = cm.admit(1)
    assert cm.try_reserve(a, 32)
    assert not cm.try_reserve(a, 64)  # the second group has 2 pages only
    assert cm.free_pages() == [2, 0]
    with pytest.raises(AlofaError, match="too few free pages"):
        cm.reserve(a, 64)
    cm.admit(2)
    with pytest.raises(AlofaError) as err:
        cm.admit(3)
    assert err.value.code == "capacity"
    with pytest.raises(AlofaError) as err:
        cm.admit(2)
    assert err.value.code == "state"
    cm.release(a)
    with pytest.raises(AlofaError) as err:
        cm.release(a)  # freed twice
    assert err.value.code == "state"
    assert cm.defects() == 0


def test_window_gives_pages_back_as_it_passes():
    cm = CacheManager([GroupSpec(16, 64), GroupSpec(16, 64, window=24)], max_requests=2, max_tokens=1024)
    s = cm.admit(1)
    length = 0
    rng = np.random.default_rng(0)
    while length < 900:
        n = int(rng.integers(1, 40))
        cm.reserve(s, length + n)
        # during the step every key a query of this portion sees must have a page
        table = cm.block_table(s, 1)
        oldest = max(0, length - 24 + 1)
        assert all(table[b] >= 0 for b in range(oldest // 16, len(table)))
        length += n
        cm.advance(s, length)
        table = cm.block_table(s, 1)
        oldest_next = max(0, length - 24 + 1)
        assert all(p < 0 for p in table[: oldest_next // 16]) and all(p >= 0 for p in table[oldest_next // 16 :])
        assert (table >= 0).sum() <= 24 // 16 + 2
        check_books(cm, [s])
    assert cm.used_pages(0) == -(-length // 16)
    cm.release(s)
    assert cm.free_pages() == [64, 64]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = np.random.default_rng(seed)
    groups = [GroupSpec(16, 24), GroupSpec(16, 12, window=int(rng.choice([8, 24, 50])))]
    cm = CacheManager(groups, max_requests=5, max_tokens=256)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            slot = cm.admit(next_id)
            assert slot not in live
            live[slot] = 0
            next_id += 1
        elif op < 0.8 and live:
            slot = int(rng.choice(list(live)))
            grow = int(rng.integers(1, 48))
            if live[slot] + grow <= 256 and cm.try_reserve(slot, live[slot] + grow):
                live[slot] += grow
                cm.advance(slot, live[slot])
        elif live:
            slot = int(rng.choice(list(live)))
            cm.release(slot)
            del live[slot]
        check_books(cm, list(live))
        for slot, n in live.items():
            assert cm.computed_len(slot) == n
    for slot in list(live):
        cm.release(slot)
    assert cm.free_pages() == [24, 12] and cm.live_requests() == 0
    c = cm.counters(0)
    assert c["allocs"] == c["frees"] and c["allocs"] > 24  # pages were used again


def test_shared_prefix_is_counted_once_per_holder():
    cm = CacheManager([GroupSpec(16, 8)], max_requests=3, max_tokens=128)
    a = cm.admit(1)
    cm.reserve(a, 40)
    cm.advance(a, 40)
    b = cm.admit(2)
    cm.share_prefix(a, b, 32)
    assert list(cm.block_table(b, 0)) == list(cm.block_table(a, 0))[:2]
    cm.reserve(b, 50)
    assert cm.defects() == 0 and cm.used_pages(0) == 3 + 2
    cm.release(a)
    assert cm.used_pages(0) == 4  # the shared pages stay with b
    cm.release(b)
    assert cm.free_pages(0) == 8 and cm.defects() == 0


def test_digest_tells_states_apart():
    def play(order):
        cm = CacheManager([GroupSpec(16, 8)], max_requests=3, max_tokens=128)
        slots = [cm.admit(i) for i in range(2)]
        for i in order:
            cm.reserve(slots[i], cm.reserved_len(slots[i]) + 16)
        return cm.digest()

    assert play([0, 1, 0]) == play([0, 1, 0])
    assert play([0, 1, 0]) != play([1, 0, 0])


def plan(cm, entries, words=4096):
    """plan_step over [(slot, tokens)], every row wanted; returns the metadata words."""
    slots = np.array([s for s, _ in entries], dtype=np.int32)
    counts = np.array([n for _, n in entries], dtype=np.int32)
    want_counts = np.ones(len(entries), dtype=np.int32)
    wants = np.zeros(len(entries), dtype=np.int32)
    meta = np.full(words, -7, dtype=np.int32)
    n_tok, n_seq = int(counts.sum()), len(entries)
    at, offsets = 0, []
    for size in [n_tok, n_tok, n_seq + 1, n_seq, n_seq, n_seq] + [n_tok, n_seq * cm.max_blocks] * len(cm.groups):
        offsets.append(at)
        at += size
    cm.plan_step(slots, counts, want_counts, wants, meta.ctypes.data, np.array(offsets, dtype=np.int32), cm.max_blocks)
    return meta


def test_a_step_that_does_not_fit_changes_nothing():
    """Two entries, the second of which does not fit: the first keeps no
    reservation, the metadata is untouched, and a smaller step goes through."""
    cm = CacheManager([GroupSpec(16, 4)], max_requests=2, max_tokens=128)
    a, b = cm.admit(1), cm.admit(2)
    with pytest.raises(AlofaError, match="too few free pages"):
        meta = plan(cm, [(a, 40), (b, 40)])  # 3 + 3 pages of 4
    assert cm.free_pages() == [4] and cm.reserved_len(a) == 0 and cm.reserved_len(b) == 0
    check_books(cm, [a, b])
    meta = plan(cm, [(a, 20), (b, 30)])  # 2 + 2 pages
    assert list(meta[:50]) == list(range(20)) + list(range(30))  # positions
    cm.commit_step(np.array([a, b], dtype=np.int32), np.array([20, 30], dtype=np.int32))
    check_books(cm, [a, b])
    # a step that was planned and never committed is taken back by the next plan
    plan(cm, [(a, 10)])
    assert cm.reserved_len(a) == 30 and cm.free_pages() == [0]
    meta = plan(cm, [(a, 4), (b, 2)])
    assert cm.reserved_len(a) == 24 and cm.reserved_len(b) == 32
    check_books(cm, [a, b])
    # a slot named twice, or a wanted place outside the entry's tokens, is refused before anything is reserved
    for bad in ([(a, 1), (a, 1)],):
        with pytest.raises(AlofaError):
            plan(cm, bad)
    assert cm.reserved_len(a) == 24
    check_books(cm, [a, b])


def test_a_manager_without_groups_hands_out_state_slots_only():
    cm = CacheManager([], max_requests=2, max_tokens=64)
    a, b = cm.admit(1), cm.admit(2)
    assert (a, b) == (0, 1) and cm.free_pages() == []
    with pytest.raises(AlofaError):
        cm.admit(3)
    meta = plan(cm, [(a, 5), (b, 7)])
    assert list(meta[:12]) == list(range(5)) + list(range(7))
    cm.commit_step(np.array([a, b], dtype=np.int32), np.array([5, 7], dtype=np.int32))
    assert cm.computed_len(a) == 5 and cm.computed_len(b) == 7 and cm.defects() == 0
    cm.release(a)
    assert cm.admit(4) == a and cm.computed_len(a) == 0
