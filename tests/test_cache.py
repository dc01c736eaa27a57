"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice."""

import random

import pytest

from models_b200.cache import CacheFull, FreeList, KvCache, KvRequest


def test_free_list_never_hands_an_id_out_twice():
    pool = FreeList(5, first=1, what="page")
    taken = [pool.take() for _ in range(5)]
    assert sorted(taken) == [1, 2, 3, 4, 5]
    with pytest.raises(CacheFull):
        pool.take()
    pool.give_back(3)
    with pytest.raises(ValueError, match="twice"):
        pool.give_back(3)
    with pytest.raises(ValueError):
        pool.give_back(99)
    assert pool.take() == 3  # a released id is the next one handed out
    pool.check()


def _cache(max_tokens=640, window=None, max_slots=None):
    full = KvRequest(2, 16, None)
    requests = [full, full, KvRequest(2, 16, window) if window else full]
    return KvCache(requests, [None, None, None], max_tokens, max_slots)


def test_groups_by_need_and_storage_shapes():
    cache = _cache(window=100)
    assert len(cache.groups) == 2
    assert cache.groups[0].runs == [0, 1] and cache.groups[1].runs == [2]
    shapes = []
    cache.allocate_storage(lambda shape: shapes.append(shape) or shape)
    # keys and values of each group: 10 pages and the spare page 0
    assert shapes == [(2, 11, 2, 64, 16), (2, 11, 2, 64, 16), (1, 11, 2, 64, 16), (1, 11, 2, 64, 16)]
    shared = KvCache([KvRequest(2, 16), KvRequest(2, 16)], [None, 0], 128)
    assert shared.run_location[1] == shared.run_location[0] and shared.groups[0].runs == [0]
    with pytest.raises(ValueError, match="kv heads"):
        KvCache([KvRequest(2, 16), KvRequest(4, 16)], [None, 0], 128)


def test_append_commit_release_and_refusals():
    cache = _cache(max_tokens=256)  # 4 pages
    a, b = cache.open_slot(), cache.open_slot()
    cache.append([(a, 65), (b, 1)])
    cache.commit([(a, 65), (b, 1)])
    assert cache.length(a) == 65 and len(cache.groups[0].tables[a]) == 2
    with pytest.raises(CacheFull):
        cache.append([(a, 64), (b, 64)])  # needs 1 + 1 more pages... a: 129 -> 3 pages, b: 65 -> 2: 5 > 4
    cache.check()
    assert cache.length(a) == 65 and len(cache.groups[0].tables[a]) == 2  # a refused step changes nothing
    with pytest.raises(ValueError, match="twice"):
        cache.append([(a, 1), (a, 1)])
    with pytest.raises(KeyError):
        cache.append([(7, 1)])
    cache.release(a)
    with pytest.raises(KeyError):
        cache.release(a)
    c = cache.open_slot()
    assert c == a and cache.length(c) == 0  # the slot is used again, empty
    cache.append([(c, 128)])
    cache.commit([(c, 128)])
    cache.check()


def test_window_group_gives_pages_back_and_rewind_knows():
    cache = _cache(max_tokens=64 * 20, window=70)
    s = cache.open_slot()
    cache.append([(s, 300)])
    cache.commit([(s, 300)])
    full, windowed = cache.groups
    assert [p >= 0 for p in full.tables[s]] == [True] * 5
    # next query is at 300 and sees keys >= 231: blocks 0..2 (positions < 192) are dead
    assert [p >= 0 for p in windowed.tables[s]] == [False, False, False, True, True]
    cache.check()
    with pytest.raises(ValueError, match="window"):
        cache.rewind(s, 200)
    cache.rewind(s, 290)
    assert cache.length(s) == 290
    cache.release(s)
    cache.check()
    assert windowed.pages.held == 0 and full.pages.held == 0


def test_random_schedule_of_batches_loses_nothing():
    rng = random.Random(0)
    cache = _cache(max_tokens=64 * 40, window=90, max_slots=6)
    live = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and cache.slots.free:
            live[cache.open_slot()] = 0
        elif action < 0.8 and live:
            chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
            appends = [(s, rng.choice([1, 1, 1, 5, 64, 130])) for s in chosen]
            try:
                cache.append(appends)
            except CacheFull:
                before = dict(cache.lengths)
                assert before == {s: live[s] for s in live}
                continue
            cache.commit(appends)
            for s, n in appends:
                live[s] += n
        elif live:
            s = rng.choice(sorted(live))
            cache.release(s)
            del live[s]
        cache.check()
        assert {s: cache.length(s) for s in live} == live
    for s in list(live):
        cache.release(s)
    cache.check()
    assert cache.slots.held == 0 and all(g.pages.held == 0 for g in cache.groups)


def test_table_stamps_change_with_the_tables_and_never_repeat():
    cache = _cache(max_tokens=64 * 12, window=70)
    seen = set()
    a = cache.open_slot()
    stamp = cache.table_stamps[a]
    seen.add(stamp)
    cache.append([(a, 10)])  # a first page
    assert cache.table_stamps[a] != stamp
    stamp = cache.table_stamps[a]
    seen.add(stamp)
    cache.commit([(a, 10)])
    cache.append([(a, 1)])  # no new page: the tables are what they were
    cache.commit([(a, 1)])
    assert cache.table_stamps[a] == stamp
    cache.append([(a, 60)])  # a second page
    cache.commit([(a, 60)])
    assert cache.table_stamps[a] not in seen
    seen.add(cache.table_stamps[a])
    cache.append([(a, 64)])
    stamp = cache.table_stamps[a]
    cache.commit([(a, 64)])  # 135 positions, window 70: the window group gives its first page back
    assert cache.groups[1].tables[a][0] == -1 and cache.table_stamps[a] != stamp
    seen.add(cache.table_stamps[a])
    cache.rewind(a, 134)
    assert cache.table_stamps[a] not in seen
    seen.add(cache.table_stamps[a])
    cache.release(a)
    assert a not in cache.table_stamps
    b = cache.open_slot()
    assert b == a and cache.table_stamps[b] not in seen  # the same slot id, another tenant: another stamp


def test_decode_rows_follow_the_tables_of_a_slot_that_is_used_again():
    """Two requests of two pages end; two others get their slots, at the same rows, with as many pages --
    the same pages in the other order.  The rows of a captured step must then hold the new tables."""
    import numpy as np

    from models_b200.engine.batch import StepLayout, pack_step
    from models_b200.engine.decode_graph import DecodeRows

    full = KvRequest(2, 16, None)
    cache = KvCache([full], [None], 64 * 8, max_slots=2)
    layout = StepLayout(2, 2, 2, 4, 1)
    buffer = np.zeros(layout.total, dtype=np.int32)
    pack_step(cache, [], layout, buffer, cache.max_slots)
    rows = DecodeRows(layout, buffer)

    def tenant_pair(prompt):
        slots = [cache.open_slot(), cache.open_slot()]
        appends = [(s, prompt) for s in slots]
        cache.append(appends)
        cache.commit(appends)
        for _ in range(3):
            step = [(s, 1) for s in slots]
            cache.append(step)
            rows.update(cache, slots, [1, 2])
            for b, s in enumerate(slots):
                table = cache.groups[0].tables[s]
                assert rows.tables_h[0][b, :len(table)].tolist() == table, (b, table)
                length = cache.lengths[s]
                assert rows.mappings_h[0][b] == table[length // 64] * 64 + length % 64
                assert rows.kv_lens_h[b] == length + 1 and rows.positions_h[b] == length
            cache.commit(step)
        return slots, [list(cache.groups[0].tables[s]) for s in slots]

    first_slots, first_tables = tenant_pair(70)
    for s in reversed(first_slots):
        cache.release(s)
    second_slots, second_tables = tenant_pair(70)
    assert second_slots == first_slots and [len(t) for t in second_tables] == [len(t) for t in first_tables]
    assert second_tables != first_tables  # the case that a (slot, page count) key cannot tell apart
    rows.update(cache, second_slots[:1], [3])  # one row falls out: it becomes padding
    assert rows.tables_h[0][1].tolist() == [0, 0, 0, 0] and rows.mappings_h[0][1] == -1 and rows.slots_h[1] == cache.max_slots


def test_key_and_value_sizes_apart_and_a_window_groups_own_budget():
    """A group's keys and values have sizes of their own; a window group is made with the pages its
    window (and the longest step) can hold, a group that keeps everything with the whole budget."""
    narrow_values = KvRequest(2, 32, None, value_dim=8)
    windowed = KvRequest(1, 16, 100)
    cache = KvCache([narrow_values, windowed, narrow_values], [None, None, 0], 64 * 200, max_slots=4, max_step_tokens=30)
    shapes = []
    cache.allocate_storage(lambda shape: shapes.append(shape) or shape)
    # window 100 and steps of up to 30 tokens: ceil(129 / 64) + 1 = 4 pages per sequence, 16 in all
    assert [g.num_pages for g in cache.groups] == [200, 16]
    assert shapes == [(1, 201, 2, 64, 32), (1, 201, 2, 64, 8), (1, 17, 1, 64, 16), (1, 17, 1, 64, 16)]
    assert cache.pools(2)[1] is cache.pools(0)[1]  # run 2 reads run 0's storage
    slots = [cache.open_slot() for _ in range(4)]
    for s in slots:  # four sequences grow to 1,000 positions in steps of 30: the window group never runs out
        for _ in range(34):
            cache.append([(s, 30)])
            cache.commit([(s, 30)])
        assert sum(p >= 0 for p in cache.groups[1].tables[s]) <= 4
    cache.check()
    with pytest.raises(CacheFull, match="window of 100"):
        cache.append([(s, 64 * 5) for s in slots])  # a step longer than promised does not fit the window group
    cache.check()
    with pytest.raises(ValueError, match="values 8"):
        KvCache([narrow_values, KvRequest(2, 32, None)], [None, 0], 128)
    unbounded = KvCache([windowed], [None], 64 * 200, max_slots=4)  # no promise about steps: the whole budget
    assert unbounded.groups[0].num_pages == 200
