"""How a step's tokens are packed into its one index buffer (no GPU): real sequences, padding
sequences of one token or of none, rows that belong to no sequence."""

import numpy as np
import pytest

from models_b200.cache import KvCache, KvRequest
from models_b200.engine.batch import StepLayout, pack_step, plan_layout


def _cache():
    full = KvRequest(2, 16, None)
    return KvCache([full, KvRequest(2, 16, 100)], [None, None], 1024, 8)  # two groups: all keys, a window


def _parts(layout, buf):
    off = [int(o) for o in layout.offsets]
    names = ["tokens", "positions", "cu_q", "kv_lens", "slots", "want"]
    parts = {n: buf[off[i]:off[i + 1]] for i, n in enumerate(names)}
    for g in range(layout.groups):
        parts[f"table{g}"] = buf[off[6 + 2 * g]:off[7 + 2 * g]].reshape(layout.sequences, layout.blocks)
        parts[f"mapping{g}"] = buf[off[7 + 2 * g]:off[8 + 2 * g]]
    return parts


def test_prompts_of_unequal_lengths_with_empty_padding():
    cache = _cache()
    a, b = cache.open_slot(), cache.open_slot()
    cache.append([(a, 70)])
    cache.commit([(a, 70)])  # a already holds 70 positions: its 5 new tokens continue there
    entries = [(a, [11, 12, 13, 14, 15], [4]), (b, [21, 22, 23], [0, 2])]
    cache.append([(a, 5), (b, 3)])
    layout = StepLayout(4, 16, 4, 4, len(cache.groups))
    buf = np.full(layout.total, 99, dtype=np.int32)
    q_lens, max_kv = pack_step(cache, entries, layout, buf, state_pad_row=cache.max_slots, empty_padding=True)
    p = _parts(layout, buf)
    assert q_lens == [5, 3, 0, 0] and max_kv == 75
    assert list(p["tokens"][:8]) == [11, 12, 13, 14, 15, 21, 22, 23] and not p["tokens"][8:].any()
    assert list(p["positions"][:8]) == [70, 71, 72, 73, 74, 0, 1, 2]
    assert list(p["cu_q"]) == [0, 5, 8, 8, 8]  # the padding sequences are empty; rows 8..15 belong to nobody
    assert list(p["kv_lens"]) == [75, 3, 1, 1]
    assert list(p["slots"]) == [a, b, cache.max_slots, cache.max_slots]
    assert list(p["want"]) == [4, 5, 7, 0]  # wanted rows in the order of the entries; the spare one points at row 0
    for g, group in enumerate(cache.groups):
        mapping = p[f"mapping{g}"]
        table_a, table_b = group.tables[a], group.tables[b]
        assert list(mapping[:5]) == [table_a[(70 + i) // 64] * 64 + (70 + i) % 64 for i in range(5)]
        assert list(mapping[5:8]) == [table_b[0] * 64 + i for i in range(3)]
        assert (mapping[8:] == -1).all()  # nothing is stored for rows of no sequence
        assert not p[f"table{g}"][2:].any()  # padding sequences read the spare page 0
    cache.commit([(a, 5), (b, 3)])
    cache.check()


def test_decode_padding_keeps_one_token_per_sequence():
    cache = _cache()
    a = cache.open_slot()
    cache.append([(a, 1)])
    layout = StepLayout(4, 4, 4, 2, len(cache.groups))
    buf = np.zeros(layout.total, dtype=np.int32)
    q_lens, _ = pack_step(cache, [(a, [7], [0])], layout, buf, state_pad_row=cache.max_slots)
    p = _parts(layout, buf)
    assert q_lens == [1, 1, 1, 1] and list(p["cu_q"]) == [0, 1, 2, 3, 4]
    assert list(p["kv_lens"]) == [1, 1, 1, 1]
    for g in range(layout.groups):
        assert p[f"mapping{g}"][0] >= 64 and (p[f"mapping{g}"][1:] == -1).all()


def test_a_step_that_does_not_fit_its_layout_is_refused():
    cache = _cache()
    a = cache.open_slot()
    cache.append([(a, 9)])
    layout = StepLayout(2, 8, 2, 2, len(cache.groups))
    with pytest.raises(ValueError, match="do not fit"):
        pack_step(cache, [(a, list(range(9)), [8])], layout, np.zeros(layout.total, dtype=np.int32), empty_padding=True)
    assert plan_layout(cache, [(a, list(range(9)), [8])]).tokens == 9


def test_context_classes_of_decode_steps():
    from models_b200.kernels.ops import LONG_KEYS, decode_span

    assert decode_span(1) == 0 and decode_span(LONG_KEYS) == 0
    assert decode_span(LONG_KEYS + 1) == 2 * LONG_KEYS
    assert decode_span(5000) == 8192 and decode_span(8192) == 8192 and decode_span(8193) == 16384
