"""The tokens of one step as one ragged batch, with everything the kernels index by.

All sequences' new tokens are packed one after another (T = sum of the entries' token counts).
Per token: its id, its absolute position in its sequence, and per cache group the flat cache
position it is stored at.  Per sequence: its first packed row (cu_q), its cache length after the
step (kv_lens), its slot, and per cache group its page table.  Padding rows that a fixed-size
decode batch may carry have slot_mapping -1 (nothing is stored), a cache length of 1 and a page
table of zeros (the never-handed-out page 0), and no logits row.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class GroupBatch:
    block_table: torch.Tensor  # int32 [sequences, blocks]
    slot_mapping: torch.Tensor  # int32 [tokens]


@dataclass
class StepBatch:
    tokens: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T]
    cu_q: torch.Tensor  # int32 [B + 1]
    kv_lens: torch.Tensor  # int32 [B]
    slots: torch.Tensor  # int32 [B]; state-area rows (padding rows point at the spare last row)
    want_rows: Optional[torch.Tensor]  # int32 [R] packed rows whose logits are wanted
    groups: List[GroupBatch]
    num_sequences: int
    num_tokens: int
    num_wanted: int
    max_q_len: int
    max_kv_len: int
    q_lens: Tuple[int, ...]  # host copies, for parts that loop on the host
    host_slots: Tuple[int, ...]


@dataclass(frozen=True)
class StepLayout:
    """Where the parts of a step lie in its one int32 buffer."""

    sequences: int
    tokens: int
    wanted: int
    blocks: int
    groups: int

    @property
    def sizes(self):
        B, T = self.sequences, self.tokens
        return [T, T, B + 1, B, B, self.wanted] + [B * self.blocks, T] * self.groups

    @property
    def offsets(self):
        return np.concatenate([[0], np.cumsum(self.sizes)]).astype(np.int64)

    @property
    def total(self) -> int:
        return int(sum(self.sizes))


def plan_layout(cache, entries, pad_sequences: int = 0, blocks: int = 0) -> StepLayout:
    B = max(len(entries), pad_sequences)
    T = sum(len(tokens) for _, tokens, _ in entries) + (B - len(entries))
    need_blocks = 1
    for slot, tokens, _ in entries:
        need_blocks = max(need_blocks, -(-(cache.lengths[slot] + len(tokens)) // cache.page_size))
    if blocks and blocks < need_blocks:
        raise ValueError(f"page table of {blocks} blocks is too narrow, the step needs {need_blocks}")
    R = sum(len(want) for _, _, want in entries)
    return StepLayout(B, T, R, blocks or need_blocks, len(cache.groups))


def pack_step(cache, entries, layout: StepLayout, buf: np.ndarray, state_pad_row: int = 0, empty_padding: bool = False):
    """Fills `buf` (int32, layout.total long) for the step; returns (q_lens, max_kv_len).  Sequences
    beyond the entries are padding: of one token each, or with `empty_padding` of none -- the rows
    that are left over then belong to no sequence (token 0, position 0, nothing stored, no logits)."""
    B, T, width, n_groups = layout.sequences, layout.tokens, layout.blocks, layout.groups
    offsets = layout.offsets
    need = sum(len(tokens) for _, tokens, _ in entries) + (0 if empty_padding else max(0, B - len(entries)))
    wanted_rows = sum(len(want) for _, _, want in entries)
    if len(entries) > B or need > T or wanted_rows > layout.wanted:
        raise ValueError(f"the step's {len(entries)} sequences, {need} tokens and {wanted_rows} wanted rows do not fit the "
                         f"layout's {B}, {T} and {layout.wanted}")
    buf[:] = 0
    tokens_a, positions_a, cu_q_a, kv_lens_a, slots_a, want_a = (buf[offsets[i]:offsets[i + 1]] for i in range(6))
    tables = [buf[offsets[6 + 2 * g]:offsets[7 + 2 * g]].reshape(B, width) for g in range(n_groups)]
    mappings = [buf[offsets[7 + 2 * g]:offsets[8 + 2 * g]] for g in range(n_groups)]
    page = cache.page_size
    q_lens = []
    row = 0
    wanted = 0
    max_kv = 1
    for b, (slot, tokens, want) in enumerate(entries):
        n = len(tokens)
        q_lens.append(n)
        start = cache.lengths[slot]
        tokens_a[row:row + n] = tokens
        pos = np.arange(start, start + n, dtype=np.int32)
        positions_a[row:row + n] = pos
        cu_q_a[b] = row
        kv_lens_a[b] = start + n
        slots_a[b] = slot
        max_kv = max(max_kv, start + n)
        for w in want:
            want_a[wanted] = row + w
            wanted += 1
        for g, group in enumerate(cache.groups):
            table = np.asarray(group.tables[slot], dtype=np.int32)
            tables[g][b, :len(table)] = np.maximum(table, 0)
            mappings[g][row:row + n] = table[pos // page] * page + pos % page
        row += n
    for b in range(len(entries), B):  # padding sequences
        q_lens.append(0 if empty_padding else 1)
        cu_q_a[b] = row
        kv_lens_a[b] = 1
        slots_a[b] = state_pad_row
        if not empty_padding:
            for g in range(n_groups):
                mappings[g][row] = -1
            row += 1
    cu_q_a[B] = row
    for g in range(n_groups):  # rows of no sequence
        mappings[g][row:] = -1
    return q_lens, max_kv


def batch_from_buffer(dev: torch.Tensor, layout: StepLayout, q_lens, max_kv: int, host_slots) -> StepBatch:
    offsets = layout.offsets
    part = [dev[int(offsets[i]):int(offsets[i + 1])] for i in range(len(layout.sizes))]
    B, width = layout.sequences, layout.blocks
    groups = [GroupBatch(part[6 + 2 * g].view(B, width), part[7 + 2 * g]) for g in range(layout.groups)]
    return StepBatch(
        tokens=part[0], positions=part[1], cu_q=part[2], kv_lens=part[3], slots=part[4],
        want_rows=part[5] if layout.wanted else None, groups=groups, num_sequences=B, num_tokens=layout.tokens,
        num_wanted=layout.wanted, max_q_len=max(q_lens), max_kv_len=max_kv, q_lens=tuple(q_lens),
        host_slots=tuple(host_slots))


def build_step_batch(cache, entries: Sequence[Tuple[int, Sequence[int], Sequence[int]]], device,
                     pad_sequences: int = 0, blocks: int = 0, state_pad_row: int = 0) -> StepBatch:
    """entries: (slot, new tokens, wanted places among them).  The cache must already have room
    (KvCache.append); lengths are still the ones before the step.  `pad_sequences` > len(entries)
    appends one-token padding sequences; `blocks` fixes the page-table width (0: as needed)."""
    layout = plan_layout(cache, entries, pad_sequences, blocks)
    buf = np.zeros(layout.total, dtype=np.int32)
    q_lens, max_kv = pack_step(cache, entries, layout, buf, state_pad_row)
    host = torch.from_numpy(buf)
    if torch.device(device).type == "cuda":
        dev = host.pin_memory().to(device, non_blocking=True)
    else:
        dev = host.to(device)
    return batch_from_buffer(dev, layout, q_lens, max_kv, [slot for slot, _, _ in entries])
