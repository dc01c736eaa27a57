"""The whole decode step as one kernel (csrc/decode_step.cu), for models whose parts it knows.

A model qualifies when every scheduled layer is the pre-norm block of RMSNorm, rotary grouped-query
attention over a cache of its own and a gated feed-forward, all bfloat16 without biases, and the
embedding and the head are the package's own.  The parts stay what they are; this module only reads
their tensors and constants into the kernel's list of phases.  Anything else -- another kind of
part, a float32 weight, a step of more than eight rows or of several tokens per sequence, an
observer -- runs part by part as before.

It is switched on by `enabled` (MODELS_B200_FUSED_DECODE=1 in the environment sets it for every
model).  It is off by default: measured on the 1B sizes it streams the large matrices faster than
the kernel-per-matrix path (gate/up 8.7 us against 16.7, the output matrix 67 against 89) but pays
about 7 us per phase for the barrier, the staging of activations and the first tile, which the
kernel-per-matrix path hides behind programmatic dependent launches: 0.92 ms against 0.83 ms per step at
batch 8.  `time_phases` shows where a step's time goes.
"""

from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from ..kernels import ops
from ..parts.attention import AttentionMixer
from ..parts.block import PreNormBlock
from ..parts.embedding import TokenEmbedding
from ..parts.feed_forward import GatedFeedForward
from ..parts.head import LinearHead
from ..parts.norm import RmsNorm

PH_EMBED, PH_QKV, PH_ATTN, PH_OUT, PH_GATE_UP, PH_DOWN, PH_HEAD = range(7)
MAX_GROUPS = 4
MAX_ROWS = 8
MAX_SPLITS = 16


class Phase(ctypes.Structure):
    """struct Phase of csrc/decode_step.cu."""

    _fields_ = [
        ("kind", ctypes.c_int), ("barrier_before", ctypes.c_int), ("w", ctypes.c_void_p), ("ldw", ctypes.c_int),
        ("rows", ctypes.c_int), ("tiles", ctypes.c_int), ("k_len", ctypes.c_int), ("k_pad", ctypes.c_int),
        ("k_begin", ctypes.c_int), ("pair_offset", ctypes.c_int), ("activation", ctypes.c_int), ("eps", ctypes.c_float),
        ("gain", ctypes.c_void_p), ("group", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int),
        ("window", ctypes.c_int), ("scale", ctypes.c_float), ("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p),
        ("cos_table", ctypes.c_void_p), ("sin_table", ctypes.c_void_p),
    ]


class Step(ctypes.Structure):
    """struct Step of csrc/decode_step.cu."""

    _fields_ = [
        ("phases", ctypes.c_void_p), ("num_phases", ctypes.c_int), ("batch", ctypes.c_int), ("hidden", ctypes.c_int),
        ("tokens", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("kv_lens", ctypes.c_void_p),
        ("embedding", ctypes.c_void_p), ("embedding_scale", ctypes.c_float), ("max_blocks", ctypes.c_int),
        ("block_tables", ctypes.c_void_p * MAX_GROUPS), ("slot_mappings", ctypes.c_void_p * MAX_GROUPS),
        ("splits", ctypes.c_int * MAX_GROUPS), ("x", ctypes.c_void_p), ("q", ctypes.c_void_p), ("ld_q", ctypes.c_int),
        ("h", ctypes.c_void_p), ("ld_h", ctypes.c_int), ("attn_o", ctypes.c_void_p), ("attn_ml", ctypes.c_void_p),
        ("attn_tickets", ctypes.c_void_p), ("a", ctypes.c_void_p), ("logits", ctypes.c_void_p), ("ld_logits", ctypes.c_int), ("barrier", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("timeline", ctypes.c_void_p),
    ]


def _bf16_matrix(t: Optional[torch.Tensor]) -> bool:
    return (t is not None and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.shape[1] % 8 == 0 and t.data_ptr() % 16 == 0)


def _norm_fits(norm, width: int) -> bool:
    return type(norm) is RmsNorm and norm.weight.dtype == torch.float32 and norm.weight.numel() == width and norm.weight.data_ptr() % 16 == 0


class FusedDecode:
    """The phases of one model, built at the first step (the cache pools are known then)."""

    def __init__(self, model):
        self.model = model
        self.lib = None
        self.phases = None  # the records, in host memory
        self.num_phases = 0
        self.head_dim = 0
        self.why_not: Optional[str] = self._check(model)
        self.enabled = bool(os.environ.get("MODELS_B200_FUSED_DECODE"))
        self.scratch = None
        self.timeline: Optional[torch.Tensor] = None  # set by `time_phases`: the kernel then records where its time goes

    # ------------------------------------------------------------------ does the model qualify

    def _check(self, model) -> Optional[str]:
        rt, spec = model.runtime, model.spec
        if rt.mode != "bfloat16":
            return "the fused decode step is a bfloat16 kernel"
        if type(model.embedding) is not TokenEmbedding or type(model.head) is not LinearHead:
            return "an embedding or a head of another kind"
        if not _bf16_matrix(model.embedding.weight) or not model.embedding.weight.is_contiguous():
            return "the embedding table is not a contiguous bfloat16 matrix"
        if not _bf16_matrix(model.head.weight) or not _norm_fits(model.final_norm, spec.hidden_size):
            return "the output matrix is not bfloat16 or the final norm is of another kind"
        hidden = spec.hidden_size
        head_dims = set()
        for entry in spec.schedule:
            if entry.cache_from is not None:
                return "a run that reads another run's cache"
            block = model.blocks[entry.layer]
            if type(block) is not PreNormBlock or type(block.mixer) is not AttentionMixer or type(block.feed_forward) is not GatedFeedForward:
                return "a block, mixer or feed-forward of another kind"
            m, f = block.mixer, block.feed_forward
            s = m.spec
            pos = m.position
            if m.b_qkv is not None or m.b_o is not None or f.b_gate_up is not None or f.b_down is not None:
                return "biases"
            if pos is None or pos.rotary_dim != s.head_dim or pos.interleaved:
                return "a position encoding other than split-half rotation over the whole head"
            if not all(_bf16_matrix(t) for t in (m.w_qkv, m.w_o, f.w_gate_up, f.w_down)):
                return "a weight matrix that is not bfloat16 with 16-byte rows"
            if not _norm_fits(block.mixer_norm, hidden) or not _norm_fits(block.feed_forward_norm, hidden):
                return "a norm of another kind"
            head_dims.add(s.head_dim)
            if s.hidden_size != hidden or f.spec.hidden_size != hidden:
                return "layers of different widths"
        if len(head_dims) != 1:
            return "layers with different head sizes"
        self.head_dim = head_dims.pop()
        if self.head_dim % 16 or self.head_dim > 128:
            return f"a head size of {self.head_dim} (the fused step takes multiples of 16 up to 128)"
        return None

    # ------------------------------------------------------------------ the list of phases

    def _build(self, runs) -> None:
        model, spec = self.model, self.model.spec
        self.lib = lib = ops.decode_step_lib(self.head_dim)
        lib.mb_decode_step_phase_bytes.restype = ctypes.c_size_t
        lib.mb_decode_step_step_bytes.restype = ctypes.c_size_t
        if lib.mb_decode_step_phase_bytes() != ctypes.sizeof(Phase) or lib.mb_decode_step_step_bytes() != ctypes.sizeof(Step):
            raise ops.KernelError("the decode step's records differ between the library and its Python face")
        max_columns, slice_columns = lib.mb_decode_step_max_columns(), lib.mb_decode_step_slice_columns()
        hidden = spec.hidden_size
        if hidden > max_columns:
            self.why_not = f"a width of {hidden} (a row of activations must fit a block's shared memory: {max_columns})"
            return
        phases: List[Phase] = []

        def pad(k):
            return -(-k // slice_columns) * slice_columns

        def matrix(kind, w, rows, tiles, barrier, k_begin=0, k_len=None, **more):
            k_len = w.shape[1] if k_len is None else k_len
            p = Phase(kind=kind, barrier_before=1 if barrier else 0, w=w.data_ptr() + 2 * k_begin, ldw=w.stride(0), rows=rows,
                      tiles=tiles, k_len=k_len, k_pad=pad(k_len), k_begin=k_begin)
            for name, value in more.items():
                setattr(p, name, value)
            phases.append(p)

        phases.append(Phase(kind=PH_EMBED))
        self.max_q_width = self.max_intermediate = self.max_heads = 0
        self.groups = set()
        for run, entry in zip(runs, spec.schedule):
            block = model.blocks[entry.layer]
            m, f = block.mixer, block.feed_forward
            s = m.spec
            if run.k_pool is None or run.k_pool.dtype != torch.bfloat16 or run.k_pool.shape[2] != 64 or not run.writes_cache:
                self.why_not = "a cache that is not bfloat16 pages of 64 positions"
                return
            if run.group >= MAX_GROUPS:
                self.why_not = f"more than {MAX_GROUPS} cache groups"
                return
            if m.q_width > max_columns:
                self.why_not = f"{m.q_width} query columns (at most {max_columns})"
                return
            self.groups.add(run.group)
            attention = dict(group=run.group, heads=s.num_heads, kv_heads=s.num_kv_heads, window=s.window or 0, scale=s.scale,
                             k_pool=run.k_pool.data_ptr(), v_pool=run.v_pool.data_ptr(), cos_table=m.position.cos.data_ptr(),
                             sin_table=m.position.sin.data_ptr())
            n1, n2 = block.mixer_norm, block.feed_forward_norm
            qkv_rows = (s.num_heads + 2 * s.num_kv_heads) * s.head_dim
            matrix(PH_QKV, m.w_qkv, qkv_rows, qkv_rows // 16, True, gain=n1.weight.data_ptr(), eps=n1.spec.eps, **attention)
            phases.append(Phase(kind=PH_ATTN, barrier_before=1, **attention))
            matrix(PH_OUT, m.w_o, hidden, -(-hidden // 16), True, **attention)
            inter = f.spec.intermediate_size
            matrix(PH_GATE_UP, f.w_gate_up, inter, -(-inter // 8), True, gain=n2.weight.data_ptr(), eps=n2.spec.eps,
                   pair_offset=inter, activation=ops.activation_code(f.spec.activation))
            # the down product's K may exceed what a block can stage: column ranges, one after the other, each adding
            # into the rows the block owns (so only the first waits for the phase before it)
            parts = -(-inter // max_columns)
            per_part = pad(-(-inter // parts))
            for i, k_begin in enumerate(range(0, inter, per_part)):
                matrix(PH_DOWN, f.w_down, hidden, -(-hidden // 16), i == 0, k_begin=k_begin, k_len=min(per_part, inter - k_begin))
            self.max_q_width = max(self.max_q_width, m.q_width)
            self.max_intermediate = max(self.max_intermediate, inter)
            self.max_heads = max(self.max_heads, s.num_heads)
        norm = model.final_norm
        vocab = model.head.weight.shape[0]
        matrix(PH_HEAD, model.head.weight, vocab, -(-vocab // 16), True, gain=norm.weight.data_ptr(), eps=norm.spec.eps)
        self.vocab = vocab
        if len(phases) > lib.mb_decode_step_max_phases():
            self.why_not = f"{len(phases)} phases (a launch carries {lib.mb_decode_step_max_phases()})"
            return
        device = model.runtime.device
        self.phases = (Phase * len(phases))(*phases)  # host memory: the launcher copies them into the launch's parameters
        self.kinds = [p.kind for p in phases]
        self.num_phases = len(phases)
        f32 = dict(dtype=torch.float32, device=device)
        self.scratch = {
            "x": torch.zeros((MAX_ROWS, hidden), **f32),
            "q": torch.zeros((MAX_ROWS, self.max_q_width), dtype=torch.bfloat16, device=device),
            "h": torch.zeros((MAX_ROWS, self.max_intermediate), dtype=torch.bfloat16, device=device),
            "attn_o": torch.zeros((MAX_ROWS * self.max_heads * MAX_SPLITS * self.head_dim,), **f32),
            "attn_ml": torch.zeros((MAX_ROWS * self.max_heads * MAX_SPLITS * 2,), **f32),
            "attn_tickets": torch.zeros((MAX_ROWS * self.max_heads,), dtype=torch.int32, device=device),  # every step leaves them zero
            "a": torch.zeros((MAX_ROWS, self.max_q_width), dtype=torch.bfloat16, device=device),
            "barrier": torch.zeros((1,), dtype=torch.int32, device=device),
            "status": torch.zeros((1,), dtype=torch.int32, device=device),
        }
        self.sms = ops.multiprocessors(device)

    # ------------------------------------------------------------------ a step

    def takes(self, batch) -> bool:
        """One new token for each of at most eight sequences, every token's logits wanted, no observer."""
        return (self.enabled and self.why_not is None and self.model.observer is None and batch.max_q_len == 1
                and batch.num_tokens == batch.num_sequences <= MAX_ROWS and batch.num_wanted == batch.num_tokens)

    def splits_for(self, sequences: int, heads: int, kv_heads: int) -> int:
        """Blocks that share a sequence's keys: what gives every block an item, a power of two of at most 16.  It does not
        depend on the sequences' lengths (a split that finds no page of its own writes an empty result)."""
        items = sequences * kv_heads * (-(-(heads // kv_heads) // 16))
        splits = 1
        if items * 3 <= self.sms:  # with a third of the blocks busy or more, splitting costs more (the combine) than it gains
            while splits * 2 <= MAX_SPLITS and items * splits * 2 <= self.sms:
                splits *= 2
        return splits

    def run(self, batch, runs) -> Optional[torch.Tensor]:
        if self.phases is None:
            self._build(runs)
            if self.why_not is not None:
                return None
        model = self.model
        scratch = self.scratch
        rows = batch.num_tokens
        logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=model.runtime.device)
        step = Step(phases=ctypes.addressof(self.phases), num_phases=self.num_phases, batch=rows, hidden=model.spec.hidden_size,
                    tokens=batch.tokens.data_ptr(), positions=batch.positions.data_ptr(), kv_lens=batch.kv_lens.data_ptr(),
                    embedding=model.embedding.weight.data_ptr(), embedding_scale=model.spec.embedding.scale,
                    max_blocks=batch.groups[0].block_table.shape[1] if batch.groups else 0,
                    x=scratch["x"].data_ptr(), q=scratch["q"].data_ptr(), ld_q=self.max_q_width, h=scratch["h"].data_ptr(),
                    ld_h=self.max_intermediate, attn_o=scratch["attn_o"].data_ptr(), attn_ml=scratch["attn_ml"].data_ptr(),
                    attn_tickets=scratch["attn_tickets"].data_ptr(), a=scratch["a"].data_ptr(),
                    logits=logits.data_ptr(), ld_logits=logits.stride(0), barrier=scratch["barrier"].data_ptr(),
                    status=scratch["status"].data_ptr(), timeline=self.timeline.data_ptr() if self.timeline is not None else None)
        for g in self.groups:
            step.block_tables[g] = batch.groups[g].block_table.data_ptr()
            step.slot_mappings[g] = batch.groups[g].slot_mapping.data_ptr()
        for run, entry in zip(runs, model.spec.schedule):  # (the layers of a group share its kv heads; the least of their answers)
            s = model.blocks[entry.layer].mixer.spec
            splits = self.splits_for(rows, s.num_heads, s.num_kv_heads)
            step.splits[run.group] = min(splits, step.splits[run.group] or splits)
        ops.decode_step(self.lib, step, self.sms)
        spec = model.spec.head
        if spec.logit_scale != 1.0 or spec.softcap != 0.0:
            ops.logit_epilogue(logits, spec.logit_scale, spec.softcap)
        return logits

    def time_phases(self, on: bool = True) -> None:
        """Makes the kernel record, for its first block, the clock when it enters each phase, passes the barrier,
        has staged the activations and is done (read with `phase_times`).  For looking at where a step's time goes."""
        self.timeline = torch.zeros((max(1, self.num_phases) * 6,), dtype=torch.int64, device=self.model.runtime.device) if on else None

    def phase_times(self):
        """(kind, cycles waiting at the barrier, cycles staging, cycles in tiles or items, of those the first tile's
        products, and its wait for the other warps) per phase of the last step."""
        kinds = self.kinds
        t = self.timeline.cpu().view(self.num_phases, 6).tolist()
        return [(kinds[i], t[i][1] - t[i][0], t[i][2] - t[i][1], t[i][3] - t[i][2], max(0, t[i][4] - t[i][2]), max(0, t[i][5] - t[i][4]))
                for i in range(self.num_phases)]

    def status(self) -> int:
        """0 unless a bounded wait inside the kernel ever gave up (1 + (phase << 8)); the barrier counter, which such a
        step leaves short, is then cleared so that the next step starts clean."""
        if self.scratch is None:
            return 0
        status = int(self.scratch["status"].item())
        if status:
            self.scratch["barrier"].zero_()
            self.scratch["status"].zero_()
        return status
