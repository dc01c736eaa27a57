"""Python faces of the CUDA launchers: shape and dtype checks, then one C call on the current stream.

There is no CPU path and no library stand-in: a tensor that is not on a CUDA device, or a kernel
library that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_library

_F32, _BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, got {dtype}")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "models_b200 kernels run on a CUDA device only (got a tensor on "
                f"{t.device}); there is no CPU path")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    """The current stream of the current device, as the raw handle the launchers take (the two
    calls below are what torch.cuda.current_stream() ends in, without its Python layers: this runs
    once per kernel launch)."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


_launches = [0]


def launch_count() -> int:
    """Launches of this package's own kernels so far (graph replays count the kernels they hold)."""
    return _launches[0]


def add_launches(n: int) -> None:
    _launches[0] += n


_recorded = [None]  # a list while launches are being recorded (see `recording`), else None


class recording:
    """`with ops.recording() as names:` collects, in order, which launcher of this module ran each of this
    package's kernels (the function's name says which form of a product it is).  For reports, not for hot loops."""

    def __enter__(self):
        self.before, _recorded[0] = _recorded[0], []
        return _recorded[0]

    def __exit__(self, *exc):
        _recorded[0] = self.before
        return False


def _run(lib, status: int):
    if status != 0:
        raise KernelError(lib.mb_last_error().decode("utf-8", "replace"))
    _launches[0] += 1
    if _recorded[0] is not None:
        import sys
        _recorded[0].append(sys._getframe(1).f_code.co_name)


def _int32(t: Optional[torch.Tensor], name: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")


# ------------------------------------------------------------------------------------ libraries

def elementwise():
    return load_library("mb_elementwise", ["elementwise.cu"])


def attention_rows():
    return load_library("mb_attention_rows", ["attention_rows.cu"])


def attention_tc(head_dim: int):
    """The tensor-core attention kernels, compiled for this head size at first use."""
    return load_library("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": int(head_dim)})


def attention_tc_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and page_size == 64


def prefill_attention_tc(head_dim: int):
    """The tcgen05 prefill attention, compiled for this head size (64 or 128) at first use."""
    return load_library("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": int(head_dim)})


TCGEN05_ATTENTION_MIN_ROWS = 33  # shorter steps go to the mma.sync kernel, whose blocks take 64 query rows


def prefill_attention_tcgen05_takes(q: torch.Tensor, out: torch.Tensor, head_dim: int, max_q_len: int) -> bool:
    """Head sizes 64 and 128, steps of more than a few tokens, rows that TMA and 16-byte stores can address."""
    return (head_dim in (64, 128) and max_q_len >= TCGEN05_ATTENTION_MIN_ROWS and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def gemm32():
    return load_library("mb_gemm_f32", ["gemm_f32.cu"])


def sampling():
    return load_library("mb_sampling", ["sampling.cu"])


def random_init():
    return load_library("mb_random_init", ["random_init.cu"])


def random_normal(out: torch.Tensor, key, mean: float, std: float) -> torch.Tensor:
    """Fills `out` (contiguous float32 or bfloat16) with mean + std * z, z standard normal from the
    counter-based generator keyed by `key` (two 32-bit words): the values of weights/philox_normal.py."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal fills a contiguous tensor")
    lib = random_init()
    _run(lib, lib.mb_random_normal(_p(out), _code(out.dtype), ctypes.c_size_t(out.numel()), ctypes.c_uint32(key[0]),
                                   ctypes.c_uint32(key[1]), ctypes.c_float(mean), ctypes.c_float(std), _stream()))
    return out


# ------------------------------------------------------------------------------------ element-wise

def embed_gather(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Rows of `table` ([vocab, width]) picked by `tokens` (int32), as the float residual stream."""
    _cuda(table, tokens)
    _int32(tokens, "tokens")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding table must be a contiguous [vocab, width] matrix")
    rows, (vocab, width) = tokens.numel(), table.shape
    out = torch.empty((rows, width), dtype=torch.float32, device=table.device)
    lib = elementwise()
    _run(lib, lib.mb_embed_gather(_p(table), _code(table.dtype), _p(tokens), _p(out), rows, width, vocab,
                                  ctypes.c_float(scale), _stream()))
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x (float residual, [T, width]) += delta, then RMSNorm with `weight` (float).  With `rows`
    only those rows are normalised (and x is left alone).  Returns the normalised rows."""
    _cuda(x, delta, weight, rows)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("the residual stream must be a contiguous float32 [rows, width] tensor")
    width = x.shape[1]
    if weight.dtype != torch.float32 or weight.numel() != width:
        raise KernelError(f"norm weight must be float32 of {width} elements, got {weight.dtype} of {weight.numel()}")
    if delta is not None and (delta.shape != x.shape or not delta.is_contiguous()):
        raise KernelError(f"delta {tuple(delta.shape)} must match the residual stream {tuple(x.shape)}")
    _int32(rows, "rows")
    out_rows = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((out_rows, width), dtype=out_dtype, device=x.device)
    lib = elementwise()
    _run(lib, lib.mb_add_rmsnorm(_p(x), _p(delta), _code(delta.dtype) if delta is not None else 0, _p(weight), _p(out),
                                 _code(out_dtype), _p(rows), out_rows, width, ctypes.c_float(eps),
                                 1 if (write_x and rows is None) else 0, _stream()))
    return out


def rope_cache_write(qkv: torch.Tensor, positions: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                     sin: Optional[torch.Tensor], k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     slot_mapping: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                     interleaved: bool, page_size: int, write_cache: bool) -> None:
    """Rotates the query heads of `qkv` ([T, (heads + 2*kv_heads) * head_dim]) in place; rotates the
    key heads and copies the value heads into the pools at `slot_mapping`."""
    _cuda(qkv, positions, cos, sin, k_pool, v_pool, slot_mapping)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("qkv must be a [tokens, columns] tensor with unit column stride")
    need = (heads + (2 * kv_heads if write_cache else 0)) * head_dim
    if qkv.shape[1] < need:
        raise KernelError(f"qkv rows have {qkv.shape[1]} columns, {need} are needed")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if rotary_dim > 0:
        if cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("rotation needs float32 cos/sin tables")
        if cos.shape[-1] != rotary_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError(f"cos/sin tables must be contiguous [positions, {rotary_dim // 2}]")
    if write_cache and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype):
        raise KernelError(f"cache pools ({k_pool.dtype}) must have the dtype of qkv ({qkv.dtype})")
    lib = elementwise()
    _run(lib, lib.mb_rope_cache_write(_p(qkv), _code(qkv.dtype), qkv.stride(0), _p(positions), _p(cos), _p(sin),
                                      _p(k_pool), _p(v_pool), _p(slot_mapping), qkv.shape[0], heads, kv_heads,
                                      head_dim, rotary_dim, 1 if interleaved else 0, page_size,
                                      1 if write_cache else 0, _stream()))


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}  # the codes of csrc/common.cuh (MB_ACT_*)


def activation_code(activation: str) -> int:
    if activation not in ACTIVATIONS:
        raise KernelError(f"gate activation {activation!r} is not built (known: {', '.join(sorted(ACTIVATIONS))})")
    return ACTIVATIONS[activation]


def gated_epilogue(activation: str = "silu") -> int:
    """The epilogue code of a gate/up product that stores act(gate) * up: EPI_SWIGLU with the
    activation in the bits above it (silu gives EPI_SWIGLU itself)."""
    return EPI_SWIGLU | (activation_code(activation) << 8)


def swiglu(gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(gate) * up for a [rows, 2*width] tensor whose first half of columns is the gate."""
    _cuda(gate_up)
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("gate_up must be a contiguous [rows, 2*width] tensor")
    rows, width = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, width), dtype=gate_up.dtype, device=gate_up.device)
    lib = elementwise()
    _run(lib, lib.mb_swiglu(_p(gate_up), _p(out), _code(gate_up.dtype), rows, width, activation_code(activation), _stream()))
    return out


def logit_epilogue(logits: torch.Tensor, scale: float, softcap: float) -> torch.Tensor:
    """In place on float32 logits [rows, vocab]: times `scale`, then softcap * tanh(logits / softcap)
    unless softcap is 0."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logit_epilogue takes float32 [rows, vocab] logits")
    lib = elementwise()
    _run(lib, lib.mb_logit_epilogue(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], ctypes.c_float(scale),
                                    ctypes.c_float(softcap), _stream()))
    return logits


def bias_add(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    _cuda(x, bias)
    if not x.is_contiguous() or bias.dtype != torch.float32 or bias.numel() != x.shape[-1]:
        raise KernelError("bias_add needs a contiguous x and a float32 bias of x's width")
    lib = elementwise()
    _run(lib, lib.mb_bias_add(_p(x), _code(x.dtype), _p(bias), x.numel() // x.shape[-1], x.shape[-1], _stream()))
    return x


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() or delta.shape != x.shape:
        raise KernelError("residual_add needs a contiguous float32 x and a delta of the same shape")
    lib = elementwise()
    _run(lib, lib.mb_residual_add(_p(x), _p(delta), _code(delta.dtype), ctypes.c_size_t(x.numel()), _stream()))
    return x


# ------------------------------------------------------------------------------------ attention

def paged_attention_rows(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int,
                         heads: int, kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> None:
    """q: [T, >= heads*head_dim] (may be a column slice of a wider tensor); out: [T, heads*head_dim].
    Pools: [pages, kv_heads, page_size, head_dim]."""
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    if k_pool.dim() != 4 or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim or not k_pool.is_contiguous():
        raise KernelError(f"k_pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pool.shape)}")
    if v_pool.shape != k_pool.shape or not v_pool.is_contiguous():
        raise KernelError("v_pool must match k_pool")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("q, out and the pools must share one dtype")
    sequences = kv_lens.numel()
    lib = attention_rows()
    _run(lib, lib.mb_paged_attention_rows(_p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool),
                                          _p(v_pool), _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens),
                                          sequences, max_q_len, heads, kv_heads, head_dim, k_pool.shape[2],
                                          window or 0, ctypes.c_float(scale), _stream()))


def _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim):
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    if k_pool.dim() != 4 or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim or not k_pool.is_contiguous():
        raise KernelError(f"k_pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pool.shape)}")
    if v_pool.shape != k_pool.shape or not v_pool.is_contiguous():
        raise KernelError("v_pool must match k_pool")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("the tensor-core attention kernels take bfloat16 q, out and pools")


_decode_block_bytes = {}


LONG_KEYS = 1024  # up to so many cached positions the split depends on the batch size alone


def decode_span(max_kv_len: int) -> int:
    """The class of context lengths that share one split of the keys: 0 up to LONG_KEYS positions, else
    the next power of two.  A captured decode step is valid for one class."""
    if max_kv_len <= LONG_KEYS:
        return 0
    span = LONG_KEYS
    while span < max_kv_len:
        span *= 2
    return span


SHARED_MEMORY_PER_SM = 227 * 1024  # what a block of sm_100a can be given


def decode_splits(sequences: int, heads: int, kv_heads: int, head_dim: int = 64, keys: int = 0,
                  window: Optional[int] = None, multiprocessors: Optional[int] = None, page_size: int = 64) -> int:
    """How many blocks share one sequence's keys.

    Up to LONG_KEYS cached positions (`keys`; 0: unknown, taken as short): a power of two, at most 8
    (they form one thread-block cluster), with which all blocks of the call are resident at once -- a
    second, partly filled round of blocks costs more than longer blocks do (measured: 16 sequences of
    1,100 positions at head size 128 take 22 us with 2 splits, 29 with 4, 38 with 8).  The kernel runs
    with three page stages when there are four or more splits (or heads of 96 and more, or blocks so
    few that all of them fit the multiprocessors with three) and with two otherwise, and a block's shared
    memory follows from that; so does the count.  It depends on the
    batch size rounded up to a power of two only, so a batch padded to such a size is split like the
    unpadded one.

    Longer contexts: what counts is that enough blocks are in flight to keep memory busy, and a
    cluster's eight are too few for one or two sequences (one sequence of 32,768 positions, head size
    64: 58 us with 8 splits, 26 us with 32).  Up to four sequences the count is what makes one round of
    blocks (at most 400: they then run with the deep page ring, and a second, partly filled round costs
    more than it gives: 2 sequences of 32,768 positions take 29 us with 16 splits, 39 with 32; 4
    sequences 57 us with 8, 65 with 16).  Larger batches have blocks enough anyway; there the count is
    one block per 16 pages (64 pages for heads wider than 64, whose pages are twice as large) within
    2,048 blocks in all (8 sequences of 65,536 positions: 175 us with 32 splits, 184 with 16; 16
    sequences of 16,384: 94 us with 16, 100 with 8).  Always at most 64 and at least 4 pages each; above
    8 the partial results meet in scratch memory and a second kernel.  `keys` is rounded up to its class
    (decode_span), so the count is the same for every length of a class.  `multiprocessors`: those of
    the device the call runs on (None: the current device's)."""
    if multiprocessors is None:
        multiprocessors = _sm_count(torch.device("cuda", torch.cuda.current_device()))
    rounded = 1
    while rounded < sequences:
        rounded *= 2
    base = rounded * kv_heads * (-(-(heads // kv_heads) // 16))
    if head_dim not in _decode_block_bytes:
        lib = attention_tc(head_dim)
        lib.mb_decode_block_bytes.restype = ctypes.c_size_t
        _decode_block_bytes[head_dim] = {stages: int(lib.mb_decode_block_bytes(stages)) + 1024 for stages in (2, 3)}
        _decode_block_bytes[head_dim]["wide"] = int(lib.mb_decode_stages(1)) == 3  # three stages whatever the split

    def power_of_two_up_to(limit: int) -> int:
        splits = 1
        while splits * 2 <= limit:
            splits *= 2
        return splits

    def fitting(stages: int) -> int:
        resident = max(1, SHARED_MEMORY_PER_SM // _decode_block_bytes[head_dim][stages])
        return power_of_two_up_to(max(1, min(8, (resident * multiprocessors) // max(1, base))))

    with_three = fitting(3)
    short = with_three if _decode_block_bytes[head_dim]["wide"] or with_three >= 4 else min(2, fitting(2))
    # (eight blocks to a sequence only for a handful of sequences: with more, a block is left with a page or two, and the
    # cluster's meeting costs more than the shorter walk saves -- batch 8: 0.772 ms per step with four, 0.810 with eight)
    short = min(short, max(4, 256 // max(1, base)))
    span = decode_span(keys)
    if span == 0:
        return short
    visible = min(span, window) if window else span
    pages = -(-visible // page_size)
    by_length = pages // (16 if head_dim <= 64 else 64)
    one_round = power_of_two_up_to(max(1, 400 // base))
    want = one_round if one_round >= 8 else max(one_round, by_length)
    want = power_of_two_up_to(max(1, min(want, 64, 2048 // base, pages // 4)))
    return want if want > 8 else short


def decode_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, heads: int, kv_heads: int,
                     head_dim: int, window: Optional[int], scale: float, splits: int, use_scratch: bool = False) -> None:
    """One query token per sequence (row cu_q[s] of q) against its cached keys and values.  The keys
    of a sequence are split over `splits` blocks; 2, 4 or 8 of them combine inside a thread-block
    cluster, other counts (or use_scratch) through scratch memory and a second kernel."""
    _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim)
    sequences = kv_lens.numel()
    lib = attention_tc(head_dim)
    scratch = None
    if splits > 1 and (use_scratch or splits not in (2, 4, 8)):
        lib.mb_decode_scratch_floats.restype = ctypes.c_size_t
        scratch = torch.empty((lib.mb_decode_scratch_floats(sequences, heads, splits),), dtype=torch.float32, device=q.device)
    _run(lib, lib.mb_decode_attention(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(v_pool),
                                      _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), sequences, heads,
                                      kv_heads, k_pool.shape[2], window or 0, ctypes.c_float(scale), splits,
                                      _p(scratch), _stream()))
    if scratch is not None:
        _launches[0] += 1  # the combine kernel


def prefill_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int, heads: int,
                      kv_heads: int, head_dim: int, window: Optional[int], scale: float, kernel: Optional[str] = None) -> None:
    """Any number of new tokens per sequence; their keys and values are already in the cache.
    `kernel`: None picks the tcgen05 kernel where it applies, else the mma.sync one; "tcgen05" or
    "mma" asks for one of them."""
    _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim)
    if kernel not in (None, "tcgen05", "mma"):
        raise KernelError(f"prefill_attention: unknown kernel {kernel!r}")
    if kernel == "tcgen05" or (kernel is None and prefill_attention_tcgen05_takes(q, out, head_dim, max_q_len)):
        if head_dim not in (64, 128):
            raise KernelError(f"the tcgen05 prefill attention is built for head sizes 64 and 128, got {head_dim}")
        lib = prefill_attention_tc(head_dim)
        _run(lib, lib.mb_prefill_attention_tcgen05(
            _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_pool), _p(v_pool), k_pool.shape[0],
            _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), kv_lens.numel(), max_q_len, heads, kv_heads,
            k_pool.shape[2], window or 0, ctypes.c_float(scale), _stream()))
        return
    lib = attention_tc(head_dim)
    _run(lib, lib.mb_prefill_attention(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(v_pool),
                                       _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), kv_lens.numel(),
                                       max_q_len, heads, kv_heads, k_pool.shape[2], window or 0, ctypes.c_float(scale),
                                       _stream()))


# ------------------------------------------------------------------------------------ matrix products

def gemm_f32(a: torch.Tensor, w: torch.Tensor, row_invariant: bool = True) -> torch.Tensor:
    """a [m, k] . w[n, k]^T in true 32-bit arithmetic."""
    _cuda(a, w)
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError(f"gemm_f32 takes float32 operands, got {a.dtype} and {w.dtype}")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not fit")
    m, k = a.shape
    n = w.shape[0]
    c = torch.empty((m, n), dtype=torch.float32, device=a.device)
    lib = gemm32()
    _run(lib, lib.mb_gemm_f32(_p(a), a.stride(0), _p(w), w.stride(0), _p(c), n, m, n, k, 1 if row_invariant else 0,
                              _stream()))
    return c


SKINNY_ROWS, SKINNY_NORM_ROWS = 32, 16
EPI_BF16, EPI_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3


def skinny():
    return load_library("mb_skinny_gemm", ["skinny_gemm.cu"])


def skinny_takes(weight: torch.Tensor, rows: int, with_norm: bool = False) -> bool:
    """Whether the decode matrix product takes this weight with this many activation rows."""
    return (weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1 and weight.shape[1] % 8 == 0
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0
            and 0 < rows <= (SKINNY_NORM_ROWS if with_norm else SKINNY_ROWS))


SKINNY_PAYS_ROWS = 8  # one 8-column MMA tile of activations: beyond it a block's activations crowd out its weight rings


def skinny_pays(weight: torch.Tensor, rows: int, with_norm: bool = False) -> bool:
    """Whether the decode matrix product is the one to use: it takes up to 32 rows, but with more than 8
    its blocks hold twice the activations in shared memory, half as many of them fit a multiprocessor,
    and a library product streams the weights faster (measured at 16 and 32 rows on every layer shape
    of the 1B, 3B and 8B models)."""
    return rows <= SKINNY_PAYS_ROWS and skinny_takes(weight, rows, with_norm)


_multiprocessors = {}


def _sm_count(device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _multiprocessors:
        _multiprocessors[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _multiprocessors[index]


def multiprocessors(device) -> int:
    """Multiprocessors of a CUDA device (asked of the driver once)."""
    return _sm_count(torch.device(device))


def skinny_gemm(weight: torch.Tensor, epilogue: int, x: Optional[torch.Tensor] = None, xf: Optional[torch.Tensor] = None,
                gain: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """Few activation rows times weight^T ([n, k] bfloat16).  Activations: `x` (bfloat16 [rows, k]), or
    `xf` (the float32 residual rows, optionally gathered by `rows`) normalised on the fly with `gain`
    and `eps`.  Epilogues: EPI_BF16 / EPI_F32 store [rows, n]; EPI_RESIDUAL adds into `out` (float32
    [rows, n]); EPI_SWIGLU takes weight = [gate rows; up rows] and stores act(gate) * up [rows, n/2].
    `norm_parts` and `emit_gain` as for wide_gemm: `x` is then the rows times a norm's gain, divided by their
    root mean square in the epilogue; a residual product can prepare the next norm's rows the same way."""
    _cuda(weight, x, xf, gain, rows, out, emit_gain)
    n, k = weight.shape
    norm = gain is not None
    if norm:
        if xf is None or xf.dtype != torch.float32 or xf.stride(1) != 1 or xf.shape[1] != k:
            raise KernelError("the norm prologue needs float32 rows of the weight's width")
        if gain.dtype != torch.float32 or gain.numel() != k:
            raise KernelError("the norm gain must be float32 of the weight's width")
        _int32(rows, "rows")
        batch = rows.numel() if rows is not None else xf.shape[0]
    else:
        if x is None or x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != k:
            raise KernelError("activations must be bfloat16 rows of the weight's width")
        batch = x.shape[0]
    if not skinny_takes(weight, batch, norm):
        raise KernelError(f"skinny_gemm does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows")
    kind = epilogue & 0xFF  # a gated epilogue carries its activation above
    out_cols = n // 2 if kind == EPI_SWIGLU else n
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (batch, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [rows, n] tensor")
    elif out is None:
        out = torch.empty((batch, out_cols), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16,
                          device=weight.device)
    if norm and norm_parts is not None:
        raise KernelError("a product normalises float32 rows itself or takes rows with parts of their sums of squares, not both")
    ssq, count, _, _, part_eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    if norm_parts is not None and norm_parts[2] != k:
        raise KernelError("the norm's width is the product's k")
    emit_rows = emit_ssq = None
    written = ctypes.c_int(0)
    if emit_gain is not None:
        if kind != EPI_RESIDUAL or emit_gain.dtype != torch.float32 or emit_gain.numel() != n:
            raise KernelError("the next norm's rows come from the residual epilogue, with a float32 gain of the output's width")
        emit_rows = torch.empty((batch, n), dtype=torch.bfloat16, device=weight.device)
        emit_ssq = torch.empty((-(-n // 16), SSQ_COLUMNS), dtype=torch.float32, device=weight.device)
    lib = skinny()
    _run(lib, lib.mb_skinny_gemm(_p(weight), weight.stride(0), n, k, batch, _p(x), x.stride(0) if x is not None else 0,
                                 _p(xf), xf.stride(0) if xf is not None else 0, _p(gain),
                                 part_eps if norm_parts is not None else ctypes.c_float(eps), _p(rows),
                                 _p(out), out.stride(0), epilogue, _sm_count(weight.device), 1, ssq, count, _p(emit_gain),
                                 _p(emit_rows), emit_rows.stride(0) if emit_rows is not None else 0, _p(emit_ssq),
                                 ctypes.byref(written), _stream()))
    if emit_gain is not None:
        return out, emit_rows, emit_ssq, written.value
    return out


def skinny_qkv_rope(weight: torch.Tensor, xf: Optional[torch.Tensor], gain: Optional[torch.Tensor], eps: float, heads: int,
                    kv_heads: int, head_dim: int, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, slot_mapping: torch.Tensor, x: Optional[torch.Tensor] = None,
                    norm_parts=None) -> torch.Tensor:
    """The q/k/v product of an attention layer on few rows with everything around it folded in: RMSNorm
    of the float32 residual rows `xf` before it, rotation of queries and keys (split-half pairs over
    the whole head) and the paged cache write of keys and values after it.  Returns the rotated
    queries, bfloat16 [rows, heads * head_dim].  In place of `xf` and `gain`: `x`, the rows times the gain as
    bfloat16, with `norm_parts` (as for wide_gemm); the division by the root mean square then happens in the epilogue."""
    _cuda(weight, xf, x, gain, positions, cos, sin, k_pool, v_pool, slot_mapping)
    if (xf is None) == (x is None) or (x is not None and norm_parts is None):
        raise KernelError("skinny_qkv_rope takes float32 rows with a gain, or gained bfloat16 rows with parts of their sums of squares")
    batch, k = (xf if xf is not None else x).shape
    if weight.shape != ((heads + 2 * kv_heads) * head_dim, k) or not skinny_takes(weight, batch, True):
        raise KernelError(f"skinny_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows")
    if xf is not None and (xf.dtype != torch.float32 or xf.stride(1) != 1 or gain.dtype != torch.float32 or gain.numel() != k):
        raise KernelError("skinny_qkv_rope needs float32 residual rows and gain")
    if x is not None and (x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16 or norm_parts[2] != k):
        raise KernelError("skinny_qkv_rope needs aligned bfloat16 rows of the weight's width")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim:
        raise KernelError("cache pools must be bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=weight.device)
    ssq, count, _, _, part_eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = skinny()
    _run(lib, lib.mb_skinny_qkv_rope(_p(weight), weight.stride(0), k, batch, _p(x), x.stride(0) if x is not None else 0, _p(xf),
                                     xf.stride(0) if xf is not None else 0, _p(gain),
                                     part_eps if norm_parts is not None else ctypes.c_float(eps), _p(q), q.stride(0), heads,
                                     kv_heads, head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool),
                                     _p(slot_mapping), k_pool.shape[2], _sm_count(weight.device), 1, ssq, count, _stream()))
    return q


def gemm_tc():
    return load_library("mb_gemm_tcgen05", ["gemm_tcgen05.cu"])


TCGEN05_MIN_ROWS = 9  # fewer rows take the narrow decode product
WIDE_ROWS = 128  # most activation rows of the wide decode product


def gemm_tcgen05_takes(weight: torch.Tensor, epilogue: int = EPI_BF16, rows: Optional[int] = None) -> bool:
    """Whether a tcgen05 matrix product takes this weight and, if `rows` is given, is the one to use for
    so many rows: above 128 the prefill form; from 9 to 128 the wide decode form (fewer rows take the
    narrow decode product)."""
    epilogue &= 0xFF
    n = weight.shape[0] // 2 if epilogue == EPI_SWIGLU else weight.shape[0]
    if rows is not None and rows < TCGEN05_MIN_ROWS:
        return False
    return (weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1 and weight.shape[1] % 8 == 0
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0 and n % 8 == 0
            and (epilogue != EPI_SWIGLU or weight.shape[0] % 2 == 0))


_split_tickets = {}


def gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                 tile_width: int = 0, pair: int = 0, arrival_order: bool = False) -> torch.Tensor:
    """a [m, k] . weight[n, k]^T on the tcgen05 tensor cores (bfloat16 in, float accumulation).
    Epilogues as for skinny_gemm: EPI_BF16 / EPI_F32 store, EPI_RESIDUAL adds into `out` (float32
    [m, n]), EPI_SWIGLU stores act(gate) * up for weight = [gate rows; up rows].  tile_width 0 lets
    the launcher choose between tiles of 128 and 256 output columns.  pair 2: tiles of 256 rows by
    256 columns on pairs of blocks (tcgen05 cta_group::2).  Where the residual epilogue splits K over
    blocks (few tiles, a long K) the parts are summed in their order through scratch memory, so a
    result is the same bits in every run; `arrival_order` lets each part add into `out` as it finishes
    instead (a little quicker, the last bit of an element then depends on timing)."""
    _cuda(a, weight, out)
    if a.dtype != torch.bfloat16 or a.dim() != 2 or a.stride(1) != 1 or a.shape[1] != weight.shape[1]:
        raise KernelError(f"gemm_tcgen05: activations {tuple(a.shape)} {a.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_takes(weight, epilogue) or a.stride(0) % 8 or a.data_ptr() % 16:
        raise KernelError(f"gemm_tcgen05 does not take a {tuple(weight.shape)} {weight.dtype} weight")
    m, k = a.shape
    n_w = weight.shape[0]
    kind = epilogue & 0xFF
    n = n_w // 2 if kind == EPI_SWIGLU else n_w
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (m, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [m, n] tensor")
    elif out is None:
        out = torch.empty((m, n), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16, device=a.device)
    lib = gemm_tc()
    sms = _sm_count(a.device)
    partial = tickets = None
    if kind == EPI_RESIDUAL and not arrival_order:
        need_partial, need_tickets = ctypes.c_size_t(0), ctypes.c_size_t(0)
        lib.mb_gemm_tcgen05_scratch(sms, ctypes.byref(need_partial), ctypes.byref(need_tickets))
        partial = torch.empty((need_partial.value,), dtype=torch.float32, device=a.device)  # touched only where K is split
        key = a.device.index if a.device.index is not None else torch.cuda.current_device()
        tickets = _split_tickets.get(key)
        if tickets is None:
            # zero once; every launch leaves the tickets at zero
            tickets = _split_tickets[key] = torch.zeros((need_tickets.value,), dtype=torch.int32, device=a.device)
    _run(lib, lib.mb_gemm_tcgen05(_p(a), a.stride(0), _p(weight), weight.stride(0), _p(out), out.stride(0), m, n_w, k,
                                  epilogue, sms, tile_width, pair, _p(partial), _p(tickets), _stream()))
    return out


def gemm_tcgen05_qkv_rope_takes(weight: torch.Tensor, rows: int, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the prefill q/k/v product with folded rotation and cache write applies: a weight the
    tcgen05 product takes for so many rows, heads of 64 or 128."""
    return (head_dim in (64, 128) and weight.shape[0] == (heads + 2 * kv_heads) * head_dim and rows > WIDE_ROWS
            and gemm_tcgen05_takes(weight, EPI_BF16, rows))


def gemm_tcgen05_qkv_rope(a: torch.Tensor, weight: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                          positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_pool: torch.Tensor,
                          v_pool: torch.Tensor, slot_mapping: torch.Tensor) -> torch.Tensor:
    """The q/k/v product of an attention layer over a whole prompt with what follows it folded into
    its epilogue: rotation of queries and keys (split-half pairs over the whole head) and the paged
    cache write of keys and values.  Returns the rotated queries, bfloat16 [rows, heads * head_dim]."""
    _cuda(a, weight, positions, cos, sin, k_pool, v_pool, slot_mapping)
    m, k = a.shape
    if a.dtype != torch.bfloat16 or a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16 or weight.shape[1] != k:
        raise KernelError(f"gemm_tcgen05_qkv_rope: activations {tuple(a.shape)} {a.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_qkv_rope_takes(weight, m, heads, kv_heads, head_dim):
        raise KernelError(f"gemm_tcgen05_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {m} rows "
                          f"and heads of {head_dim}")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if positions.numel() < m or slot_mapping.numel() < m:
        raise KernelError("positions and slot_mapping must hold one entry per row")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if (k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.dim() != 4 or k_pool.shape[1] != kv_heads
            or k_pool.shape[3] != head_dim or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError("cache pools must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((m, heads * head_dim), dtype=torch.bfloat16, device=a.device)
    lib = gemm_tc()
    _run(lib, lib.mb_gemm_tcgen05_qkv_rope(_p(a), a.stride(0), _p(weight), weight.stride(0), _p(q), q.stride(0), m, k, heads,
                                           kv_heads, head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool),
                                           _p(slot_mapping), k_pool.shape[2], _sm_count(a.device), _stream()))
    return q


def wide_gemm_lib():
    return load_library("mb_wide_gemm_tcgen05", ["wide_gemm_tcgen05.cu"])


SSQ_COLUMNS = 128  # columns of a table of parts of sums of squares: one per activation row


def _norm_args(norm_parts, rows: int, columns: Optional[int] = None):
    """(ssq_parts, count, row stride, width, eps) of a product whose activations still lack the division by the
    root mean square, as the C launchers take them.  The table is [parts, columns] float32 with a column per
    activation row (`columns` given: exactly so many)."""
    if norm_parts is None:
        return None, 0, 0, 0, ctypes.c_float(0.0)
    ssq, count, width, eps = norm_parts
    if (ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.stride(1) != 1 or ssq.shape[1] < rows or ssq.shape[0] < count or count <= 0
            or (columns is not None and (ssq.shape[1] != columns or ssq.stride(0) != columns))):
        raise KernelError(f"parts of sums of squares must be a float32 [parts, {columns or 'rows'}] table with a column per row")
    return _p(ssq), int(count), ssq.stride(0), int(width), ctypes.c_float(eps)


def wide_gemm(x: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
              norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """Up to 128 activation rows times weight^T on the tcgen05 tensor cores with the weights as the
    128-row operand (decode at wide batches); K is split over the blocks of a cluster where a matrix has
    few row tiles, their sums meeting in distributed shared memory in a fixed order.  Epilogues as for
    skinny_gemm.

    The RMSNorm before a product can ride in it: `x` is then the rows times the norm's gain, and
    `norm_parts` = (parts of the rows' sums of squares [parts, 128], how many parts, the rows' width, eps);
    the results are scaled by 1 / rms.  The residual epilogue can prepare the NEXT norm the same way: with
    `emit_gain` (that norm's gain) it returns (out, rows of the new `out` times the gain as bfloat16, parts of
    their sums of squares, how many parts)."""
    _cuda(x, weight, out, emit_gain)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != weight.shape[1] or x.shape[0] > WIDE_ROWS:
        raise KernelError(f"wide_gemm: activations {tuple(x.shape)} {x.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_takes(weight, epilogue) or x.stride(0) % 8 or x.data_ptr() % 16:
        raise KernelError(f"wide_gemm does not take a {tuple(weight.shape)} {weight.dtype} weight")
    batch, k = x.shape
    n_w = weight.shape[0]
    kind = epilogue & 0xFF
    n = n_w // 2 if kind == EPI_SWIGLU else n_w
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (batch, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [rows, n] tensor")
    elif out is None:
        out = torch.empty((batch, n), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16, device=x.device)
    emit_rows = emit_ssq = None
    written = ctypes.c_int(0)
    if emit_gain is not None:
        if kind != EPI_RESIDUAL or emit_gain.dtype != torch.float32 or emit_gain.numel() != n:
            raise KernelError("the next norm's rows come from the residual epilogue, with a float32 gain of the output's width")
        emit_rows = torch.empty((batch, n), dtype=torch.bfloat16, device=x.device)
        emit_ssq = torch.empty((8 * -(-n // 128), SSQ_COLUMNS), dtype=torch.float32, device=x.device)
    ssq, count, _, width, eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = wide_gemm_lib()
    _run(lib, lib.mb_wide_gemm(_p(x), x.stride(0), _p(weight), weight.stride(0), _p(out), out.stride(0), batch, n_w, k,
                               epilogue, _sm_count(x.device), ssq, count, width, eps, _p(emit_gain), _p(emit_rows),
                               emit_rows.stride(0) if emit_rows is not None else 0, _p(emit_ssq), ctypes.byref(written), _stream()))
    if emit_gain is not None:
        return out, emit_rows, emit_ssq, written.value
    return out


def wide_qkv_rope_takes(weight: torch.Tensor, rows: int, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the wide q/k/v product with folded rotation and cache write applies: a bfloat16 weight the
    tcgen05 products take, 9 to 128 rows, a head size that divides 128."""
    return (head_dim >= 16 and 128 % head_dim == 0 and weight.shape[0] == (heads + 2 * kv_heads) * head_dim
            and SKINNY_PAYS_ROWS < rows <= WIDE_ROWS and gemm_tcgen05_takes(weight, EPI_BF16))


def wide_qkv_rope(x: torch.Tensor, weight: torch.Tensor, heads: int, kv_heads: int, head_dim: int, positions: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  slot_mapping: torch.Tensor, norm_parts=None) -> torch.Tensor:
    """The q/k/v product of an attention layer on 9 to 128 rows with what follows it folded in: rotation of
    queries and keys (split-half pairs over the whole head) and the paged cache write of keys and values.
    Returns the rotated queries, bfloat16 [rows, heads * head_dim].  `norm_parts` as for wide_gemm."""
    _cuda(x, weight, positions, cos, sin, k_pool, v_pool, slot_mapping)
    batch, k = x.shape
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16 or weight.shape[1] != k:
        raise KernelError(f"wide_qkv_rope: activations {tuple(x.shape)} {x.dtype} do not fit the weight {tuple(weight.shape)}")
    if not wide_qkv_rope_takes(weight, batch, heads, kv_heads, head_dim):
        raise KernelError(f"wide_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows and heads of {head_dim}")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if positions.numel() < batch or slot_mapping.numel() < batch:
        raise KernelError("positions and slot_mapping must hold one entry per row")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if (k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.dim() != 4 or k_pool.shape[1] != kv_heads
            or k_pool.shape[3] != head_dim or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError("cache pools must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=x.device)
    ssq, count, _, width, eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = wide_gemm_lib()
    _run(lib, lib.mb_wide_qkv_rope(_p(x), x.stride(0), _p(weight), weight.stride(0), _p(q), q.stride(0), batch, k, heads, kv_heads,
                                   head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool), _p(slot_mapping),
                                   k_pool.shape[2], _sm_count(x.device), ssq, count, width, eps, _stream()))
    return q


def tensor_core_gemm(a: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                     norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """The tcgen05 product for this many rows: up to 128 the wide decode form, above the prefill form.  The norms
    around a product ride in the wide form only (`norm_parts`, `emit_gain`, see wide_gemm): over a whole prompt a
    norm kernel runs at the speed of memory, and a residual epilogue that does its work, one tile per block with
    nothing to hide behind, was measured to cost as much (4 us each at 2,048 rows of 2,048)."""
    if a.shape[0] <= WIDE_ROWS:
        return wide_gemm(a, weight, epilogue, out, norm_parts=norm_parts, emit_gain=emit_gain)
    if norm_parts is not None or emit_gain is not None:
        raise KernelError("the norms ride in the products of up to 128 rows only")
    return gemm_tcgen05(a, weight, epilogue, out)


def prefill_attention_tcgen05_status(head_dim: int) -> int:
    """0 unless a bounded wait inside the tcgen05 prefill attention ever gave up (1 + (role << 8))."""
    return int(prefill_attention_tc(head_dim).mb_prefill_attention_tc_status())


def gemm_tcgen05_status() -> int:
    """0 unless a bounded wait inside a tcgen05 kernel ever gave up (then it names the role)."""
    return int(gemm_tc().mb_gemm_tc_status()) or int(wide_gemm_lib().mb_wide_gemm_status())


# ------------------------------------------------------------------------------------ the fused decode step

def decode_step_lib(head_dim: int):
    """The whole-step decode kernel, compiled for this head size at first use."""
    return load_library("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": int(head_dim)})


def decode_step(lib, step, sms: int) -> None:
    """Launches csrc/decode_step.cu with the ctypes record `step` (engine/fused_decode.py builds it)."""
    _run(lib, lib.mb_decode_step(ctypes.byref(step), sms, _stream()))


# ------------------------------------------------------------------------------------ sampling

def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax_rows takes float32 [rows, vocab] logits")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    lib = sampling()
    _run(lib, lib.mb_argmax_rows(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(out), _stream()))
    return out


def sample_max_sorted() -> int:
    return int(sampling().mb_sample_max_sorted())


def sample_rows(logits: torch.Tensor, work: torch.Tensor, counts: Optional[torch.Tensor], temperature: torch.Tensor,
                top_k: torch.Tensor, top_p: torch.Tensor, penalty: torch.Tensor, history: Optional[torch.Tensor],
                history_len: Optional[torch.Tensor], seeds: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                uniforms: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                max_candidates: int = 0, history_rows: Optional[torch.Tensor] = None, append: bool = False) -> torch.Tensor:
    """One token per row of `logits` by the sampling pipeline.  `max_candidates`: the caller's bound on
    min(top_k, vocabulary) over the rows, 0 if it has none; when every row keeps at most
    sample_max_sorted() candidates a row is spread over a cluster of blocks instead of one block.
    The earlier tokens of the rows (for the repetition penalty) are the rows of `history`, or the int32
    arrays whose device addresses `history_rows` (int64 per row, 0: none) holds; `history_len` counts
    them either way.  With `append` the kernel stores each row's new id behind its history (the arrays
    of `history_rows` need room for it)."""
    _cuda(logits, work, counts, temperature, top_k, top_p, penalty, history, history_len, seeds, counters, uniforms, history_rows)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample_rows takes float32 [rows, vocab] logits")
    rows, vocab = logits.shape
    if work.dtype != torch.float32 or work.numel() < rows * vocab:
        raise KernelError("sample_rows needs rows*vocab floats of scratch")
    if counts is not None and (counts.dtype != torch.int32 or counts.numel() < rows * vocab):
        raise KernelError("sample_rows needs rows*vocab int32 counters for the repetition penalty")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("penalty", penalty, torch.float32)):
        if t.dtype != dt or t.numel() < rows:
            raise KernelError(f"{name} must hold {rows} values of {dt}")
    _int32(history, "history")
    _int32(history_len, "history_len")
    if (history is not None or history_rows is not None) and (counts is None or history_len is None):
        raise KernelError("a token history needs its lengths and the counters scratch")
    if history_rows is not None and (history is not None or history_rows.dtype != torch.int64 or history_rows.numel() < rows):
        raise KernelError(f"history_rows must hold {rows} int64 addresses and comes instead of a history matrix")
    if append and history_rows is None:
        raise KernelError("appending needs history_rows: a row of a history matrix has no room of its own")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = sampling()
    _run(lib, lib.mb_sample_rows(_p(logits), logits.stride(0), rows, vocab, _p(work), _p(counts), _p(temperature),
                                 _p(top_k), _p(top_p), _p(penalty), _p(history),
                                 history.stride(0) if history is not None else 0, _p(history_rows), 1 if append else 0,
                                 _p(history_len), _p(seeds),
                                 _p(counters), _p(uniforms), _p(out), int(max_candidates), _stream()))
    return out
