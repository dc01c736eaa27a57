"""The decode attention entry point that allocates nothing, called through its exported C symbol.

It exists for hosts that run the kernels without this package's Python side and cannot allocate
device memory where they call it (all memory already given to an arena of their own, or a serving
loop in which cudaMalloc may not appear): its scratch is an array built into the library.  Here it
must give what the ordinary entry point gives, on two calls in a row that share that array.
This file sorts last so that a run that stops at the first failure has run everything else."""

import ctypes
import math

import pytest
import torch

from plain import plain_llama

pytestmark = pytest.mark.gpu


def plain_decode_attention(q, k_pool, v_pool, table, kv_lens, heads, kv_heads, head_dim):
    """One query token per sequence against its cached positions, by the plain whole-sequence
    attention: the query sits in the last row, and that row's output is taken."""
    page = k_pool.shape[2]
    out = torch.zeros(len(kv_lens), heads * head_dim)
    for b, total in enumerate(kv_lens):
        pos = torch.arange(total)
        pages = table[b][pos // page].long()
        k = k_pool.float()[pages, :, pos % page, :]
        v = v_pool.float()[pages, :, pos % page, :]
        q_full = torch.zeros(total, heads, head_dim)
        q_full[-1] = q[b].float().reshape(heads, head_dim)
        out[b] = plain_llama.causal_gqa_attention(q_full, k, v)[-1].reshape(-1)
    return out


def test_static_scratch_decode_matches_the_allocating_entry_point(cuda_device):
    from models_b200.kernels import ops

    heads, kv_heads, head_dim, page = 8, 2, 64, 64
    lib = ops.attention_tc(head_dim)
    lib.mb_decode_attention_static_capacity.restype = ctypes.c_size_t
    lib.mb_decode_scratch_floats.restype = ctypes.c_size_t
    capacity = lib.mb_decode_attention_static_capacity()
    assert capacity == 1 << 20

    def pointer(t):
        return ctypes.c_void_p(t.data_ptr())

    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the third call splits 2,000 positions over 16 blocks: more than a cluster holds, and few enough
    # blocks that the kernel runs with its deep page ring
    for call, (kv_lens, splits, seed) in enumerate((([300, 1, 65, 128], 4, 1), ([17, 200, 64], 7, 2), ([2000, 1100], 16, 3))):
        g = torch.Generator().manual_seed(seed)
        sequences = len(kv_lens)
        pages_needed = [-(-n // page) for n in kv_lens]
        total_pages = sum(pages_needed) + 1
        k_pool = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).bfloat16().cuda()
        v_pool = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).bfloat16().cuda()
        table = torch.zeros(sequences, max(pages_needed), dtype=torch.int32)
        order = torch.randperm(total_pages - 1, generator=g) + 1
        at = 0
        for b, n in enumerate(pages_needed):
            table[b, :n] = order[at:at + n].int()
            at += n
        host_table, host_k, host_v = table, k_pool.cpu(), v_pool.cpu()
        table = table.cuda()
        q = torch.randn(sequences, heads * head_dim, generator=g).bfloat16().cuda()
        cu_q = torch.arange(sequences + 1, dtype=torch.int32).cuda()
        lens = torch.tensor(kv_lens, dtype=torch.int32).cuda()
        scale = 1.0 / math.sqrt(head_dim)

        expected = torch.zeros(sequences, heads * head_dim, dtype=torch.bfloat16, device="cuda")
        ops.decode_attention(q, expected, k_pool, v_pool, table, cu_q, lens, heads, kv_heads, head_dim, None, scale, splits)

        got = torch.zeros_like(expected)
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)  # allocations the framework ever made
        free_before = torch.cuda.mem_get_info()[0]  # the driver's count: an allocation by anyone in this process lowers it
        status = lib.mb_decode_attention_static(
            pointer(q), q.stride(0), pointer(got), got.stride(0), pointer(k_pool), pointer(v_pool), pointer(table),
            table.shape[1], pointer(cu_q), pointer(lens), sequences, heads, kv_heads, page, 0, ctypes.c_float(scale), splits,
            stream)
        assert status == 0, lib.mb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before
        assert torch.cuda.mem_get_info()[0] >= free_before
        worst = float((got.float() - expected.float()).abs().max())
        assert worst <= 1e-2 * float(expected.float().abs().max()), (call, worst)
        plain = plain_decode_attention(q.cpu(), host_k, host_v, host_table, kv_lens, heads, kv_heads, head_dim)
        worst = float((got.float().cpu() - plain).abs().max())
        assert worst <= 1e-2 * float(plain.abs().max()), ("against the plain attention", call, worst)

    # a request beyond the built-in array is refused with a message, and nothing runs
    too_many = 4096
    assert lib.mb_decode_scratch_floats(too_many, heads, 16) > capacity
    status = lib.mb_decode_attention_static(
        pointer(q), q.stride(0), pointer(got), got.stride(0), pointer(k_pool), pointer(v_pool), pointer(table), table.shape[1],
        pointer(cu_q), pointer(lens), too_many, heads, kv_heads, page, 0, ctypes.c_float(scale), 16, stream)
    assert status != 0 and "built-in" in lib.mb_last_error().decode()
