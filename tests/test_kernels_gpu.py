"""Each kernel alone against a plain float32 reference of the same operation, at sizes that are
not the engine's: widths and vocabularies that are no power of two, head sizes in steps of 16,
odd numbers of heads and groups, rows that do not fill a tile."""

import math

import numpy as np
import pytest
import torch

from plain import plain_llama

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 1e-2


def close(actual, expected, dtype, scale=None):
    actual, expected = actual.double().cpu(), expected.double().cpu()
    bound = tol(dtype) * (scale if scale is not None else float(expected.abs().max().clamp_min(1e-30)))
    worst = float((actual - expected).abs().max())
    assert worst <= bound, f"max abs error {worst} > {bound}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(cuda_device, dtype):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(0)
    table = torch.randn(203, 72, generator=g).to(dtype)
    tokens = torch.tensor([0, 202, 5, 5, 17], dtype=torch.int32)
    out = ops.embed_gather(table.cuda(), tokens.cuda(), scale=1.5)
    assert out.dtype == torch.float32
    close(out, table.float()[tokens.long()] * 1.5, torch.float32)


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("width,count", [(72, 7), (2048, 7), (5000, 7), (72, 300), (264, 300), (1028, 261), (2048, 300),
                                         (3080, 259), (4096, 257), (5000, 260)])
def test_add_rmsnorm(cuda_device, out_dtype, width, count):
    """Few rows: a block per row; from 256 rows on, a warp per row (widths up to 4,096)."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(1)
    x = torch.randn(count, width, generator=g) * 3
    delta = (torch.randn(count, width, generator=g)).to(out_dtype)
    weight = 1 + 0.1 * torch.randn(width, generator=g)
    eps = 3e-6
    xd = x.cuda()
    out = ops.add_rmsnorm(xd, delta.cuda(), weight.cuda(), eps, out_dtype)
    summed = x + delta.float()
    close(xd, summed, torch.float32)
    close(out, plain_llama.rms_norm(summed, weight, eps), out_dtype)
    # without a delta, on chosen rows, x untouched
    rows = torch.tensor([6, 0, 3], dtype=torch.int32) if count < 256 else torch.randperm(count, generator=g)[:257].int()
    before = xd.clone()
    out = ops.add_rmsnorm(xd, None, weight.cuda(), eps, out_dtype, rows=rows.cuda())
    assert torch.equal(before, xd)
    close(out, plain_llama.rms_norm(summed[rows.long()], weight, eps), out_dtype)
    # a delta on chosen rows is added for the norm only
    out = ops.add_rmsnorm(xd, delta.cuda(), weight.cuda(), eps, out_dtype, rows=rows.cuda())
    assert torch.equal(before, xd)
    close(out, plain_llama.rms_norm((summed + delta.float())[rows.long()], weight, eps), out_dtype)


@pytest.mark.parametrize("m,n,k", [(1, 72, 40), (5, 203, 136), (70, 130, 97), (130, 64, 256)])
def test_gemm_f32(cuda_device, m, n, k):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(2)
    a, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    expected = (a.double() @ w.double().t())
    for invariant in (True, False):
        out = ops.gemm_f32(a.cuda(), w.cuda(), row_invariant=invariant)
        close(out, expected, torch.float32, scale=float(expected.abs().max()) * 4)
    # a row's result does not depend on the other rows of the call
    alone = ops.gemm_f32(a[:1].cuda(), w.cuda(), row_invariant=True)
    together = ops.gemm_f32(a.cuda(), w.cuda(), row_invariant=True)
    assert torch.equal(alone[0], together[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_bias(cuda_device, dtype):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(3)
    gate_up = (torch.randn(5, 2 * 136, generator=g) * 4).to(dtype)
    out = ops.swiglu(gate_up.cuda())
    f = gate_up.float()
    close(out, plain_llama.swiglu(f[:, :136], f[:, 136:]), dtype)
    x = torch.randn(5, 203, generator=g).to(dtype)
    bias = torch.randn(203, generator=g)
    got = ops.bias_add(x.cuda().clone(), bias.cuda())
    close(got, x.float() + bias, dtype)


def _pools(pages, kv_heads, page_size, head_dim, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    k = (torch.randn(pages, kv_heads, page_size, head_dim, generator=g)).to(dtype)
    v = (torch.randn(pages, kv_heads, page_size, head_dim, generator=g)).to(dtype)
    return k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("head_dim,rotary_dim", [(16, 16), (48, 48), (64, 32)])
def test_rope_cache_write(cuda_device, dtype, pairing, head_dim, rotary_dim):
    from models_b200.kernels import ops

    heads, kv_heads, page = 3, 2, 64
    tokens = 9
    g = torch.Generator().manual_seed(4)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(tokens, width + 8, generator=g).to(dtype)  # wider rows: the stride is honoured
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 130, 7, 8], dtype=torch.int32)
    freqs = plain_llama.rope_pair_frequencies(rotary_dim, 12345.0)
    cos, sin = plain_llama.rope_cos_sin(torch.arange(200), freqs, None)
    pages = 5
    k_pool, v_pool = _pools(pages, kv_heads, page, head_dim, dtype, 5)
    slot_mapping = torch.tensor([64 * 1 + 0, 64 * 1 + 1, 64 * 1 + 2, 64 * 1 + 63, 64 * 3 + 0, 64 * 3 + 1, 64 * 4 + 2, -1,
                                 64 * 2 + 8], dtype=torch.int32)
    qkv_d, k_d, v_d = qkv.cuda(), k_pool.cuda(), v_pool.cuda()
    view = qkv_d[:, :width]
    ops.rope_cache_write(view, positions.cuda(), cos.cuda(), sin.cuda(), k_d, v_d, slot_mapping.cuda(), heads, kv_heads,
                         head_dim, rotary_dim, pairing == "interleaved", page, True)

    def rotate(x, pos):  # x [T, h, hd] float
        c, s = cos[pos.long()], sin[pos.long()]
        if pairing == "half":
            return plain_llama.rope_rotate_split_half(x, c, s)
        pairs = rotary_dim // 2
        x0, x1 = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        r0, r1 = x0 * c[:, None, :] - x1 * s[:, None, :], x0 * s[:, None, :] + x1 * c[:, None, :]
        out = x.clone()
        out[..., 0:rotary_dim:2], out[..., 1:rotary_dim:2] = r0, r1
        return out

    f = qkv.float()[:, :width]
    q = f[:, : heads * head_dim].reshape(tokens, heads, head_dim)
    k = f[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    v = f[:, (heads + kv_heads) * head_dim:].reshape(tokens, kv_heads, head_dim)
    close(qkv_d[:, : heads * head_dim], rotate(q, positions).reshape(tokens, -1), dtype)
    assert torch.equal(qkv_d[:, width:].cpu(), qkv[:, width:])  # columns beyond the heads are untouched
    ek, ev = k_pool.float().clone(), v_pool.float().clone()
    rk = rotate(k, positions)
    for t in range(tokens):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        ek[s // page, :, s % page, :] = rk[t]
        ev[s // page, :, s % page, :] = v[t]
    close(k_d, ek, dtype)
    close(v_d, ev, dtype)


def _reference_attention(q, k_pool, v_pool, block_table, q_lens, kv_lens, heads, kv_heads, head_dim, window, scale):
    """q [T, heads*hd] float; whole-sequence plain attention per sequence, keys gathered from the pages."""
    page = k_pool.shape[2]
    out = torch.zeros(q.shape[0], heads * head_dim)
    row = 0
    for b, (n, total) in enumerate(zip(q_lens, kv_lens)):
        pos = torch.arange(total)
        pages = block_table[b][pos // page].long()
        k = k_pool.float()[pages, :, pos % page, :]  # [total, kv, hd]
        v = v_pool.float()[pages, :, pos % page, :]
        qfull = torch.zeros(total, heads, head_dim)
        qfull[total - n:] = q[row:row + n].reshape(n, heads, head_dim)
        full = plain_llama.causal_gqa_attention(qfull * (scale * math.sqrt(head_dim)), k, v, window)
        out[row:row + n] = full[total - n:]
        row += n
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (3, 1, 32, None), (6, 3, 48, None),
                                                            (8, 2, 128, None), (5, 5, 80, 37), (4, 1, 64, 64)])
def test_paged_attention_rows(cuda_device, dtype, heads, kv_heads, head_dim, window):
    from models_b200.kernels import ops

    page = 64
    q_lens = [1, 70, 5, 1]
    kv_lens = [1, 70, 133, 200]
    pages_needed = [-(-n // page) for n in kv_lens]
    total_pages = sum(pages_needed) + 1
    k_pool, v_pool = _pools(total_pages, kv_heads, page, head_dim, dtype, 6)
    order = torch.randperm(total_pages - 1, generator=torch.Generator().manual_seed(7)) + 1
    block_table = torch.zeros(len(q_lens), max(pages_needed), dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_needed):
        block_table[b, :n] = order[at:at + n].int()
        at += n
    T = sum(q_lens)
    g = torch.Generator().manual_seed(8)
    q = torch.randn(T, heads * head_dim + 16, generator=g).to(dtype)
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    out = torch.zeros(T, heads * head_dim, dtype=dtype, device="cuda")
    scale = 0.7 / math.sqrt(head_dim)
    ops.paged_attention_rows(q.cuda()[:, : heads * head_dim], out, k_pool.cuda(), v_pool.cuda(), block_table.cuda(),
                             cu_q.cuda(), torch.tensor(kv_lens, dtype=torch.int32).cuda(), max(q_lens), heads, kv_heads,
                             head_dim, window, scale)
    expected = _reference_attention(q.float()[:, : heads * head_dim], k_pool, v_pool, block_table, q_lens, kv_lens, heads,
                                    kv_heads, head_dim, window, scale)
    close(out, expected, dtype)


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (3, 1, 32, None), (6, 3, 48, None),
                                                            (32, 8, 64, None), (8, 2, 128, None), (5, 5, 80, 37),
                                                            (4, 1, 64, 64), (40, 2, 64, None), (2, 1, 256, 100)])
def test_tensor_core_attention(cuda_device, heads, kv_heads, head_dim, window):
    """Prefill (unequal new-token counts on top of unequal cached lengths) and decode (one token each,
    with 1, 3 and 16 splits of the keys) against the plain attention."""
    from models_b200.kernels import ops

    dtype, page = torch.bfloat16, 64
    for q_lens, kv_lens in (([1, 70, 5, 64, 130], [1, 70, 133, 200, 130]), ([1, 1, 1, 1], [1, 64, 65, 300])):
        pages_needed = [-(-n // page) for n in kv_lens]
        total_pages = sum(pages_needed) + 1
        k_pool, v_pool = _pools(total_pages, kv_heads, page, head_dim, dtype, 6)
        order = torch.randperm(total_pages - 1, generator=torch.Generator().manual_seed(7)) + 1
        block_table = torch.zeros(len(q_lens), max(pages_needed) + 2, dtype=torch.int32)
        at = 0
        for b, n in enumerate(pages_needed):
            block_table[b, :n] = order[at:at + n].int()
            at += n
        T = sum(q_lens)
        q = torch.randn(T, heads * head_dim + 16, generator=torch.Generator().manual_seed(8)).to(dtype)
        cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
        scale = 0.7 / math.sqrt(head_dim)
        expected = _reference_attention(q.float()[:, : heads * head_dim], k_pool, v_pool, block_table, q_lens, kv_lens,
                                        heads, kv_heads, head_dim, window, scale)
        common = (k_pool.cuda(), v_pool.cuda(), block_table.cuda(), cu_q.cuda(), torch.tensor(kv_lens, dtype=torch.int32).cuda())
        qd = q.cuda()[:, : heads * head_dim]
        if max(q_lens) > 1:
            for kernel in ("mma", "tcgen05") if head_dim in (64, 128) else ("mma",):
                out = torch.zeros(T, heads * head_dim, dtype=dtype, device="cuda")
                ops.prefill_attention(qd, out, *common, max(q_lens), heads, kv_heads, head_dim, window, scale, kernel=kernel)
                close(out, expected, dtype)
        else:
            for splits, use_scratch in ((1, False), (2, False), (4, False), (8, False), (3, False), (16, False), (4, True)):
                out = torch.zeros(T, heads * head_dim, dtype=dtype, device="cuda")
                ops.decode_attention(qd, out, *common, heads, kv_heads, head_dim, window, scale, splits, use_scratch)
                close(out, expected, dtype)


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(8, 2, 64, None), (3, 3, 128, None), (4, 1, 64, 100),
                                                            (2, 1, 128, 257), (12, 4, 64, 64)])
def test_tcgen05_prefill_attention(cuda_device, heads, kv_heads, head_dim, window):
    """The tcgen05 kernel alone at sizes that turn its rings over several times: many pages per
    block, several 128-row blocks per sequence, new tokens on top of cached ones, a sequence of one
    token beside long ones, pages scattered over the pool."""
    from models_b200.kernels import ops

    dtype, page = torch.bfloat16, 64
    q_lens = [300, 1, 129, 700, 64, 128]
    kv_lens = [300, 50, 500, 700, 449, 128]
    pages_needed = [-(-n // page) for n in kv_lens]
    total_pages = sum(pages_needed) + 3
    k_pool, v_pool = _pools(total_pages, kv_heads, page, head_dim, dtype, 16)
    order = torch.randperm(total_pages - 1, generator=torch.Generator().manual_seed(17)) + 1
    block_table = torch.zeros(len(q_lens), max(pages_needed) + 1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_needed):
        block_table[b, :n] = order[at:at + n].int()
        at += n
    T = sum(q_lens)
    q = torch.randn(T, heads * head_dim + 24, generator=torch.Generator().manual_seed(18)).to(dtype)
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    scale = 1.3 / math.sqrt(head_dim)
    expected = _reference_attention(q.float()[:, : heads * head_dim], k_pool, v_pool, block_table, q_lens, kv_lens,
                                    heads, kv_heads, head_dim, window, scale)
    out = torch.full((T, heads * head_dim), 7.0, dtype=dtype, device="cuda")
    ops.prefill_attention(q.cuda()[:, : heads * head_dim], out, k_pool.cuda(), v_pool.cuda(), block_table.cuda(), cu_q.cuda(),
                          torch.tensor(kv_lens, dtype=torch.int32).cuda(), max(q_lens), heads, kv_heads, head_dim, window,
                          scale, kernel="tcgen05")
    torch.cuda.synchronize()
    assert ops.prefill_attention_tcgen05_status(head_dim) == 0
    close(out, expected, dtype)


@pytest.mark.parametrize("head_dim", [64, 128])
def test_tcgen05_prefill_attention_finds_one_far_key(cuda_device, head_dim):
    """One key among 600 stands out.  Every query row at or after it must return that key's value
    row; every row before it sees equal scores and must return the mean of the values it can see."""
    from models_b200.kernels import ops

    heads, kv_heads, page, total, new = 2, 1, 64, 600, 250
    for far in (0, 349, 350, 383, 384, 511, 599):
        k_pool = torch.zeros(11, kv_heads, page, head_dim)
        v_pool = torch.randn(11, kv_heads, page, head_dim, generator=torch.Generator().manual_seed(far))
        table = torch.tensor([[5, 2, 10, 1, 3, 9, 7, 4, 8, 6]], dtype=torch.int32)
        k_pool[table[0, far // page], 0, far % page, :] = 10.0
        q = torch.ones(new, heads * head_dim).bfloat16()
        out = torch.zeros(new, heads * head_dim, device="cuda", dtype=torch.bfloat16)
        ops.prefill_attention(q.cuda(), out, k_pool.bfloat16().cuda(), v_pool.bfloat16().cuda(), table.cuda(),
                              torch.tensor([0, new], dtype=torch.int32).cuda(), torch.tensor([total], dtype=torch.int32).cuda(),
                              new, heads, kv_heads, head_dim, None, 1.0, kernel="tcgen05")
        values = v_pool.bfloat16().float()
        flat = torch.stack([values[table[0, p // page], 0, p % page, :] for p in range(total)])  # [total, hd]
        for row in range(new):
            pos = total - new + row
            want = flat[far] if pos >= far else flat[: pos + 1].mean(dim=0)
            for h in range(heads):
                got = out[row, h * head_dim:(h + 1) * head_dim].float().cpu()
                assert torch.allclose(got, want, atol=2e-2), (far, row, h, float((got - want).abs().max()))


def test_window_edge_and_stale_pages_do_not_leak(cuda_device):
    """The key just outside the window, the positions beyond a sequence's length in its last page, and
    a page that belongs to nobody are all made to attract the query; none may be seen."""
    from models_b200.kernels import ops

    heads, kv_heads, head_dim, page, window = 4, 1, 64, 64, 50
    kv_len = 150
    loud = 30.0
    k_pool = torch.zeros(5, kv_heads, page, head_dim)
    v_pool = torch.zeros(5, kv_heads, page, head_dim)
    k_pool[:] = loud  # every key attracts ...
    v_pool[:] = 1000.0  # ... and would wreck the output
    table = torch.tensor([[2, 4, 1, 0]], dtype=torch.int32)
    first = kv_len - window  # the decode query sits at 149 and sees 100..149
    for p in range(first, kv_len):  # the visible keys are quiet and carry the value 1
        k_pool[table[0, p // page], 0, p % page, :] = 0.0
        v_pool[table[0, p // page], 0, p % page, :] = 1.0
    q = torch.ones(1, heads * head_dim)
    for dtype in (torch.bfloat16, torch.float32):
        args = (k_pool.to(dtype).cuda(), v_pool.to(dtype).cuda(), table.cuda(), torch.tensor([0, 1], dtype=torch.int32).cuda(),
                torch.tensor([kv_len], dtype=torch.int32).cuda())
        out = torch.zeros(1, heads * head_dim, dtype=dtype, device="cuda")
        ops.paged_attention_rows(q.to(dtype).cuda(), out, *args, 1, heads, kv_heads, head_dim, window, 1.0)
        assert torch.allclose(out.float().cpu(), torch.ones(1, heads * head_dim)), dtype
        if dtype == torch.bfloat16:
            for splits in (1, 2, 4):
                out = torch.zeros(1, heads * head_dim, dtype=dtype, device="cuda")
                ops.decode_attention(q.to(dtype).cuda(), out, *args, heads, kv_heads, head_dim, window, 1.0, splits)
                assert torch.allclose(out.float().cpu(), torch.ones(1, heads * head_dim)), splits
            # prefill of the last 3 tokens: each sees its own 50 positions; make 97..99 quiet for them
            for p in range(first - 2, first):
                k_pool[table[0, p // page], 0, p % page, :] = 0.0
                v_pool[table[0, p // page], 0, p % page, :] = 1.0
            args = (k_pool.to(dtype).cuda(), v_pool.to(dtype).cuda()) + args[2:3] + (
                torch.tensor([0, 3], dtype=torch.int32).cuda(), args[4])
            out = torch.zeros(3, heads * head_dim, dtype=dtype, device="cuda")
            ops.prefill_attention(q.to(dtype).cuda().expand(3, -1).contiguous(), out, *args, 3, heads, kv_heads, head_dim,
                                  window, 1.0)
            assert torch.allclose(out.float().cpu(), torch.ones(3, heads * head_dim))


def test_attention_finds_one_far_key(cuda_device):
    """One key among hundreds is made to stand out; the output must be that key's value row."""
    from models_b200.kernels import ops

    heads, kv_heads, head_dim, page = 2, 1, 32, 64
    total = 300
    for far in (0, 63, 64, 191, 299):
        k_pool = torch.zeros(6, kv_heads, page, head_dim)
        v_pool = torch.randn(6, kv_heads, page, head_dim, generator=torch.Generator().manual_seed(far))
        table = torch.tensor([[5, 2, 4, 1, 3]], dtype=torch.int32)
        k_pool[table[0, far // page], 0, far % page, :] = 10.0
        q = torch.ones(1, heads * head_dim)
        out = torch.zeros(1, heads * head_dim, device="cuda")
        ops.paged_attention_rows(q.cuda(), out, k_pool.cuda(), v_pool.cuda(), table.cuda(),
                                 torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                 torch.tensor([total], dtype=torch.int32).cuda(), 1, heads, kv_heads, head_dim, None, 1.0)
        expected = v_pool[table[0, far // page], 0, far % page, :]
        for h in range(heads):
            assert torch.allclose(out[0, h * head_dim:(h + 1) * head_dim].cpu(), expected, atol=1e-5), far
        for splits in (1, 5):
            out16 = torch.zeros(1, heads * head_dim, device="cuda", dtype=torch.bfloat16)
            ops.decode_attention(q.bfloat16().cuda(), out16, k_pool.bfloat16().cuda(), v_pool.bfloat16().cuda(), table.cuda(),
                                 torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                 torch.tensor([total], dtype=torch.int32).cuda(), heads, kv_heads, head_dim, None, 1.0, splits)
            for h in range(heads):
                assert torch.allclose(out16[0, h * head_dim:(h + 1) * head_dim].float().cpu(), expected.bfloat16().float(),
                                      atol=1e-2), (far, splits)


def test_decode_attention_finds_one_far_key_in_a_long_context(cuda_device):
    """5,000 cached positions split over 16 to 64 blocks (partial results through scratch memory): the one
    key that stands out may lie in any split, also the first and the last, and in a split's last page."""
    from models_b200.kernels import ops

    heads, kv_heads, head_dim, page = 8, 2, 64, 64
    total = 5000
    pages = -(-total // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(3)).to(torch.int32) + 1
    table = order.reshape(1, pages)
    for far in (0, 63, 2047, 2048, 3333, 4992, 4999):
        k_pool = torch.zeros(pages + 1, kv_heads, page, head_dim)
        v_pool = torch.randn(pages + 1, kv_heads, page, head_dim, generator=torch.Generator().manual_seed(far))
        k_pool[table[0, far // page], :, far % page, :] = 4.0
        q = torch.ones(1, heads * head_dim)
        for splits in (16, 32, 64):
            assert ops.decode_splits(1, heads, kv_heads, head_dim, total) > 8  # what the engine would choose is of this kind
            out = torch.zeros(1, heads * head_dim, device="cuda", dtype=torch.bfloat16)
            ops.decode_attention(q.bfloat16().cuda(), out, k_pool.bfloat16().cuda(), v_pool.bfloat16().cuda(), table.cuda(),
                                 torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                 torch.tensor([total], dtype=torch.int32).cuda(), heads, kv_heads, head_dim, None, 1.0, splits)
            for h in range(heads):
                expected = v_pool[table[0, far // page], h // (heads // kv_heads), far % page, :]
                assert torch.allclose(out[0, h * head_dim:(h + 1) * head_dim].float().cpu(), expected.bfloat16().float(),
                                      atol=1e-2), (far, splits, h)


def test_decode_splits_follow_the_context_class(cuda_device):
    """Short contexts: the split depends on the batch size alone and stays within a cluster.  Long ones:
    more blocks for few sequences, the same count for every length of a class."""
    from models_b200.kernels import ops

    short = ops.decode_splits(1, 32, 8, 64)
    assert short <= 8 and short == ops.decode_splits(1, 32, 8, 64, 1) == ops.decode_splits(1, 32, 8, 64, ops.LONG_KEYS)
    assert ops.decode_span(ops.LONG_KEYS) == 0 and ops.decode_span(ops.LONG_KEYS + 1) == 2 * ops.LONG_KEYS
    assert ops.decode_span(5000) == 8192 and ops.decode_span(8192) == 8192
    for keys in (4097, 5000, 8192):
        assert ops.decode_splits(1, 32, 8, 64, keys) == ops.decode_splits(1, 32, 8, 64, 8192) > 8
    assert ops.decode_splits(1, 32, 8, 64, 32768) == 32
    assert ops.decode_splits(8, 32, 8, 64, 65536) == 32  # 2,048 blocks at most
    assert ops.decode_splits(64, 32, 8, 64, 16384) <= 8
    assert ops.decode_splits(1, 32, 8, 64, 32768, window=512) == short  # a window's few pages need no more blocks


def test_argmax_first_maximum(cuda_device):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(9)
    logits = torch.randn(5, 5003, generator=g)
    logits[1, 4000] = logits[1, 77] = 50.0  # a tie: the lower id wins
    logits[2, 0] = 60.0
    logits[3, 5002] = 60.0
    got = ops.argmax_rows(logits.cuda()).cpu().tolist()
    assert got == [plain_llama.plain_argmax(row) for row in logits]
    assert got[1] == 77


@pytest.mark.parametrize("batch", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(48, 64), (203, 136), (3072, 2048), (130, 8192)])
def test_skinny_gemm_all_prologues_and_epilogues(cuda_device, batch, n, k):
    """The decode matrix product against float64: plain, with the folded RMSNorm (and a row gather),
    with the residual add, and with the gated activation, at widths that do not fill its tiles."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(batch * 1000 + n)
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    x = torch.randn(batch, k, generator=g).bfloat16()
    wd, xd = w.cuda(), x.cuda()
    exact = x.double() @ w.double().t()
    scale = float(exact.abs().max())
    out = ops.skinny_gemm(wd, ops.EPI_F32, x=xd)
    assert float((out.double().cpu() - exact).abs().max()) < 2e-5 * scale * math.sqrt(k)
    out = ops.skinny_gemm(wd, ops.EPI_BF16, x=xd)
    assert out.dtype == torch.bfloat16 and float((out.double().cpu() - exact).abs().max()) < 1e-2 * scale
    residual = torch.randn(batch, n, generator=g)
    rd = residual.cuda()
    ops.skinny_gemm(wd, ops.EPI_RESIDUAL, x=xd, out=rd)
    assert float((rd.double().cpu() - (residual.double() + exact)).abs().max()) < 2e-5 * (scale + 4) * math.sqrt(k)
    if n % 2 == 0:
        gated = ops.skinny_gemm(wd, ops.EPI_SWIGLU, x=xd)
        want = plain_llama.swiglu(exact[:, : n // 2], exact[:, n // 2:])
        assert gated.shape == (batch, n // 2)
        assert float((gated.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
    if batch <= 16:
        rows_total = batch + 3
        xf = torch.randn(rows_total, k, generator=g) * 2
        gain = 1 + 0.1 * torch.randn(k, generator=g)
        pick = torch.randperm(rows_total, generator=g)[:batch].int()
        eps = 1e-5
        normed = plain_llama.rms_norm(xf.double(), gain.double(), eps)[pick.long()]
        want = normed @ w.double().t()
        got = ops.skinny_gemm(wd, ops.EPI_F32, xf=xf.cuda(), gain=gain.cuda(), eps=eps, rows=pick.cuda())
        # the normalised rows are rounded to bfloat16 before the product
        assert float((got.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
        if n % 2 == 0:
            got = ops.skinny_gemm(wd, ops.EPI_SWIGLU, xf=xf.cuda()[:batch].contiguous(), gain=gain.cuda(), eps=eps)
            full = plain_llama.rms_norm(xf.double()[:batch], gain.double(), eps) @ w.double().t()
            want = plain_llama.swiglu(full[:, : n // 2], full[:, n // 2:])
            assert float((got.double().cpu() - want).abs().max()) < 2e-2 * float(want.abs().max())
    else:
        with pytest.raises(ops.KernelError):
            ops.skinny_gemm(wd, ops.EPI_F32, xf=x.float().cuda(), gain=torch.ones(k).cuda(), eps=1e-5)
    with pytest.raises(ops.KernelError):
        ops.skinny_gemm(wd, ops.EPI_F32, x=torch.zeros(33, k, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("batch", [1, 5, 16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,hidden", [(4, 2, 16, 64), (3, 1, 32, 96), (32, 8, 64, 2048), (6, 3, 48, 72)])
@pytest.mark.parametrize("prepared", [False, True])
def test_skinny_qkv_with_norm_rotation_and_cache_write(cuda_device, batch, heads, kv_heads, head_dim, hidden, prepared):
    """The folded decode kernel (norm, q/k/v product, rotation, cache write) against the plain parts.
    `prepared`: the rows arrive as x times the gain in bfloat16 with parts of their sums of squares (as the
    product before leaves them) instead of as float32 rows that the kernel normalises itself."""
    from models_b200.kernels import ops

    page = 64
    g = torch.Generator().manual_seed(batch + head_dim)
    n = (heads + 2 * kv_heads) * head_dim
    w = (torch.randn(n, hidden, generator=g) * 0.05).bfloat16()
    xf = torch.randn(batch, hidden, generator=g) * 2
    gain = 1 + 0.1 * torch.randn(hidden, generator=g)
    eps = 1e-5
    positions = torch.randint(0, 300, (batch,), generator=g).int()
    cos, sin = plain_llama.rope_cos_sin(torch.arange(300), plain_llama.rope_pair_frequencies(head_dim, 50000.0), None)
    pages = batch + 2
    k_pool, v_pool = _pools(pages, kv_heads, page, head_dim, torch.bfloat16, 3)
    slots = (torch.randperm(pages - 1, generator=g)[:batch] + 1) * page + torch.randint(0, page, (batch,), generator=g)
    slots = slots.int()
    if batch > 1:
        slots[1] = -1  # a padding row stores nothing
    kd, vd = k_pool.cuda(), v_pool.cuda()
    if prepared:
        squares = (xf.double() ** 2).sum(1)
        share = torch.rand(5, batch, generator=g).double()
        ssq = torch.zeros(7, ops.SSQ_COLUMNS)  # five parts that add up to the rows' sums of squares, two that do not count
        ssq[:5, :batch] = (share / share.sum(0) * squares).float()
        ssq[5:] = 1e6
        q = ops.skinny_qkv_rope(w.cuda(), None, None, 0.0, heads, kv_heads, head_dim, positions.cuda(), cos.cuda(), sin.cuda(),
                                kd, vd, slots.cuda(), x=(xf * gain).bfloat16().cuda(), norm_parts=(ssq.cuda(), 5, hidden, eps))
    else:
        q = ops.skinny_qkv_rope(w.cuda(), xf.cuda(), gain.cuda(), eps, heads, kv_heads, head_dim, positions.cuda(), cos.cuda(),
                                sin.cuda(), kd, vd, slots.cuda())
    qkv = plain_llama.rms_norm(xf, gain, eps) @ w.float().t()
    c, s_ = cos[positions.long()], sin[positions.long()]
    want_q = plain_llama.rope_rotate_split_half(qkv[:, : heads * head_dim].reshape(batch, heads, head_dim), c, s_)
    want_k = plain_llama.rope_rotate_split_half(
        qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(batch, kv_heads, head_dim), c, s_)
    want_v = qkv[:, (heads + kv_heads) * head_dim:].reshape(batch, kv_heads, head_dim)
    scale = float(qkv.abs().max())
    assert float((q.float().cpu() - want_q.reshape(batch, -1)).abs().max()) < 2e-2 * scale
    ek, ev = k_pool.float().clone(), v_pool.float().clone()
    for b in range(batch):
        slot = int(slots[b])
        if slot >= 0:
            ek[slot // page, :, slot % page, :] = want_k[b]
            ev[slot // page, :, slot % page, :] = want_v[b]
    assert float((kd.float().cpu() - ek).abs().max()) < 2e-2 * max(scale, 4.0)
    assert float((vd.float().cpu() - ev).abs().max()) < 2e-2 * max(scale, 4.0)
    untouched = torch.ones(pages, dtype=torch.bool)
    untouched[[int(x) // page for x in slots if x >= 0]] = False
    assert torch.equal(kd.cpu()[untouched], k_pool[untouched])  # pages of other sequences are left alone


@pytest.mark.parametrize("rows,heads,kv_heads,head_dim,hidden", [(129, 8, 2, 64, 512), (300, 3, 3, 128, 264), (700, 5, 1, 64, 328),
                                                               (257, 2, 2, 128, 1024), (1500, 28, 4, 64, 136)])
def test_tcgen05_qkv_product_with_rotation_and_cache_write(cuda_device, rows, heads, kv_heads, head_dim, hidden):
    """The prefill q/k/v product with rotation and paged cache write in its epilogue against the plain
    parts: head counts that leave the last tile partly empty, rows that do not fill the last row tile,
    padding rows that must store nothing, positions scattered over the table."""
    from models_b200.kernels import ops

    page = 64
    g = torch.Generator().manual_seed(rows + head_dim)
    n = (heads + 2 * kv_heads) * head_dim
    w = (torch.randn(n, hidden, generator=g) * 0.05).bfloat16()
    a = torch.randn(rows, hidden, generator=g).bfloat16()
    positions = torch.randint(0, 900, (rows,), generator=g).int()
    cos, sin = plain_llama.rope_cos_sin(torch.arange(900), plain_llama.rope_pair_frequencies(head_dim, 50000.0), None)
    pages = -(-rows // page) + 3
    k_pool, v_pool = _pools(pages, kv_heads, page, head_dim, torch.bfloat16, 3)
    slots = (torch.randperm((pages - 1) * page, generator=g)[:rows] + page).int()  # distinct cache positions, none in page 0
    slots[1] = -1  # padding rows store nothing
    slots[rows - 1] = -1
    kd, vd = k_pool.cuda(), v_pool.cuda()
    q = ops.gemm_tcgen05_qkv_rope(a.cuda(), w.cuda(), heads, kv_heads, head_dim, positions.cuda(), cos.cuda(), sin.cuda(), kd, vd,
                                  slots.cuda())
    torch.cuda.synchronize()
    assert ops.gemm_tcgen05_status() == 0
    qkv = (a.float() @ w.float().t()).bfloat16().float()  # the product passes through bfloat16 before the rotation
    c, s_ = cos[positions.long()], sin[positions.long()]
    want_q = plain_llama.rope_rotate_split_half(qkv[:, : heads * head_dim].reshape(rows, heads, head_dim), c, s_)
    want_k = plain_llama.rope_rotate_split_half(
        qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(rows, kv_heads, head_dim), c, s_)
    want_v = qkv[:, (heads + kv_heads) * head_dim:].reshape(rows, kv_heads, head_dim)
    scale = float(qkv.abs().max())
    assert q.shape == (rows, heads * head_dim)
    assert float((q.float().cpu() - want_q.reshape(rows, -1)).abs().max()) < 1.5e-2 * scale
    ek, ev = k_pool.float().clone(), v_pool.float().clone()
    for b in range(rows):
        slot = int(slots[b])
        if slot >= 0:
            ek[slot // page, :, slot % page, :] = want_k[b]
            ev[slot // page, :, slot % page, :] = want_v[b]
    assert float((kd.float().cpu() - ek).abs().max()) < 1.5e-2 * max(scale, 4.0)
    assert float((vd.float().cpu() - ev).abs().max()) < 1.5e-2 * max(scale, 4.0)
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[slots[slots >= 0].long()] = True
    untouched = ~written.reshape(pages, page)
    assert torch.equal(kd.cpu().permute(0, 2, 1, 3)[untouched], k_pool.permute(0, 2, 1, 3)[untouched])  # nothing else was stored
    assert torch.equal(vd.cpu().permute(0, 2, 1, 3)[untouched], v_pool.permute(0, 2, 1, 3)[untouched])
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05_qkv_rope(a.cuda(), w.cuda(), heads, kv_heads, 48, positions.cuda(), cos.cuda(), sin.cuda(), kd, vd, slots.cuda())


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (70, 144, 136), (300, 272, 200), (1, 512, 2048), (513, 1040, 328),
                                   (2100, 5136, 264), (200, 528, 4136), (520, 272, 1288)])
def test_tcgen05_gemm_all_epilogues(cuda_device, m, n, k):
    """The prefill matrix product (TMA, tcgen05.mma, accumulator in tensor memory) against float64,
    at sizes that do not fill its 128 x 256 x 64 tiles; no bounded wait may have given up.  With few
    tiles and a long K the residual epilogue splits K over blocks (the last part shorter than the rest)."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    exact = a.double() @ w.double().t()
    scale = float(exact.abs().max())
    # the launcher's choice; both tile widths of single blocks by name; pairs of blocks (cta_group::2)
    for tile_width, pair in ((0, 0), (128, 1), (256, 1), (0, 2)):
        out = ops.gemm_tcgen05(a.cuda(), w.cuda(), ops.EPI_F32, tile_width=tile_width, pair=pair)
        assert float((out.double().cpu() - exact).abs().max()) < 2e-5 * scale * math.sqrt(k)
        out = ops.gemm_tcgen05(a.cuda(), w.cuda(), ops.EPI_BF16, tile_width=tile_width, pair=pair)
        assert out.dtype == torch.bfloat16 and float((out.double().cpu() - exact).abs().max()) < 1e-2 * scale
        residual = torch.randn(m, n, generator=g)
        rd = residual.cuda()
        ops.gemm_tcgen05(a.cuda(), w.cuda(), ops.EPI_RESIDUAL, out=rd, tile_width=tile_width, pair=pair)
        assert float((rd.double().cpu() - (residual.double() + exact)).abs().max()) < 2e-5 * (scale + 4) * math.sqrt(k)
    with pytest.raises(ops.KernelError, match="256"):
        ops.gemm_tcgen05(a.cuda(), w.cuda(), ops.EPI_SWIGLU, tile_width=128)
    want = plain_llama.swiglu(exact[:, : n // 2], exact[:, n // 2:])
    for pair in (1, 2):
        gated = ops.gemm_tcgen05(a.cuda(), w.cuda(), ops.EPI_SWIGLU, pair=pair)
        assert gated.shape == (m, n // 2)
        assert float((gated.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
    # a strided view of wider activations is taken as it is
    wide = torch.randn(m, k + 24, generator=g).bfloat16().cuda()
    out = ops.gemm_tcgen05(wide[:, 8:8 + k], w.cuda(), ops.EPI_F32)
    want = wide[:, 8:8 + k].double().cpu() @ w.double().t()
    assert float((out.double().cpu() - want).abs().max()) < 2e-5 * float(want.abs().max()) * math.sqrt(k)
    assert ops.gemm_tcgen05_status() == 0
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05(a.cuda(), torch.zeros(n + 4, k, dtype=torch.bfloat16, device="cuda"), ops.EPI_BF16)


@pytest.mark.parametrize("batch", [9, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(144, 136), (2048, 2048), (272, 8192), (1040, 328)])
def test_wide_decode_gemm_all_epilogues(cuda_device, batch, n, k):
    """The wide decode product (weights as the 128-row tcgen05 operand, K split over the blocks of a
    cluster whose sums meet in distributed shared memory) against float64; a second call gives the
    same bits."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(batch + n + k)
    a = torch.randn(batch, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    ad, wd = a.cuda(), w.cuda()
    exact = a.double() @ w.double().t()
    scale = float(exact.abs().max())
    out = ops.wide_gemm(ad, wd, ops.EPI_F32)
    assert float((out.double().cpu() - exact).abs().max()) < 2e-5 * scale * math.sqrt(k)
    assert torch.equal(out, ops.wide_gemm(ad, wd, ops.EPI_F32))
    out = ops.wide_gemm(ad, wd, ops.EPI_BF16)
    assert out.dtype == torch.bfloat16 and float((out.double().cpu() - exact).abs().max()) < 1e-2 * scale
    residual = torch.randn(batch, n, generator=g)
    rd = residual.cuda()
    ops.wide_gemm(ad, wd, ops.EPI_RESIDUAL, out=rd)
    assert float((rd.double().cpu() - (residual.double() + exact)).abs().max()) < 2e-5 * (scale + 4) * math.sqrt(k)
    gated = ops.wide_gemm(ad, wd, ops.EPI_SWIGLU)
    want = plain_llama.swiglu(exact[:, : n // 2], exact[:, n // 2:])
    assert gated.shape == (batch, n // 2)
    assert float((gated.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("rows", [1, 5, 8, 9, 33, 64, 100, 128])
@pytest.mark.parametrize("width,inner", [(264, 520), (2048, 2048), (272, 4136), (3088, 264), (1040, 8200)])
def test_the_norm_rides_in_the_products_around_it(cuda_device, rows, width, inner):
    """x = x + h . Wd^T with the next RMSNorm half done in the same kernel (x * gain as bfloat16, and parts of
    every row's sum of squares), then a product that divides by the root mean square in its own epilogue:
    against float64 of the same steps (y = x / sqrt(mean(x^2) + eps) * gain, integrallis/models,
    backend-java/.../ops/TensorOps.java:45-58).  These are the decode products (the narrow ones up to 8 rows, the
    wide ones from 9 to 128); over more rows the norms keep kernels of their own, and the products say so."""
    from models_b200.kernels import ops

    def product(a, w, epilogue, **more):
        if rows <= ops.SKINNY_PAYS_ROWS:
            return ops.skinny_gemm(w, epilogue, x=a, **more)
        return ops.tensor_core_gemm(a, w, epilogue, **more)

    g = torch.Generator().manual_seed(rows + width + inner)
    eps = 3e-5
    h = torch.randn(rows, inner, generator=g).bfloat16()
    w_down = (torch.randn(width, inner, generator=g) * 0.05).bfloat16()
    w_next = (torch.randn(144, width, generator=g) * 0.05).bfloat16()
    gain = (1.0 + 0.2 * torch.randn(width, generator=g)).float()
    x = (3.0 * torch.randn(rows, width, generator=g)).float()
    xd = x.cuda()
    out, gained, ssq, count = product(h.cuda(), w_down.cuda(), ops.EPI_RESIDUAL, out=xd, emit_gain=gain.cuda())
    assert out is xd and gained.shape == (rows, width) and gained.dtype == torch.bfloat16
    exact_x = x.double() + h.double() @ w_down.double().t()
    scale = float(exact_x.abs().max())
    assert float((xd.double().cpu() - exact_x).abs().max()) < 2e-5 * scale * math.sqrt(inner)
    # the gained rows are the kernel's own new x times the gain, rounded once
    assert torch.equal(gained.cpu(), (xd.cpu() * gain).bfloat16())
    squares = ssq[:count, :rows].double().sum(0).cpu()
    want_squares = (xd.double().cpu() ** 2).sum(1)
    assert float(((squares - want_squares) / want_squares).abs().max()) < 1e-5
    parts = (ssq, count, width, eps)
    inv_rms = 1.0 / torch.sqrt(want_squares / width + eps)
    normed = gained.double().cpu() * inv_rms[:, None]
    exact = normed @ w_next.double().t()
    got = product(gained, w_next.cuda(), ops.EPI_F32, norm_parts=parts)
    assert float((got.double().cpu() - exact).abs().max()) < 2e-5 * float(exact.abs().max()) * math.sqrt(width)
    got = product(gained, w_next.cuda(), ops.EPI_SWIGLU, norm_parts=parts)
    want = plain_llama.swiglu(exact[:, :72], exact[:, 72:])
    assert float((got.double().cpu() - want).abs().max()) < 1e-2 * float(want.abs().max())
    # the same bits in a second run (ordered sums everywhere)
    xd2 = x.cuda()
    _, gained2, ssq2, count2 = product(h.cuda(), w_down.cuda(), ops.EPI_RESIDUAL, out=xd2, emit_gain=gain.cuda())
    assert torch.equal(xd, xd2) and torch.equal(gained, gained2) and count == count2 and torch.equal(ssq[:count, :rows], ssq2[:count, :rows])
    assert ops.gemm_tcgen05_status() == 0
    with pytest.raises(ops.KernelError, match="128 rows"):
        ops.tensor_core_gemm(torch.zeros(129, width, dtype=torch.bfloat16, device="cuda"), w_next.cuda(), ops.EPI_F32, norm_parts=parts)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count", [1, 3, 4, 1001, 262147])
def test_random_weights_are_the_same_bits_on_host_and_device(cuda_device, dtype, count):
    """The counter-based normal generator of random-weights mode: the device kernel and its numpy twin
    evaluate the same polynomials with the same roundings."""
    from models_b200.weights.philox_normal import normal_float32, tensor_key

    from models_b200.kernels import ops

    torch_dtype = dtype
    for mean, std, name in ((0.0, 0.02, "a.weight"), (1.0, 0.1, "b.weight"), (0.0, 1.0, "c")):
        key = tensor_key(count, name)
        device = ops.random_normal(torch.empty(count, dtype=torch_dtype, device="cuda"), key, mean, std)
        host = torch.from_numpy(normal_float32(count, key, mean, std)).to(torch_dtype)
        assert torch.equal(device.cpu(), host), (count, name)


def test_a_random_model_is_the_same_from_a_file_and_on_the_device(cuda_device, tmp_path):
    """`engine_from_config` (weights drawn on the GPU) and `write_random_model` (drawn on the host, written,
    read back) give one model: the same tensors, so the same logits."""
    from models_b200.config import config_from_dict
    from models_b200.engine import StepEntry
    from models_b200.engine.loading import engine_from_config, engine_from_folder
    from tiny import TINY_B, make_folder, random_tokens

    folder = make_folder(TINY_B, 9, tmp_path)
    from_file = engine_from_folder(folder, "bfloat16", 256)
    on_device = engine_from_config(config_from_dict(TINY_B), 9, "bfloat16", 256)
    assert torch.equal(from_file.model.embedding.weight, on_device.model.embedding.weight)
    assert torch.equal(from_file.model.head.weight, on_device.model.head.weight)
    assert torch.equal(from_file.model.final_norm.weight, on_device.model.final_norm.weight)
    for a, b in zip(from_file.model.blocks, on_device.model.blocks):
        assert torch.equal(a.mixer.w_qkv, b.mixer.w_qkv) and torch.equal(a.feed_forward.w_down, b.feed_forward.w_down)
        assert torch.equal(a.mixer_norm.weight, b.mixer_norm.weight)
    tokens = random_tokens(TINY_B["vocab_size"], 50, 1)
    outs = []
    for engine in (from_file, on_device):
        slot = engine.open_slot()
        outs.append(engine.step([StepEntry(slot, tokens, [49])]))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gated_products_take_their_activation_as_an_argument(cuda_device, activation):
    """act(gate) * up with the gate's activation as an argument of every kernel that applies it: the
    stand-alone kernel (float32 and bfloat16), the decode product (with and without the folded norm),
    the wide tcgen05 product and the prefill tcgen05 product."""
    from models_b200.kernels import ops

    act = {"silu": P_swiglu, "gelu_tanh": plain_llama.gelu_glu}[activation]
    g = torch.Generator().manual_seed(5)
    n, k = 272, 264
    w = (torch.randn(2 * n, k, generator=g) * 0.2).to(torch.bfloat16)
    gain = 1.0 + 0.1 * torch.randn(k, generator=g)
    for dtype in DTYPES:
        both = (torch.randn(37, 2 * 203, generator=g) * 2).to(dtype)
        expected = act(both[:, :203].float(), both[:, 203:].float())
        close(ops.swiglu(both.cuda(), activation), expected, dtype)
    code = ops.gated_epilogue(activation)
    for rows in (5, 16, 64, 300):
        x = (torch.randn(rows, k, generator=g)).to(torch.bfloat16)
        product = x.float() @ w.float().t()
        expected = act(product[:, :n], product[:, n:])
        if rows <= 32:
            close(ops.skinny_gemm(w.cuda(), code, x=x.cuda()), expected, torch.bfloat16)
        if rows <= 16:
            xf = torch.randn(rows, k, generator=g)
            normed = plain_llama.rms_norm(xf, gain, 1e-5).to(torch.bfloat16).float() @ w.float().t()
            got = ops.skinny_gemm(w.cuda(), code, xf=xf.cuda(), gain=gain.cuda(), eps=1e-5)
            want = act(normed[:, :n], normed[:, n:])
            # as for silu in the test of all epilogues: two roundings to bfloat16 (rows, result) around a product of two sums
            assert float((got.double().cpu() - want.double()).abs().max()) < 2e-2 * float(want.abs().max())
        if rows <= 128:
            close(ops.wide_gemm(x.cuda(), w.cuda(), code), expected, torch.bfloat16)
        close(ops.gemm_tcgen05(x.cuda(), w.cuda(), code), expected, torch.bfloat16)
    with pytest.raises(ops.KernelError, match="not built"):
        ops.gated_epilogue("relu")
    assert ops.gemm_tcgen05_status() == 0


def P_swiglu(gate, up):
    return plain_llama.swiglu(gate, up)


def test_logit_epilogue(cuda_device):
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(9)
    logits = torch.randn(5, 203, generator=g) * 3
    wide = torch.zeros(5, 256)
    wide[:, :203] = logits
    view = wide.cuda()[:, :203]  # rows wider than the vocabulary: the stride is an argument
    close(ops.logit_epilogue(view, 2.0, 5.0), plain_llama.softcap_logits(logits * 2.0, 5.0), torch.float32)
    close(ops.logit_epilogue(logits.clone().cuda(), 0.5, 0.0), logits * 0.5, torch.float32)


def test_split_k_residual_product_is_the_same_bits_every_time(cuda_device):
    """Few tiles and a long K: the residual product splits K over blocks.  The parts are summed in their
    order, so ten runs give one result, bit for bit, and it is the plain product; letting the parts add
    in as they finish is still there as an option and gives the same numbers within rounding."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(11)
    for m, n, k in ((256, 2048, 8192), (200, 520, 4096), (129, 264, 2048)):
        a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
        x0 = torch.randn(m, n, generator=g).cuda()
        expected = x0.double().cpu() + a.double().cpu() @ w.double().cpu().t()
        results = []
        for _ in range(10):
            x = x0.clone()
            ops.gemm_tcgen05(a, w, ops.EPI_RESIDUAL, out=x)
            results.append(x)
        for other in results[1:]:
            assert torch.equal(results[0], other), (m, n, k)
        close(results[0], expected, torch.float32, scale=float(expected.abs().max()) * 1e3)  # bfloat16 inputs, float sums
        loose = ops.gemm_tcgen05(a, w, ops.EPI_RESIDUAL, out=x0.clone(), arrival_order=True)
        close(loose, expected, torch.float32, scale=float(expected.abs().max()) * 1e3)
    tickets = ops._split_tickets[torch.cuda.current_device()]
    assert int(tickets.abs().sum()) == 0  # every launch leaves them as it found them
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("batch", [9, 40, 64, 128])
@pytest.mark.parametrize("heads,kv_heads,head_dim,hidden", [(4, 2, 16, 64), (3, 1, 32, 96), (32, 8, 64, 2048), (6, 3, 128, 264)])
@pytest.mark.parametrize("normed", [False, True])
def test_wide_qkv_product_with_rotation_and_cache_write(cuda_device, batch, heads, kv_heads, head_dim, hidden, normed):
    """The q/k/v product of a decode step of 9 to 128 sequences with rotation and cache write folded in,
    against the plain functions: queries rotated by each row's own position, keys rotated and values
    as they are at each row's cache position, rows without a position of their own storing nothing.
    `normed`: the division by the rows' root mean square happens in the product's epilogue, from parts
    of their sums of squares."""
    from models_b200.kernels import ops

    g = torch.Generator().manual_seed(batch * 7 + head_dim)
    rows_w = (heads + 2 * kv_heads) * head_dim
    w = (torch.randn(rows_w, hidden, generator=g) * 0.05).bfloat16()
    x = torch.randn(batch, hidden, generator=g).bfloat16()
    positions = torch.randint(0, 300, (batch,), generator=g).int()
    freqs = plain_llama.rope_pair_frequencies(head_dim, 10000.0)
    cos, sin = plain_llama.rope_cos_sin(torch.arange(300), freqs, None)
    pages, page = 2 * batch + 1, 64
    k_pool = torch.zeros(pages, kv_heads, page, head_dim, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    slots = torch.randperm(pages * page - page, generator=g)[:batch].int() + page
    slots[batch // 2] = -1  # a padding row: nothing is stored for it
    kd, vd = k_pool.cuda(), v_pool.cuda()
    parts, inv_rms = None, torch.ones(batch, dtype=torch.float64)
    if normed:
        ssq = torch.rand(7, ops.SSQ_COLUMNS, generator=g) * hidden  # (two more parts than are counted)
        parts = (ssq.cuda(), 5, hidden, 2e-5)
        inv_rms = 1.0 / torch.sqrt(ssq[:5, :batch].double().sum(0) / hidden + 2e-5)
    q = ops.wide_qkv_rope(x.cuda(), w.cuda(), heads, kv_heads, head_dim, positions.cuda(), cos.cuda(), sin.cuda(), kd, vd, slots.cuda(),
                          norm_parts=parts)
    full = ((x.double() @ w.double().t()) * inv_rms[:, None]).float()
    qe = full[:, : heads * head_dim].bfloat16().float().reshape(batch, heads, head_dim)
    ke = full[:, heads * head_dim:(heads + kv_heads) * head_dim].bfloat16().float().reshape(batch, kv_heads, head_dim)
    ve = full[:, (heads + kv_heads) * head_dim:].reshape(batch, kv_heads, head_dim)
    c, s = cos[positions.long()], sin[positions.long()]
    qe, ke = plain_llama.rope_rotate_split_half(qe, c, s), plain_llama.rope_rotate_split_half(ke, c, s)
    close(q.reshape(batch, heads, head_dim), qe, torch.bfloat16)
    kflat, vflat = kd.cpu().permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim), vd.cpu().permute(0, 2, 1, 3).reshape(-1, kv_heads, head_dim)
    for b in range(batch):
        if slots[b] < 0:
            continue
        close(kflat[slots[b]], ke[b], torch.bfloat16, scale=float(ke.abs().max()))
        close(vflat[slots[b]], ve[b], torch.bfloat16, scale=float(ve.abs().max()))
    stored = (kflat.abs().sum(dim=(1, 2)) > 0).sum()
    assert int(stored) == batch - 1  # exactly the rows with a cache position wrote
    assert ops.gemm_tcgen05_status() == 0
