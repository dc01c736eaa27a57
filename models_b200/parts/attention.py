"""Grouped-query attention over the paged cache (the Llama mixer).

q = Wq.xn, k = Wk.xn, v = Wv.xn (optional biases); rotation of every query and key head; keys and
values stored at the token's position; per head softmax(q.K * scale) . V over the visible positions
with kvHead = head / (heads / kv_heads); then Wo (integrallis/models,
backend-java/.../llama/LlamaForwardPass.java:1061-1138,1543-1593).  q, k and v are one matrix
product over the row-concatenated weights, which is how the reference groups them at execution
time (tripleMatmulDispatch, backend-java/.../llama/LlamaForwardPass.java:1044-1059).
"""

from __future__ import annotations

import torch

from ..cache.kv_cache import KvRequest
from ..kernels import ops
from ..weights.loader import ParamRequest
from .base import Mixer, Prenormed, RunContext
from .linear import linear
from .registry import build_part, register_part


class AttentionMixer(Mixer):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are no multiple of {spec.num_kv_heads} kv heads")
        if spec.window is not None and spec.window <= 0:
            raise ValueError(f"attention window must be positive, got {spec.window}")
        self.q_width = spec.num_heads * spec.head_dim
        self.kv_width = spec.num_kv_heads * spec.head_dim
        self.position = None
        if spec.position is not None:
            if spec.position.rotary_dim > spec.head_dim:
                raise ValueError(f"rotary_dim {spec.position.rotary_dim} exceeds head_dim {spec.head_dim}")
            key = ("position", spec.position, runtime.max_positions)
            if key not in runtime.shared:
                runtime.shared[key] = build_part("position", spec.position, runtime)
            self.position = runtime.shared[key]

    def parameters(self):
        s, n = self.spec, self.spec.weights
        out = [
            ParamRequest(n["q"], (self.q_width, s.hidden_size)),
            ParamRequest(n["k"], (self.kv_width, s.hidden_size)),
            ParamRequest(n["v"], (self.kv_width, s.hidden_size)),
            ParamRequest(n["o"], (s.hidden_size, self.q_width)),
        ]
        if s.bias:
            out += [
                ParamRequest(n["q_bias"], (self.q_width,), "bias"),
                ParamRequest(n["k_bias"], (self.kv_width,), "bias"),
                ParamRequest(n["v_bias"], (self.kv_width,), "bias"),
                ParamRequest(n["o_bias"], (s.hidden_size,), "bias"),
            ]
        return out

    def load(self, tensors):
        n, rt = self.spec.weights, self.runtime
        q, k, v = (rt.matrix(tensors[n[r]]) for r in ("q", "k", "v"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.q_width]
        self.w_o = rt.matrix(tensors[n["o"]])
        self.b_qkv = self.b_o = None
        if self.spec.bias:
            self.b_qkv = torch.cat([rt.vector(tensors[n[r]]) for r in ("q_bias", "k_bias", "v_bias")]).contiguous()
            self.b_q = self.b_qkv[: self.q_width].contiguous()
            self.b_o = rt.vector(tensors[n["o_bias"]])

    def kv_request(self):
        return KvRequest(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def folds(self, rows: int, norm) -> bool:
        """Whether `forward_residual` applies: bfloat16 weights, few rows, no biases, a foldable norm."""
        return (self.b_qkv is None and self.b_o is None and getattr(norm, "foldable", False)
                and ops.skinny_pays(self.w_qkv, rows, with_norm=True) and ops.skinny_pays(self.w_o, rows))

    def forward_residual(self, x: torch.Tensor, norm, batch, run: RunContext) -> None:
        """x += Wo . attention(rotate(Wqkv . norm(x))): the norm rides in the q/k/v product, the
        residual add in the output product."""
        writes, s, pos = run.writes_cache, self.spec, self.position
        if (writes and pos is not None and pos.rotary_dim == s.head_dim and not pos.interleaved and s.head_dim % 16 == 0
                and run.k_pool is not None and run.k_pool.dtype == torch.bfloat16):
            # rotation and cache write ride in the q/k/v product too
            group = batch.groups[run.group]
            q = ops.skinny_qkv_rope(self.w_qkv, x, norm.weight, norm.spec.eps, s.num_heads, s.num_kv_heads, s.head_dim,
                                    batch.positions, pos.cos, pos.sin, run.k_pool, run.v_pool, group.slot_mapping)
            attended = torch.empty((q.shape[0], self.q_width), dtype=q.dtype, device=q.device)
            self.attend(q, attended, batch, group, run)
        else:
            qkv = ops.skinny_gemm(self.w_qkv if writes else self.w_q, ops.EPI_BF16, xf=x, gain=norm.weight, eps=norm.spec.eps)
            attended = self._rotate_store_attend(qkv, batch, run)
        ops.skinny_gemm(self.w_o, ops.EPI_RESIDUAL, x=attended, out=x)

    def adds(self, xn: torch.Tensor) -> bool:
        """Whether `forward_into` applies (any number of rows): a bfloat16 output matrix the tcgen05
        kernel takes, no output bias."""
        return self.b_o is None and xn.dtype == torch.bfloat16 and ops.gemm_tcgen05_takes(self.w_o, rows=xn.shape[0])

    def forward_into(self, x: torch.Tensor, xn: torch.Tensor, batch, run: RunContext) -> None:
        """x += Wo . attention(...): the residual add rides in the output product, and (whole heads of
        64 or 128, split-half pairs over the whole head) rotation and cache write in the q/k/v product."""
        writes, s, pos = run.writes_cache, self.spec, self.position
        rows = xn.shape[0]
        folds_rotation = (writes and self.b_qkv is None and pos is not None and pos.rotary_dim == s.head_dim and not pos.interleaved
                          and run.k_pool is not None and run.k_pool.dtype == torch.bfloat16)
        if folds_rotation and ops.gemm_tcgen05_qkv_rope_takes(self.w_qkv, rows, s.num_heads, s.num_kv_heads, s.head_dim):
            group = batch.groups[run.group]
            q = ops.gemm_tcgen05_qkv_rope(xn, self.w_qkv, s.num_heads, s.num_kv_heads, s.head_dim, batch.positions, pos.cos,
                                          pos.sin, run.k_pool, run.v_pool, group.slot_mapping)
            attended = torch.empty((q.shape[0], self.q_width), dtype=q.dtype, device=q.device)
            self.attend(q, attended, batch, group, run)
        elif folds_rotation and ops.wide_qkv_rope_takes(self.w_qkv, rows, s.num_heads, s.num_kv_heads, s.head_dim):
            group = batch.groups[run.group]  # 9 to 128 rows: the wide decode product, rotation and cache write in it too
            q = ops.wide_qkv_rope(xn, self.w_qkv, s.num_heads, s.num_kv_heads, s.head_dim, batch.positions, pos.cos, pos.sin,
                                  run.k_pool, run.v_pool, group.slot_mapping)
            attended = torch.empty((q.shape[0], self.q_width), dtype=q.dtype, device=q.device)
            self.attend(q, attended, batch, group, run)
        else:
            qkv = linear(xn, self.w_qkv if writes else self.w_q, self.runtime.compute_dtype)
            if self.b_qkv is not None:
                ops.bias_add(qkv, self.b_qkv if writes else self.b_q)
            attended = self._rotate_store_attend(qkv, batch, run)
        ops.tensor_core_gemm(attended, self.w_o, ops.EPI_RESIDUAL, out=x)

    def chains(self, rows: int, run: RunContext, next_norm) -> bool:
        """Whether `forward_chain` applies: up to 128 rows (the narrow decode products up to 8, the wide ones above),
        rotation and cache write folded into the q/k/v product, no biases, and a next norm whose gain a residual
        product can apply."""
        s, pos = self.spec, self.position
        if not (self.b_qkv is None and self.b_o is None and run.writes_cache and pos is not None
                and pos.rotary_dim == s.head_dim and not pos.interleaved and run.k_pool is not None
                and run.k_pool.dtype == torch.bfloat16 and getattr(next_norm, "foldable", False)):
            return False
        if rows <= ops.SKINNY_PAYS_ROWS:
            return s.head_dim % 16 == 0 and ops.skinny_pays(self.w_qkv, rows, with_norm=True) and ops.skinny_pays(self.w_o, rows)
        return (ops.wide_qkv_rope_takes(self.w_qkv, rows, s.num_heads, s.num_kv_heads, s.head_dim)
                and ops.gemm_tcgen05_takes(self.w_o, ops.EPI_RESIDUAL, rows))

    def forward_chain(self, x: torch.Tensor, scaled, batch, run: RunContext, next_norm, norm=None) -> Prenormed:
        """x += Wo . attention(rotate(Wqkv . norm(x))) for up to 128 rows, in three kernels and with no kernel for
        either norm: `scaled` is the normalised rows, or a Prenormed whose division by the root mean square the
        q/k/v product does itself, or None (few rows only): the product then normalises x with `norm` itself.  The
        output product adds into x and prepares the rows of `next_norm`."""
        s, pos = self.spec, self.position
        group = batch.groups[run.group]
        rows, parts = (scaled.rows, scaled.norm_parts()) if isinstance(scaled, Prenormed) else (scaled, None)
        tables = (batch.positions, pos.cos, pos.sin, run.k_pool, run.v_pool, group.slot_mapping)
        few = x.shape[0] <= ops.SKINNY_PAYS_ROWS
        if few and rows is None:
            q = ops.skinny_qkv_rope(self.w_qkv, x, norm.weight, norm.spec.eps, s.num_heads, s.num_kv_heads, s.head_dim, *tables)
        elif few:
            q = ops.skinny_qkv_rope(self.w_qkv, None, None, 0.0, s.num_heads, s.num_kv_heads, s.head_dim, *tables, x=rows,
                                    norm_parts=parts)
        else:
            q = ops.wide_qkv_rope(rows, self.w_qkv, s.num_heads, s.num_kv_heads, s.head_dim, *tables, norm_parts=parts)
        attended = torch.empty((q.shape[0], self.q_width), dtype=q.dtype, device=q.device)
        self.attend(q, attended, batch, group, run)
        if few:
            _, gained, ssq, count = ops.skinny_gemm(self.w_o, ops.EPI_RESIDUAL, x=attended, out=x, emit_gain=next_norm.weight)
        else:
            _, gained, ssq, count = ops.wide_gemm(attended, self.w_o, ops.EPI_RESIDUAL, out=x, emit_gain=next_norm.weight)
        return Prenormed(gained, ssq, count, x.shape[1], next_norm.spec.eps, next_norm)

    def forward(self, xn: torch.Tensor, batch, run: RunContext) -> torch.Tensor:
        dtype = self.runtime.compute_dtype
        writes = run.writes_cache
        qkv = linear(xn, self.w_qkv if writes else self.w_q, dtype)
        if self.b_qkv is not None:
            ops.bias_add(qkv, self.b_qkv if writes else self.b_q)
        attended = self._rotate_store_attend(qkv, batch, run)
        delta = linear(attended, self.w_o, dtype)
        if self.b_o is not None:
            ops.bias_add(delta, self.b_o)
        return delta

    def _rotate_store_attend(self, qkv: torch.Tensor, batch, run: RunContext) -> torch.Tensor:
        s, dtype = self.spec, self.runtime.compute_dtype
        if run.k_pool is None:
            raise RuntimeError("the attention mixer needs cache pools; its run has none")
        writes = run.writes_cache
        group = batch.groups[run.group]
        pos = self.position
        ops.rope_cache_write(
            qkv, batch.positions, pos.cos if pos else None, pos.sin if pos else None, run.k_pool, run.v_pool,
            group.slot_mapping, s.num_heads, s.num_kv_heads, s.head_dim, pos.rotary_dim if pos else 0,
            pos.interleaved if pos else False, run.k_pool.shape[2], writes)
        attended = torch.empty((qkv.shape[0], self.q_width), dtype=dtype, device=qkv.device)
        self.attend(qkv, attended, batch, group, run)
        return attended

    def decode_class(self, sequences: int, max_kv_len: int):
        """What of a decode step's launches depends on the context length: how many blocks share a
        sequence's keys.  Steps of one class can replay one capture."""
        s = self.spec
        if self.runtime.compute_dtype != torch.bfloat16 or s.head_dim % 16 or s.head_dim > 256:
            return 0  # the plain-arithmetic kernel: one launch shape for every length
        return ops.decode_splits(sequences, s.num_heads, s.num_kv_heads, s.head_dim, max_kv_len, s.window,
                                 ops.multiprocessors(self.runtime.device))

    def attend(self, qkv, attended, batch, group, run):
        """Tensor-core kernels where they apply (bfloat16, head size a multiple of 16, pages of 64);
        otherwise the plain-arithmetic kernel, which takes every size and is the 32-bit path's."""
        s = self.spec
        args = (qkv, attended, run.k_pool, run.v_pool, group.block_table, batch.cu_q, batch.kv_lens)
        if ops.attention_tc_takes(qkv.dtype, s.head_dim, run.k_pool.shape[2]):
            if batch.max_q_len == 1:
                splits = ops.decode_splits(batch.num_sequences, s.num_heads, s.num_kv_heads, s.head_dim, batch.max_kv_len,
                                           s.window, ops.multiprocessors(qkv.device), run.k_pool.shape[2])
                ops.decode_attention(*args, s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.scale, splits)
            else:
                ops.prefill_attention(*args, batch.max_q_len, s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.scale)
            return
        ops.paged_attention_rows(*args, batch.max_q_len, s.num_heads, s.num_kv_heads, s.head_dim, s.window, s.scale)


register_part("mixer", "attention", AttentionMixer)
