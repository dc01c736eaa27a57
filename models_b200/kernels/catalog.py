"""Every kernel library of the package, for building them all ahead of time."""

from __future__ import annotations

from .build import build_library

# (name, sources, definitions)
LIBRARIES = [
    ("mb_elementwise", ["elementwise.cu"], {}),
    ("mb_attention_rows", ["attention_rows.cu"], {}),
    ("mb_gemm_f32", ["gemm_f32.cu"], {}),
    ("mb_sampling", ["sampling.cu"], {}),
    ("mb_random_init", ["random_init.cu"], {}),
    ("mb_skinny_gemm", ["skinny_gemm.cu"], {}),
    ("mb_gemm_tcgen05", ["gemm_tcgen05.cu"], {}),
    ("mb_wide_gemm_tcgen05", ["wide_gemm_tcgen05.cu"], {}),
    # the tensor-core attention is compiled per head size when a model first needs it; these are
    # the sizes of the benchmark models and of the tests
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 16}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 32}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 48}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 128}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 16}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 32}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 48}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 128}),
    ("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": 128}),
]


def build_all(quiet: bool = False):
    return [build_library(name, sources, defines, quiet=quiet) for name, sources, defines in LIBRARIES]
