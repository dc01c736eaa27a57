"""Every kernel library of the package, for building them all ahead of time."""

from __future__ import annotations

from .build import build_library

# (name, sources, definitions)
LIBRARIES = [
    ("mb_elementwise", ["elementwise.cu"], {}),
    ("mb_attention_rows", ["attention_rows.cu"], {}),
    ("mb_gemm_f32", ["gemm_f32.cu"], {}),
    ("mb_sampling", ["sampling.cu"], {}),
]


def build_all(quiet: bool = False):
    return [build_library(name, sources, defines, quiet=quiet) for name, sources, defines in LIBRARIES]
