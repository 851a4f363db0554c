"""TEST INFRASTRUCTURE — not part of the product.

CPU oracle for the causal depthwise conv1d hot path: a ctypes front end over
``libcc1d_oracle.so`` (built from ``cc1d_oracle.c`` by ``oracle/Makefile``).  Only the
tests, the smoke check and the benchmark's CPU-baseline leg import this package; the
product package never does.

Every function takes torch tensors of any dtype / layout, evaluates the restated
algorithm in float64 on dense channel-first copies and returns float64 tensors (so the
caller decides how to round).  ``*_f32`` variants exist for timing only.
"""
from .oracle import (  # noqa: F401
    build,
    lib,
    fwd,
    bwd,
    update,
    varlen_states,
    prefill_varlen,
    round_to,
    max_threads,
    set_threads,
    fwd_f32_timed,
    bwd_f32_timed,
    update_f32_timed,
)
