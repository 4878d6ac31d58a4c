"""Where one kernel path hands over to another. These numbers change speed, never results: the tests
run the paths on both sides of each. They were measured on one B200 at the layer sizes named beside
them; a model of other sizes may want others. Set them on `TUNING` before an engine is built (a
recorded CUDA graph keeps the path it was recorded with)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Tuning:
    # Steps of at most so many rows run in the folded form (five kernels a layer: the products'
    # epilogues do norm, rotation, cache write, activation and residual) on this package's few-token
    # product; above it the library product and separate kernels take over. Measured at hidden 2,048 /
    # intermediate 8,192: a decode step of 64 rows is 15 % slower in the folded form, one of 32 rows
    # 22 % faster. At most 64 (what the fused kernels take).
    few_rows: int = 32
    # From so many rows the gate/up product runs on the two-SM kernel with the SwiGLU epilogue instead
    # of the library product plus the activation kernel. Measured on whole prefill steps at hidden
    # 2,048 / intermediate 8,192: 512 / 640 / 768 / 896 rows take 1.47 / 1.70 / 1.78 / 2.15 ms with it
    # and 1.53 / 1.80 / 1.89 / 2.25 ms without; at 384 rows it loses (1.33 against 1.26 ms).
    pair_gemm_from_rows: int = 512
    # A step in which some request has more keys than this counts as one of long contexts: decode
    # attention then shares a request's keys over up to 64 blocks that merge through global memory
    # instead of a cluster of 8. Measured on whole decode steps with 8 kv heads of 64: at 4,096 keys
    # the cluster wins at batch 1, 2 and 4 (0.764 / 0.791 / 0.825 against 0.767 / 0.808 / 0.854 ms), at
    # 6,000 keys the wider grid wins at batch 1 and 2 (0.794 / 0.837 against 0.819 / 0.857 ms) and
    # ties at batch 4.
    long_context_keys: int = 5120


TUNING = Tuning()
