"""Switches of the kernel path, as one typed object that a model is loaded with.

Two engines in one process may differ in them. The defaults are what measured best on B200 with
LFM2 sizes; the other values exist for comparisons and for the tests that pin down what a switch
changes. Nothing on the hot path reads the environment: ``KernelOptions.from_env`` exists for
benchmark scripts and tests that want to flip a switch from the command line.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields
from typing import Mapping, Optional


@dataclass
class KernelOptions:
    # Products of more than 16 rows on the bfloat16 path: "swiglu" = the gate|up product with its activation
    # runs on this package's tcgen05 kernel from ``tensor_core_min_rows`` rows up, the others on cuBLAS;
    # "all" = every such product on the tcgen05 kernel; "none" = cuBLAS for all of them.
    tensor_core_products: str = "swiglu"
    # Below this many rows the library product followed by the activation kernel still wins (few 128-row
    # tiles in too few waves). Measured, 2,048 prompt tokens in portions of 256 / 512 / 1,024 / 1,536 / 2,048
    # rows: 9.70 / 6.51 / 4.66 / 4.84 / 3.99 ms with this package's kernel against 9.34 / 6.15 / 4.59 / 4.76 /
    # 4.13 ms with the library's.
    tensor_core_min_rows: int = 2048
    # ... and below this width of the model (the product's k) too: at 2,048 rows and a width of 1,024 the library
    # with its activation kernel takes 52 us where this package's kernel takes 62 (a tile's 16 k-steps are too
    # few to hide its start and its epilogue); at 1,536 it is 78 against 76, at 2,048 117 against 106.
    tensor_core_min_width: int = 1536
    # -1: the host chooses the tile shape of the tcgen05 product; 0..3 force one (for measurements)
    tensor_core_variant: int = -1
    # decode steps of few rows: residual add + RMSNorm split over the products before and after it
    split_norms: bool = True
    # decode steps: q/k norm + rotation + cache write inside the attention kernel (False: a kernel of their own)
    fuse_decode_qk: bool = True
    # prompt-portion attention of head size 64 on tcgen05 (False: the mma.sync kernel)
    tcgen05_attention: bool = True
    # Each small-batch product asks this much of its successor's weights into the L2 (0: off). Measured at
    # batch 8 with LFM2-1.2B sizes: 0.736 ms a step without, 0.723 with 4 MiB, 0.714 with 8, 0.734 with 16.
    prefetch_mb: float = 8.0
    # decode steps of at most 16 rows run the fused small-batch products (False: the general path)
    fuse_small_batches: bool = True

    def validate(self) -> None:
        if self.tensor_core_products not in ("none", "swiglu", "all"):
            raise ValueError(f"tensor_core_products must be none, swiglu or all, got {self.tensor_core_products!r}")
        if not -1 <= self.tensor_core_variant <= 3:
            raise ValueError("tensor_core_variant must lie in -1..3")
        if self.tensor_core_min_rows < 1 or self.tensor_core_min_width < 1 or self.prefetch_mb < 0:
            raise ValueError("tensor_core_min_rows and tensor_core_min_width must be positive and prefetch_mb must "
                             "not be negative")

    @classmethod
    def from_env(cls, environ: Optional[Mapping[str, str]] = None, prefix: str = "CELEG_B200_") -> "KernelOptions":
        """Defaults overridden by variables named ``<prefix><FIELD>`` (upper case): for scripts and tests."""
        environ = os.environ if environ is None else environ
        options = cls()
        for item in fields(cls):
            text = environ.get(prefix + item.name.upper())
            if text is None:
                continue
            current = getattr(options, item.name)
            if isinstance(current, bool):
                value = text.strip().lower() not in ("0", "false", "no", "off", "")
            elif isinstance(current, int):
                value = int(text)
            elif isinstance(current, float):
                value = float(text)
            else:
                value = text
            setattr(options, item.name, value)
        options.validate()
        return options
