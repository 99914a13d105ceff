"""The crossover points between kernels: measured, not derived, and kept in one place.

Each value says from where on one kernel hands over to another.  They are no limits (a kernel refuses
what it cannot take on its own) and nothing depends on them for correctness; they were measured on one
B200 at the layer sizes named beside them, and another width or another GPU may want others.  Any of
them can be overridden for a process with ``QIL_TUNE_<NAME>=<number>`` (read once, at import) or by
assigning to the attribute before the first step.
"""
from __future__ import annotations

import os


def _tuned(name, default):
    raw = os.environ.get(f"QIL_TUNE_{name}")
    return type(default)(raw) if raw is not None else default


#: Most rows the weight-streaming decode product takes (``gemm_small_m``); the kernel's own limit is 16.
SMALL_M_MAX_ROWS = _tuned("SMALL_M_MAX_ROWS", 16)
#: With 9 to 16 rows the decode product keeps three stages in flight instead of four; on a matrix of at
#: least this many elements it then loses to the library (151936 x 4096 vocabulary head, 16 rows: 274 us
#: against 211 us).
SMALL_M_LIBRARY_ELEMENTS = _tuned("SMALL_M_LIBRARY_ELEMENTS", 1 << 28)
#: With at most 8 rows the decode product gives a block 32 output features instead of 16 when that still leaves
#: this many blocks (one for each of the 148 SMs: 4096 features make 128 and lose, 19.7 -> 22.9 us at K 12288)
#: and the matrix has fewer than this many elements (a stream as long as a vocabulary head's runs 3 % faster on
#: the longer row segments of the 16-feature blocks: 194.7 against 200.9 us).  In between the wider block wins by
#: its fewer instructions per weight byte (6144 x 4096 with the norm: 20.3 -> 18.5 us; 24576 x 4096: 37.2 -> 36.2).
SMALL_M_WIDE_MIN_BLOCKS = _tuned("SMALL_M_WIDE_MIN_BLOCKS", 148)
SMALL_M_WIDE_MAX_ELEMENTS = _tuned("SMALL_M_WIDE_MAX_ELEMENTS", 1 << 28)
#: From this many rows on the gate/up product runs on the tcgen05 tile kernel (the first row count the decode
#: product does not take).
TILE_KERNEL_MIN_ROWS = _tuned("TILE_KERNEL_MIN_ROWS", 17)
#: From this many rows on the q/k/v product runs on the tcgen05 kernels with its tail fused; below, the pair
#: kernel has too few 256 x 256 tiles for the SM pairs and the library product plus the tail kernel win
#: (6144 x 4096 at 2048 rows: 86 us against 75 + 24 us; at 256 rows the library wins).
QKV_TAIL_MIN_ROWS = _tuned("QKV_TAIL_MIN_ROWS", 512)
#: The single-token attention's cost model, in units of the time a block takes to stream one 64-key tile:
#: a block's start-up (its description, page ids and first tile arrive one after the other) and what each
#: further span adds to the merge.  Fitted to the recorded decode step of 32/8 heads of 128 at a context of
#: 8192 (batch 8: 4.84 ms with 5 or 6 spans, 4.97 with 4, 5.1 with 7 to 9; batch 1 flat from 16 to 43 spans).
SPAN_STARTUP_TILES = _tuned("SPAN_STARTUP_TILES", 2.0)
SPAN_MERGE_TILES = _tuned("SPAN_MERGE_TILES", 0.15)
