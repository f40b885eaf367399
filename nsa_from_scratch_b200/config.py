"""Hyper-parameter bag with the reference's field names (nsa/reference.py:17-29) plus the
optional extensions.  Any object with these attributes is accepted by `nsa_forward`; the
extension fields are read with getattr and default to the reference's behaviour."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class NSAConfig:
    block_size_c: int = 64
    block_size_n: int = 64
    block_size_m: int = 64
    top_k: int = 16
    window_size: int = 512
    causal: bool = True
    pool: str = "mean"
    gate_activation: str = "sigmoid"
    scale: Optional[float] = None
    precision: str = "bf16"
    # extensions (None / 0 = the reference's behaviour)
    stride_c: Optional[int] = None   # compression stride < block_size_c: overlapping windows
    force_first: int = 0             # always select the first n blocks
    force_local: int = 0             # always select the last n causally legal blocks
    select_per_group: bool = False   # one block list per KV head (shared by its query heads), scored by
                                     # the sum of the heads' scores; False = one list per query head
    scorer: str = "mean"             # "mean": the reference's block-mean scores; "compressed": probability mass
                                     # of the compressed branch per selection block (scoring.py)
