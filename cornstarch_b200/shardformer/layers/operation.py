"""``gather_forward_split_backward`` at the import path of the reference (cornstarch/shardformer/layers/operation.py)."""

from ...parallel.comm import (  # noqa: F401
    all_to_all_comm,
    gather_forward_split_backward,
    split_forward_gather_backward,
)
