"""The reference's ``models.gpt_utils`` import path (models/gpt_utils.py:7-160): the shard readers and the two
data loaders under the reference's names."""

from .data import (  # noqa: F401
    ArithmeticDistributedDataLoader,
    DistributedDataLoader,
    _map_shard,
    _read_header,
)

_peek_data_shard = _read_header   # number of tokens a shard's header claims
_load_data_shard = _map_shard     # the shard's uint16 tokens (memory-mapped, header checked)
