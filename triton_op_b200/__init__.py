"""B200 (sm_100a) paged-attention decode: split-KV partition kernel + log-sum-exp reduce.

Public surface:
  paged_attention_decode   the reference operator's entry point (see ``pa_decode``)
  inputs                   KV-cache layouts, quantisers and the seeded benchmark workloads
  sharding                 multi-GPU planning (sequence sharding, KV-partition sharding + merge)
  cache_write              the write side: new K/V tokens quantised and scattered into the paged caches

The compute path is the CUDA library ``lib/libpa_decode_sm100.so`` (``python -m
triton_op_b200.build``); importing the operator without it raises.
"""
from .pa_decode import (PaArgumentError, SEQUENCE_PARTITION_SIZE, get_workspaces,
                        paged_attention_decode, query_launch)

__all__ = ["paged_attention_decode", "query_launch", "get_workspaces", "PaArgumentError",
           "SEQUENCE_PARTITION_SIZE"]
