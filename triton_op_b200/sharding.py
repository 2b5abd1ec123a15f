"""Multi-GPU use of the decode operator: one process per GPU, two ways to split the work.

* **By sequence** (large batches): every rank owns whole sequences, their pages and block-table
  rows, and calls :func:`triton_op_b200.paged_attention_decode` on them.  No collective is
  involved; the only question is which rank gets which sequences.  :func:`shard_sequences`
  deals them out in contiguous runs or balanced by token count (decode time is proportional to
  the KV bytes read, i.e. to the tokens a rank holds).

* **By KV partition** (few, very long sequences): rank ``g`` holds a contiguous range of every
  sequence's tokens, computes attention over that range and reduces it to one
  ``(max, sum, normalised output)`` triple per output row (the reduce kernel's triple output,
  pa_decode_triton_gluon_fp8.py:1266-1313 stopped one step early).  The triples are all-gathered
  (520 bytes per row and rank) and merged with the same log-sum-exp formula across ranks.
  :func:`plan_kv_shards` computes the ranges, :func:`decode_kv_shard` runs one rank's part and
  :func:`gather_and_merge` does the exchange and the merge.

The planning functions are pure host code (``torch`` CPU tensors / Python ints) and run without
a GPU; the exchange works on any ``torch.distributed`` backend (NCCL on GPUs).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch

__all__ = [
    "shard_sequences", "shard_token_counts", "KvShard", "plan_kv_shards", "local_block_table",
    "decode_kv_shard", "all_gather_triples", "merge_triples_cuda", "gather_and_merge", "KvShardedDecoder",
    "PeerExchange",
]


# ----------------------------------------------------------------------------- by sequence
def shard_sequences(context_lens: Sequence[int], world_size: int, policy: str = "balanced") -> List[List[int]]:
    """Sequence indices owned by each rank.

    ``policy="contiguous"``: equal counts in index order (rank r gets ``[r*n/W, (r+1)*n/W)``).
    ``policy="balanced"``: longest-first greedy assignment to the rank with the fewest tokens so
    far (ties: fewer sequences, then lower rank); every list is returned in ascending index order.
    Deterministic, so every rank can compute the same plan from the same lengths.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    lens = [int(x) for x in context_lens]
    n = len(lens)
    if policy == "contiguous":
        return [list(range(r * n // world_size, (r + 1) * n // world_size)) for r in range(world_size)]
    if policy != "balanced":
        raise ValueError(f"unknown policy {policy!r}")
    order = sorted(range(n), key=lambda i: (-lens[i], i))
    load = [0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], len(owned[k]), k))
        owned[r].append(i)
        load[r] += lens[i]
    return [sorted(o) for o in owned]


def shard_token_counts(context_lens: Sequence[int], shards: List[List[int]]) -> List[int]:
    """Tokens (KV rows) each rank reads per decode call under ``shards``."""
    lens = [int(x) for x in context_lens]
    return [sum(lens[i] for i in s) for s in shards]


# ----------------------------------------------------------------------------- by KV partition
@dataclass(frozen=True)
class KvShard:
    """One rank's part of one sequence: tokens ``[begin, end)`` of a context of ``context_len``."""
    begin: int
    end: int
    context_len: int
    query_len: int

    @property
    def tokens(self) -> int:
        return self.end - self.begin

    @property
    def holds_tail(self) -> bool:
        """True when the range ends at the end of the context (or the range is empty)."""
        return self.end >= self.context_len

    @property
    def local_context_len(self) -> int:
        return self.tokens

    @property
    def local_query_len(self) -> int:
        """``query_len`` to call the operator with.

        The causal rule -- row ``t`` sees key ``j`` iff ``(L-1-t) + j < context_len``
        (pa_decode_triton_gluon_fp8.py:915-920) -- only ever hides the last ``L-1`` keys of the
        context.  A range that ends before them is attended to by every row alike, which is the
        operator's ``query_len = 1`` with a group of ``L*G`` rows (the query layout is the same).
        """
        return self.query_len if self.holds_tail else 1


def plan_kv_shards(context_lens: Sequence[int], world_size: int, partition_size: int,
                   query_len: int = 1) -> List[List[KvShard]]:
    """``plan[rank][seq]``: contiguous token ranges, cut at multiples of ``partition_size``.

    The partitions of a sequence are dealt out as evenly as possible, earlier ranks taking the
    remainder.  The range that ends at the context's end always holds at least ``query_len - 1``
    tokens (the keys the causal rule can hide), so that only that range needs the rule; when
    the last partition is shorter than that, the cut before it is removed.  Ranks with nothing
    to do for a sequence get an empty range at the end of the context.
    """
    if world_size < 1 or partition_size < 1 or query_len < 1:
        raise ValueError("world_size, partition_size and query_len must be positive")
    plan: List[List[KvShard]] = [[] for _ in range(world_size)]
    for ctx in (int(c) for c in context_lens):
        ctx = max(ctx, 0)
        parts = (ctx + partition_size - 1) // partition_size
        base, extra = divmod(parts, world_size)
        cuts = [0]
        for r in range(world_size):
            cuts.append(cuts[-1] + base + (1 if r < extra else 0))
        bounds = [min(c * partition_size, ctx) for c in cuts]
        # the range holding the end of the context needs >= query_len - 1 tokens
        last = max((r for r in range(world_size) if bounds[r + 1] > bounds[r]), default=None)
        if last is not None and last > 0 and bounds[last + 1] - bounds[last] < query_len - 1:
            bounds[last] = bounds[last + 1]      # give the short tail to the previous non-empty range
        for r in range(world_size):
            plan[r].append(KvShard(bounds[r], bounds[r + 1], ctx, query_len))
    return plan


def local_block_table(block_table: torch.Tensor, shards: Sequence[KvShard], block_size: int) -> torch.Tensor:
    """Block-table rows restricted to each sequence's range (``[S, max local blocks]`` int32).

    A range begins at a multiple of the partition size, which is a multiple of the block size for
    every block size below it; for 1024-token blocks the partition size must be a multiple of
    the block size as well, so that the range starts at a block boundary.
    """
    S = block_table.shape[0]
    if len(shards) != S:
        raise ValueError("one shard per sequence expected")
    for sh in shards:
        if sh.tokens > 0 and sh.begin % block_size != 0:
            raise ValueError(f"range start {sh.begin} is not a multiple of the block size {block_size}")
    widths = [(sh.tokens + block_size - 1) // block_size for sh in shards]
    out = torch.zeros((S, max(1, max(widths, default=1))), dtype=torch.int32, device=block_table.device)
    for s, (sh, w) in enumerate(zip(shards, widths)):
        if w:
            first = sh.begin // block_size
            out[s, :w] = block_table[s, first:first + w]
    return out


def decode_kv_shard(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                    shards: Sequence[KvShard], local_tables: torch.Tensor, softmax_scale: float,
                    key_scale, value_scale, *, partition_size: int = 256,
                    query_scale: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """This rank's ``(m, l, o)`` triples for its ranges: partition kernel + reduce kernel.

    ``query`` ``[S, Hkv*L*G, D]`` is the full query (every rank has it); ``key_cache`` /
    ``value_cache`` are this rank's pools and ``local_tables`` (from :func:`local_block_table`)
    indexes them.  With ``query_len > 1`` the ranges that hold the end of their context and those
    that do not are computed by two launches (they differ in ``query_len``, see
    :attr:`KvShard.local_query_len`).  Returns fp32 ``m, l`` ``[R]`` and ``o`` ``[R, D]`` with
    ``R = S * Hkv * L * G`` rows in query order; rows of empty ranges hold ``m = -inf, l = 0``.
    """
    from . import _lib
    from .pa_decode import build_params

    if not query.is_cuda:
        raise RuntimeError("decode_kv_shard runs on CUDA tensors only; there is no CPU fallback")
    S, rows_per_seq, D = query.shape
    if len(shards) != S:
        raise ValueError("one shard per sequence expected")
    dev = query.device
    R = S * rows_per_seq
    L = _lib.lib()

    def run(qlen: int, lens: List[int]):
        ctx = torch.tensor(lens, dtype=torch.int32).to(dev)
        out = torch.empty_like(query)     # the reduce kernel also writes the bf16 rows; unused here
        m = torch.empty(R, dtype=torch.float32, device=dev)
        l = torch.empty(R, dtype=torch.float32, device=dev)
        o = torch.empty((R, D), dtype=torch.float32, device=dev)
        p, keep = build_params(out, query, key_cache, value_cache, ctx, local_tables, softmax_scale, qlen,
                               max(lens + [1]), None, query_scale, key_scale, value_scale, None, partition_size,
                               None, None, None, status, None)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(L.pa_partition_sm100(C.byref(p), stream), "pa_partition_sm100")
            _lib.check(L.pa_reduce_sm100(C.byref(p), m.data_ptr(), l.data_ptr(), o.data_ptr(), stream),
                       "pa_reduce_sm100")
        del keep
        return m, l, o

    kinds = sorted({sh.local_query_len for sh in shards if sh.tokens > 0})
    if len(kinds) <= 1:
        return run(kinds[0] if kinds else 1, [sh.local_context_len for sh in shards])
    # two kinds of ranges: one launch each with the other kind's lengths set to zero, then every
    # sequence takes its rows from the launch of its kind
    parts = [run(k, [sh.local_context_len if sh.local_query_len == k else 0 for sh in shards]) for k in kinds]
    first = torch.tensor([sh.local_query_len == kinds[0] for sh in shards], device=dev)
    pick = first.repeat_interleave(rows_per_seq)
    m = torch.where(pick, parts[0][0], parts[1][0])
    l = torch.where(pick, parts[0][1], parts[1][1])
    o = torch.where(pick[:, None], parts[0][2], parts[1][2])
    return m, l, o


def all_gather_triples(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, group=None
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """All-gather of the triples over ``group``: ``[R]``, ``[R]``, ``[R, D]`` -> ``[W, R]``, ``[W, R]``,
    ``[W, R, D]``.  ``m`` and ``l`` travel as one ``[2, R]`` message, so a call is two collectives."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ml = torch.stack([m, l]).contiguous()                    # [2, R]
    R, D = o.shape
    # outputs are the ranks' tensors concatenated along dim 0 (the form every backend accepts)
    ml_all = torch.empty((world * 2, R), dtype=ml.dtype, device=ml.device)
    o_all = torch.empty((world * R, D), dtype=o.dtype, device=o.device)
    dist.all_gather_into_tensor(ml_all, ml, group=group)
    dist.all_gather_into_tensor(o_all, o.contiguous(), group=group)
    ml_all = ml_all.view(world, 2, R)
    return ml_all[:, 0].contiguous(), ml_all[:, 1].contiguous(), o_all.view(world, R, D)


def merge_triples_cuda(m_all: torch.Tensor, l_all: torch.Tensor, o_all: torch.Tensor,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Log-sum-exp merge over the shard axis with the library's merge kernel; returns bf16 ``[R, D]``."""
    from . import _lib

    if not o_all.is_cuda:
        raise RuntimeError("merge_triples_cuda runs on CUDA tensors only; there is no CPU fallback")
    W, R, D = o_all.shape
    if out is None:
        out = torch.empty((R, D), dtype=torch.bfloat16, device=o_all.device)
    flat = out.view(-1, D)
    if flat.shape[0] != R or flat.stride(1) != 1:
        raise ValueError("out must hold R rows of D contiguous elements")
    m_all, l_all, o_all = m_all.contiguous(), l_all.contiguous(), o_all.contiguous()
    L = _lib.lib()
    with torch.cuda.device(o_all.device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(L.pa_merge_triples_sm100(flat.data_ptr(), flat.stride(0), m_all.data_ptr(), l_all.data_ptr(),
                                            o_all.data_ptr(), W, R, D, stream), "pa_merge_triples_sm100")
    return out


def gather_and_merge(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, group=None,
                     merge: Optional[Callable] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exchange this rank's triples and merge them; every rank ends up with the full result.

    ``merge`` defaults to :func:`merge_triples_cuda`; tests of the host logic on a CPU backend
    pass their own statement of the merge.
    """
    m_all, l_all, o_all = all_gather_triples(m, l, o, group)
    if merge is not None:
        return merge(m_all, l_all, o_all)
    return merge_triples_cuda(m_all, l_all, o_all, out)


class PeerExchange:
    """The triple exchange over NVLink peer stores instead of an all-gather.

    Every rank owns a receive buffer (two parities x world x rows of flagged 16-byte lines); the
    constructor maps all ranks' buffers into this rank's device through CUDA IPC (ranks of one
    node, one process each).  Per decode step, :meth:`reduce_push` runs the reduce kernel with
    its triples stored straight into every rank's buffer, and :meth:`merge` merges the rows from
    the local buffer, waiting (bounded) for lines that have not arrived.  Data only ever moves
    by stores into the consumer's memory; the step number is counted on the device, so both
    launches take the same arguments every step and can be captured in a CUDA graph.
    """

    def __init__(self, num_rows: int, head_size: int, device: torch.device, group=None):
        import torch.distributed as dist
        from . import _lib

        self._lib = _lib
        self._L = _lib.lib()
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_rows, self.head_size = num_rows, head_size
        nbytes = int(self._L.pa_exchange_bytes(self.world, num_rows, head_size))
        if nbytes <= 0:
            raise ValueError("nothing to exchange (no rows, or an unsupported head size)")
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)   # [1]: steps merged, counted on the device
        # an allocation of its own per rank: an inter-process handle names a whole allocation
        handle = C.create_string_buffer(_lib.PA_IPC_HANDLE_BYTES)
        own = C.c_void_p()
        with torch.cuda.device(device):
            _lib.check(self._L.pa_exchange_alloc(nbytes, C.byref(own), handle), "pa_exchange_alloc")
        self._own = own.value
        everyone: List = [None] * self.world
        dist.all_gather_object(everyone, handle.raw, group=group)
        self._mapped: List[int] = []      # what close() has to unmap
        bases = []
        for g, raw in enumerate(everyone):
            if g == self.rank:
                bases.append(self._own)
                continue
            ptr = C.c_void_p()
            with torch.cuda.device(device):   # the mapping belongs to the device that is current here
                _lib.check(self._L.pa_exchange_open(raw, C.byref(ptr)), "pa_exchange_open")
            self._mapped.append(ptr.value)
            bases.append(ptr.value)
        self._recv_ptrs = (C.c_void_p * self.world)(*bases)
        dist.barrier(group)       # every rank has mapped every buffer before anybody stores

    def close(self) -> None:
        """Unmaps the peers' buffers, then (after every rank has done so) frees this rank's.
        Collective: all ranks call it, with no step in flight."""
        import torch.distributed as dist
        if self._own is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for ptr in self._mapped:
                self._lib.check(self._L.pa_exchange_close(ptr), "pa_exchange_close")
            self._mapped = []
            dist.barrier(self.group)
            self._lib.check(self._L.pa_exchange_free(self._own), "pa_exchange_free")
        self._own = None

    def reduce_push(self, params) -> None:
        """Next step: the reduce over this rank's partitions, its triples stored into every rank's buffer."""
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            self._lib.check(self._L.pa_reduce_push_sm100(C.byref(params), self._recv_ptrs, self.counters.data_ptr(),
                                                         self.world, self.rank, 0, stream), "pa_reduce_push_sm100")

    def merge(self, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Merges the current step's triples of all ranks into ``out`` (bf16), waiting for late ones."""
        flat = out.view(-1, self.head_size)
        with torch.cuda.device(out.device):
            stream = torch.cuda.current_stream().cuda_stream
            self._lib.check(self._L.pa_merge_wait_sm100(flat.data_ptr(), flat.stride(0), self._own,
                                                        self.counters.data_ptr(),
                                                        status.data_ptr() if status is not None else None,
                                                        self.world, 0, self.num_rows, self.head_size, stream),
                            "pa_merge_wait_sm100")
        return out


class KvShardedDecoder:
    """One rank's side of KV-partition-sharded decode with everything per-batch prepared once.

    The parameter block, the local block tables, the workspaces and the exchange buffers are
    built in the constructor; :meth:`step` then only launches (partition kernel, reduce kernel
    with triples, one all-gather, merge kernel), so a decode loop pays no per-step host work
    beyond the launches.  The kernels read the context lengths from device memory on every
    step, so ``self.context_lens`` may be updated in place between steps as sequences grow
    within their last partition.  Restricted to batches whose ranges need one launch
    (``query_len == 1``, or all ranges of this rank of one kind).
    """

    def __init__(self, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                 shards: Sequence[KvShard], block_tables: torch.Tensor, softmax_scale: float,
                 key_scale, value_scale, *, partition_size: int = 256, group=None,
                 status: Optional[torch.Tensor] = None, exchange: str = "nccl"):
        import torch.distributed as dist
        from . import _lib
        from .pa_decode import build_params

        if not query.is_cuda:
            raise RuntimeError("KvShardedDecoder runs on CUDA tensors only; there is no CPU fallback")
        kinds = sorted({sh.local_query_len for sh in shards if sh.tokens > 0})
        if len(kinds) > 1:
            raise ValueError("ranges of two kinds need decode_kv_shard (two launches)")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        dev = query.device
        S, rows, D = query.shape
        R = S * rows
        block_size = value_cache.shape[-1]
        self.query = query
        self.tables = local_block_table(block_tables, shards, block_size)
        lens = [sh.local_context_len for sh in shards]
        self.context_lens = torch.tensor(lens, dtype=torch.int32).to(dev)
        self.kv_bytes = sum(lens) * key_cache.shape[1] * D * 2 * key_cache.element_size()
        self._scratch_out = torch.empty_like(query)
        self._lib = _lib
        self._L = _lib.lib()
        # this rank's message m | l | pad | o, and the gathered messages of all ranks
        self.msg_floats = int(self._L.pa_packed_triple_floats(R, D))
        self.msg = torch.empty(self.msg_floats, dtype=torch.float32, device=dev)
        self.msg_all = torch.empty(self.world * self.msg_floats, dtype=torch.float32, device=dev)
        self._o_off = self.msg_floats - R * D
        self._rows = R
        self.out = torch.empty((S, rows, D), dtype=torch.bfloat16, device=dev)
        self.params, self._keep = build_params(
            self._scratch_out, query, key_cache, value_cache, self.context_lens, self.tables, softmax_scale,
            kinds[0] if kinds else 1, max(lens + [1]), None, None, key_scale, value_scale, None, partition_size,
            None, None, None, status, None)
        self.launches_per_step = 3
        # the exchange: one NCCL all-gather, or peer stores over NVLink ("p2p", ranks of one node)
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.status = status
        self.peer = PeerExchange(R, D, dev, group) if (exchange == "p2p" and self.world > 1) else None

    def close(self) -> None:
        """Releases the peer exchange's mapped buffers (collective; a no-op for the NCCL exchange)."""
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def capture(self) -> "torch.cuda.CUDAGraph":
        """One step captured in a CUDA graph (collective: every rank calls it).  The launches of a
        step take the same arguments every time (the peer exchange counts its steps on the
        device), and three short kernels per step are otherwise bound by the host's launch rate."""
        self.step()                       # anything lazy (communicator set-up) happens outside the capture
        torch.cuda.synchronize(self.query.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step()
        return graph

    def step(self) -> torch.Tensor:
        """Launches one decode step on the current stream; returns the merged bf16 output
        ``[S, Hkv*L*G, D]`` (the same tensor every step)."""
        import torch.distributed as dist
        L, lib = self._L, self._lib
        R, D = self._rows, self.out.shape[-1]
        base = self.msg.data_ptr()
        with torch.cuda.device(self.query.device):
            stream = torch.cuda.current_stream().cuda_stream
            lib.check(L.pa_partition_sm100(C.byref(self.params), stream), "pa_partition_sm100")
            if self.peer is not None:   # the reduce stores into every rank's buffer; merge what arrives here
                self.peer.reduce_push(self.params)
                return self.peer.merge(self.out, self.status)
            lib.check(L.pa_reduce_sm100(C.byref(self.params), base, base + 4 * R, base + 4 * self._o_off, stream),
                      "pa_reduce_sm100")
            gathered = self.msg
            if self.world > 1:      # one collective per step
                dist.all_gather_into_tensor(self.msg_all, self.msg, group=self.group)
                gathered = self.msg_all
            lib.check(L.pa_merge_packed_triples_sm100(self.out.data_ptr(), D, gathered.data_ptr(), self.world, R, D,
                                                      stream), "pa_merge_packed_triples_sm100")
        return self.out
