"""Single-request long-context decode with the KV pages split over GPUs.

The reference library is single-device; its serving patch merges per-device
attention states with `_merge_states` (patches/tpu-inference.patch:7174-7186 of
the reference project).  Here one process per GPU holds every world-th logical
page of the request (round-robin) in its own pool; every decode step each rank runs
the split-KV decode kernel over its own pages in partial-state mode; then the
sink-free `(o, lse)` states (33 KB per rank for 64 heads) are exchanged and
merged.  Two exchanges are built: "p2p" (default) - the decode launch's combine
kernel stores the rank's state straight into every rank's exchange buffer over
NVLink as {value, epoch} pairs, and the merge kernel polls its own buffer until
all ranks' pairs carry the step's epoch (fw_sharded_decode_step: three launches
per step, no flag, fence or collective library on the data path); "nccl" - an
NCCL all-gather followed by `fw_lse_combine`.  The rank that owns the page
holding position `cache_len` appends the new token; which rank that is, and how
many tokens each rank holds, is worked out on the device every step (by the
merge kernel for the next step, or by fw_shard_step), so one captured CUDA graph
serves a whole generation.

Requests and KV heads need none of this: they shard with no communication
(`request_shard`, `kv_head_shard`).
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch
import torch.distributed as dist

from flywheel_tpu.softmax_attention import _arrays, _native


def owned_pages(total_pages: int, world: int, rank: int) -> range:
    """Logical pages of `rank`: page p lives on rank p % world, as that rank's
    local page p // world.  Round-robin keeps the growing tail of a generation
    moving from GPU to GPU, so every rank holds the same number of pages to
    within one at every length."""
    return range(rank, total_pages, world)


def owner_of_page(page: int, world: int) -> int:
    """Rank that holds logical page `page`."""
    return page % world


def local_length(global_len: int, page_size: int, world: int, rank: int) -> int:
    """How many of the first `global_len` tokens live in `rank`'s pages.  They
    fill a prefix of its local page list, so this is the rank's cache_seqlens."""
    full_pages, tail = divmod(global_len, page_size)
    owned_full = len(range(rank, full_pages, world))
    return owned_full * page_size + (tail if full_pages % world == rank else 0)


def kv_head_shard(nheads: int, nheads_k: int, world: int, rank: int) -> tuple[slice, slice]:
    """(query-head slice, KV-head slice) of `rank` when the KV heads are split
    over `world` GPUs: each GPU keeps nheads_k / world KV heads of every page
    (its pool is (num_pages, page_size, 2 * nheads_k / world, d), same block
    table everywhere) and the query heads that share them.  No communication:
    the ranks' outputs are disjoint head slices of the full output."""
    if nheads_k % world:
        raise ValueError(f"nheads_k={nheads_k} must be a multiple of the {world} ranks.")
    if nheads % nheads_k:
        raise ValueError(f"{nheads=} must be a multiple of {nheads_k=}.")
    per_rank, group = nheads_k // world, nheads // nheads_k
    kv = slice(rank * per_rank, (rank + 1) * per_rank)
    return slice(kv.start * group, kv.stop * group), kv


def request_shard(lengths, world: int, rank: int) -> list[int]:
    """Requests of `rank` when the batch is split over `world` GPUs with no
    communication: longest first, each to the GPU with the fewest cached tokens
    so far, so the ranks stream about the same number of KV bytes."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load, mine = [0] * world, []
    for index in order:
        target = min(range(world), key=lambda r: (load[r], r))
        load[target] += int(lengths[index])
        if target == rank:
            mine.append(index)
    return sorted(mine)


def pack_state(partial_out: torch.Tensor, partial_lse: torch.Tensor) -> torch.Tensor:
    """(rows, d) f32 and (rows,) f32 -> one (rows * (d + 1),) buffer: all o rows,
    then all lse, so the gathered buffer splits back without a copy."""
    return torch.cat([partial_out.reshape(-1), partial_lse.reshape(-1)])


def unpack_states(gathered: torch.Tensor, world: int, rows: int, d: int):
    """Views of a gathered buffer: (world, rows, d) states and (world, rows)
    lse.  Consecutive ranks are rows * (d + 1) elements apart in both."""
    per_rank = gathered.view(world, rows * (d + 1))
    outs = per_rank[:, : rows * d].unflatten(1, (rows, d))
    lses = per_rank[:, rows * d:]
    return outs, lses


@dataclasses.dataclass
class ShardedDecoder:
    """Per-rank state of a long-context decode whose pages are dealt round-robin
    over the ranks of `group`.  `pool` holds this rank's pages (any physical
    order); `table` is this rank's (1, local_pages) block table over its own
    pool, local page i being logical page rank + i * world."""

    pool: torch.Tensor
    table: torch.Tensor
    nheads: int
    nheads_k: int
    group: dist.ProcessGroup | None = None
    softmax_scale: float | None = None
    sinks: torch.Tensor | None = None
    exchange: str = "p2p"

    def __post_init__(self):
        self.device = self.pool.device
        # without a process group there is one rank: it holds every page
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        self.page_size = self.pool.shape[1]
        self.head_dim = self.pool.shape[3]
        rows = self.nheads
        f32 = dict(dtype=torch.float32, device=self.device)
        self.state = torch.empty(rows * (self.head_dim + 1), **f32)
        self.gathered = torch.empty(self.world * rows * (self.head_dim + 1), **f32)
        # [tokens cached (all ranks), tokens on this rank, does this rank append]
        self.counters = torch.zeros(3, dtype=torch.int32, device=self.device)
        self.out = torch.empty((1, 1, self.nheads, self.head_dim), dtype=torch.bfloat16,
                               device=self.device)
        self.lse = torch.empty((1, self.nheads, 1), **f32)
        self.scale = self.softmax_scale or self.head_dim ** -0.5
        self.lib = _native.library()
        self.scratch = None
        self.peers = None
        if self.exchange not in ("p2p", "nccl"):
            raise ValueError(f"exchange must be 'p2p' or 'nccl'; got {self.exchange!r}.")
        if self.exchange == "p2p" and self.world > 1:
            self._open_exchange_buffers()
            self._shard_step(advance=0)   # bookkeeping of length 0, as the fused step expects to find it

    def _open_exchange_buffers(self):
        """Allocates this rank's exchange buffer, passes its IPC handle to the
        peers and maps theirs.  Collective over `group`; set-up, not the step."""
        rows, d = self.nheads, self.head_dim
        nbytes = self.lib.fw_exchange_buffer_bytes(self.world, rows, d)
        if nbytes == 0:
            raise RuntimeError(_native.last_error())
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _native.check(self.lib.fw_peer_alloc(nbytes, ctypes.byref(own), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=self.group)
            pointers = []
            for rank, raw in enumerate(handles):
                if rank == self.rank:
                    pointers.append(own.value)
                    continue
                mapped = ctypes.c_void_p()
                _native.check(self.lib.fw_peer_open(raw, ctypes.byref(mapped)))
                pointers.append(mapped.value)
        self.peers = (ctypes.c_void_p * self.world)(*pointers)
        dist.barrier(group=self.group)   # every rank has mapped every buffer

    def close(self):
        """Unmaps the peers' buffers and frees this rank's.  Collective: no rank
        may still be stepping."""
        if self.peers is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for rank in range(self.world):
                if rank != self.rank:
                    _native.check(self.lib.fw_peer_close(self.peers[rank]))
            dist.barrier(group=self.group)  # nobody maps this buffer any more
            _native.check(self.lib.fw_peer_free(self.peers[self.rank]))
        self.peers = None

    def set_length(self, global_len: int) -> None:
        """Sets the number of tokens cached so far (over all ranks).  Every step
        that carries a new token advances it on the device."""
        self.counters[0:1].fill_(int(global_len))
        if self._fused:
            # the fused step advances the bookkeeping at its end, for the next step: prime it
            self._shard_step(advance=0)

    @property
    def _fused(self) -> bool:
        return self.world > 1 and self.exchange == "p2p"

    def _shard_step(self, advance: int) -> None:
        base = self.counters.data_ptr()
        shard = _native.FwShardStepArgs(
            global_len=base, local_len=base + 4, append_enable=base + 8,
            page_size=self.page_size, world=self.world, rank=self.rank, advance=advance)
        _native.check(self.lib.fw_shard_step(ctypes.byref(shard), _native.current_stream(self.device)))

    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, global_len: int | None = None):
        """One decode step: q (1, 1, nheads, d), new k / v (1, 1, nheads_k, d).
        `global_len`, when given, resets the cached length first; otherwise the
        device counter carries on from the previous step.  Returns (out, lse);
        the new token is appended on the rank that owns its page."""
        if global_len is not None:
            self.set_length(global_len)
        return self._enqueue(q, k, v)

    def capture(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                global_len: int) -> torch.cuda.CUDAGraph:
        """A CUDA graph of one decode step starting at `global_len` cached tokens.
        The cached length, each rank's share of it and which rank appends all
        live on the device and are advanced inside the graph, so the graph can be
        replayed for as long as the block tables have pages; q / k / v are read
        from the given tensors at every replay, so refill them in place between
        replays.  A step is latency-bound (tens of microseconds of HBM time), so
        launching it as one graph matters."""
        self.set_length(global_len)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):            # warm-up outside capture
            self._enqueue(q, k, v, advance=0)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        # thread_local: the process group's watchdog thread may query events meanwhile
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self._enqueue(q, k, v)
        return graph

    def _enqueue(self, q, k, v, advance=1):
        rows, d = self.nheads, self.head_dim
        partial_out = self.state[: rows * d]
        partial_lse = self.state[rows * d:]
        alone = self.world == 1   # one rank holds every page: no partial state, no exchange
        stream = _native.current_stream(self.device)
        base = self.counters.data_ptr()
        advance = advance if k is not None else 0
        fused = self._fused
        if not fused:
            self._shard_step(advance)
        merged = alone or fused   # out / lse / sinks describe the final result
        args = _native.FwDecodeArgs(
            q=q.data_ptr(), out=self.out.data_ptr() if merged else 0, lse=self.lse.data_ptr() if merged else 0,
            kv_cache=self.pool.data_ptr(), v_cache=0,
            k_new=_arrays.data_ptr(k), v_new=_arrays.data_ptr(v), append_enable=base + 8,
            cache_seqlens=base + 4, block_table=self.table.data_ptr(),
            sinks=_arrays.data_ptr(self.sinks) if merged else 0,
            partial_out=0 if merged else partial_out.data_ptr(),
            partial_lse=0 if merged else partial_lse.data_ptr(),
            num_pages=self.pool.shape[0], page_size=self.page_size,
            pages_per_seq=self.table.shape[1], batch=1, seqlen_q=1, nheads=self.nheads,
            nheads_k=self.nheads_k, head_dim=d,
            kv_dtype=_native.DTYPE_CODE[_arrays.dtype_name(self.pool.dtype)],
            # one query token on the last position: every local key is visible
            causal=0, window_left=-1, softmax_scale=self.scale, softcap=0.0, num_ctas=0)
        if self.scratch is None:
            nbytes = self.lib.fw_decode_workspace_bytes(ctypes.byref(args))
            if nbytes == 0:
                raise RuntimeError(_native.last_error())
            self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        args.workspace, args.workspace_bytes = self.scratch.data_ptr(), self.scratch.numel()
        if fused:
            if self.peers is None:
                raise RuntimeError("the exchange buffers were closed.")
            whole = _native.FwShardedDecodeArgs(
                decode=args, peer_buffers=ctypes.cast(self.peers, ctypes.c_void_p), world=self.world,
                rank=self.rank, global_len=base, local_len=base + 4, append_enable=base + 8, advance=advance)
            _native.check(self.lib.fw_sharded_decode_step(ctypes.byref(whole), stream))
            return self.out, self.lse
        _native.check(self.lib.fw_decode_kvcache(ctypes.byref(args), stream))
        if alone:
            return self.out, self.lse
        dist.all_gather_into_tensor(self.gathered, self.state, group=self.group)
        outs, lses = unpack_states(self.gathered, self.world, rows, d)
        merge = _native.FwCombineArgs(
            partial_out=outs.data_ptr(), partial_lse=lses.data_ptr(),
            sinks=_arrays.data_ptr(self.sinks), out=self.out.data_ptr(), lse=self.lse.data_ptr(),
            parts=self.world, rows=rows, nheads=self.nheads, head_dim=d, lse_head_stride=1,
            lse_token_stride=self.nheads, part_stride_out=rows * (d + 1),
            part_stride_lse=rows * (d + 1))
        _native.check(self.lib.fw_lse_combine(ctypes.byref(merge), stream))
        return self.out, self.lse
