"""Sharding of a large GEMM over the GPUs of one box: column-wise (N) with the gather of the bf16 slices, and
K-wise (row-parallel layers) with the reduce-scatter of fp32 partials.

The reference is single-GPU (no collective call sites anywhere in its tree).  Output columns of
``x @ y.T`` are independent, so rank r keeps rows ``[n0, n1)`` of the weight ``y`` (and the matching rows
of the 128x128-block weight scales), every rank holds the full activation ``x``, and each computes its
``[M, n1 - n0]`` slice with the unchanged single-GPU kernel: no communication inside the GEMM.  Only when
the caller needs the whole matrix are the slices exchanged: with one NCCL all-gather over NVLink
(`all_gather_slices`), or by the GEMM kernel itself, whose epilogue stores every block into every rank's matrix
through mapped peer memory (`FusedGatherGemm`).  With K sharded instead, every rank computes fp32 partial sums of
the whole output over its K slice; row blocks are exchanged by one all-to-all (`matmul_blockwise_ksharded`) or
stored by the GEMM epilogue straight into the owning rank's receive area (`FusedReduceScatterGemm`), and added in
rank order.

One process per GPU; ``torch.distributed`` must be initialised by the caller (backend "nccl" on GPUs;
the index logic also runs under "gloo" on CPU tensors, which is how it is tested without GPUs).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

KBLOCK = 128


def shard_bounds(N: int, world: int, rank: int, block: int = KBLOCK) -> tuple[int, int]:
    """Rows [n0, n1) of the weight owned by `rank`: whole 128-row blocks, as even as possible, so that a
    shard never splits a weight-scale block.  Trailing ranks may own fewer (or zero) rows."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    nb = -(-N // block)
    base, extra = divmod(nb, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * block, N), min(b1 * block, N)


def shard_weight(y: torch.Tensor, w_scale: Optional[torch.Tensor], rank: int, world: int):
    """Returns this rank's (y rows, weight-scale rows) as contiguous tensors."""
    n0, n1 = shard_bounds(y.shape[0], world, rank)
    ys = y[n0:n1].contiguous()
    if w_scale is None:
        return ys, None
    if w_scale.dim() == 1:  # per-output-channel scales [N]
        return ys, w_scale[n0:n1].contiguous()
    return ys, w_scale[n0 // KBLOCK: -(-n1 // KBLOCK)].contiguous()


def uniform_shards(N: int, world: int) -> bool:
    sizes = {shard_bounds(N, world, r)[1] - shard_bounds(N, world, r)[0] for r in range(world)}
    return len(sizes) == 1


def all_gather_slices(local: torch.Tensor, out: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """All-gathers equal-sized ``[M, n_local]`` slices into ``[world, M, n_local]`` (block layout: slice r is
    the r-th column block of the full matrix).  One collective, no copy; `out` may be preallocated."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    # concatenation along dim 0 of the flattened view == stacking into [world, M, n_local]
    dist.all_gather_into_tensor(out.view(world * local.shape[0], *local.shape[1:]), local.contiguous(), group=group)
    return out


def assemble_row_major(blocks: torch.Tensor) -> torch.Tensor:
    """``[world, M, n_local]`` block layout -> row-major ``[M, world * n_local]`` (one permuting copy)."""
    g, M, n = blocks.shape
    return blocks.permute(1, 0, 2).reshape(M, g * n)


def all_gather_ragged(local: torch.Tensor, N: int, group=None) -> torch.Tensor:
    """Gather for shard widths that differ between ranks: every slice is padded to the widest shard, gathered
    with the same single collective, and the padding is dropped while assembling row-major ``[M, N]``."""
    world = dist.get_world_size(group)
    M = local.shape[0]
    bounds = [shard_bounds(N, world, r) for r in range(world)]
    widest = max(n1 - n0 for n0, n1 in bounds)
    padded = local
    if local.shape[1] != widest:
        padded = torch.zeros((M, widest), dtype=local.dtype, device=local.device)
        padded[:, : local.shape[1]] = local
    blocks = all_gather_slices(padded, group=group)
    return torch.cat([blocks[r, :, : n1 - n0] for r, (n0, n1) in enumerate(bounds)], dim=1)


def matmul_blockwise_nsharded(x_q: torch.Tensor, w_q_shard: torch.Tensor, x_scale: torch.Tensor,
                              w_scale_shard: torch.Tensor, N: int, gather: bool = True, row_major: bool = True,
                              group=None, compute: Optional[Callable] = None) -> torch.Tensor:
    """Blockwise W8A8 GEMM with the weight sharded over N.

    Each rank passes the full activations and ITS weight shard (see `shard_weight`).  With ``gather=False``
    the local ``[M, n_local]`` slice is returned and nothing is communicated.  With ``gather=True`` every rank
    gets the full result: row-major ``[M, N]`` (``row_major=True``, costs one permuting copy) or the
    ``[world, M, n_local]`` block layout straight out of the collective.
    `compute` replaces the local GEMM (tests inject a CPU checker there); by default it is the CUDA op.
    """
    if compute is None:
        from . import matmul_blockwise as compute
    local = compute(x_q, w_q_shard, x_scale, w_scale_shard)
    if not gather:
        return local
    world = dist.get_world_size(group)
    if uniform_shards(N, world):
        blocks = all_gather_slices(local, group=group)
        return assemble_row_major(blocks) if row_major else blocks
    return all_gather_ragged(local, N, group=group)


def kshard_bounds(K: int, world: int, rank: int, block: int = KBLOCK) -> tuple[int, int]:
    """Columns [k0, k1) of x and of the weight owned by `rank` in a K-sharded (row-parallel) layer: whole 128-wide
    K blocks, as even as possible, so that no scale block is split."""
    return shard_bounds(K, world, rank, block)


def matmul_blockwise_ksharded(x_q_shard: torch.Tensor, w_q_shard: torch.Tensor, x_scale_shard: torch.Tensor,
                              w_scale_shard: torch.Tensor, group=None, compute: Optional[Callable] = None,
                              reduce: Optional[Callable] = None) -> torch.Tensor:
    """Blockwise W8A8 GEMM with K sharded over the ranks (a row-parallel layer), reduce-scattered over token rows.

    Rank r passes its K slice of everything: ``x_q[:, k0:k1]``, ``w_q[:, k0:k1]`` and the matching columns of both
    scale arrays (see `kshard_bounds`).  Every rank computes the fp32 accumulators of its slice for the whole
    ``[M, N]`` output (one fused multiply-add per K block, ascending, as the unsharded kernel does), the ranks
    exchange row blocks with one all-to-all (rank j receives rows ``[j M/g, (j+1) M/g)`` of every rank's partial:
    the bytes of a reduce-scatter), and each rank adds the g partials of its rows IN RANK ORDER and casts to bf16.
    The result therefore is ``bf16(((acc_0 + acc_1) + acc_2) + ...)`` with acc_r the chain over rank r's K blocks --
    a fixed order, which a CPU restatement reproduces bit for bit; it is not the unsharded kernel's single chain
    (the difference is fp32 rounding of g - 1 additions).  M must be a multiple of the world size.
    Returns this rank's bf16 ``[M / g, N]`` rows.
    `compute` / `reduce` replace the local GEMM and the ordered sum (tests inject CPU checkers there).
    """
    if compute is None:
        from . import matmul_blockwise_f32 as compute
    if reduce is None:
        from . import sum_parts_bf16 as reduce
    world = dist.get_world_size(group)
    part = compute(x_q_shard, w_q_shard, x_scale_shard, w_scale_shard)  # fp32 [M, N]
    M, N = part.shape
    if M % world:
        raise ValueError(f"M={M} must be a multiple of the world size {world}")
    if world == 1:
        return reduce(part.reshape(1, M, N))
    recv = torch.empty((world, M // world, N), dtype=part.dtype, device=part.device)
    # send buffer viewed as [world, M/world, N]: block j goes to rank j; received block r came from rank r
    dist.all_to_all_single(recv.view(-1), part.contiguous().view(-1), group=group)
    return reduce(recv)


class FusedGatherGemm:
    """N-sharded blockwise GEMM whose epilogue writes every output block straight into every rank's full
    [M, N] matrix (TMA stores through mapped peer memory), so the all-gather rides on the GEMM tile by tile and no
    collective or permuting copy follows.

    Set-up (once per output shape): every rank allocates TWO [M, N] bf16 matrices with the library's peer allocator,
    the CUDA IPC handles are exchanged through `torch.distributed` (object all-gather: host side, any backend), and
    each rank maps the others' matrices.  Per call: one kernel launch, then a barrier after which the returned
    matrix is complete on every rank.  Ranks must be processes on one node with peer access between their GPUs;
    no multicast is used.

    Lifetime of a result.  Peers write into this rank's matrix, so a result can be overwritten from outside.  Calls
    alternate between the two matrices: the matrix returned by call i is written again by call i + 2, and a peer
    can start its call i + 2 only after the barrier of call i + 1 has completed, i.e. after THIS rank's stream has
    reached its own barrier of call i + 1.  Hence the rule: consume the result of call i on the stream `run` was
    called on (or make that stream wait for the consumer) before calling `run` for the second time after it; with
    that, no cross-rank write-after-read can happen.  The barrier must be stream-ordered (NCCL); with a host-only
    backend `run` synchronises the stream before the barrier instead.
    """

    def __init__(self, M: int, N: int, group=None):
        import ctypes

        import torch.distributed as dist

        from . import _C, _lib

        self._C, self._lib, self._ct = _C, _lib, ctypes
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("FusedGatherGemm supports at most 8 ranks")
        self.M, self.N = M, N
        self.lo, self.hi = shard_bounds(N, self.world, self.rank)
        if N % 8 or self.lo % 32 or (self.hi % 32 and self.hi != N):
            raise ValueError("N must be a multiple of 8 and every shard a multiple of 32 columns")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._stream_ordered = dist.get_backend(group) == "nccl"
        nbytes = M * N * 2
        self._own, self._mapped, self._outs, self._views = [], [], [], []
        for _ in range(2):
            own = ctypes.c_void_p()
            _lib.check(_C, _C.gi8_peer_alloc(ctypes.byref(own), nbytes))
            self._own.append(own)
            handle = (ctypes.c_ubyte * 64)()
            _lib.check(_C, _C.gi8_peer_export(own, handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(own.value)
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = ctypes.c_void_p()
                _lib.check(_C, _C.gi8_peer_import(buf, ctypes.byref(p)))
                self._mapped.append(p)
                ptrs.append(p.value)
            # own matrix first, then the peers in cyclic order from this rank on (the entry point takes any order; the
            # kernel stores every block to the matrices in this order, so at any moment the ranks address different peers)
            order = [(self.rank + i) % self.world for i in range(self.world)]
            self._outs.append((ctypes.c_void_p * self.world)(*[ptrs[r] for r in order]))
            self._views.append(_tensor_from_ptr(own.value, (M, N), self.device))
        self._turn = 0
        dist.barrier(group=group)  # every rank has mapped every matrix before anyone writes

    def run(self, x_q: torch.Tensor, w_q_shard: torch.Tensor, x_scale: torch.Tensor, w_scale_shard: torch.Tensor,
            barrier: bool = True) -> torch.Tensor:
        """Launches the GEMM on the current stream; with `barrier` also the cross-rank barrier after which the
        returned [M, N] bf16 tensor (one of this rank's two matrices) is complete.  See the class docstring for how
        long the returned tensor stays valid."""
        import torch.distributed as dist

        M, K = x_q.shape
        n_local = w_q_shard.shape[0]
        if M != self.M or n_local != self.hi - self.lo:
            raise ValueError("operand shapes do not match the gather buffers")
        turn = self._turn
        self._turn ^= 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._C.gi8_matmul_blockwise_allgather(
            x_q.data_ptr(), w_q_shard.data_ptr(), x_scale.data_ptr(), x_scale.stride(0), w_scale_shard.data_ptr(),
            w_scale_shard.stride(0), self._outs[turn], self.world, M, n_local, K, self.N, self.lo, stream)
        self._lib.check(self._C, rc)
        if barrier:
            if not self._stream_ordered:
                torch.cuda.current_stream(self.device).synchronize()  # a host-only barrier orders nothing on the GPU
            dist.barrier(group=self.group)
        return self._views[turn]

    def result(self) -> torch.Tensor:
        """The matrix the most recent `run` wrote."""
        return self._views[self._turn ^ 1]

    def close(self) -> None:
        """Unmaps the peers' matrices and frees this rank's (collective: every rank must call it)."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._mapped:
            self._lib.check(self._C, self._C.gi8_peer_release(p))
        self._mapped = []
        self._views = []
        dist.barrier(group=self.group)  # nobody frees while a peer still has the matrix mapped
        for own in self._own:
            self._lib.check(self._C, self._C.gi8_peer_free(own))
        self._own = []


class FusedReduceScatterGemm:
    """K-sharded (row-parallel) blockwise GEMM whose epilogue stores the fp32 accumulators of every row block straight
    into the receive area of the rank that owns those rows (TMA stores through mapped peer memory), followed by a
    barrier and the ordered sum + cast (`sum_parts_bf16`): the data movement of the reduce-scatter rides on the GEMM
    tile by tile, and the result is bit-identical to `matmul_blockwise_ksharded` (same chains, same order of the sum).

    Set-up (once per output shape): every rank allocates TWO receive areas, float ``[world, M / world, N]``, with the
    library's peer allocator; CUDA IPC handles are exchanged through `torch.distributed`.  Calls alternate between the
    two areas, which closes the cross-rank write-after-read window exactly as in `FusedGatherGemm` (consume the
    result of call i before calling `run` for the second time after it; the barrier must be stream-ordered, i.e. NCCL,
    otherwise `run` synchronises the stream first).  M must be a multiple of 32 * world, N of 4; at most 8 ranks.
    """

    def __init__(self, M: int, N: int, group=None):
        import ctypes

        import torch.distributed as dist

        from . import _C, _lib

        self._C, self._lib, self._ct = _C, _lib, ctypes
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("FusedReduceScatterGemm supports at most 8 ranks")
        if M % (32 * self.world) or N % 4:
            raise ValueError("M must be a multiple of 32 x world size and N a multiple of 4")
        self.M, self.N, self.rows = M, N, M // self.world
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._stream_ordered = dist.get_backend(group) == "nccl"
        nbytes = self.world * self.rows * N * 4
        self._own, self._mapped, self._recv, self._views = [], [], [], []
        for _ in range(2):
            own = ctypes.c_void_p()
            _lib.check(_C, _C.gi8_peer_alloc(ctypes.byref(own), nbytes))
            self._own.append(own)
            handle = (ctypes.c_ubyte * 64)()
            _lib.check(_C, _C.gi8_peer_export(own, handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(own.value)
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = ctypes.c_void_p()
                _lib.check(_C, _C.gi8_peer_import(buf, ctypes.byref(p)))
                self._mapped.append(p)
                ptrs.append(p.value)
            self._recv.append((ctypes.c_void_p * self.world)(*ptrs))   # indexed by owning rank
            self._views.append(_tensor_from_ptr(own.value, (self.world, self.rows, N), self.device, torch.float32))
        self._turn = 0
        dist.barrier(group=group)  # every rank has mapped every area before anyone writes

    def run(self, x_q_shard: torch.Tensor, w_q_shard: torch.Tensor, x_scale_shard: torch.Tensor,
            w_scale_shard: torch.Tensor) -> torch.Tensor:
        """One kernel launch on the current stream, the cross-rank barrier, the ordered sum: returns this rank's bf16
        ``[M / world, N]`` rows."""
        import torch.distributed as dist

        from . import sum_parts_bf16

        M, _ = x_q_shard.shape
        N = w_q_shard.shape[0]
        if M != self.M or N != self.N:
            raise ValueError("operand shapes do not match the receive areas")
        turn = self._turn
        self._turn ^= 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._C.gi8_matmul_blockwise_f32_scatter(
            x_q_shard.data_ptr(), w_q_shard.data_ptr(), x_scale_shard.data_ptr(), x_scale_shard.stride(0),
            w_scale_shard.data_ptr(), w_scale_shard.stride(0), self._recv[turn], self.world, self.rank, M, N,
            x_q_shard.shape[1], stream)
        self._lib.check(self._C, rc)
        if not self._stream_ordered:
            torch.cuda.current_stream(self.device).synchronize()  # a host-only barrier orders nothing on the GPU
        dist.barrier(group=self.group)
        return sum_parts_bf16(self._views[turn])

    def close(self) -> None:
        """Unmaps the peers' areas and frees this rank's (collective: every rank must call it)."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._mapped:
            self._lib.check(self._C, self._C.gi8_peer_release(p))
        self._mapped = []
        self._views = []
        dist.barrier(group=self.group)  # nobody frees while a peer still has the area mapped
        for own in self._own:
            self._lib.check(self._C, self._C.gi8_peer_free(own))
        self._own = []


def _tensor_from_ptr(ptr: int, shape, device: torch.device, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """A bf16 (or fp32) tensor over device memory the library allocated (kept alive by its owner, not by the tensor)."""
    n = 1
    for d in shape:
        n *= d
    typestr, raw = ("<i2", torch.int16) if dtype == torch.bfloat16 else ("<i4", torch.int32)

    class _Mem:
        __cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3}

    t = torch.as_tensor(_Mem(), device=device)
    assert t.dtype == raw
    return t.view(dtype).view(*shape)
