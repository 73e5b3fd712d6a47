"""Tensor-parallel sharding of packed RPTC layers.

Rows of a weight matrix are independent trellis streams, so a column-parallel layer (split by
output rows) is a plain slice of the packed codes.  A row-parallel layer (split by input columns)
cuts every row's stream: the shard on the right needs the 16 bits that precede its first unit,
which are the low half of the last word of the shard on its left (`carry_in`); nothing is
re-encoded.  Both helpers work on the TILED layout [m/32][units][32][4].
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import LAYOUT_TILED, check, lib, ptr, stream_ptr
from .linear import RPTCLinear, hadamard_block


def _need_tiled(lin: RPTCLinear) -> None:
    if lin.fmt.layout != LAYOUT_TILED:
        raise ValueError("sharding works on the TILED layout; repack first")


def shard_rows(lin: RPTCLinear, rank: int, world: int) -> RPTCLinear:
    """Column-parallel shard: output rows [rank*m/world, (rank+1)*m/world)."""
    _need_tiled(lin)
    m = lin.out_features
    if m % (32 * world):
        raise ValueError("out_features must be a multiple of 32 * world")
    ml = m // world
    codes = lin.codes[rank * ml // 32:(rank + 1) * ml // 32].contiguous()
    so = None if lin.signs_out is None else lin.signs_out[rank * ml:(rank + 1) * ml].contiguous()
    ci = None if lin.carry_in is None else lin.carry_in[rank * ml:(rank + 1) * ml].contiguous()
    out = RPTCLinear(lin.in_features, ml, lin.fmt, codes, lin.lut, lin.scale, lin.signs_in, so, ci)
    out.block_in = lin.block_in
    out.block_out = min(lin.block_out, hadamard_block(ml))
    if lin.incoherent and ml % lin.block_out:
        raise ValueError("a Hadamard block of the output transform straddles the shard boundary")
    return out


def shard_cols(lin: RPTCLinear, rank: int, world: int) -> RPTCLinear:
    """Row-parallel shard: input columns [rank*n/world, (rank+1)*n/world); partial outputs must be summed."""
    _need_tiled(lin)
    nu = lin.codes.shape[1]
    if nu % world:
        raise ValueError("the number of 128-bit units per row must be divisible by world")
    ul = nu // world
    nl = lin.in_features // world
    if lin.incoherent and nl % lin.block_in:
        raise ValueError("a Hadamard block of the input transform straddles the shard boundary")
    u0 = rank * ul
    codes = lin.codes[:, u0:u0 + ul].contiguous()
    if u0 == 0:
        ci = lin.carry_in
    else:
        ci = lin.codes[:, u0 - 1, :, 3].reshape(-1).contiguous()        # last word of the unit to the left, per row
    si = None if lin.signs_in is None else lin.signs_in[rank * nl:(rank + 1) * nl].contiguous()
    out = RPTCLinear(nl, lin.out_features, lin.fmt, codes, lin.lut, lin.scale, si, lin.signs_out, ci)
    out.block_in, out.block_out = lin.block_in, lin.block_out
    return out


class PeerAllReduce:
    """Exchange buffers for `rptc_peer_finish`: the output transform of a row-parallel layer, the all-reduce
    over the tensor-parallel ranks and the residual add as one kernel over NVLink peer memory.

    Each rank allocates a data buffer of [2][world][rows*n/2] 64-bit (payload, epoch) words, exports its CUDA IPC handle
    through `group` (any torch.distributed backend) and maps its peers' buffers.  One object serves every
    row-parallel layer of a model whose output width is `n` (they run one after another on one stream)."""

    def __init__(self, rows: int, n: int, block: int, rank: int, world: int, group=None, timeout_ms: int = 2000):
        import torch.distributed as dist
        self.rows, self.n, self.block, self.rank, self.world, self.timeout_ms = rows, n, block, rank, world, timeout_ms
        chunk = max(block, 256)
        self.n_ctas = rows * (n // chunk)
        L = lib()
        self._own = []
        self._mapped = []

        def alloc(nbytes: int) -> int:
            p = ctypes.c_void_p()
            check(L.rptc_peer_alloc(nbytes, ctypes.byref(p)), "rptc_peer_alloc")
            self._own.append(p.value)
            return p.value

        data = alloc(2 * world * rows * n * 4)      # (payload word, epoch) pairs: twice the fp16 payload
        flags = alloc(world * self.n_ctas * 4)
        self.epochs = torch.zeros(self.n_ctas, dtype=torch.int32, device="cuda")
        handles = []
        for p in (data, flags):
            buf = ctypes.create_string_buffer(64)
            check(L.rptc_peer_export(p, buf), "rptc_peer_export")
            handles.append(buf.raw)
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, handles, group=group)
        else:
            gathered[0] = handles
        self.data_ptrs = (ctypes.c_void_p * world)()
        self.flag_ptrs = (ctypes.c_void_p * world)()
        for r in range(world):
            if r == rank:
                self.data_ptrs[r], self.flag_ptrs[r] = data, flags
                continue
            for k, arr in enumerate((self.data_ptrs, self.flag_ptrs)):
                q = ctypes.c_void_p()
                check(L.rptc_peer_import(gathered[r][k], ctypes.byref(q)), "rptc_peer_import")
                self._mapped.append(q.value)
                arr[r] = q.value
        if world > 1:
            dist.barrier(group=group)

    def finish(self, lin: RPTCLinear, acc: torch.Tensor, h: torch.Tensor) -> None:
        """h += sum over ranks of lin's output transform of acc (acc is cleared)."""
        rows, n = h.shape
        assert rows == self.rows and n == self.n and lin.block_out == self.block
        check(lib().rptc_peer_finish(ptr(acc), acc.stride(0) if rows > 1 else max(n, acc.stride(0)), ptr(lin.signs_out), lin.scale,
                                     ptr(h), h.stride(0) if rows > 1 else max(n, h.stride(0)), self.data_ptrs, self.flag_ptrs,
                                     ptr(self.epochs), self.rank, self.world, rows, n, self.block, self.timeout_ms, stream_ptr()),
              "rptc_peer_finish")

    def close(self) -> None:
        torch.cuda.synchronize()
        for q in self._mapped:
            lib().rptc_peer_close(q)
        for p in self._own:
            lib().rptc_peer_free(p)
        self._mapped, self._own = [], []
