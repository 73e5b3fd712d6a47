"""Tensor-parallel sharding of packed RPTC layers.

Rows of a weight matrix are independent trellis streams, so a column-parallel layer (split by
output rows) is a plain slice of the packed codes.  A row-parallel layer (split by input columns)
cuts every row's stream: the shard on the right needs the 16 bits that precede its first unit,
which are the low half of the last word of the shard on its left (`carry_in`); nothing is
re-encoded.  Both helpers work on the TILED layout [m/32][units][32][4].
"""
from __future__ import annotations

import torch

from ._lib import LAYOUT_TILED
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
