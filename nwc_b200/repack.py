"""Cutting a compressed matrix into tensor-parallel shards without decoding it.

Blocks are coded independently and share only the per-tensor symbol table (`lut`), and they are stored row-group-major
with their payloads contiguous in block order (reference: csrc/nwc_ops.cu:87-98 for the geometry, 288-316 for the block
order and the `bases` offsets).  So a shard is a re-pack, not a re-encode:

  rows (column-parallel: q/k/v, gate/up, lm_head)   whole row groups [r0, r1): one contiguous span of `data`, a slice of
        `bases` (rebased), `hdr` and of the raw plane(s); several ranges (the q, k and v parts of a fused projection) are
        concatenated in order;
  cols (row-parallel: o, down)   whole column blocks [c0, c1): per row group one contiguous run of blocks, runs
        concatenated; the raw planes are sliced by columns (layout 0) or by super-chunk slots (layouts 1, 2).

`lut` (and `scale` for row slices) carry over unchanged.  Everything here is index arithmetic on torch tensors, on any
device; nothing imports the CUDA library, so it is tested on the CPU against the oracle's decoder.
"""
from dataclasses import dataclass

import torch

LANES, BLOCK_COLS, RAW_SLACK, DATA_SLACK = 32, 512, 512, 64


@dataclass
class Geometry:
    """Sizes of an M x K matrix in layout 0 (8-row blocks) or 1 / 2 (16-row blocks); the formulas of the format."""
    M: int
    K: int
    layout: int
    fp8: bool

    def __post_init__(self):
        self.rows = 16 if self.layout else 8
        self.K16 = (self.K + 15) // 16 * 16
        self.CB = (self.K + BLOCK_COLS - 1) // BLOCK_COLS
        self.groups = (self.M + self.rows - 1) // self.rows
        self.nb = self.groups * self.CB
        last_chunks = (self.K16 - (self.CB - 1) * BLOCK_COLS) // 16
        self.last_super = (last_chunks + 1) // 2
        self.slots = 16 * (self.CB - 1) + self.last_super                       # super-chunk slots per row group (layouts 1, 2)
        self.pair_slots = 8 * (self.CB - 1) + (self.last_super + 1) // 2       # layout 2 fp8 raw plane
        self.unit = (2 if self.fp8 else 3) if self.layout == 2 else 4          # bytes per hdr count: exception entry / stream word

    @property
    def nibble_plane(self): return self.groups * self.slots * LANES * 8

    @property
    def raw_bytes(self):
        if self.layout == 2:
            return self.nibble_plane + (self.groups * self.pair_slots * 3 * LANES * 4 if self.fp8 else self.groups * self.slots * LANES * 16)
        if self.layout == 1: return self.groups * self.slots * LANES * (8 if self.fp8 else 16)
        return self.M * (self.K16 // 2 if self.fp8 else self.K16)


@dataclass
class Compressed:
    """The tensors of one compressed matrix (what a checkpoint stores per matrix) with its shape and coding."""
    M: int
    K: int
    layout: int
    elem: str                   # "bf16" | "fp8"
    data: torch.Tensor          # uint8
    bases: torch.Tensor         # int32 (u32 byte offsets)
    hdr: torch.Tensor           # uint8 [nb * 32]
    lut: torch.Tensor           # int32 [4096]
    low: torch.Tensor           # uint8, raw plane(s), with or without the 512 bytes of slack
    scale: torch.Tensor = None  # fp32 [M] (fp8)

    @property
    def geometry(self): return Geometry(self.M, self.K, self.layout, self.elem == "fp8")


def _block_ends(c: Compressed, g: Geometry):
    """End offset (exclusive, rounded up to the 8-byte block alignment) of every block's payload inside data."""
    bases = c.bases.to(torch.int64) & 0xFFFFFFFF
    per_block = c.hdr.view(g.nb, LANES).to(torch.int64).sum(1) * g.unit
    return bases, (bases + per_block + 7) // 8 * 8


def _concat_spans(c: Compressed, starts, ends):
    """data bytes of the spans [starts[i], ends[i]) back to back (+ slack), and where each span starts in the result."""
    lengths = [int(e - s) for s, e in zip(starts, ends)]
    offsets, total = [], 0
    for n in lengths: offsets.append(total); total += n
    out = torch.zeros(total + 2 * DATA_SLACK, dtype=torch.uint8, device=c.data.device)
    have = c.data.numel()
    for s, n, o in zip(starts, lengths, offsets):
        take = max(0, min(n, have - int(s)))                               # the 8-byte padding of the very last block may lie past the stored bytes
        if take: out[o:o + take] = c.data[int(s):int(s) + take]
    return out, offsets


def take_rows(c: Compressed, ranges) -> Compressed:
    """Rows [r0, r1) for every (r0, r1) in `ranges`, concatenated in order.  Every r0 must be a multiple of the block height
    (8 for layout 0, 16 otherwise) and so must every r1; only the last range may instead end with the matrix."""
    g = c.geometry
    ranges = [(int(a), int(b)) for a, b in ranges]
    for i, (r0, r1) in enumerate(ranges):
        if not (0 <= r0 < r1 <= c.M) or r0 % g.rows or (r1 % g.rows and not (i + 1 == len(ranges) and r1 == c.M)):
            raise ValueError(f"rows [{r0}, {r1}) of {c.M} do not fall on {g.rows}-row block boundaries")
    bases, ends = _block_ends(c, g)
    starts_b, ends_b, hdr_parts, base_parts = [], [], [], []
    for r0, r1 in ranges:
        b0, b1 = r0 // g.rows * g.CB, (r1 + g.rows - 1) // g.rows * g.CB
        starts_b.append(int(bases[b0])); ends_b.append(int(ends[b1 - 1]))
        hdr_parts.append(c.hdr[b0 * LANES:b1 * LANES]); base_parts.append((b0, b1))
    data, offsets = _concat_spans(c, starts_b, ends_b)
    new_bases = torch.cat([bases[b0:b1] - s + o for (b0, b1), s, o in zip(base_parts, starts_b, offsets)]).to(torch.int32)
    M = sum(r1 - r0 for r0, r1 in ranges)
    ng = Geometry(M, c.K, c.layout, g.fp8)
    low = c.low[:g.raw_bytes]
    if c.layout == 0:
        stride = g.K16 // 2 if g.fp8 else g.K16
        new_low = torch.cat([low.view(c.M, stride)[r0:r1] for r0, r1 in ranges]).reshape(-1)
    else:
        def plane(t, per_group):                                           # [groups][per_group bytes] -> the groups of the ranges
            v = t.view(g.groups, per_group)
            return torch.cat([v[r0 // g.rows:(r1 + g.rows - 1) // g.rows] for r0, r1 in ranges]).reshape(-1)
        if c.layout == 1: new_low = plane(low, g.slots * LANES * (8 if g.fp8 else 16))
        else:
            nib, raw = low[:g.nibble_plane], low[g.nibble_plane:]
            new_low = torch.cat([plane(nib, g.slots * LANES * 8), plane(raw, g.pair_slots * 3 * LANES * 4 if g.fp8 else g.slots * LANES * 16)])
    assert new_low.numel() == ng.raw_bytes
    new_low = torch.cat([new_low, torch.zeros(RAW_SLACK, dtype=torch.uint8, device=new_low.device)])
    scale = None if c.scale is None else torch.cat([c.scale[r0:r1] for r0, r1 in ranges])
    return Compressed(M, c.K, c.layout, c.elem, data, new_bases, torch.cat(hdr_parts).contiguous(), c.lut, new_low, scale)


def take_cols(c: Compressed, c0: int, c1: int) -> Compressed:
    """Columns [c0, c1): c0 a multiple of 512, c1 a multiple of 512 or K."""
    g = c.geometry
    if not (0 <= c0 < c1 <= c.K) or c0 % BLOCK_COLS or (c1 % BLOCK_COLS and c1 != c.K):
        raise ValueError(f"columns [{c0}, {c1}) of {c.K} do not fall on 512-column block boundaries")
    cb0, cb1 = c0 // BLOCK_COLS, (c1 + BLOCK_COLS - 1) // BLOCK_COLS
    ng = Geometry(c.M, c1 - c0, c.layout, g.fp8)
    bases, ends = _block_ends(c, g)
    first = torch.arange(g.groups, device=c.bases.device) * g.CB + cb0     # first block of every row group's run
    starts_b, ends_b = bases[first].tolist(), ends[first + (cb1 - cb0) - 1].tolist()
    data, offsets = _concat_spans(c, starts_b, ends_b)
    keep = (first[:, None] + torch.arange(cb1 - cb0, device=first.device)[None, :])                # [groups][CB'] old block ids
    shift = (torch.tensor(offsets, dtype=torch.int64, device=first.device) - bases[first])[:, None]
    new_bases = (bases[keep] + shift).reshape(-1).to(torch.int32)
    new_hdr = c.hdr.view(g.nb, LANES)[keep.reshape(-1)].reshape(-1).contiguous()
    low = c.low[:g.raw_bytes]
    if c.layout == 0:
        if g.fp8: new_low = low.view(c.M, g.K16 // 2)[:, c0 // 2:c0 // 2 + ng.K16 // 2]
        else: new_low = low.view(c.M, g.K16)[:, c0:c0 + ng.K16]
        new_low = new_low.contiguous().reshape(-1)
    else:
        s0 = cb0 * 16
        def plane(t, per_slot, n_old, first_slot, n_new):
            return t.view(g.groups, n_old, per_slot)[:, first_slot:first_slot + n_new].contiguous().reshape(-1)
        if c.layout == 1: new_low = plane(low, LANES * (8 if g.fp8 else 16), g.slots, s0, ng.slots)
        else:
            nib, raw = low[:g.nibble_plane], low[g.nibble_plane:]
            raw_new = plane(raw, 3 * LANES * 4, g.pair_slots, s0 // 2, ng.pair_slots) if g.fp8 else plane(raw, LANES * 16, g.slots, s0, ng.slots)
            new_low = torch.cat([plane(nib, LANES * 8, g.slots, s0, ng.slots), raw_new])
    assert new_low.numel() == ng.raw_bytes
    new_low = torch.cat([new_low, torch.zeros(RAW_SLACK, dtype=torch.uint8, device=new_low.device)])
    return Compressed(c.M, c1 - c0, c.layout, c.elem, data, new_bases, new_hdr, c.lut, new_low, c.scale)


def rows_divisible(layout: int, *sizes) -> bool:
    """True when row sections of these sizes can be cut without re-encoding."""
    rows = 16 if layout else 8
    return all(s % rows == 0 for s in sizes)
