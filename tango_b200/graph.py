"""DGL-free graph container and seeded synthetic graph generator.

`Graph` exposes the attributes the reference operators read after `graph_preprocess`
(cuda/util.py:5-11 in the reference): `adj_csr`, `adj_csc` = (indptr, indices, edge_ids), `coo` = (src, dst) in
edge-id order, `inc_in` / `inc_out` = [2, E] (node, edge id) pairs, and `num_nodes()`.  Indices are int32 (the
reference uses DGL's int64; halving the index traffic matters for memory-bound kernels).

`rmat_graph` builds the R-MAT graphs (a=0.57, b=c=0.19, d=0.05) that stand in for the public datasets the
reference's scripts load.  It uses only wrapping int64 arithmetic, so the same seed gives the same graph on CPU and
on GPU.
"""
from __future__ import annotations

import contextlib
import math
from typing import Optional, Tuple

import torch

_M64 = (1 << 64) - 1


def _s64(x: int) -> int:
    """Python int -> the signed 64-bit value with the same low 64 bits."""
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


_C1 = _s64(0xBF58476D1CE4E5B9)
_C2 = _s64(0x94D049BB133111EB)
_GOLD = _s64(0x9E3779B97F4A7C15)


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    return (x >> s) & ((1 << (64 - s)) - 1)


def mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on int64 tensors (wrapping arithmetic)."""
    x = (x ^ _lsr(x, 30)) * _C1
    x = (x ^ _lsr(x, 27)) * _C2
    return x ^ _lsr(x, 31)


def _rmat_batch(n_nodes: int, start: int, count: int, seed: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    levels = max(1, math.ceil(math.log2(max(2, n_nodes))))
    i = torch.arange(start, start + count, dtype=torch.int64, device=device)
    base = mix64(i * _GOLD + _s64(seed * 0x2545F4914F6CDD1D + 0x1234567))
    src = torch.zeros(count, dtype=torch.int64, device=device)
    dst = torch.zeros(count, dtype=torch.int64, device=device)
    ta, tb, tc = int(0.57 * (1 << 24)), int(0.76 * (1 << 24)), int(0.95 * (1 << 24))
    for lvl in range(levels):
        u = _lsr(mix64(base + _s64((lvl + 1) * 0xD6E8FEB86659FD93)), 40)  # 24 uniform bits
        sbit = (u >= tb).to(torch.int64)                                   # quadrants c, d: source bit set
        dbit = (((u >= ta) & (u < tb)) | (u >= tc)).to(torch.int64)       # quadrants b, d: destination bit set
        src = (src << 1) | sbit
        dst = (dst << 1) | dbit
    return src, dst


def rmat_edges(n_nodes: int, n_edges: int, seed: int, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """`n_edges` distinct directed non-loop edges (src, dst) of an R-MAT graph, sorted by (src, dst)."""
    keys = torch.empty(0, dtype=torch.int64, device=device)
    start = 0
    while keys.numel() < n_edges:
        need = n_edges - keys.numel()
        count = max(1024, int(need * 1.5) + 1024)
        s, d = _rmat_batch(n_nodes, start, count, seed, device)
        start += count
        ok = (s < n_nodes) & (d < n_nodes) & (s != d)
        new = torch.unique(s[ok] * n_nodes + d[ok])
        del s, d, ok
        if keys.numel():
            pos = torch.searchsorted(keys, new).clamp_(max=keys.numel() - 1)
            new = new[keys[pos] != new]
        if new.numel() > need:  # keep a pseudo-random, seed-determined subset of the last batch
            order = torch.argsort(mix64(new ^ _s64(seed)))
            new = new[order[:need]]
        keys = torch.sort(torch.cat([keys, new]))[0]
    return (keys // n_nodes).to(torch.int32), (keys % n_nodes).to(torch.int32)


class Graph:
    """Homogeneous directed graph held as int32 index tensors on one device."""

    is_block = False

    def __init__(self, src: torch.Tensor, dst: torch.Tensor, n_nodes: int):
        assert src.shape == dst.shape and src.dim() == 1
        self._src = src.to(torch.int32).contiguous()
        self._dst = dst.to(torch.int32).contiguous()
        self._n = int(n_nodes)
        self.ndata = {}
        self.edata = {}
        self.srcdata = self.ndata
        self.dstdata = self.ndata
        self._csr = None
        self._csc = None
        self._plans = {}
        self._deg = {}
        self._identity = {}   # fmt -> True when slot k of that format holds edge k (edge ids follow the format's order)
        self.n_classes = None

    # ---- DGL-like surface used by the operators and the layers
    @property
    def device(self):
        return self._src.device

    def num_nodes(self) -> int:
        return self._n

    number_of_nodes = num_nodes

    def num_edges(self) -> int:
        return int(self._src.numel())

    number_of_edges = num_edges

    def number_of_dst_nodes(self) -> int:
        return self._n

    def edges(self):
        return self._src, self._dst

    def in_degrees(self) -> torch.Tensor:
        if "in" not in self._deg:
            self._deg["in"] = torch.bincount(self._dst.long(), minlength=self._n)
        return self._deg["in"]

    def out_degrees(self) -> torch.Tensor:
        if "out" not in self._deg:
            self._deg["out"] = torch.bincount(self._src.long(), minlength=self._n)
        return self._deg["out"]

    @contextlib.contextmanager
    def local_scope(self):
        yield self

    def to(self, device) -> "Graph":
        g = Graph(self._src.to(device), self._dst.to(device), self._n)
        g.n_classes = self.n_classes
        g.ndata = {k: v.to(device) for k, v in self.ndata.items() if torch.is_tensor(v)}
        g.srcdata = g.dstdata = g.ndata
        return g

    # ---- sparse formats
    def adj_sparse(self, fmt: str):
        """(indptr, indices, edge_ids); 'csr' rows are sources, 'csc' rows are destinations.  Columns are sorted."""
        if fmt == "coo":
            return self._src, self._dst
        rows, cols = (self._src, self._dst) if fmt == "csr" else (self._dst, self._src)
        cached = self._csr if fmt == "csr" else self._csc
        if cached is None:
            key = rows.long() * self._n + cols.long()
            key, perm = torch.sort(key, stable=True)
            counts = torch.bincount(rows.long(), minlength=self._n)
            indptr = torch.zeros(self._n + 1, dtype=torch.int64, device=self.device)
            torch.cumsum(counts, 0, out=indptr[1:])
            cached = (indptr.to(torch.int32), (key % self._n).to(torch.int32), perm.to(torch.int32))
            self._identity[fmt] = bool((perm == torch.arange(perm.numel(), device=perm.device)).all())
            if fmt == "csr":
                self._csr = cached
            else:
                self._csc = cached
        return cached

    @property
    def adj_csr(self):
        return self.adj_sparse("csr")

    @property
    def adj_csc(self):
        return self.adj_sparse("csc")

    @property
    def coo(self):
        return self._src, self._dst

    def _inc(self, fmt: str) -> torch.Tensor:
        indptr, _, eids = self.adj_sparse(fmt)
        nodes = torch.repeat_interleave(torch.arange(self._n, dtype=torch.int32, device=self.device),
                                        (indptr[1:] - indptr[:-1]).long())
        return torch.stack([nodes, eids])

    @property
    def inc_in(self):
        return self._inc("csc")

    @property
    def inc_out(self):
        return self._inc("csr")


def add_self_loop(src: torch.Tensor, dst: torch.Tensor, n_nodes: int):
    """Drops existing loops and appends one loop per node (dgl.remove_self_loop + add_self_loop,
    evaluation/util.py:28 in the reference)."""
    keep = src != dst
    loop = torch.arange(n_nodes, dtype=src.dtype, device=src.device)
    return torch.cat([src[keep], loop]), torch.cat([dst[keep], loop])


def graph_from_edge_list(path: str, n_nodes: Optional[int] = None, device="cpu", self_loops: bool = True,
                         symmetric: bool = False) -> Graph:
    """Reads a whitespace-separated "src dst" edge list (the SNAP text format the reference's loader parses for its
    DBLP / Amazon graphs, evaluation/util.py:15-22; lines starting with '#' are comments), optionally adds the reverse
    edges, drops duplicates, and applies the reference's remove_self_loop + add_self_loop."""
    import numpy as np
    arr = np.loadtxt(path, dtype=np.int64, comments="#", ndmin=2)
    src, dst = torch.from_numpy(arr[:, 0].copy()), torch.from_numpy(arr[:, 1].copy())
    if symmetric:
        src, dst = torch.cat([src, dst]), torch.cat([dst, src])
    n = int(max(int(src.max()), int(dst.max())) + 1) if n_nodes is None else int(n_nodes)
    key = torch.unique(src * n + dst)
    src, dst = (key // n).to(torch.int32), (key % n).to(torch.int32)
    if self_loops:
        src, dst = add_self_loop(src, dst, n)
    order = torch.argsort(dst.long() * n + src.long())
    return Graph(src[order].contiguous(), dst[order].contiguous(), n).to(device)


def rmat_graph(n_nodes: int, n_edges: int, seed: int, device="cpu", self_loops: bool = True,
               edge_order: str = "dst") -> Graph:
    """Seeded R-MAT graph.  edge_order='dst' numbers the edges by (destination, source), so that edge ids follow the
    CSC order and every per-edge tensor is streamed by the destination-major kernels; 'append' keeps the generator's
    (source, destination) order with the self loops appended, as dgl.add_self_loop leaves them."""
    src, dst = rmat_edges(n_nodes, n_edges, seed, device)
    if self_loops:
        src, dst = add_self_loop(src, dst, n_nodes)
    if edge_order == "dst":
        order = torch.argsort(dst.long() * n_nodes + src.long())
        src, dst = src[order].contiguous(), dst[order].contiguous()
    return Graph(src, dst, n_nodes)


# ----------------------------------------------------------------------------------------------------------------
# Schedules for rows that are too long for one warp, and 1-D row partitions for multi-GPU training.
# ----------------------------------------------------------------------------------------------------------------
SPLIT_THRESHOLD = 4096
BLOCK_ROW_NNZ = 1024
SHORT_ROW_NNZ = 48      # rows up to this length are processed by a group of lanes instead of a whole warp
UNIT_NNZ = 2048


class SpmmSchedule:
    """Device arrays consumed by the SpMM kernels: `units` [n_units, 4] = (segment row, begin, end, scratch slot)
    for every slice of a row longer than the threshold, and `heavy_rows` = those rows.

    force_heavy (optional, nseg == 1): row ids that are finished through the int32 scratch whatever their length (the
    rows of a dense hub block, in the block's row order); they come first in `heavy_rows`, every heavy row comes
    first in `row_order`, and `n_skip` = n_heavy tells the row kernels to start after them."""

    def __init__(self, indptr: torch.Tensor, nseg: int = 1, threshold: Optional[int] = None,
                 unit: Optional[int] = None, force_heavy: Optional[torch.Tensor] = None):
        if threshold is None:
            # A row is worked on by one warp, neighbour batch after neighbour batch, so the longest unsplit row sets
            # the critical path of the kernel.  Keep it short relative to the total work: about nnz / 16384 (one
            # batch-chain per resident warp slot), between 256 and SPLIT_THRESHOLD.
            nnz = int(indptr[-1]) if indptr.numel() else 0
            threshold = 256
            while threshold < SPLIT_THRESHOLD and threshold * 16384 < nnz:
                threshold *= 2
        if unit is None:
            unit = max(128, threshold // 2)
        self.nseg = nseg
        self.threshold = threshold
        n_rows = (indptr.numel() - 1) // nseg
        ip = indptr.long()
        row_deg = ip[nseg::nseg] - ip[:-1:nseg][:n_rows] if nseg > 1 else ip[1:] - ip[:-1]
        self.n_skip = 0
        if force_heavy is None:
            # rows in order of decreasing length: the warps of a CTA then work on rows of similar length and the
            # longest rows start first
            # (the short rows, too: taking them in natural order instead -- neighbouring lane groups on neighbouring
            # rows -- measured 20-60 % slower, rows of unequal length in one warp cost more than the locality gains)
            self.row_order = torch.argsort(row_deg, descending=True, stable=True).to(torch.int32)
            self.n_long = int((row_deg > SHORT_ROW_NNZ).sum())
            heavy = torch.nonzero(row_deg > threshold).flatten()
        else:
            assert nseg == 1
            forced = force_heavy.long()
            is_forced = torch.zeros(n_rows, dtype=torch.bool, device=indptr.device)
            is_forced[forced] = True
            heavy = torch.cat([forced, torch.nonzero((row_deg > threshold) & ~is_forced).flatten()])
            is_heavy = is_forced.clone()
            is_heavy[heavy] = True
            rest = torch.nonzero(~is_heavy).flatten()
            rest = rest[torch.argsort(row_deg[rest], descending=True, stable=True)]
            n_rest_long = int((row_deg[rest] > SHORT_ROW_NNZ).sum())
            self.row_order = torch.cat([heavy, rest]).to(torch.int32)
            self.n_skip = int(heavy.numel())
            self.n_long = self.n_skip + n_rest_long
        self.n_block_rows = int((row_deg > BLOCK_ROW_NNZ).sum())   # rows that deserve a whole CTA in row-team kernels
        self.n_heavy = int(heavy.numel())
        self.heavy_rows = heavy.to(torch.int32)
        if self.n_heavy == 0:
            self.units = torch.zeros((0, 4), dtype=torch.int32, device=indptr.device)
            self.n_units = 0
            return
        # segment rows of the heavy rows, their scratch slots, and the slices of each
        seg_rows = (heavy[:, None] * nseg + torch.arange(nseg, device=indptr.device)[None, :]).flatten()
        slots = torch.arange(seg_rows.numel(), device=indptr.device)
        beg, end = ip[seg_rows], ip[seg_rows + 1]
        n_chunks = (end - beg + unit - 1) // unit
        rep = torch.repeat_interleave(torch.arange(seg_rows.numel(), device=indptr.device), n_chunks)
        first = torch.cumsum(n_chunks, 0) - n_chunks
        k = torch.arange(rep.numel(), device=indptr.device) - first[rep]
        ub = beg[rep] + k * unit
        ue = torch.minimum(ub + unit, end[rep])
        units = torch.stack([seg_rows[rep], ub, ue, slots[rep]], dim=1)
        # longest slices first
        self.units = units.to(torch.int32).contiguous()
        self.n_units = int(self.units.shape[0])


HUB_BLOCK_MIN_DENSITY = 0.035   # a 128 x 128 tile below this density costs more as a dense int8 product than its
                                # edges cost to gather (break-even measured at about 2.7 %)
HUB_TILE = 128


class HubBlock:
    """The dense hub region of an aggregation matrix (CSR-like `indptr`, `indices` over `n_cols` feature rows).

    Rows are ranked by length and columns by how often they are referenced; in that order the matrix of a power-law
    graph is densest in its top-left corner and thins out smoothly, so the region worth multiplying as a dense 0/1
    int8 matrix on the tensor cores is a staircase: row tile i (128 rows) keeps its first `kend[i]` column tiles
    (128 columns each), the prefix that maximises (edges covered x cost of gathering an edge - tiles x cost of a tile
    product) for tiles of at least `min_density`.  The region is stored tile by tile (`dense`: [n_tiles * 128, 128]
    int8, multiplicities), cut into work items `units` = (row tile, first stored tile, first column tile, tiles) of
    bounded length for the GEMM kernel; `cols` lists the feature rows of the columns used.  The edges outside the
    region form a CSR of their own (`indptr`, `indices`), whose row schedule forces the region's rows through the
    int32 scratch, where the tensor-core product and the gathered remainder meet.  Exact int32 either way, so results
    do not change by a bit.

    On the 232,965-node / 114.6 M-edge graph the region holds about two thirds of the edges in 24 K tiles (0.4 GB)."""

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, n_cols: int, max_rows: int = 163840,
                 max_cols: int = 163840, min_density: float = HUB_BLOCK_MIN_DENSITY):
        dev = indptr.device
        T = HUB_TILE
        ip = indptr.long()
        n_rows = ip.numel() - 1
        row_deg = ip[1:] - ip[:-1]
        ntr = min(max_rows, n_rows) // T
        ntc = min(max_cols, n_cols) // T
        self.ok = False
        if ntr <= 0 or ntc <= 0 or indices.numel() == 0:
            return
        col_deg = torch.bincount(indices.long(), minlength=n_cols)
        rows = torch.argsort(row_deg, descending=True, stable=True)[:ntr * T]
        cols = torch.argsort(col_deg, descending=True, stable=True)[:ntc * T]
        row_slot = torch.full((n_rows,), -1, dtype=torch.int64, device=dev)
        row_slot[rows] = torch.arange(ntr * T, device=dev)
        col_pos = torch.full((n_cols,), -1, dtype=torch.int64, device=dev)
        col_pos[cols] = torch.arange(ntc * T, device=dev)
        edge_row = torch.repeat_interleave(torch.arange(n_rows, device=dev), row_deg)
        rs, cp = row_slot[edge_row], col_pos[indices.long()]
        cand = (rs >= 0) & (cp >= 0)
        cnt = torch.bincount((rs[cand] // T) * ntc + cp[cand] // T, minlength=ntr * ntc).view(ntr, ntc)
        # per row tile: the prefix of column tiles with the largest net benefit; one tile costs as much as gathering
        # min_density * T * T edges (min_density == 0: every tile inside the caps is taken)
        if min_density > 0:
            gain = torch.cumsum(cnt.double() - min_density * T * T, dim=1)
            best, arg = gain.max(dim=1)
            # a row tile also costs a fixed amount (its own work item: pipeline fill, 32 K atomics, its rows routed
            # through the scratch), about as much as six tile products
            kend = torch.where(best > 6 * min_density * T * T, arg + 1, torch.zeros_like(arg))
        else:
            kend = torch.full((ntr,), ntc, dtype=torch.int64, device=dev)
        used = torch.nonzero(kend > 0).flatten()
        if used.numel() == 0:
            return
        ntr = int(used.max()) + 1                      # row tiles 0 .. ntr-1 take part (some may have no tile)
        kend = kend[:ntr]
        self.kend = kend
        tile_base = torch.cumsum(kend, 0) - kend
        n_tiles = int(kend.sum())
        ks = int(kend.max()) * T
        in_blk = cand & (rs < ntr * T)
        in_blk &= (cp // T) < kend[(rs // T).clamp(max=ntr - 1)]
        self.n_block_edges = int(in_blk.sum())
        self.n_tiles = n_tiles
        self.density = self.n_block_edges / float(n_tiles * T * T)
        rb, cb = rs[in_blk], cp[in_blk]
        tile = tile_base[rb // T] + cb // T
        dense = torch.zeros(n_tiles * T * T, dtype=torch.int8, device=dev)
        dense.index_put_(((tile * T + rb % T) * T + cb % T,),
                         torch.ones(1, dtype=torch.int8, device=dev).expand(self.n_block_edges), accumulate=True)
        self.dense = dense.view(n_tiles * T, T)
        # GEMM work items of bounded length, longest first
        chunk = max(8, min(128, -(-n_tiles // (148 * 4))))
        n_chunks = (kend + chunk - 1) // chunk
        rep = torch.repeat_interleave(torch.arange(ntr, device=dev), n_chunks)
        first = torch.cumsum(n_chunks, 0) - n_chunks
        k0 = (torch.arange(rep.numel(), device=dev) - first[rep]) * chunk
        length = torch.minimum(kend[rep] - k0, torch.full_like(k0, chunk))
        order = torch.argsort(length, descending=True, stable=True)
        self.units = torch.stack([rep, tile_base[rep] + k0, k0, length], dim=1)[order].to(torch.int32).contiguous()
        keep = ~in_blk
        self.indices = indices[keep].contiguous()
        tail_deg = row_deg - torch.bincount(edge_row[in_blk], minlength=n_rows)
        tip = torch.zeros(n_rows + 1, dtype=torch.int64, device=dev)
        torch.cumsum(tail_deg, 0, out=tip[1:])
        self.indptr = tip.to(torch.int32)
        self.rows = rows[:ntr * T].to(torch.int32)
        self.cols = cols[:ks].to(torch.int32).contiguous()
        self.schedule = SpmmSchedule(self.indptr, force_heavy=rows[:ntr * T])
        self.schedule.hub = self
        self.ok = True

    def to_dense(self) -> torch.Tensor:
        """The region as an ordinary [rows, cols] int32 matrix (zero outside the staircase); for tests."""
        T = HUB_TILE
        out = torch.zeros((self.rows.numel(), self.cols.numel()), dtype=torch.int32, device=self.dense.device)
        base = torch.cumsum(self.kend, 0) - self.kend
        for i in range(self.kend.numel()):
            for k in range(int(self.kend[i])):
                t = int(base[i]) + k
                out[i * T:(i + 1) * T, k * T:(k + 1) * T] = self.dense[t * T:(t + 1) * T].int()
        return out


def balanced_bounds(weights: torch.Tensor, world: int):
    """Contiguous row blocks [b_k, b_k+1) with (nearly) equal total weight -- e.g. in-degree + out-degree, so that
    the skewed rows of a power-law graph do not all land on rank 0.  Returns a list of world + 1 Python ints."""
    n = weights.numel()
    cum = torch.cumsum(weights.double(), 0)
    total = float(cum[-1]) if n else 0.0
    targets = torch.tensor([total * k / world for k in range(1, world)], dtype=torch.float64, device=weights.device)
    cuts = torch.searchsorted(cum, targets).tolist() if world > 1 else []
    b = [0] + [min(n, int(c) + 1) for c in cuts] + [n]
    for k in range(1, len(b)):            # keep the boundaries monotone
        b[k] = max(b[k], b[k - 1])
    return b


def uniform_bounds(n_nodes: int, world: int):
    step = (n_nodes + world - 1) // world
    return [min(n_nodes, k * step) for k in range(world)] + [n_nodes]


class RowPartition:
    """The rows of a CSR/CSC that one rank owns, with column ids rewritten for the all-gathered feature buffer, in
    which rank k's rows start at k * shard_rows (shard_rows = the largest shard; shorter shards are padded).

    layout='block' : rank k owns the contiguous rows [bounds[k], bounds[k+1]);
    layout='cyclic': rank k owns rows k, k + world, k + 2*world, ... (equal row counts, no padding);
    layout='dealt' : the rows of `order` (e.g. nodes sorted by degree) are dealt round-robin, order[i] going to rank
                     i % world at local position i // world -- equal row counts and, for a degree-sorted order,
                     nearly equal edge counts even on power-law graphs.
    `local_ids` lists the global ids of the owned rows in local order.  `indptr` has n_local * world + 1 entries: row v
    owns `world` consecutive segments, segment k holding the columns that live on rank k; `indptr_flat` is the same
    structure without that cut (n_local + 1 entries)."""

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, edge_ids: Optional[torch.Tensor], n_nodes: int,
                 rank: int, world: int, bounds=None, layout: str = "block", order: Optional[torch.Tensor] = None):
        assert layout in ("block", "cyclic", "dealt")
        self.world, self.rank, self.layout = world, rank, layout
        dev = indptr.device
        ip = indptr.long()
        if layout == "block":
            self.bounds = list(bounds) if bounds is not None else uniform_bounds(n_nodes, world)
            assert len(self.bounds) == world + 1 and self.bounds[0] == 0 and self.bounds[-1] == n_nodes
            self.shard_rows = max(1, max(self.bounds[k + 1] - self.bounds[k] for k in range(world)))
            self.r0, self.r1 = self.bounds[rank], self.bounds[rank + 1]
            self.local_ids = torch.arange(self.r0, self.r1, device=dev)
            bt = torch.tensor(self.bounds, dtype=torch.int64, device=dev)

            def place(cols):
                owner = torch.searchsorted(bt, cols, right=True) - 1
                return owner * self.shard_rows + (cols - bt[owner])
        elif layout == "cyclic":
            self.bounds = None
            self.shard_rows = max(1, (n_nodes + world - 1) // world)
            self.local_ids = torch.arange(rank, n_nodes, world, device=dev)
            self.r0, self.r1 = None, None

            def place(cols):
                return (cols % world) * self.shard_rows + cols // world
        else:
            assert order is not None and order.numel() == n_nodes
            self.bounds = None
            self.shard_rows = max(1, (n_nodes + world - 1) // world)
            order = order.long()
            self.local_ids = order[rank::world].contiguous()
            self.r0, self.r1 = None, None
            slot = torch.empty(n_nodes, dtype=torch.int64, device=dev)      # node -> row in the gathered buffer
            i = torch.arange(n_nodes, device=dev)
            slot[order] = (i % world) * self.shard_rows + i // world

            def place(cols):
                return slot[cols]
        self.n_local = int(self.local_ids.numel())
        beg, end = ip[self.local_ids], ip[self.local_ids + 1]
        lens = end - beg
        total = int(lens.sum())
        first = torch.cumsum(lens, 0) - lens
        rows = torch.repeat_interleave(torch.arange(self.n_local, device=dev), lens)
        pos = torch.arange(total, device=dev) - first[rows] + beg[rows]          # slots of the owned rows, row by row
        remapped = place(indices[pos].long())
        span = self.shard_rows * world
        key = rows * span + remapped
        if layout != "block":                       # the rewritten columns are no longer sorted inside a row
            key, order = torch.sort(key)
            pos = pos[order]
            remapped = key - rows * span
        self.indices = remapped.to(torch.int32).contiguous()
        self.edge_ids = None if edge_ids is None else edge_ids[pos].contiguous()
        seg_bounds = (torch.arange(self.n_local, device=dev)[:, None] * span
                      + torch.arange(world, device=dev)[None, :] * self.shard_rows).flatten()
        seg = torch.searchsorted(key, seg_bounds)
        self.indptr = torch.cat([seg, torch.tensor([total], device=dev)]).to(torch.int32)
        self.schedule = SpmmSchedule(self.indptr, nseg=world)
        # the same rows without the per-shard cut, for aggregation with one scale shared by all ranks
        self.indptr_flat = self.indptr[::world].contiguous()
        self.schedule_flat = SpmmSchedule(self.indptr_flat, nseg=1)
