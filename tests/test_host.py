"""Host-side logic that needs no GPU: graph generator and index bundles, long-row schedules, row partitions, shape
helpers, rounding-mode switch, and the 2-rank all-gather path over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tango_oracle as O
from tango_b200 import config
from tango_b200.graph import Graph, HubBlock, RowPartition, SpmmSchedule, add_self_loop, rmat_edges, rmat_graph
from tango_b200.kernels import alloc_int8, infer_broadcast_shape


def test_rmat_is_seeded_distinct_and_loop_free():
    s1, d1 = rmat_edges(1000, 8000, 5)
    s2, d2 = rmat_edges(1000, 8000, 5)
    s3, _ = rmat_edges(1000, 8000, 6)
    assert torch.equal(s1, s2) and torch.equal(d1, d2) and not torch.equal(s1, s3)
    assert s1.numel() == 8000 and int((s1 == d1).sum()) == 0
    key = s1.long() * 1000 + d1.long()
    assert key.unique().numel() == 8000 and int(s1.max()) < 1000 and int(d1.max()) < 1000
    deg = torch.bincount(s1.long(), minlength=1000)
    assert deg.max() > 8 * deg.float().mean()            # power-law skew


def test_graph_index_bundles():
    g = rmat_graph(500, 4000, 3)
    src, dst = g.coo
    assert g.num_edges() == 4500 and int(g.in_degrees().min()) >= 1      # one self loop per node
    for fmt, rows, cols in (("csr", src, dst), ("csc", dst, src)):
        indptr, indices, eids = g.adj_sparse(fmt)
        assert indptr.dtype == torch.int32 and int(indptr[-1]) == 4500
        assert torch.equal(cols[eids.long()], indices)
        r = torch.repeat_interleave(torch.arange(500), (indptr[1:] - indptr[:-1]).long())
        assert torch.equal(rows[eids.long()].long(), r)
        for v in (0, 7, 499):                                            # columns sorted inside a row
            seg = indices[indptr[v]:indptr[v + 1]]
            assert torch.equal(seg, seg.sort()[0])
    inc = g.inc_in
    assert inc.shape == (2, 4500) and torch.equal(dst[inc[1].long()], inc[0])
    assert torch.equal(src[g.inc_out[1].long()], g.inc_out[0])


def test_add_self_loop_replaces_existing_loops():
    s = torch.tensor([0, 1, 2, 2], dtype=torch.int32)
    d = torch.tensor([0, 2, 2, 1], dtype=torch.int32)
    s2, d2 = add_self_loop(s, d, 3)
    assert s2.tolist() == [1, 2, 0, 1, 2] and d2.tolist() == [2, 1, 0, 1, 2]


@pytest.mark.parametrize("nseg", [1, 3])
def test_schedule_covers_long_rows_exactly_once(nseg):
    g = rmat_graph(2000, 60000, 9)
    indptr, indices, _ = g.adj_csc
    if nseg > 1:
        part = RowPartition(indptr, indices, None, 2000, 0, nseg)
        indptr = part.indptr
    s = SpmmSchedule(indptr, nseg=nseg, threshold=100, unit=64)
    ip = indptr.long()
    n_rows = (ip.numel() - 1) // nseg
    deg = ip[nseg::nseg] - ip[:-1:nseg]
    assert s.n_heavy == int((deg > 100).sum()) and s.n_heavy > 0
    cov = torch.zeros(int(ip[-1]), dtype=torch.int32)
    for vrow, b, e, slot in s.units.tolist():
        assert 0 < e - b <= 64 and ip[vrow] <= b and e <= ip[vrow + 1]
        assert s.heavy_rows[slot // nseg] == vrow // nseg and slot % nseg == vrow % nseg
        cov[b:e] += 1
    assert int(cov.max()) == 1 and int(cov.sum()) == int(deg[s.heavy_rows.long()].sum())
    assert n_rows * nseg + 1 == ip.numel()


def test_row_partition_segments():
    g = rmat_graph(1003, 20000, 4)
    indptr, indices, _ = g.adj_csc
    world = 4
    seen = 0
    for r in range(world):
        p = RowPartition(indptr, indices, None, 1003, r, world)
        assert p.shard_rows == 251 and p.indptr.numel() == p.n_local * world + 1
        ip = p.indptr.long()
        for v in (0, p.n_local // 2, p.n_local - 1):
            for k in range(world):
                seg = p.indices[ip[v * world + k]:ip[v * world + k + 1]]
                assert bool(((seg // p.shard_rows) == k).all())
        seen += p.indices.numel()
    assert seen == g.num_edges()


def test_alloc_int8_padding_and_broadcast_shapes():
    t = alloc_int8((10, 41), "cpu")
    assert t.shape == (10, 41) and t.stride() == (48, 1)
    t = alloc_int8((10, 4, 64), "cpu")
    assert t.is_contiguous()
    t = alloc_int8((10, 2, 24), "cpu")
    assert t.shape == (10, 2, 24) and t.stride() == (48, 24, 1)
    assert alloc_int8((7, 4), "cpu", align=1).is_contiguous()
    assert infer_broadcast_shape("dot", (4, 64), (4, 64)) == (4, 1)
    assert infer_broadcast_shape("add", (4, 1), (4, 1)) == (4, 1)
    assert infer_broadcast_shape("mul", (4, 16), (1, 16)) == (4, 16)
    with pytest.raises(ValueError):
        infer_broadcast_shape("add", (4, 3), (4, 5))


def test_rounding_switch():
    from tango_b200._lib import ROUND_NEAREST, ROUND_STOCHASTIC, ROUND_TRUNC
    config.set_rounding("reference")
    assert config.mode_for("gemm_fwd") == ROUND_TRUNC and config.mode_for("quantize") == ROUND_NEAREST
    config.set_rounding("stochastic", seed=9)
    assert config.mode_for("gemm_fwd") == ROUND_STOCHASTIC and config.seed() == 9
    config.set_rounding("reference")
    with pytest.raises(ValueError):
        config.set_rounding("bogus")


# ------------------------------------------------------------------------------------------- 2 ranks over gloo
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tango_b200.dist import all_gather_quantized
    n, f = 301, 24                                       # ragged: the last shard is shorter
    g = rmat_graph(n, 5000, 21)
    indptr, indices, _ = g.adj_csc
    part = RowPartition(indptr, indices, None, n, rank, world)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, f)).astype(np.float32) * (1 + np.arange(n)[:, None] / 100)
    x_loc = x[part.r0:part.r1]
    s_loc = O.absmax_scale(x_loc)
    q_loc = torch.zeros((part.n_local, 32), dtype=torch.int8)          # padded rows, as the quantizer writes them
    q_loc[:, :f] = torch.from_numpy(O.quantize(x_loc, s_loc))
    q_all, scales = all_gather_quantized(q_loc, torch.tensor([s_loc]), part.shard_rows)
    assert q_all.shape == (world * part.shard_rows, 32)
    out = O.spmm_copy_u(part.indptr.numpy().astype(np.int64)[::world], part.indices.numpy().astype(np.int64),
                        q_all[:, :f].numpy(), scales.numpy(), shard_rows=part.shard_rows)
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    np.save(os.path.join(out_dir, f"scales{rank}.npy"), scales.numpy())
    # transport selection is a host-side decision taken alike on all ranks: no CUDA device -> library collectives
    from tango_b200.dist import DistGraph
    dg = DistGraph(g, rank, world, transport="auto")
    assert dg.transport == "nccl" and dg.peer is None and dg.n_local == dg.fwd.n_local and not dg.hubs
    # an expired rendezvous on ONE rank reaches every rank through the gradient all-reduce (host logic of the peer
    # transport's status word, with a stand-in for the transport: no GPU here)
    from tango_b200._lib import TangoError
    from tango_b200.dist import allreduce_grads
    from tango_b200.peer import PeerTransport

    class FakePeer:
        status_word = PeerTransport.status_word
        raise_if_expired = PeerTransport.raise_if_expired
        reset_status = PeerTransport.reset_status

        def __init__(self, expired):
            self._status = torch.tensor([-4 if expired else 0], dtype=torch.int32)
            self.group_status = torch.zeros(1)

    lin = torch.nn.Linear(3, 2)
    for p_ in lin.parameters():
        p_.grad = torch.full_like(p_, float(rank + 1))
    peer = FakePeer(expired=(rank == 1))
    allreduce_grads(lin, peer=peer)
    assert all(bool((p_.grad == 3.0).all()) for p_ in lin.parameters())        # 1 + 2: the gradients are untouched
    assert float(peer.group_status) == 4.0
    try:
        peer.raise_if_expired()
        raised = False
    except TangoError:
        raised = True
    assert raised                                                               # on rank 0 too, whose own word is 0
    peer.reset_status()
    for p_ in lin.parameters():
        p_.grad = torch.ones_like(p_)
    allreduce_grads(lin, peer=peer)
    peer.raise_if_expired()                                                     # nothing expired since the reset
    dist.destroy_process_group()


def test_two_rank_gather_and_aggregate(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    n, f = 301, 24
    g = rmat_graph(n, 5000, 21)
    indptr, indices, _ = [t.numpy().astype(np.int64) for t in g.adj_csc]
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, f)).astype(np.float32) * (1 + np.arange(n)[:, None] / 100)
    shard = (n + world - 1) // world
    scales = np.array([O.absmax_scale(x[k * shard:(k + 1) * shard]) for k in range(world)], dtype=np.float32)
    q = np.concatenate([O.quantize(x[k * shard:(k + 1) * shard], scales[k]) for k in range(world)])
    ref = O.spmm_copy_u(indptr, indices, q, scales, shard_rows=shard)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    np.testing.assert_array_equal(np.load(tmp_path / "scales0.npy"), scales)
    np.testing.assert_array_equal(got, ref)
    # and the per-shard-scale result stays within the stated tolerance of the fp32 aggregation
    a = np.zeros((n, f)); rows = np.repeat(np.arange(n), np.diff(indptr)); np.add.at(a, rows, x[indices])
    assert np.abs(got - a).max() / np.abs(a).max() < 1e-2


@pytest.mark.parametrize("layout", ["block", "cyclic", "dealt"])
def test_partition_layouts_reproduce_the_unpartitioned_aggregation(layout):
    """Every rank aggregates its rows from a buffer laid out like the all-gather result (rank k's rows at
    k * shard_rows); together they must give the plain aggregation, for contiguous and for round-robin placement."""
    from tango_b200.graph import balanced_bounds
    n, world, f = 1003, 4, 8
    g = rmat_graph(n, 20000, 4)
    indptr, indices, eids = g.adj_csc
    nq = np.random.default_rng(0).integers(-127, 128, (n, f), dtype=np.int8)
    ref = O.spmm_copy_u(indptr.numpy().astype(np.int64), indices.numpy().astype(np.int64), nq, np.float32(0.5))
    bounds = balanced_bounds(g.in_degrees() + g.out_degrees() + 10, world) if layout == "block" else None
    order = torch.argsort(g.in_degrees() + g.out_degrees(), descending=True, stable=True) if layout == "dealt" else None
    parts = [RowPartition(indptr, indices, eids, n, r, world, bounds, layout, order) for r in range(world)]
    if layout == "dealt":
        nnz = [p.indices.numel() for p in parts]
        assert max(nnz) < 1.1 * min(nnz)
    shard = parts[0].shard_rows
    gathered = np.zeros((world * shard, f), dtype=np.int8)
    for p in parts:
        ids = p.local_ids.numpy()
        gathered[p.rank * shard:p.rank * shard + len(ids)] = nq[ids]
    seen = 0
    for p in parts:
        out = O.spmm_copy_u(p.indptr_flat.numpy().astype(np.int64), p.indices.numpy().astype(np.int64), gathered,
                            np.float32(0.5))
        np.testing.assert_array_equal(out, ref[p.local_ids.numpy()])
        ip = p.indptr.long()
        for v in (0, p.n_local - 1):                       # segment k only holds columns stored in rank k's slice
            for k in range(world):
                seg = p.indices[ip[v * world + k]:ip[v * world + k + 1]]
                assert bool(((seg // shard) == k).all())
        src, dst = g.coo                                   # edge ids follow their slots through the re-ordering
        assert torch.equal(dst[p.edge_ids.long()].long(),
                           p.local_ids[torch.repeat_interleave(torch.arange(p.n_local),
                                                               (p.indptr_flat[1:] - p.indptr_flat[:-1]).long())])
        seen += p.indices.numel()
    assert seen == g.num_edges()


def test_graph_from_edge_list(tmp_path):
    from tango_b200.graph import graph_from_edge_list
    f = tmp_path / "g.txt"
    f.write_text("# comment\n0 1\n1 2\n1 2\n2 2\n3 0\n")
    g = graph_from_edge_list(str(f), symmetric=True)
    src, dst = g.coo
    pairs = set(zip(src.tolist(), dst.tolist()))
    assert pairs == {(0, 1), (1, 0), (1, 2), (2, 1), (3, 0), (0, 3), (0, 0), (1, 1), (2, 2), (3, 3)}
    assert g.num_nodes() == 4 and g.adj_csc[0].tolist() == [0, 3, 6, 8, 10]
    assert g._identity["csc"]


def test_rendezvous_protocol_model():
    """Host-side model of the one-CTA rendezvous kernel (csrc/peer.cu): rank r writes (round, value) into word
    bank(round) * world + r of every rank's slot array, then waits for the `world` words of that bank in its own
    array.  Ranks run as threads with random delays; every round must return the maximum of that round's values on
    every rank although fast ranks are already writing the next round while slow ones still read (two banks)."""
    import random
    import threading
    import time
    world, rounds = 4, 200
    slots = [[(0, 0.0)] * (2 * world) for _ in range(world)]      # slots[k][bank * world + r] = (round, value)
    results = [[None] * rounds for _ in range(world)]
    rng = random.Random(5)
    values = [[rng.random() for _ in range(rounds)] for _ in range(world)]
    errors = []

    def rank_main(r):
        local = random.Random(100 + r)
        for e in range(1, rounds + 1):
            bank = (e & 1) * world
            if local.random() < 0.3:
                time.sleep(local.random() * 1e-4)
            for k in range(world):                                 # "release" stores into every rank's array
                slots[k][bank + r] = (e, values[r][e - 1])
            got = []
            for t in range(world):                                 # bounded wait on the own array
                t0 = time.time()
                while slots[r][bank + t][0] < e:
                    if time.time() - t0 > 5.0:
                        errors.append((r, e, t))
                        return
                    time.sleep(0)
                got.append(slots[r][bank + t])
            # a word may already carry a LATER round of the same bank only if that rank passed round e + 1, which
            # needs this rank's round e + 1 store -- impossible while this rank is still in round e
            if any(rd != e for rd, _ in got):
                errors.append((r, e, "overwritten"))
                return
            results[r][e - 1] = max(v for _, v in got)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
    for e in range(rounds):
        want = max(values[r][e] for r in range(world))
        assert all(results[r][e] == want for r in range(world))


def test_reference_import_names_resolve_to_one_copy_of_each_module():
    """The reference's scripts do `from cuda.kernels import *` and call `cuda_kernels.get_scale`
    (evaluation/test_fuse.py:48-49, evaluation/SPMM_broadcast.py:15); after install_as_cuda() those names are the same
    objects as tango_b200's, and a setting made through one name is seen through the other."""
    import importlib
    import sys
    import tango_b200
    tango_b200.install_as_cuda()
    try:
        ns = {}
        exec("from cuda.kernels import *\nfrom cuda.QLinear import QLinear, Qlinear_func, Qlinear_func_reduce\n"
             "from cuda.SPMM import spmm_copy_u, spmm_u_mul_e\nfrom cuda.SDDMM import sddmm_u_add_v\n"
             "from cuda.util import graph_preprocess\nimport cuda, cuda.config", ns)
        assert ns["cuda"] is tango_b200
        assert ns["cuda_kernels"] is tango_b200.kernels.cuda_kernels
        assert ns["cuda_kernels"].get_scale is tango_b200.kernels._get_scale
        for name in ("quantize", "mySDDMM_int8", "QGEMM_forward", "QGEMM_backward", "transpose_quant",
                     "multi_cusparse_SPMM", "incidence_SPMM", "csr_SPMM", "multi_cusparse_SPMV"):
            assert ns[name] is getattr(tango_b200.kernels, name), name
        assert ns["QLinear"] is tango_b200.QLinear and ns["spmm_copy_u"] is tango_b200.spmm_copy_u
        assert ns["sddmm_u_add_v"] is tango_b200.sddmm_u_add_v and ns["graph_preprocess"] is tango_b200.graph_preprocess
        assert importlib.import_module("cuda.kernels") is tango_b200.kernels
        assert importlib.import_module("cuda.QLinear") is sys.modules["tango_b200.QLinear"]
        old = config.get_rounding()
        try:
            ns["cuda"].config.set_rounding("stochastic", seed=5)
            assert tango_b200.config.get_rounding() == "stochastic" and tango_b200.config.seed() == 5
            assert sys.modules["cuda.config"].mode_for("quantize") == tango_b200.kernels.ROUND_STOCHASTIC
        finally:
            config.set_rounding(old)
    finally:
        for k in [k for k in sys.modules if k == "cuda" or k.startswith("cuda.")]:
            if sys.modules[k] is tango_b200 or getattr(sys.modules[k], "__name__", "").startswith("tango_b200"):
                del sys.modules[k]


def test_dw_workspace_query_saturates_instead_of_wrapping():
    from tango_b200 import _lib
    L = _lib.lib
    assert L.tango_qgemm_dw_workspace_bytes(256, 602) == 256 * 604 * 4
    big = 2 ** 62
    assert L.tango_qgemm_dw_workspace_bytes(big, big) == 2 ** 63 - 1
    assert L.tango_qgemm_dw_workspace_bytes(3, 2 ** 63 - 2) == 2 ** 63 - 1
    # the entry point with built-in scratch refuses such sizes before any CUDA call
    assert L.tango_qgemm_dw_noalloc(None, 16, None, 16, 8, 2 ** 31, 2 ** 31, None, None, None, 2 ** 31, None, None) == -5
    assert L.tango_qgemm_dw_noalloc(None, 16, None, 16, 8, 2 ** 40, 4, None, None, None, 4, None, None) == -5


def test_hub_block_partitions_the_edges_exactly():
    """Dense hub region (stored tile by tile) + remaining CSR = the original adjacency, edge for edge; the region's
    rows lead heavy_rows and row_order, the row kernels are told to skip them, and the GEMM work items cover every
    stored tile exactly once."""
    g = rmat_graph(3000, 60000, 5, device="cpu")
    ip, idx, _ = g.adj_csc
    n = g.num_nodes()
    full = torch.zeros((n, n), dtype=torch.int32)
    rows = torch.repeat_interleave(torch.arange(n), (ip[1:] - ip[:-1]).long())
    full.index_put_((rows, idx.long()), torch.ones(1, dtype=torch.int32).expand(idx.numel()), accumulate=True)
    for caps in ((256, 384, 0.0), (1024, 1024, 0.035)):
        hub = HubBlock(ip, idx, n, *caps)
        assert hub.ok and 0 < hub.density < 1 and hub.dense.shape == (hub.n_tiles * 128, 128)
        if caps[2] == 0.0:
            assert hub.kend.tolist() == [3, 3]                      # every tile inside the caps
        else:
            assert hub.kend[0] == hub.kend.max() and hub.kend.min() >= 0   # a staircase
        rest = torch.zeros_like(full)
        trows = torch.repeat_interleave(torch.arange(n), (hub.indptr[1:] - hub.indptr[:-1]).long())
        rest.index_put_((trows, hub.indices.long()), torch.ones(1, dtype=torch.int32).expand(hub.indices.numel()),
                        accumulate=True)
        rest[hub.rows.long()[:, None], hub.cols.long()[None, :]] += hub.to_dense()
        assert torch.equal(full, rest)
        covered = torch.zeros(hub.n_tiles, dtype=torch.int32)
        base = torch.cumsum(hub.kend, 0) - hub.kend
        for rt, t0, k0, cnt in hub.units.tolist():
            assert t0 == int(base[rt]) + k0 and k0 + cnt <= int(hub.kend[rt])
            covered[t0:t0 + cnt] += 1
        assert bool((covered == 1).all())
        s = hub.schedule
        nr = hub.rows.numel()
        assert s.n_skip == s.n_heavy >= nr and torch.equal(s.heavy_rows[:nr], hub.rows)
        assert torch.equal(s.row_order[:s.n_skip], s.heavy_rows)
        assert sorted(s.row_order.tolist()) == list(range(n))
        tail_deg = (hub.indptr[1:] - hub.indptr[:-1]).long()
        assert bool((tail_deg[s.row_order[s.n_skip:].long()] <= s.threshold).all())
    # nothing is dense enough at a bar of 90 %
    assert not HubBlock(ip, idx, n, 256, 384, 0.9).ok


def _emulate_hub_aggregation(hub, feats_i64):
    """What the kernels do with a HubBlock, in NumPy: every GEMM work item adds its run of stored tiles times the
    matching 128-row slices of the packed hub features into the scratch rows of its row tile; the remaining edges are
    gathered; both meet as exact integers."""
    T = 128
    n_rows = hub.indptr.numel() - 1
    acc = np.zeros((n_rows, feats_i64.shape[1]), dtype=np.int64)
    packed = feats_i64[hub.cols.numpy().astype(np.int64)]                       # gather_rows_kernel
    dense = hub.dense.numpy().astype(np.int64)
    rows = hub.rows.numpy().astype(np.int64)
    for rt, t0, k0, cnt in hub.units.tolist():                                  # igemm_kernel, tile-list mode
        part = np.zeros((T, feats_i64.shape[1]), dtype=np.int64)
        for t in range(cnt):
            part += dense[(t0 + t) * T:(t0 + t + 1) * T] @ packed[(k0 + t) * T:(k0 + t + 1) * T]
        acc[rows[rt * T:(rt + 1) * T]] += part
    ip = hub.indptr.numpy().astype(np.int64)
    idx = hub.indices.numpy().astype(np.int64)
    np.add.at(acc, np.repeat(np.arange(n_rows), np.diff(ip)), feats_i64[idx])    # the gather kernels on the remainder
    return acc


def test_hub_region_work_items_reproduce_the_aggregation():
    g = rmat_graph(3000, 90000, 7, device="cpu")
    ip, idx, _ = g.adj_csc
    rng = np.random.default_rng(0)
    nq = rng.integers(-127, 128, (3000, 24)).astype(np.int64)
    want = O.spmm_copy_u_acc(ip.numpy().astype(np.int64), idx.numpy().astype(np.int64), nq)
    for caps in ((512, 640, 0.0), (2048, 2048, 0.03)):
        hub = HubBlock(ip, idx, 3000, *caps)
        assert hub.ok and hub.units.shape[0] >= hub.kend.numel() - int((hub.kend == 0).sum())
        np.testing.assert_array_equal(_emulate_hub_aggregation(hub, nq), want)


def test_hub_region_on_a_row_partition_reproduces_the_aggregation():
    """The multi-GPU form: every rank builds the hub region of ITS rows over the columns of the gathered table (rank
    k's rows at k * shard_rows); emulated in NumPy, the ranks together give the unpartitioned aggregation."""
    n, world = 2500, 3
    g = rmat_graph(n, 80000, 9, device="cpu")
    ip, idx, _ = g.adj_csc
    rng = np.random.default_rng(1)
    nq = rng.integers(-127, 128, (n, 16)).astype(np.int64)
    want = O.spmm_copy_u_acc(ip.numpy().astype(np.int64), idx.numpy().astype(np.int64), nq)
    order = torch.argsort(g.in_degrees() + g.out_degrees(), descending=True, stable=True)
    parts = [RowPartition(ip, idx, None, n, r, world, None, "dealt", order) for r in range(world)]
    shard = parts[0].shard_rows
    table = np.zeros((world * shard, 16), dtype=np.int64)                        # what the exchange leaves on every rank
    for r, p in enumerate(parts):
        table[r * shard:r * shard + p.n_local] = nq[p.local_ids.numpy()]
    for p in parts:
        hub = HubBlock(p.indptr_flat, p.indices, world * shard, 256, 384, 0.0)
        assert hub.ok and hub.n_block_edges > 0
        got = _emulate_hub_aggregation(hub, table)
        np.testing.assert_array_equal(got, want[p.local_ids.numpy()])


def test_hub_self_check_accepts_a_faithful_region_and_rejects_a_lossy_one(monkeypatch):
    """kernels.hub_self_check compares the aggregation with and without the dense hub region on one random table.
    With the native call replaced by the NumPy emulation it must say yes; with an emulation that forgets the dense
    part (what a broken GEMM pass would amount to) it must say no."""
    from tango_b200 import kernels as K
    g = rmat_graph(2000, 60000, 3, device="cpu")
    ip, idx, _ = g.adj_csc
    hub = HubBlock(ip, idx, 2000, 512, 512, 0.0)
    assert hub.ok and hub.n_block_edges > 0

    def fake(drop_dense):
        def _csr_spmm(out, indptr, indices, U, scaleU, sched=None, nseg=1, *a, **k):
            feats = U.numpy().astype(np.int64)
            if getattr(sched, "hub", None) is not None and not drop_dense:
                acc = _emulate_hub_aggregation(sched.hub, feats)
            else:
                acc = O.spmm_copy_u_acc(indptr.numpy().astype(np.int64), indices.numpy().astype(np.int64), feats)
            out.copy_(torch.from_numpy(acc.astype(np.float32)))
        return _csr_spmm

    assert hub.schedule.hub is hub
    monkeypatch.setattr(K, "_csr_spmm", fake(False))
    assert K.hub_self_check(hub, ip, idx, SpmmSchedule(ip), 2000, f=16)
    monkeypatch.setattr(K, "_csr_spmm", fake(True))
    assert not K.hub_self_check(hub, ip, idx, SpmmSchedule(ip), 2000, f=16)
