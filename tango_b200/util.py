"""graph_preprocess of the reference's cuda/util.py:5-11, for the DGL-free `Graph`."""
from __future__ import annotations

import warnings

from . import config
from .graph import HUB_BLOCK_MIN_DENSITY, Graph, HubBlock, SpmmSchedule

HUB_BLOCK_MIN_EDGES = 4_000_000     # smaller graphs are launch-bound: the extra launches would cost more than they save


def graph_preprocess(graph: Graph, hub_block=None) -> Graph:
    """Materialises the CSR / CSC index bundles (and the long-row schedules of the SpMM kernels) once, so that no
    operator call pays for a sort.  `graph.coo`, `graph.inc_in` and `graph.inc_out` are derived on access.

    hub_block: largest side (rows, columns) of the dense hub region that the unweighted aggregation (csr_SPMM /
    spmm_copy_u) multiplies on the tensor cores instead of gathering (see graph.HubBlock); None takes
    config.hub_block() (0 = off), and the region is then only built for graphs large enough to profit and only from
    tiles dense enough to pay; an explicit side is always honoured and takes every tile inside it."""
    assert graph.device.type == "cuda", "graph must be on GPU"
    side = config.hub_block() if hub_block is None else int(hub_block)
    forced = hub_block is not None
    graph._hubs = {}
    for fmt in ("csr", "csc"):
        indptr, indices, _ = graph.adj_sparse(fmt)
        graph._plans[fmt] = SpmmSchedule(indptr)
        if side > 0 and (forced or graph.num_edges() >= HUB_BLOCK_MIN_EDGES):
            hub = HubBlock(indptr, indices, graph.num_nodes(), side, side, 0.0 if forced else HUB_BLOCK_MIN_DENSITY)
            if hub.ok:
                from . import kernels
                if kernels.hub_self_check(hub, indptr, indices, graph._plans[fmt], graph.num_nodes()):
                    graph._hubs[fmt] = hub
                else:
                    warnings.warn(f"dense hub region of the {fmt} aggregation did not reproduce the gathered result; "
                                  "not used", RuntimeWarning)
    return graph
