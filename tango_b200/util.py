"""graph_preprocess of the reference's cuda/util.py:5-11, for the DGL-free `Graph`."""
from __future__ import annotations

from .graph import Graph, SpmmSchedule


def graph_preprocess(graph: Graph) -> Graph:
    """Materialises the CSR / CSC index bundles (and the long-row schedules of the SpMM kernels) once, so that no
    operator call pays for a sort.  `graph.coo`, `graph.inc_in` and `graph.inc_out` are derived on access."""
    assert graph.device.type == "cuda", "graph must be on GPU"
    for fmt in ("csr", "csc"):
        indptr, _, _ = graph.adj_sparse(fmt)
        graph._plans[fmt] = SpmmSchedule(indptr)
    return graph
