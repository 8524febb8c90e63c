"""The GAT attention path that never materialises the attention weights in fp32: softmax statistics per destination,
int8 weights written once, a backward pass that recomputes the weights -- against the path that writes the weights
as fp32 [E, H] and quantizes them afterwards (itself held to the oracle in test_gpu_primitives / test_gpu_models)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _setup(n=1500, e=20000, seed=3):
    import tango_b200 as T
    from tango_b200.graph import rmat_graph
    g = rmat_graph(n, e, seed, device="cuda")
    T.graph_preprocess(g)
    return g


@pytest.mark.parametrize("rounding", ["reference", "stochastic"])
def test_gat_without_fp32_attention_is_bit_identical(cuda, rounding):
    """The GAT layer that never materialises the attention weights in fp32 (softmax statistics -> int8 weights
    written once -> backward recomputes the weights) against the path that writes them as fp32 [E, H] and quantizes
    them afterwards: same int8 weights, hence identical logits and identical gradients, in the deterministic modes
    and with the seeded stochastic stream."""
    from tango_b200 import config, kernels as K
    from tango_b200.gnn import GAT
    g = _setup(1500, 40000, 37)
    n = g.num_nodes()
    torch.manual_seed(8)
    x = torch.randn(n, 64, device="cuda")
    y = torch.randint(0, 6, (n,), device="cuda")
    res = []
    config.set_rounding(rounding, seed=77)
    try:
        for fused in (True, "int8"):
            torch.manual_seed(9)
            K.set_call_counter(100)
            m = GAT(g, 2, 64, 16, 6, [4, 1], fused=fused).cuda()
            logits = m(x)
            F.cross_entropy(logits, y).backward()
            res.append((logits.detach(), [p.grad.clone() for p in m.parameters()]))
    finally:
        config.set_rounding("reference")
    if rounding == "reference":
        assert torch.equal(res[0][0], res[1][0])
        for a, b in zip(res[0][1], res[1][1]):
            assert torch.equal(a, b)
    else:
        # the two paths draw their per-call counters in a different order, so the noise differs: same statistics only
        assert (res[0][0] - res[1][0]).abs().max() / res[1][0].abs().max() < 0.1


def test_gat_int8_attention_weights_match_the_quantized_fp32_weights(cuda):
    """Kernel level: stats + quantized emit == quantize(edge_softmax fp32) with the scale max|a| / 127, in all three
    rounding modes, on an arbitrarily numbered graph (edge_ids indirection) with a long row."""
    from tango_b200 import kernels as K
    from tango_b200.graph import rmat_graph
    import tango_b200 as T
    g = rmat_graph(800, 30000, 23, device="cuda", edge_order="append")
    T.graph_preprocess(g)
    n, e = g.num_nodes(), g.num_edges()
    torch.manual_seed(1)
    for h in (4, 1, 3):
        el = torch.randint(-127, 128, (n, h), dtype=torch.int8, device="cuda")
        er = torch.randint(-127, 128, (n, h), dtype=torch.int8, device="cuda")
        sl, sr = torch.tensor([0.02], device="cuda"), torch.tensor([0.015], device="cuda")
        a, sa = K.gat_edge_softmax(g, el, er, sl, sr, 0.2, want_scale=True)
        m, inv, sa2 = K.gat_edge_softmax_stats(g, el, er, sl, sr, 0.2)
        assert sa2.item() == sa.item()
        for mode in (0, 1, 2):
            want, _ = K.quantize(a, sa, mode=mode, seed=5, call=9, align=1)
            got = K.gat_edge_softmax_quantized(g, el, er, sl, sr, m, inv, sa2, 0.2, mode, 5, 9)
            assert torch.equal(got, want.reshape(e, h)), (h, mode)
        da = torch.randn(e, h, device="cuda")
        dz1, s1 = K.gat_edge_softmax_bwd(g, el, er, sl, sr, a, da, 0.2, want_scale=True)
        dz2, s2 = K.gat_edge_softmax_bwd_stats(g, el, er, sl, sr, m, inv, da, 0.2)
        assert torch.equal(dz1, dz2) and s1.item() == s2.item()
