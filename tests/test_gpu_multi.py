"""Row-partitioned training on 2 GPUs against the single-GPU model (needs >= 2 CUDA devices; skipped otherwise).
NVLS is switched off for these child processes."""
import os
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn_with_deadline(fn, args, world, deadline_s=300):
    """mp.spawn, but a rank that never comes back fails the test instead of blocking the whole run: after the
    deadline the children started here (and only those) are terminated."""
    ctx = mp.spawn(fn, args=args, nprocs=world, join=False)
    t0 = time.monotonic()
    while not ctx.join(timeout=5):          # raises if a child raised (and ends the others)
        if time.monotonic() - t0 > deadline_s:
            for p in ctx.processes:
                if p.is_alive():
                    p.terminate()
            for p in ctx.processes:
                p.join(10)
                if p.is_alive():
                    p.kill()
            pytest.fail(f"ranks still running after {deadline_s} s")


def _worker(rank, world, port, out_dir, balance, scale_mode, transport="nccl", hub=0):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import torch.nn.functional as F
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import tango_b200.dist as tdist
    from tango_b200 import config
    from tango_b200.dist import DistGCN, DistGraph, allreduce_grads
    from tango_b200.graph import rmat_graph
    n = 5003
    g = rmat_graph(n, 120000, 17, device=dev)
    config.set_hub_block(hub)
    if hub:
        tdist.HUB_BLOCK_MIN_EDGES = 0          # force the dense hub region on this small graph:
        tdist.HUB_BLOCK_MIN_DENSITY = 0.0      # every tile inside the 256 x 256 caps
    dg = DistGraph(g, rank, world, balance=balance, scale_mode=scale_mode, transport=transport)
    assert bool(dg.hubs) == bool(hub)
    torch.manual_seed(4)
    model = DistGCN(dg, 100, 32, 7, 1).to(dev)
    gen = torch.Generator().manual_seed(9)
    x = torch.randn((n, 100), generator=gen)[dg.local_ids.cpu()].to(dev)
    y = torch.randint(0, 7, (n,), generator=gen)[dg.local_ids.cpu()].to(dev)
    logits = model(x)
    loss = F.cross_entropy(logits, y, reduction="sum") / n
    loss.backward()
    allreduce_grads(model, peer=dg.peer)
    if dg.peer is not None:
        dg.peer.raise_if_expired()
    lt = loss.detach().clone()
    dist.all_reduce(lt)
    torch.save({"logits": logits.detach().cpu(), "ids": dg.local_ids.cpu(), "loss": lt.cpu(),
                "grads": [p.grad.cpu() for p in model.parameters()],
                "peer_status": dg.peer.status() if dg.peer is not None else 0}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("balance,scale_mode,transport",
                         [("dealt", "global", "nccl"), ("nnz", "global", "nccl"), ("rows", "shard", "nccl"),
                          ("dealt", "shard", "nccl"), ("cyclic", "global", "nccl"), ("dealt", "global", "peer"),
                          ("nnz", "global", "peer")])
def test_two_gpu_gcn_matches_single_gpu(cuda, tmp_path, balance, scale_mode, transport):
    check_two_gpu_gcn(tmp_path, balance, scale_mode, transport, 0)


def check_two_gpu_gcn(tmp_path, balance, scale_mode, transport, hub):
    """One training step on 2 ranks against the single-GPU model (also used, with the dense hub region forced on the
    ranks' partitions, by test_zzz_gpu_multi_hub.py)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.nn.functional as F
    import tango_b200 as T
    from tango_b200.gnn import GCN
    from tango_b200.graph import rmat_graph
    world = 2
    _spawn_with_deadline(_worker, (world, _free_port(), str(tmp_path), balance, scale_mode, transport, hub), world)
    n = 5003
    g = rmat_graph(n, 120000, 17, device="cuda")
    T.graph_preprocess(g)
    torch.manual_seed(4)
    model = GCN(g, 100, 32, 7, 1).cuda()
    gen = torch.Generator().manual_seed(9)
    x = torch.randn((n, 100), generator=gen).cuda()
    y = torch.randint(0, 7, (n,), generator=gen).cuda()
    logits = model(x)
    loss = F.cross_entropy(logits, y)
    loss.backward()
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert all(p["peer_status"] == 0 for p in parts)          # no rendezvous wait expired
    ref = logits.detach().cpu()
    got = torch.empty_like(ref)
    for p in parts:
        got[p["ids"]] = p["logits"]
    if scale_mode == "global":
        # one scale agreed by all ranks: every int8 tensor, hence every logit, equals the single-GPU run's
        assert torch.equal(got, ref)
    else:
        # per-shard scales: same math, slightly different quantisation grid
        # (the int8 grid of each shard differs from the single-GPU grid by the ratio of the absmax values, so the
        # difference is of the order of the quantisation error itself: a few percent of the logits' norm)
        assert (got - ref).abs().max() / ref.abs().max() < 1e-1
        assert (got - ref).norm() / ref.norm() < 5e-2
    assert abs(parts[0]["loss"].item() - loss.item()) / loss.item() < 1e-3
    for gq, p in zip(parts[0]["grads"], model.parameters()):
        gr = p.grad.cpu()
        cos = torch.dot(gq.flatten(), gr.flatten()) / (gq.norm() * gr.norm())
        assert cos > 0.99, cos
