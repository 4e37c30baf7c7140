"""Partitioned GAT on real GPUs (skipped with fewer than two): NCCL ranks running the
CUDA kernels must reproduce the single-GPU model's logits, loss and gradients, with both
exchange schemes (all-gather of every rank's rows; halo: only the rows a block references, moved by
an all-to-all; peer: the same rows stored straight into the receivers' buffers over NVLink)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.util import assert_close, power_law_graph

pytestmark = pytest.mark.gpu


def _inputs():
    g = power_law_graph(4000, 40, seed=5)
    x = torch.randn(g.n, 20, generator=torch.Generator().manual_seed(1))
    y = torch.randint(0, 6, (g.n,), generator=torch.Generator().manual_seed(2))
    return g, x, y


def _worker(rank, world, port, results, exchange="gather"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
        from ae_mlsys_gnn_b200.partition import PartitionedGAT, build_partition

        torch.manual_seed(0)
        g, x, y = _inputs()
        g = g.to(dev)
        cp, ri, _ = csr2csc(g.row_ptr, g.col_ind)
        blocks = exchange == "peer-blocks"  # projections by row blocks, finished blocks pushed early
        if blocks:
            from ae_mlsys_gnn_b200.halo import HaloGATConv

            HaloGATConv.OVERLAP_MIN_ROWS, HaloGATConv.OVERLAP_MIN_WIDTH = 128, 1
            exchange = "peer"
        if exchange in ("halo", "peer"):
            from ae_mlsys_gnn_b200.halo import HaloGAT, build_halo_partition

            part = build_halo_partition(g.row_ptr, g.col_ind, cp, ri, rank, world)
            model = HaloGAT(20, [16, 16], [4, 4], 6, 1, exchange="peer" if exchange == "peer" else "nccl").to(dev)
            if blocks:  # both kinds of work beside the main stream
                for layer in model.gat_layers:
                    layer.overlap_blocks, layer.side_weight_grads = 4, True
            max_n = max(part.bounds[r + 1] - part.bounds[r] for r in range(world))
        else:
            part = build_partition(g.row_ptr, g.col_ind, cp, ri, rank, world, pieces=1 if world == 2 else 3)
            model = PartitionedGAT(20, [16, 16], [4, 4], 6, 1).to(dev)
            max_n = part.max_n
        for _ in range(3 if exchange == "peer" else 1):  # both buffers of every exchange point get used
            model.zero_grad()
            out = model(part, part.pad_rows(part.local_slice(x.to(dev))))
            loss = model.loss(part, out, part.local_slice(y.to(dev)))
            loss.backward()
        model.all_reduce_grads(world)
        total = loss.detach().clone()
        dist.all_reduce(total)
        padded = out.detach().new_zeros(max_n, out.shape[1])
        padded[: out.shape[0]] = out.detach()
        gathered = torch.empty(world * max_n, out.shape[1], device=dev)
        dist.all_gather_into_tensor(gathered, padded)
        torch.cuda.synchronize()
        if rank == 0:
            full = torch.cat([gathered[r * max_n: r * max_n + part.bounds[r + 1] - part.bounds[r]]
                              for r in range(world)])  # plain rank-major gather of the outputs
            results["out"] = full.cpu()
            results["loss"] = total.cpu()
            results["grads"] = {k: p.grad.cpu() for k, p in model.named_parameters()}
            results["state"] = {k: v.cpu() for k, v in model.state_dict().items()}
        if hasattr(model, "close"):
            model.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("exchange", ["gather", "halo", "peer", "peer-blocks"])
@pytest.mark.parametrize("world", [2, 4])
def test_partitioned_gat_matches_single_gpu(cuda, world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from ae_mlsys_gnn_b200.models import GAT
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, results, exchange), nprocs=world, join=True)

    g, x, y = _inputs()
    g = g.to(cuda)
    cp, ri, _ = csr2csc(g.row_ptr, g.col_ind)
    model = GAT(20, [16, 16], [4, 4], 6, 1).to(cuda)
    model.load_state_dict({k: v.to(cuda) for k, v in results["state"].items()})
    out = model(g.row_ptr, g.col_ind, cp, ri, x.to(cuda))
    loss = torch.nn.functional.cross_entropy(out, y.to(cuda))
    loss.backward()
    assert_close(results["out"], out, "logits")
    assert_close(results["loss"], loss, "loss")
    for k, p in model.named_parameters():
        assert_close(results["grads"][k], p.grad, f"grad {k}", scale_atol=True)
