"""Whole models on the benchmark configurations' shapes against the float64 CPU models of the
oracle: logits, loss and every parameter gradient.

C1 (2,708-node GAT 8x8 -> 1x7 with ELU) and C4 (19,717-node MoNet, K=3, D=2, tanh pseudo
projection) run at full size; C2, C3 and C5 run the benchmark's own generators at a reduced
scale (same architecture, same degree law, fewer nodes).  Parameters are copied from the GPU
model into the CPU model, so both compute the same function.

Tolerance: |a - e| <= 1e-5 * max(1, max|e|) + 1e-4 * |e| (several layers of fp32 sums; the
dense projections go through the 3xTF32 tensor-core GEMM).
"""
import pytest
import torch
import torch.nn.functional as F

from tests.util import assert_close

pytestmark = pytest.mark.gpu

SCALES = {"C1": 1.0, "C2": 1.0 / 64, "C3": 1.0 / 8, "C4": 1.0, "C5": 1.0 / 256}


def _copy_params(kind, gpu_model, cpu_model):
    """GPU model parameters -> the CPU model's differently organised parameters."""
    with torch.no_grad():
        if kind == "gat":
            for i, layer in enumerate(gpu_model.gat_layers):
                cpu_model.W[i].copy_(layer.W.cpu())
                cpu_model.al[i].copy_(layer.attn_l.cpu())
                cpu_model.ar[i].copy_(layer.attn_r.cpu())
        elif kind == "edgeconv":
            for i, conv in enumerate(gpu_model.conv):
                cpu_model.theta[i].weight.copy_(conv.theta.weight.cpu())
                cpu_model.phi[i].weight.copy_(conv.phi.weight.cpu())
            cpu_model.proj_output.load_state_dict({k: v.cpu() for k, v in gpu_model.proj_output.state_dict().items()})
        else:
            for i, layer in enumerate(gpu_model.layers):
                cpu_model.fc[i].weight.copy_(layer.fc.weight.cpu())
                cpu_model.mu[i].copy_(layer.mu.cpu())
                cpu_model.inv_sigma[i].copy_(layer.inv_sigma.cpu())
                cpu_model.bias[i].copy_(layer.bias.cpu())
                cpu_model.pseudo_proj[i].load_state_dict(
                    {k: v.cpu() for k, v in gpu_model.pseudo_proj[i].state_dict().items()})


def _param_pairs(kind, gpu_model, cpu_model):
    if kind == "gat":
        for i, layer in enumerate(gpu_model.gat_layers):
            yield f"layer{i}.W", layer.W, cpu_model.W[i]
            yield f"layer{i}.attn_l", layer.attn_l, cpu_model.al[i]
            yield f"layer{i}.attn_r", layer.attn_r, cpu_model.ar[i]
    elif kind == "edgeconv":
        for i, conv in enumerate(gpu_model.conv):
            yield f"conv{i}.theta", conv.theta.weight, cpu_model.theta[i].weight
            yield f"conv{i}.phi", conv.phi.weight, cpu_model.phi[i].weight
        yield "proj.weight", gpu_model.proj_output.weight, cpu_model.proj_output.weight
        yield "proj.bias", gpu_model.proj_output.bias, cpu_model.proj_output.bias
    else:
        for i, layer in enumerate(gpu_model.layers):
            yield f"layer{i}.fc", layer.fc.weight, cpu_model.fc[i].weight
            yield f"layer{i}.mu", layer.mu, cpu_model.mu[i]
            yield f"layer{i}.inv_sigma", layer.inv_sigma, cpu_model.inv_sigma[i]
            yield f"layer{i}.bias", layer.bias, cpu_model.bias[i]
            yield f"layer{i}.pseudo.weight", gpu_model.pseudo_proj[i][0].weight, cpu_model.pseudo_proj[i][0].weight
            yield f"layer{i}.pseudo.bias", gpu_model.pseudo_proj[i][0].bias, cpu_model.pseudo_proj[i][0].bias


@pytest.mark.parametrize("name", ["C1", "C2", "C3", "C4", "C5"])
def test_model_matches_cpu_model(cuda, name):
    import bench
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from oracle import cpu_models

    wl = dict(bench.WORKLOADS[name], name=name)
    kind = wl["kind"]
    d = bench.build_inputs(wl, "cpu", seed=3, scale=SCALES[name])
    torch.manual_seed(5)
    model = bench.make_model(wl).to(cuda)
    if kind == "gat":
        cpu = cpu_models.CpuGAT(wl["in_dim"], wl["hidden"], wl["heads"], wl["classes"], 1, dtype=torch.float64)
    elif kind == "edgeconv":
        cpu = cpu_models.CpuDGCNN(wl["k"], wl["dims"], wl["classes"], dtype=torch.float64)
    else:
        cpu = cpu_models.CpuMoNet(wl["in_dim"], wl["hidden"], wl["classes"], 2, wl["dim"], wl["kernels"],
                                  dtype=torch.float64)
    cpu = cpu.double()
    if kind == "gmm":  # non-trivial Gaussian parameters and bias (the initial values are 1 and 0)
        with torch.no_grad():
            for layer in model.layers:
                layer.inv_sigma.uniform_(0.5, 1.5)
                layer.bias.normal_(0, 0.1)
    _copy_params(kind, model, cpu)

    labels = d["labels"]
    if kind == "edgeconv":
        out = model(d["points"].to(cuda), d["src"].to(cuda))
        eo = cpu(d["points"].double(), d["src"])
    else:
        g = d["graph"]
        rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
        cp, ri, pm = csr2csc(rp, ci)
        if kind == "gat":
            out = model(rp, ci, cp, ri, d["x"].to(cuda))
            eo = cpu(g.row_ptr, g.col_ind, d["x"].double())
        else:
            out = model(rp, ci, cp, ri, pm, d["x"].to(cuda), d["pseudo"].to(cuda))
            eo = cpu(g.row_ptr, g.col_ind, d["x"].double(), d["pseudo"].double())
    loss = bench.mean_cross_entropy(out, labels.to(cuda))
    loss.backward()
    eloss = F.cross_entropy(eo, labels)
    eloss.backward()

    assert_close(out, eo, f"{name} logits", scale_atol=True)
    assert_close(loss, eloss, f"{name} loss")
    for what, p, q in _param_pairs(kind, model, cpu):
        assert p.grad is not None and q.grad is not None, what
        assert_close(p.grad, q.grad, f"{name} grad {what}", scale_atol=True)
